"""The Vozinex architecture without a GPU: its configuration reader, its schedule, the cache bookkeeping for windows
that keep first positions, and the plain implementation's own sanity (the planted key decides a probe's logits)."""
import copy

import numpy as np
import pytest
import torch

import plain_vozinex as PV
import tiny_vozinex as TV
from kindi_b200.cache.pages import PAGE, PageMap
from kindi_b200.cache.sequence_cache import SequenceCache
from kindi_b200.config import ConfigError
from kindi_b200.config.registry import model_from_config
from kindi_b200.parts.base import KVNeed
from kindi_b200.parts.model import cache_needs, expected_tensors


def test_config_reads_every_size_from_the_nested_keys():
    cfg, spec = model_from_config(TV.VZ_A)
    assert (cfg.vocab, cfg.width, cfg.eps) == (211, 64, 1e-5)
    assert [l.mlp is None for l in cfg.layers] == [False, True, False]
    m = cfg.layers[2].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.rot_dims, m.window, m.keep_first) == \
        (4, 4, 16, 8, 0.25, 16, 33, 1)
    assert cfg.to_dict() == TV.VZ_A
    names = expected_tensors(spec)
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.v"] == (48, 64) and names["l0.mix.o"] == (64, 96)
    assert names["l0.mix.q.norm"] == (64,) and names["l0.mix.k.norm"] == (32,)
    assert names["l0.norm1.b"] == (64,) and names["final.norm"] == (64,) and names["head"] == (211, 64)
    assert names["l0.mlp.router"] == (5, 64) and names["l0.mlp.router.b"] == (5,)
    assert names["l2.mlp.e4.up"] == (24, 64) and names["l2.mlp.e4.down"] == (64, 24)
    assert not any(n.startswith("l1.mlp") or n.startswith("l1.norm2") for n in names)
    assert spec.may_ignore == ("l1.norm2", "l1.norm2.b")       # (a folder may still store the unused norm)


@pytest.mark.parametrize("change,word", [
    (lambda c: c.update(bogus=1), "bogus"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=3.0), "softcap"),
    (lambda c: c["layers"][0].update(type="recurrent"), "recurrent"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "dense"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    c = copy.deepcopy(TV.VZ_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        model_from_config(c)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(TV.TINY))
def test_schedule_repeats_the_stretch_with_caches_of_its_own(name):
    raw = TV.TINY[name][0]
    cfg, spec = model_from_config(raw)
    want = PV.run_order(raw)
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == want
    assert [e.cache for e in spec.schedule] == list(range(len(want)))          # a cache entry per run
    needs = cache_needs(spec)
    for e in spec.schedule:
        m = cfg.layers[e.layer].mixer
        n = needs[e.cache]
        assert isinstance(n, KVNeed) and n.n_kv_heads == m.kv_heads and n.window == m.window
        assert n.keep_first == (m.keep_first if m.window else 0) and n.head_dim >= max(m.dim, m.vdim)


def test_no_loop_and_a_stretch_that_runs_once_add_nothing():
    c = copy.deepcopy(TV.VZ_A)
    c["loop"] = None
    _, spec = model_from_config(c)
    assert [(e.layer, e.add_embedding) for e in spec.schedule] == [(0, False), (1, False), (2, False)]
    c["loop"] = {"start": 0, "stop": 3, "times": 1}
    _, spec = model_from_config(c)
    assert not any(e.add_embedding for e in spec.schedule)


@pytest.mark.parametrize("window,keep", [(20, 3), (64, 0), (40, 70), (130, 64), (70, 65), (1, 1)])
def test_pages_behind_the_window_are_given_back_but_not_the_first_ones(window, keep):
    pm = PageMap(64, 2, window, keep)
    held_by_keep = -(-keep // PAGE)
    for length in list(range(1, 700, 7)) + [700]:
        pm.ensure(0, length)
        pm.trim(0, length)
        pm.check()
        blocks = set(pm.rows[0])
        first_needed = max(0, length - window + 1)            # the oldest position the NEXT query still reads
        for b in range(-(-length // PAGE)):
            needed = (b + 1) * PAGE > first_needed or b * PAGE < keep
            assert (b in blocks) == needed, (length, b)
        assert len(blocks) <= held_by_keep + -(-window // PAGE) + 1
    pm.release(0)
    pm.check()
    assert pm.pool.n_held == 0
    need = KVNeed(2, 16, window, keep)
    assert SequenceCache.group_pages(need, 1000, 4, 256) >= 4 * (held_by_keep + -(-window // PAGE) + 1) + 4


def test_mask_edges():
    v = PV.visible(12, 4, 2)
    assert v[9].tolist() == [True, True, False, False, False, False, True, True, True, True, False, False]
    assert v[3].tolist()[:5] == [True, True, True, True, False]
    assert PV.visible(5, None, 0)[4].all()


@pytest.mark.parametrize("name", ["A", "C"])
def test_the_planted_key_decides_a_probes_logits(tmp_path, name):
    """what the engine tests rest on: on the plain model, a probe row's logits move by many times the bfloat16
    tolerance when the needle's key is hidden from it, and not at all when the needle is out of its sight anyway"""
    folder = TV.make_model(tmp_path, name, "float32")
    raw = TV.TINY[name][0]
    m = PV.load_model(folder)
    import random
    rng = random.Random(5)
    window = min(l["mixer"]["mask"]["size"] for l in raw["layers"])
    widest = max(l["mixer"]["mask"]["size"] for l in raw["layers"])
    at = 2 + max(l["mixer"]["mask"]["keep_first"] for l in raw["layers"])      # past every layer's kept positions
    n = at + widest + 20
    inside, outside = at + window - 1, at + widest
    toks = TV.needle_request(raw["vocab"], n, at, [inside, outside], rng)
    full = PV.forward(m, toks).numpy()
    hidden = PV.forward(m, toks, hide=at).numpy()
    scale = np.abs(full).max()
    assert np.abs(full[inside] - hidden[inside]).max() > 0.15 * scale
    # (rows past the window see the needle only through what earlier rows made of it)
    assert np.abs(full[inside] - hidden[inside]).max() > 2 * np.abs(full[outside] - hidden[outside]).max()


@pytest.mark.parametrize("name", sorted(TV.TINY))
def test_no_routing_decision_of_the_test_models_is_a_close_call(tmp_path, name):
    """what lets the bfloat16 runs be compared row by row: in the test models the last chosen expert's logit lies well
    above the first one not chosen, in every row of every layer run"""
    import random
    folder = TV.make_model(tmp_path, name, "float32")
    raw = TV.TINY[name][0]
    m = PV.load_model(folder)
    rng = random.Random(8)
    toks = TV.needle_request(raw["vocab"], 300, 7, list(range(250, 300, 3)), rng)
    margins = []
    PV.forward(m, toks, margins=margins)
    if margins:
        assert float(torch.cat(margins).min()) > 0.1
