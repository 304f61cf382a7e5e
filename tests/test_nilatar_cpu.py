"""The Nilatar architecture without a GPU: its configuration reader, its schedule and cache needs (layers that read an
earlier layer's keys and values, state for the recurrent layers), the stretched rotation's frequencies, and the plain
implementation's own sanity (the planted key and the sinks decide a probe's logits; the recurrence and the absorbed
form of latent attention are what their definitions say)."""
import copy
import math
import random

import numpy as np
import pytest
import torch

import plain_nilatar as PN
import tiny_nilatar as TN
from kindi_b200.cache.sequence_cache import SequenceCache
from kindi_b200.config import ConfigError
from kindi_b200.config.registry import model_from_config
from kindi_b200.parts.base import KVNeed, StateNeed
from kindi_b200.parts.model import cache_needs, expected_tensors, tensor_inits
from kindi_b200.parts.rope import yarn_frequencies


def test_config_reads_every_size_from_the_nested_keys():
    cfg, spec = model_from_config(TN.NL_A)
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.embedding_scale) == (211, 64, 1e-5, 1.7)
    assert [l.kind for l in cfg.layers] == ["attention", "latent_attention", "lightning", "attention"]
    assert [l.ff for l in cfg.layers] == [40, 48, None, 40]
    m = cfg.layers[3].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.window, m.kv_from) == (4, 2, 16, 24, 0.25, 33, 0)
    m = cfg.layers[1].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.rot.base, m.rot.scaling) == \
        (4, 16, 8, 12, 24, 20, 10000.0, None)
    assert cfg.layers[2].mixer.decay == (0.9, 0.97)
    assert cfg.to_dict() == TN.NL_A
    assert model_from_config(TN.NL_B)[0].to_dict() == TN.NL_B
    names = expected_tensors(spec)
    assert names["embed"] == (211, 64) and names["head"] == (211, 64) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mix.g"] == (96, 64) and names["l0.mix.o"] == (64, 96) and names["l0.mix.sink"] == (4,)
    assert names["l0.ls1"] == (64,) and names["l0.ls2"] == (64,) and names["l0.norm2"] == (64,)
    assert names["l1.mix.dq"] == (24, 64) and names["l1.mix.dq.norm"] == (24,) and names["l1.mix.uq"] == (96, 24)
    assert names["l1.mix.dkv"] == (28, 64) and names["l1.mix.dkv.norm"] == (20,)
    assert names["l1.mix.uk"] == (64, 20) and names["l1.mix.uv"] == (48, 20) and names["l1.mix.g"] == (48, 64)
    assert names["l2.mix.q"] == (32, 64) and names["l2.mix.v"] == (48, 64) and names["l2.mix.norm"] == (48,)
    assert names["l2.mix.g"] == (48, 64) and names["l2.mix.o"] == (64, 48) and names["l2.ls1"] == (64,)
    assert not any(n.startswith(("l2.mlp", "l2.norm2", "l2.ls2")) for n in names)
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and names["l3.mix.q"] == (64, 64)
    assert names["l1.mlp.gate"] == (48, 64) and names["l1.mlp.down"] == (64, 48)
    inits = tensor_inits(spec)
    assert inits["l0.ls1"] == "gain" and inits["l1.mix.dq.norm"] == "gain" and inits["l2.mix.norm"] == "gain"


@pytest.mark.parametrize("change,word", [
    (lambda c: c.update(bogus=1), "bogus"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=3.0), "softcap"),
    (lambda c: c["layers"][0].update(type="recurrent"), "recurrent"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "moe"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(rot_dim=7), "rot_dim"),
    (lambda c: c["layers"][2]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=8), "differ"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    c = copy.deepcopy(TN.NL_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        model_from_config(c)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(TN.TINY))
def test_cache_needs_follow_the_mixers(name):
    raw = TN.TINY[name][0]
    cfg, spec = model_from_config(raw)
    needs = cache_needs(spec)
    assert [e.layer for e in spec.schedule] == list(range(len(raw["layers"])))
    for i, (layer, e) in enumerate(zip(raw["layers"], spec.schedule)):
        m = layer["mixer"]
        if layer["type"] == "lightning":
            assert needs[e.cache] == StateNeed((m["heads"], m["vdim"], m["dim"])) and e.reads_cache_of is None
        elif layer["type"] == "latent_attention":
            n = needs[e.cache]
            assert isinstance(n, KVNeed) and n.n_kv_heads == 1 and n.window is None
            assert n.head_dim >= m["kv_rank"] + m["rot_dim"]
        elif "kv_from" in m:
            assert e.reads_cache_of == m["kv_from"] and needs[e.cache] is None
        else:
            # the cache keeps what the widest window that reads it needs (all of it when one of them has no window)
            readers = [l["mixer"] for j, l in enumerate(raw["layers"])
                       if l["type"] == "attention" and (j == i or l["mixer"].get("kv_from") == i)]
            sizes = [r.get("mask", {}).get("size") for r in readers]
            n = needs[e.cache]
            assert isinstance(n, KVNeed) and n.n_kv_heads == m["kv_heads"] and n.head_dim >= max(m["dim"], m["vdim"])
            assert n.window == (None if None in sizes else max(sizes))
    # sizing the cache needs nothing but the needs
    assert SequenceCache.bytes_needed(needs, 1024, 4, torch.bfloat16, 256) > 0


def test_stretched_frequencies():
    """plain pairs keep base ** (-2 i / dims); with scaling the fast pairs stay, the slow pairs are divided by the
    factor, the pairs between are blended, and cosines and sines grow by 0.1 ln(factor) + 1"""
    f, m = yarn_frequencies(10000.0, 16, None)
    assert m == 1.0 and torch.allclose(f, torch.tensor([10000.0 ** (-2.0 * i / 16) for i in range(8)], dtype=torch.float64))
    sc = {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 1.0}
    f2, m2 = yarn_frequencies(40000.0, 16, sc)
    plain, _ = yarn_frequencies(40000.0, 16, None)
    dim_of = lambda t: 16 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(40000.0))
    lo, hi = max(math.floor(dim_of(4.0)), 0), min(math.ceil(dim_of(1.0)), 15)
    assert 0 <= lo < hi < 8                                   # the ramp lies inside the pairs
    for i in range(8):
        r = min(1.0, max(0.0, (i - lo) / (hi - lo)))
        assert abs(float(f2[i]) - float(plain[i]) * (r / 8.0 + 1.0 - r)) < 1e-15
    assert float(f2[0]) == float(plain[0]) and abs(float(f2[7]) - float(plain[7]) / 8.0) < 1e-18
    assert abs(m2 - (0.1 * math.log(8.0) + 1.0)) < 1e-15
    for raw in (TN.NL_B, TN.NL_C, TN.NL_D, TN.NL_E):
        for l in raw["layers"]:
            if l["type"] == "latent_attention":
                a, am = PN.rotation_table(l["mixer"]["rot"])
                b, bm = yarn_frequencies(l["mixer"]["rot"]["base"], l["mixer"]["rot"]["dims"],
                                         l["mixer"]["rot"].get("scaling"))
                assert float((a - b).abs().max()) < 1e-15 and abs(am - bm) < 1e-15


def test_rotation_pairs_neighbours():
    x = torch.arange(8, dtype=torch.float64).view(1, 8) + 1
    freq = torch.tensor([0.5, 0.25, 0.125, 1.0], dtype=torch.float64)
    y = PN.rotate_pairs(x, torch.tensor([3]), freq, 1.25)
    for i in range(4):
        a = 3 * float(freq[i])
        u, v = float(x[0, 2 * i]), float(x[0, 2 * i + 1])
        assert abs(float(y[0, 2 * i]) - 1.25 * (u * math.cos(a) - v * math.sin(a))) < 1e-12
        assert abs(float(y[0, 2 * i + 1]) - 1.25 * (v * math.cos(a) + u * math.sin(a))) < 1e-12


def test_window_and_sink_edges():
    q = torch.zeros(1, 6, 2, dtype=torch.float64)
    k = torch.zeros(1, 6, 2, dtype=torch.float64)
    v = torch.eye(6, dtype=torch.float64)[None]
    o = PN.softmax_attention(q, k, v, 1.0, 3, None)
    assert torch.allclose(o[0, 5], torch.tensor([0, 0, 0, 1 / 3, 1 / 3, 1 / 3], dtype=torch.float64))
    assert torch.allclose(o[0, 1], torch.tensor([0.5, 0.5, 0, 0, 0, 0], dtype=torch.float64))
    # a sink of ln 3 counts like three more keys of score 0, once, and has no value
    o = PN.softmax_attention(q, k, v, 1.0, 3, torch.tensor([math.log(3.0)]))
    assert torch.allclose(o[0, 5], torch.tensor([0, 0, 0, 1 / 6, 1 / 6, 1 / 6], dtype=torch.float64))
    assert torch.allclose(o[0, 0], torch.tensor([1 / 4, 0, 0, 0, 0, 0], dtype=torch.float64))
    o = PN.softmax_attention(q, k, v, 1.0, 1, None)
    assert torch.allclose(o[0], torch.eye(6, dtype=torch.float64))


def test_absorbed_latent_attention_is_the_same_function():
    """scores through W_uk^T q against the cached latent, values through W_uv after the weighted sum of latents: what
    the engine computes equals the expanded form of the definition"""
    raw = TN.NL_C["layers"][2]["mixer"]
    H, d, r, dv, qr, kr = raw["heads"], raw["dim"], raw["rot_dim"], raw["vdim"], raw["q_rank"], raw["kv_rank"]
    g = torch.Generator().manual_seed(1)
    width, T = 50, 30
    w = {n: torch.randn(s, generator=g, dtype=torch.float64) * 0.3 for n, s in {
        "dq": (qr, width), "uq": (H * (d + r), qr), "dkv": (kr + r, width), "uk": (H * d, kr), "uv": (H * dv, kr),
        "g": (H * dv, width), "o": (width, H * dv)}.items()}
    w["dq.norm"], w["dkv.norm"] = torch.rand(qr, generator=g, dtype=torch.float64) + 0.5, torch.rand(kr, generator=g, dtype=torch.float64) + 0.5
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    want = PN.latent_attention(h, w, raw, 1e-6)
    pos = torch.arange(T)
    freq, mult = PN.rotation_table(raw["rot"])
    cq = PN.rms_norm(h @ w["dq"].T, w["dq.norm"], 1e-6)
    q = (cq @ w["uq"].T).view(T, H, d + r)
    ckv = h @ w["dkv"].T
    c = PN.rms_norm(ckv[:, :kr], w["dkv.norm"], 1e-6)
    key = torch.cat([c, PN.rotate_pairs(ckv[:, kr:], pos, freq, mult)], dim=1)                      # [T, kr + r]
    q_abs = torch.einsum("thd,hdk->thk", q[..., :d], w["uk"].view(H, d, kr))
    qf = torch.cat([q_abs, PN.rotate_pairs(q[..., d:].transpose(0, 1), pos, freq, mult).transpose(0, 1)], dim=-1)
    o_lat = PN.softmax_attention(qf.transpose(0, 1), key[None].expand(H, T, kr + r), c[None].expand(H, T, kr),
                                 raw["scale"], None, None)
    o = torch.einsum("htk,hvk->thv", o_lat, w["uv"].view(H, dv, kr)).reshape(T, H * dv)
    got = (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert float((got - want).abs().max()) < 1e-12 * float(want.abs().max()) + 1e-13


def test_recurrence_equals_the_decayed_sum():
    """o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j"""
    m = {"heads": 2, "dim": 5, "vdim": 3, "decay": [0.8, 1.0]}
    g = torch.Generator().manual_seed(2)
    width, T = 12, 17
    w = {"q": torch.randn(10, width, generator=g, dtype=torch.float64), "k": torch.randn(10, width, generator=g, dtype=torch.float64),
         "v": torch.randn(6, width, generator=g, dtype=torch.float64), "g": torch.randn(6, width, generator=g, dtype=torch.float64),
         "o": torch.eye(6, dtype=torch.float64), "norm": torch.ones(6, dtype=torch.float64)}
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    got = PN.lightning(h, w, m, 1e-6)
    q, k, v = (PN.silu(h @ w[n].T) for n in "qkv")
    o = torch.zeros(T, 2, 3, dtype=torch.float64)
    for hd, lam in enumerate(m["decay"]):
        for t in range(T):
            for j in range(t + 1):
                o[t, hd] += lam ** (t - j) * (q[t, hd * 5:hd * 5 + 5] @ k[j, hd * 5:hd * 5 + 5]) * v[j, hd * 3:hd * 3 + 3]
    want = PN.rms_norm(o.view(T, 6), w["norm"], 1e-6) * torch.sigmoid(h @ w["g"].T)
    assert float((got - want).abs().max()) < 1e-12


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_the_planted_key_and_the_sinks_decide_a_probes_logits(tmp_path, name):
    """what the engine tests rest on: on the plain model, a probe row's logits move by many times the bfloat16
    tolerance when the needle is taken away, and by more than the 32-bit tolerance when the sinks are"""
    folder = TN.make_model(tmp_path, name, "float32")
    raw = TN.TINY[name][0]
    cfg, w = PN.load_model(folder)
    rng = random.Random(5)
    toks = TN.needle_request(raw["vocab"], 200, 150, list(range(194, 200)), rng)
    full = PN.forward(cfg, w, toks).numpy()
    gone = list(toks)
    gone[150] = 7
    hidden = PN.forward(cfg, w, gone).numpy()
    scale = np.abs(full).max()
    assert np.abs(full[194:] - hidden[194:]).max() > 0.1 * scale
    no_sink = {n: (t - 50.0 if n.endswith(".sink") else t) for n, t in w.items()}
    assert np.abs(PN.forward(cfg, no_sink, toks).numpy() - full).max() > 1e-3 * scale
