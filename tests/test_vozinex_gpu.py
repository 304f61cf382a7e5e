"""The Vozinex architecture on the GPU against the plain implementation (``plain_vozinex``): each mechanism's kernel
alone, then whole models of five small configurations through the engine's step function, its cache and its
generation loop, in true 32-bit and in bfloat16.

The models carry a planted key (``tiny_vozinex.make_model``): a probe token's attention rests on one needle token,
so a dropped key, a window or a kept stretch that is one position off, a page of another sequence or a slot's old
content changes a probe's logits by many times the tolerance (``test_vozinex_cpu`` measures that on the plain model).
"""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vozinex as PV
import tiny
import tiny_vozinex as TV

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 3e-5, "bfloat16": 2e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def K():
    from kindi_b200.kernels import lib
    lib.load()
    return lib


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-30))


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("T,E,planes,ydtype", [(1, 64, 0, "float32"), (5, 200, 3, "float32"), (33, 72, 1, "bfloat16"),
                                               (3, 4100, 2, "float32"), (130, 256, 9, "bfloat16"),
                                               (2, 14000, 1, "float32")])
def test_add_layernorm(K, T, E, planes, ydtype):
    g = torch.Generator().manual_seed(T * 1000 + E)
    x = torch.randn(T, E, generator=g) * 3 + 1.5             # a mean that matters
    d = torch.randn(planes, T, E, generator=g) if planes else None
    w, b = torch.randn(E, generator=g) + 1, torch.randn(E, generator=g)
    v = x.double() + (d.double().sum(0) if planes else 0)
    want = PV.layer_norm(v, w.double(), b.double(), 1e-5)
    xd, out = x.cuda(), torch.empty(T, E, dtype=DT[ydtype], device="cuda")
    st = _status()
    K.add_layernorm(xd, d.cuda() if planes else None, w.cuda(), b.cuda(), 1e-5, out, None, planes > 0, st)
    assert _rel(out, want) < (1e-5 if ydtype == "float32" else 8e-3) and int(st.item()) == 0
    if planes:
        assert _rel(xd, v) < 1e-6                             # the sum was written back
    # chosen rows, nothing written back
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    x2, out2 = x.cuda(), torch.empty(2, E, dtype=DT[ydtype], device="cuda")
    K.add_layernorm(x2, d.cuda() if planes else None, w.cuda(), b.cuda(), 1e-5, out2, rows, False, st)
    assert torch.equal(out2, out[[T - 1, 0]]) and torch.equal(x2.cpu(), x)


def test_residual_add(K):
    g = torch.Generator().manual_seed(1)
    x, d, e = torch.randn(37, 50, generator=g), torch.randn(3, 37, 50, generator=g), torch.randn(37, 50, generator=g)
    xd = x.cuda()
    K.residual_add(xd, d.cuda(), e.cuda())
    assert _rel(xd, x.double() + d.double().sum(0) + e.double()) < 1e-6
    xd = x.cuda()
    K.residual_add(xd, None, e.cuda())
    assert torch.equal(xd.cpu(), x + e)


def _cache(lengths, nkv, hd, dtype, seed, extra=3):
    """pool [pages, 2, nkv, 64, hd] with every sequence's pages scattered, and the page table"""
    rng = random.Random(seed)
    n_blocks = [-(-n // 64) for n in lengths]
    n_pages = sum(n_blocks) + extra
    order = list(range(n_pages))
    rng.shuffle(order)
    table = torch.full((len(lengths), max(n_blocks) + 1), -1, dtype=torch.int32)
    at = 0
    for s, nb in enumerate(n_blocks):
        for b in range(nb):
            table[s, b] = order[at]
            at += 1
    # (what a page holds past its sequence's end is some other sequence's old content: finite, and large here)
    pool = (torch.randn((n_pages, 2, nkv, 64, hd), generator=torch.Generator().manual_seed(seed)) * 50).to(dtype)
    return pool, table, n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,nh,nkv,d,hd,rot,planes", [(7, 4, 2, 16, 16, 8, 1), (40, 6, 2, 64, 64, 32, 3),
                                                     (3, 4, 1, 24, 64, 24, 2), (65, 5, 5, 24, 24, 0, 1),
                                                     (9, 8, 1, 64, 128, 64, 4)])
def test_projection_norm_rotation_and_store(K, dtype, T, nh, nkv, d, hd, rot, planes):
    """q and k are normalised over the whole projection (its true size d per head, whatever the cache's head size hd),
    rotated over their first `rot` dimensions and stored; from rows and from 32-bit planes"""
    g = torch.Generator().manual_seed(T + nh)
    tdt = DT[dtype]
    q, k, v = (torch.randn(T, n, d, generator=g) for n in (nh, nkv, nkv))
    wq, wk = ((torch.rand(n, d, generator=g) + 0.5).to(tdt).float() for n in (nh, nkv))
    if planes == 1:
        q, k, v = (x.to(tdt).float() for x in (q, k, v))          # the rows as the kernel reads them
    pos = torch.tensor([3 * t + 60 for t in range(T)], dtype=torch.int32)      # positions that cross a page
    pos[0] = 0
    qn = PV.projection_rms_norm(q.double().view(T, -1), wq.double().view(-1), 1e-5).view(T, nh, d)
    kn = PV.projection_rms_norm(k.double().view(T, -1), wk.double().view(-1), 1e-5).view(T, nkv, d)
    qn, kn = PV.rotate_first_dims(qn, pos, rot, 10000.0), PV.rotate_first_dims(kn, pos, rot, 10000.0)

    def pad(t):
        out = torch.zeros(t.shape[:-1] + (hd,), dtype=t.dtype)
        out[..., :d] = t
        return out
    row = torch.cat([pad(q).view(T, -1), pad(k).view(T, -1), pad(v).view(T, -1)], dim=1)
    if planes > 1:
        parts = torch.randn(planes, *row.shape, generator=g)
        parts[0] = row - parts[1:].sum(0)
        src = parts.cuda()
    else:
        src = row.to(tdt).cuda()
    pool, table, n_pages = _cache([int(pos.max()) + 1], nkv, hd, tdt, seed=T)
    pool, table = pool.cuda(), table.cuda()
    inv = torch.tensor([10000.0 ** (-2.0 * i / max(rot, 1)) for i in range(max(1, rot // 2))], dtype=torch.float32)
    qout = torch.empty(T, nh * hd, dtype=tdt, device="cuda")
    zeros = torch.zeros(T, dtype=torch.int32, device="cuda")
    st = _status()
    K.norm_rope_store(src, qout, pad(wq).view(-1).to(tdt).cuda(), pad(wk).view(-1).to(tdt).cuda(), 1e-5, nh * d,
                      nkv * d, inv.cuda(), rot, pos.cuda(), zeros, zeros[:1], nh, nkv, nkv, hd, pool, table, n_pages, st)
    assert int(st.item()) == 0
    tol = 2e-5 if dtype == "float32" else 1.2e-2
    got_q = qout.view(T, nh, hd)
    assert _rel(got_q[..., :d], qn) < tol and float(got_q[..., d:].float().abs().max() if hd > d else 0) == 0
    for t in range(T):
        p = int(pos[t])
        page = int(table[0, p // 64])
        assert _rel(pool[page, 0, :, p % 64, :d], kn[t]) < tol
        assert _rel(pool[page, 1, :, p % 64, :d], v[t]) < tol


def _attention_case(K, kind, dtype, nh, nkv, hd, q_lens, kv_lens, window, keep, seed, boost):
    """rows q_lens[b] at the end of sequences of kv_lens[b] positions; `boost` = (sequence, key position): that key
    and every query are scaled so that its score stands out"""
    g = torch.Generator().manual_seed(seed)
    tdt = DT[dtype]
    B = len(q_lens)
    pool, table, n_pages = _cache(kv_lens, nkv, hd, tdt, seed)
    ks = [torch.randn(n, nkv, hd, generator=g) for n in kv_lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in kv_lens]
    qs = [torch.randn(n, nh, hd, generator=g) for n in q_lens]
    if boost is not None:
        b, p = boost
        ks[b][p, :, 0] = 30.0
        for q in qs:
            q[:, :, 0] = 2.0
    scale = 0.17
    want = []
    for b in range(B):
        k, v, q = ks[b].to(tdt).double(), vs[b].to(tdt).double(), qs[b].to(tdt).double()
        full = torch.zeros(kv_lens[b], nh, hd, dtype=torch.float64)
        full[kv_lens[b] - q_lens[b]:] = q
        o = PV.grouped_attention(full, k, v, scale, PV.visible(kv_lens[b], window, keep))
        want.append(o[kv_lens[b] - q_lens[b]:])
        for p in range(kv_lens[b]):
            page = int(table[b, p // 64])
            pool[page, 0, :, p % 64] = ks[b][p].to(tdt)
            pool[page, 1, :, p % 64] = vs[b][p].to(tdt)
    q = torch.cat([x.reshape(x.shape[0], -1) for x in qs]).to(tdt).cuda()
    out = torch.full_like(q, float("nan"))
    pos = torch.cat([torch.arange(kv_lens[b] - q_lens[b], kv_lens[b]) for b in range(B)]).to(torch.int32).cuda()
    seq = torch.cat([torch.full((q_lens[b],), b) for b in range(B)]).to(torch.int32).cuda()
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    st = _status()
    pool, table = pool.cuda(), table.cuda()
    if kind == "generic":
        K.attn_generic(q, out, pos, seq, slot, nh, nkv, hd, scale, window or 0, pool, table, n_pages, st, keep)
    elif kind == "tc":
        K.attn_tc(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, window or 0, pool, table, n_pages,
                  grid_x=-(-max(q_lens) // (128 // (nh // nkv))), status=st, keep_first=keep)
    elif kind == "mma":
        K.attn_mma(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, window or 0, pool, table, n_pages, decode=False,
                   grid_x=-(-max(q_lens) * (nh // nkv) // 64), status=st, keep_first=keep)
    else:
        K.attn_mma(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, window or 0, pool, table, n_pages, decode=True,
                   grid_x=int(kind[3:]), status=st, keep_first=keep)
    assert int(st.item()) == 0
    return _rel(out.view(-1, nh, hd), torch.cat(want))


@pytest.mark.parametrize("kind,dtype,hd", [("generic", "float32", 24), ("generic", "bfloat16", 64), ("tc", "bfloat16", 64),
                                           ("tc", "bfloat16", 128), ("mma", "bfloat16", 64), ("dec1", "bfloat16", 128),
                                           ("dec3", "bfloat16", 64), ("dec7", "bfloat16", 64)])
@pytest.mark.parametrize("window,keep", [(70, 5), (40, 70), (64, 64), (130, 1), (33, 129), (70, 0)])
def test_attention_with_kept_first_positions(K, kind, dtype, hd, window, keep):
    """a key that stands out, placed just inside and just outside the window and the kept stretch, at page borders
    and far back: prompt rows and single decoded rows"""
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    dec = kind.startswith("dec")
    for L in (321,):
        places = {0, keep - 1, keep, L - window - 1, L - window, L - window + 1, 63, 64, L - 1}
        for p in sorted(x for x in places if 0 <= x < L):
            q_lens = [1, 1] if dec else [L - 200, 37]
            err = _attention_case(K, kind, dtype, 6, 2, hd, q_lens, [L, 150], window, keep, seed=L + p, boost=(0, p))
            assert err < tol, (kind, L, p, err)


@pytest.mark.parametrize("T,E,top", [(1, 5, 2), (77, 11, 3), (300, 7, 7), (40, 64, 1), (9, 130, 8)])
def test_router_pick_and_weights(K, T, E, top):
    g = torch.Generator().manual_seed(T + E)
    z, b = torch.randn(T, E, generator=g), torch.randn(E, generator=g)
    idx, w = K.moe_topk(z.cuda(), b.cuda(), top)
    widx, ww = PV.route((z + b).double(), top)
    assert torch.equal(idx.cpu().long(), widx) and _rel(w, ww) < 1e-6
    idx, w = K.moe_topk(z.cuda(), None, top)                                    # no bias
    assert torch.equal(idx.cpu().long(), PV.route(z.double(), top)[0])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,top,width,F", [(1, 5, 2, 64, 24), (150, 6, 1, 128, 64), (70, 4, 4, 96, 40),
                                             (333, 7, 3, 72, 20), (64, 16, 2, 256, 128), (700, 3, 2, 64, 264)])
def test_experts_grouped_products(K, dtype, T, E, top, width, F):
    """the experts' outputs as planes: plane k of a row is its k-th expert's output times its weight; experts that no
    row picked and experts that most rows picked"""
    from kindi_b200.kernels import moe as M
    from kindi_b200.parts.base import StepContext
    g = torch.Generator().manual_seed(T * E)
    tdt = DT[dtype]
    y = torch.randn(T, width, generator=g).to(tdt)
    up, down = (torch.randn(E, F, width, generator=g) * 0.2).to(tdt), (torch.randn(E, width, F, generator=g) * 0.2).to(tdt)
    z = torch.randn(T, E, generator=g)
    z[:, 0] += 2.0                                           # most rows pick expert 0
    if E > 2:
        z[:, E - 1] -= 50.0                                  # nobody picks the last one (unless all are picked)
    idx, w = PV.route(z.double(), top)
    want = torch.zeros(top, T, width, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            want[k, t] = w[t, k] * (down[e].double() @ PV.relu_squared(up[e].double() @ y[t].double()))
    for fast in ([False, True] if dtype == "bfloat16" else [False]):
        ctx = StepContext(T=T, B=1, tok=None, pos=None, seq=None, slot=None, q_start=None, kv_len=None, h_slot=None,
                          h_q_start=None, h_kv_len=None, decode=False, max_q=T, max_kv=T, dtype=tdt,
                          device=torch.device("cuda"), status=_status(), fast=fast)
        got = M.experts(ctx, y.cuda(), idx.to(torch.int32).cuda(), w.float().cuda(), up.cuda(), down.cuda(), top,
                        "relu2", tdt)
        assert int(ctx.status.item()) == 0
        assert _rel(got, want) < (2e-5 if dtype == "float32" else 1.5e-2), (fast,)
        assert _rel(got.sum(0), want.sum(0)) < (2e-5 if dtype == "float32" else 1.5e-2)


# ------------------------------------------------------------------------------------------- whole models
def _plain(folder, reqs):
    m = PV.load_model(folder)
    return {rid: PV.forward(m, toks).numpy() for rid, toks in reqs.items()}


def _compare(got, reqs, want, tol, what):
    for rid, toks in reqs.items():
        mine = np.stack([got[(rid, i)] for i in range(len(toks))])
        err = tiny.rel_err(mine, want[rid])
        row = int(np.argmax(np.max(np.abs(mine - want[rid]), axis=1)))
        assert err <= tol, "%s %s: %.3g at position %d of %d" % (what, rid, err, row, len(toks))


def _edge_requests(raw, seed):
    """requests whose needle stands at the places that matter - the first position, the last kept one and the first
    that is not kept, just inside and just outside each window as seen from the probes at the end, at a page border
    - with probes over the last positions; and the shortest sequences there are"""
    rng = random.Random(seed)
    vocab = raw["vocab"]
    masks = [l["mixer"]["mask"] for l in raw["layers"] if l["mixer"]["mask"]]
    windows = sorted({m["size"] for m in masks}) or [50]
    keeps = sorted({m["keep_first"] for m in masks}) or [0]
    reqs = {}
    L = max(windows) + max(keeps) + 90
    places = {0, 63, 64}
    for k in keeps:
        places |= {k - 1, k}
    for w in windows:
        places |= {L - 4 - w, L - 3 - w, L - 2 - w, L - 1 - w}
    for p in sorted(x for x in places if 0 <= x < L - 8):
        reqs["n%d" % p] = TV.needle_request(vocab, L, p, list(range(L - 6, L)), rng)
    reqs["one"] = [rng.randrange(5, vocab)]
    reqs["two"] = [rng.randrange(5, vocab), TV.PROBE]
    return reqs


def _engine(folder, steps, dtype, **kw):
    from kindi_b200.engine.engine import Engine
    return Engine(folder, ctx=tiny.max_live_tokens(steps) + 64, dtype=dtype,
                  max_batch=max(len(s["entries"]) for s in steps), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TV.TINY))
def test_whole_prompts_and_token_by_token(tmp_path, name, dtype):
    """every request whole in one step, then again with its last 40 tokens one by one (the windows pass over decoded
    tokens, the needle leaves and the kept positions stay), in the same engine, slots and pages"""
    raw = TV.TINY[name][0]
    folder = TV.make_model(tmp_path, name, dtype)
    reqs = _edge_requests(raw, seed=3)
    want = _plain(folder, reqs)
    steps = tiny.trace_whole(reqs)
    later = tiny.trace_last_n(reqs, 40)
    for s in later:
        s["step"] += len(steps)
    eng = _engine(folder, steps + later, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s whole" % (name, dtype))
    tiny.run_replay(eng, later, out)
    _compare(tiny.collect(out, later, raw["vocab"]), reqs, want, TOL[dtype], "%s %s decoded" % (name, dtype))
    eng.check_status()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_prompts_in_portions(tmp_path, name, dtype):
    """a prompt cut into portions of 2, 3, 31, 64 and 65 tokens, and a step limit that cuts it inside the engine: the
    logits are those of the whole prompt (in 32-bit to the last bits)"""
    from kindi_b200.engine.engine import Engine
    raw = TV.TINY[name][0]
    folder = TV.make_model(tmp_path, name, dtype)
    reqs = {k: v for k, v in _edge_requests(raw, seed=4).items() if k in ("n0", "n64", "two")}
    widest = max([l["mixer"]["mask"]["size"] for l in raw["layers"] if l["mixer"]["mask"]] or [50])
    want = _plain(folder, reqs)
    for portion in (2, 3, 31, 64, 65):
        steps = []
        for rid, toks in reqs.items():
            for a in range(0, len(toks), portion):
                part = toks[a:a + portion]
                steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": part,
                                                               "want": list(range(len(part)))}],
                              "end": [rid] if a + portion >= len(toks) else []})
        eng = _engine(folder, steps, dtype)
        out = str(tmp_path / ("out%d" % portion))
        tiny.run_replay(eng, steps, out)
        eng.check_status()
        _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s by %d" % (name, dtype, portion))
    steps = tiny.trace_whole(reqs)
    eng = Engine(folder, ctx=tiny.max_live_tokens(steps) + 64, dtype=dtype, max_batch=2, max_step_tokens=64)
    out = str(tmp_path / "outcut")
    tiny.run_replay(eng, steps, out)
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s cut inside" % (name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TV.TINY))
def test_unequal_batches_and_reused_slots(tmp_path, name, dtype):
    """batches of unequal requests that start together and are decoded together, shorter ones ending earlier, a
    second batch in the slots and pages the first gave back: every row as if its request ran alone"""
    raw = TV.TINY[name][0]
    folder = TV.make_model(tmp_path, name, dtype)
    reqs = _edge_requests(raw, seed=5)
    ids = list(reqs)
    rng = random.Random(9)
    decode = {r: min(len(reqs[r]) - 1, rng.choice([0, 3, 9, 30])) for r in ids}
    half = len(ids) // 2
    steps = tiny.trace_group({r: reqs[r] for r in ids[:half]}, decode)
    steps += tiny.trace_group({r: reqs[r] for r in ids[half:]}, decode, first_step=len(steps))
    want = _plain(folder, reqs)
    eng = _engine(folder, steps, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s batches" % (name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_in_a_batch(tmp_path, dtype):
    """three requests decoded together for 330 steps (recorded decode steps; the windows' pages are given back and the
    kept pages stay), probes all the way"""
    raw = TV.TINY["C"][0]
    folder = TV.make_model(tmp_path, "C", dtype)
    rng = random.Random(2)
    reqs = {"a": TV.needle_request(raw["vocab"], 400, 2, list(range(60, 400, 3)), rng),
            "b": TV.needle_request(raw["vocab"], 350, 69, list(range(200, 350, 2)), rng),
            "c": TV.needle_request(raw["vocab"], 340, 70, list(range(100, 340, 5)), rng)}
    steps = tiny.trace_group(reqs, {"a": 330, "b": 330, "c": 330})
    want = _plain(folder, reqs)
    eng = _engine(folder, steps, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    assert eng.graph_replays > 300
    # the window groups hold what the windows and the kept stretch touch, not the sequences
    for g in eng.cache.groups:
        assert g.n_pool_pages <= 3 * (-(-g.need.window // 64) + 4 + -(-g.need.keep_first // 64)) + 128
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "long %s" % dtype)


@pytest.mark.parametrize("dtype,tie", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("name", ["B", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype, tie):
    from kindi_b200 import Engine
    raw = TV.TINY[name][0]
    folder = TV.make_model(tmp_path, name, dtype)
    m = PV.load_model(folder)
    eng = Engine(folder, ctx=2048, dtype=dtype, max_batch=3)
    prompts = list(tiny.random_requests(raw["vocab"], [5, 9, 1, 80, 13], seed=3).values())
    res = eng.generate_batch(prompts, temperature=0.0, max_tokens=10, stop_token_ids=())
    assert res.stats.batches == 2 and eng.cache.slots.n_held == 0
    for p, got in zip(prompts, res.tokens):
        assert len(got) == 10
        seq = list(p)
        for t in got:
            z = PV.forward(m, seq)[-1].numpy()
            best = int(np.argmax(z))
            assert t == best or z[best] - z[t] <= tie * np.abs(z).max(), (len(seq), t, best)
            seq.append(t)
    eng.cache.check()


def test_trace_run_and_command_line_as_programs(tmp_path):
    folder = TV.make_model(tmp_path, "A", "bfloat16")
    vocab = TV.VZ_A["vocab"]
    reqs = tiny.random_requests(vocab, [5, 40], seed=2)
    steps = tiny.trace_batched(reqs, batch=2, decode=4)
    out = str(tmp_path / "out")
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "bfloat16", "--out", out,
                        "--max-tokens", str(tiny.max_live_tokens(steps))],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = tiny.collect(out, steps, vocab)
    _compare(got, reqs, _plain(folder, reqs), TOL["bfloat16"], "trace_run")
    r = subprocess.run([sys.executable, "-m", "kindi_b200", "--model", folder, "--ctx", "512", "generate",
                        "--prompt-ids", "1,2,3", "--prompt-ids", "9 8", "--temperature", "0", "--max-tokens", "5"],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.strip().split("\n")]
    assert len(lines) == 2 and all(len(l["tokens"]) == 5 for l in lines)
    r = subprocess.run([sys.executable, "-m", "kindi_b200", "--model", folder, "info"], capture_output=True, text=True,
                       cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0 and "Vozinex" in r.stdout + r.stderr, r.stderr[-2000:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_recorded_prompt_steps_and_their_padding_rows(tmp_path, name, dtype):
    """short prompt steps are padded to a multiple of 64 rows and replayed from a recording once their shape has come
    twice: the padding rows go through the norms, the router and the experts like any row, store nothing and change no
    other row; in 32-bit a recorded step gives the bits of an engine that records nothing"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    raw = TV.TINY[name][0]
    folder = TV.make_model(tmp_path, name, dtype)
    m = PV.load_model(folder)
    rng = random.Random(9)
    eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=4)
    plain_eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=4, cuda_graphs=False)

    def run(e, groups, follow=3):
        out = []
        for group in groups:
            slots = [e.alloc() for _ in group]
            k = [len(t) - follow for t in group]
            logits = e.step([StepEntry(s, tuple(t[:n]), (n - 1,)) for s, t, n in zip(slots, group, k)])
            rows = [[logits[i].cpu().numpy()] for i in range(len(group))]
            for j in range(follow):
                lg = e.step([StepEntry(s, (t[n + j],), (0,)) for s, t, n in zip(slots, group, k)])
                for i in range(len(group)):
                    rows[i].append(lg[i].cpu().numpy())
            e.check_status()
            for s in slots:
                e.free(s)
            out.append([np.stack(r) for r in rows])
        return out

    lengths = [[103], [93], [131], [68], [73], [40, 71], [64, 9], [8, 100], [200], [260], [300]]
    groups = [[TV.needle_request(raw["vocab"], n, 1, list(range(n - 5, n)), rng) for n in g] for g in lengths]
    got = run(eng, groups)
    assert sum(1 for k in eng._graphs if k[0] == "prompt") >= 2 and eng.graph_replays >= 6
    same = run(plain_eng, groups)
    for g, mine, other in zip(groups, got, same):
        for toks, a, b in zip(g, mine, other):
            want = PV.forward(m, toks).numpy()[len(toks) - 4:]
            assert tiny.rel_err(a, want) <= TOL[dtype], (len(toks), tiny.rel_err(a, want))
            if dtype == "float32":
                assert np.array_equal(a, b), len(toks)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
