"""Small Vozinex configurations with seeded random weights for the tests, with one key that stands out.

The configurations differ in every size and option: head counts and groups (one key/value head per query head up to
one for all), value heads wider and narrower than key heads, rotations over part of a head and over all of it,
windows below, at and above a cache page with none, few and many kept first positions (more than a page, more than the
window), layers without a window and layers without a feed-forward, one expert per row up to all experts, a repeated
stretch at the start, in the middle, and none.
"""
from __future__ import annotations

import json
import os
import random
import zlib
from typing import List

NEEDLE, PROBE = 3, 4            # token ids: the needle's key stands out for every probe's query
CODE = 3.0                      # the size of the planted embedding features, far above the random ones


def _layer(heads, kv, dim, vdim, scale, rot, base, window, keep, experts=None, top=None, ff=None):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
             "rot": {"base": base, "dims": rot},
             "mask": None if window is None else {"size": window, "keep_first": keep}}
    mlp = None if experts is None else {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _config(vocab, width, eps, layers, loop):
    return {"architecture": "Vozinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
            "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}}


# A: values wider than keys, part of the head rotated, a window well below a page with three kept positions, a layer
#    without feed-forward, the last two layers run twice
VZ_A = _config(211, 64, 1e-5, [
    _layer(4, 2, 16, 24, 0.3, 8, 10000.0, 20, 3, 5, 2, 24),
    _layer(4, 2, 16, 24, 0.3, 8, 10000.0, 20, 3),
    _layer(4, 4, 16, 8, 0.25, 16, 10000.0, 33, 1, 5, 2, 24)], (1, 3, 2))
# B: as many key/value heads as query heads, the whole head rotated, a window of exactly a page, nothing kept, every
#    row uses all experts, no repeated stretch
VZ_B = _config(300, 96, 1e-6, [
    _layer(3, 3, 32, 32, 0.125, 32, 500000.0, 64, 0, 4, 4, 40),
    _layer(3, 3, 32, 32, 0.125, 32, 500000.0, 64, 0, 4, 4, 40)], (0, 0, 1))
# C: head size 64 (the tensor-core attention kernels run in bfloat16), three query heads per key/value head, windows
#    of 70 and 40 with 5 and 70 kept positions (more than a page, more than the window), one expert per row, the
#    first two layers run three times
VZ_C = _config(333, 128, 1e-5, [
    _layer(6, 2, 64, 64, 0.2, 32, 10000.0, 70, 5, 6, 1, 64),
    _layer(6, 2, 64, 64, 0.2, 32, 10000.0, 40, 70, 6, 1, 64),
    _layer(6, 2, 64, 64, 0.15, 64, 1000000.0, 70, 5, 6, 2, 64)], (0, 2, 3))
# D: head size 128 with values of 64 (widened in the cache), one key/value head, a layer without a window, a window of
#    130 that keeps exactly a page, eight experts of which three, a width that is no power of two
VZ_D = _config(257, 200, 2e-6, [
    _layer(4, 1, 128, 64, 0.09, 64, 10000.0, None, 0, 8, 3, 136),
    _layer(4, 1, 128, 64, 0.09, 64, 10000.0, 130, 64, 8, 3, 136)], (1, 2, 2))
# E: odd sizes nothing is tuned for: width 72, head size 24, 5 heads in one group, 3 of 7 experts of size 20
VZ_E = _config(131, 72, 1e-5, [
    _layer(5, 1, 24, 24, 0.2, 12, 30000.0, 17, 2, 7, 3, 20),
    _layer(5, 5, 24, 10, 0.2, 24, 30000.0, 17, 2, 7, 3, 20)], (0, 1, 2))
# F: sizes that no vector load or tensor-core tile takes: width 100, heads of 10 with values of 6, then heads of an odd
#    size (9), experts of 18, a window of 9 that keeps 2, a layer without a window, both layers run twice
VZ_F = _config(97, 100, 1e-5, [
    _layer(2, 1, 10, 6, 0.31, 4, 10000.0, 9, 2, 3, 2, 18),
    _layer(2, 2, 9, 9, 0.31, 8, 10000.0, None, 0, 3, 2, 18)], (0, 2, 2))
# G: keys of 32 and values of 48, both widened to the 64 the tensor-core attention kernels take (five query heads per
#    key/value head); then a layer with a key/value head per query head at head size 64; ten experts of 96, three per
#    row; the middle layers run twice
VZ_G = _config(401, 320, 1e-5, [
    _layer(10, 2, 32, 48, 0.22, 16, 10000.0, 100, 6, 10, 3, 96),
    _layer(10, 2, 32, 48, 0.22, 16, 10000.0, 100, 6, 10, 3, 96),
    _layer(4, 4, 64, 64, 0.125, 64, 10000.0, 128, 64, 10, 3, 96),
    _layer(4, 4, 64, 64, 0.125, 64, 10000.0, 65, 1)], (1, 3, 2))
TINY = {"A": (VZ_A, 11), "B": (VZ_B, 12), "C": (VZ_C, 13), "D": (VZ_D, 14), "E": (VZ_E, 15), "F": (VZ_F, 16),
        "G": (VZ_G, 17)}


def make_model(tmp_path, name: str, dtype: str = "bfloat16", strength: float = 12.0) -> str:
    """a model folder with random weights N(0, 0.02) (norm gains around one, biases zero) in which the score of a
    PROBE token's query against a NEEDLE token's key stands out in every layer, wherever the two stand.

    How: the needle's embedding row has one large feature (column 0), a probe's another (column 1), which the layer
    norms pass on. In every layer the key projection of the first key/value head reads column 0 into one dimension -
    the last one when it is not rotated, else the first of the slowest rotated pair - and the query projections of
    that group's heads read column 1 into the same dimension; the value projection reads column 0 with a large
    weight, so that a row that sees the needle gets a value unlike any other. The norm over the whole projection then makes that
    dimension about sqrt(elements of the projection) large, so the query gain of that dimension is set to what brings
    the score to about `strength`. With plain random weights attention is nearly uniform, and a key that is dropped or
    a window that is one position off moves the logits by less than the rounding error of bfloat16."""
    import torch
    from kindi_b200.config.registry import model_from_config
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    from kindi_b200.weights.safetensors_io import write_file
    cfg, seed = TINY[name]
    d = os.path.join(str(tmp_path), "vz_%s_%s" % (name, dtype))
    if os.path.isfile(os.path.join(d, "model.safetensors")):
        return d
    os.makedirs(d, exist_ok=True)
    _, spec = model_from_config(cfg)
    t = random_tensors(expected_tensors(spec), seed, dtype=torch.float32, inits=tensor_inits(spec))
    emb = t["embed"]
    emb[:, 0:2] = 0.0
    emb[NEEDLE, 0] = CODE
    emb[PROBE, 1] = CODE
    # columns 2.. carry a code of the token: a shuffled ladder of well separated levels, one column per expert
    n_code = max([l["mlp"]["router"]["experts"] for l in cfg["layers"] if l["mlp"]] or [0])
    g = torch.Generator().manual_seed(seed + 7)
    for tok in range(cfg["vocab"]):
        emb[tok, 2:2 + n_code] = CODE * torch.randperm(n_code, generator=g).float() / max(1, n_code - 1)
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        H, G, dim, r = m["heads"], m["kv_heads"], m["dim"], m["rot"]["dims"]
        at = dim - 1 if r < dim else r // 2 - 1
        p = "l%d.mix." % i
        t[p + "k"][at, 0] = 1.0
        t[p + "k.norm"][at] = 1.0
        t[p + "v"][:, 0] = 0.25 * torch.sign(t[p + "v"][:, 1])        # the needle's value is large too
        for h in range(H // G):
            t[p + "q"][h * dim + at, 1] = 1.0
            t[p + "q.norm"][h * dim + at] = strength / (m["scale"] * (H * dim * G * dim) ** 0.5)
        # The router reads the token's code, expert e from column 2 + e: with plain random weights a row's logits lie
        # so close together that bfloat16 rounding picks other experts than the plain model in many rows, and the
        # comparison would say nothing. (test_vozinex_cpu measures the margins.) The router's bias is zero in a random
        # model; a bias that matters shows a router that forgets it.
        if layer["mlp"] is not None:
            E = layer["mlp"]["router"]["experts"]
            g = torch.Generator().manual_seed(seed * 100 + i)
            t["l%d.mlp.router" % i].zero_()
            for e in range(E):
                t["l%d.mlp.router" % i][e, 2 + e] = 3.0
            t["l%d.mlp.router.b" % i] = torch.randn(E, generator=g) * 0.2
    # no branch writes into the planted columns: what the routers and the planted key read stays the tokens' own
    for n in list(t):
        if n.endswith(".mix.o") or n.endswith(".down"):
            t[n][0:2 + n_code, :] = 0.0
    for n in list(t):
        if n.endswith(".b") and ("norm" in n):
            g = torch.Generator().manual_seed(zlib.crc32(n.encode()) % 100000)
            t[n] = torch.randn(t[n].shape, generator=g) * 0.05
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    t = {n: v.to(tdt) for n, v in t.items()}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(d, "model.safetensors"), t, metadata={"format": "pt"})
    return d


def needle_request(vocab: int, length: int, needle_at: int, probes: List[int], rng: random.Random) -> List[int]:
    """random tokens (neither needle nor probe) with the needle at `needle_at` and probes at the listed places"""
    toks = []
    for i in range(length):
        t = rng.randrange(vocab)
        while t in (NEEDLE, PROBE):
            t = rng.randrange(vocab)
        toks.append(NEEDLE if i == needle_at else PROBE if i in probes else t)
    return toks
