"""Small Nilatar configurations with seeded random weights for the tests, with one key that stands out.

The configurations differ in every size and option: the order of the three mixers, head counts and groups, values
wider and narrower than keys, windows of one position, below, at and above a cache page and none at all, layers that
read an earlier layer's keys and values through a wider and through a narrower window, latent sizes whose cached head
is 64, 128 and odd sizes, rotations with and without stretched frequencies, decays of one and near zero, layers with
and without a feed-forward, embedding scales above and below one.
"""
from __future__ import annotations

import json
import os
import random
from typing import List

NEEDLE, PROBE = 3, 4            # token ids: the needle's key stands out for every probe's query
CODE = 3.0                      # the size of the planted embedding features, far above the random ones


def _att(heads, kv, dim, vdim, scale, window, kv_from=None, ff=None):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lat(heads, dim, rot, vdim, q_rank, kv_rank, scale, base, scaling=None, ff=None):
    r = {"base": base, "dims": rot}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": scale, "rot": r}
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lin(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, eps, emb_scale, layers):
    return {"architecture": "Nilatar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": emb_scale}, "layers": layers}


# A: small everything; values wider than keys; a window well below a page; a later layer reads layer 0's keys and
#    values through a WIDER window; plain rotation of part of the latent head; a linear-attention layer without
#    feed-forward
NL_A = _config(211, 64, 1e-5, 1.7, [
    _att(4, 2, 16, 24, 0.3, 20, ff=40),
    _lat(4, 16, 8, 12, 24, 20, 0.2, 10000.0, ff=48),
    _lin(2, 16, 24, [0.9, 0.97]),
    _att(4, 2, 16, 24, 0.25, 33, kv_from=0, ff=40)])
# B: head size 64 (the tensor-core attention kernels run in bfloat16), three query heads per key/value head, a cached
#    latent head of exactly 64, stretched frequencies whose ramp lies inside the rotated pairs, a window above a page
#    and a layer that reads it through a narrower one, a layer without a window
NL_B = _config(300, 128, 1e-6, 0.6, [
    _lat(8, 32, 16, 32, 64, 48, 0.15, 40000.0, (8.0, 64, 4.0, 1.0), ff=96),
    _att(6, 2, 64, 64, 0.125, 70, ff=96),
    _lin(4, 32, 64, [0.5, 0.9, 0.99, 1.0], ff=64),
    _att(6, 2, 64, 64, 0.11, 44, kv_from=1),
    _att(2, 2, 64, 64, 0.125, None, ff=96)])
# C: head size 128 with values of 64 (widened in the cache), one key/value head, a cached latent head of 128 with five
#    query heads on it, a window of exactly a page, a width that is no power of two
NL_C = _config(257, 200, 2e-6, 14.142, [
    _lin(1, 64, 32, [0.75]),
    _att(4, 1, 128, 64, 0.09, 64, ff=136),
    _lat(5, 24, 32, 40, 72, 96, 0.1, 10000.0, (4.0, 32, 8.0, 0.5), ff=136),
    _lat(5, 24, 32, 40, 72, 96, 0.1, 10000.0, None)])
# D: sizes that no vector load or tensor-core tile takes: width 72, heads of 24 with values of 10, a key/value head per
#    query head, a window of 9 and a window of ONE position, latent sizes 20 / 18 with a rotated part of 6, a decay of
#    almost nothing, two layers reading layer 0
NL_D = _config(131, 72, 1e-5, 1.0, [
    _att(5, 5, 24, 10, 0.2, 9, ff=20),
    _lat(3, 10, 6, 14, 20, 18, 0.31, 30000.0, (2.0, 16, 2.0, 1.0), ff=20),
    _att(5, 5, 24, 10, 0.2, 1, kv_from=0),
    _lin(3, 40, 9, [1e-3, 0.6, 1.0], ff=28),
    _att(5, 5, 24, 10, 0.3, 17, kv_from=0, ff=20)])
# E: a cached latent head above 128 (the general attention kernel in both dtypes), a window of 130, keys narrower than
#    values
NL_E = _config(401, 160, 1e-5, 2.5, [
    _lat(2, 16, 64, 16, 40, 100, 0.2, 1000000.0, (16.0, 128, 32.0, 1.0), ff=64),
    _att(8, 4, 32, 48, 0.22, 130, ff=64),
    _lin(2, 128, 16, [0.95, 0.8])])
TINY = {"A": (NL_A, 21), "B": (NL_B, 22), "C": (NL_C, 23), "D": (NL_D, 24), "E": (NL_E, 25)}


def make_model(tmp_path, name: str, dtype: str = "bfloat16", strength: float = 12.0) -> str:
    """a model folder with random weights N(0, 0.02) (gains and layer scales around one) in which the score of a PROBE
    token's query against a NEEDLE token's key stands out in every attention layer, wherever the two stand, and in
    which the sinks carry a good part of a softmax's mass.

    How: the needle's embedding row has one large feature (column 0), a probe's another (column 1); the RMS norm
    makes each about sqrt(width). In a windowed-attention layer the key projection of the first key/value head reads
    column 0 into its last dimension and the query projections of that group's heads read column 1 into the same
    dimension; the value projection reads column 0 with a large weight. In a latent-attention layer the key/value
    latent's first element reads column 0, the query latent's first element column 1 (their norms make them about
    sqrt(rank)), and the up-projections carry them into the last plain dimension of every head. Sinks are drawn
    around 2, so that exp(sink) weighs like seven ordinary keys. With plain random weights attention is nearly uniform,
    and a key that is dropped, a window that is one position off or a forgotten sink moves the logits by less than
    the rounding error of bfloat16."""
    import torch
    from kindi_b200.config.registry import model_from_config
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    from kindi_b200.weights.safetensors_io import write_file
    cfg, seed = TINY[name]
    d = os.path.join(str(tmp_path), "nl_%s_%s" % (name, dtype))
    if os.path.isfile(os.path.join(d, "model.safetensors")):
        return d
    os.makedirs(d, exist_ok=True)
    _, spec = model_from_config(cfg)
    t = random_tensors(expected_tensors(spec), seed, dtype=torch.float32, inits=tensor_inits(spec))
    width = cfg["width"]
    emb = t["embed"]
    emb[:, 0:2] = 0.0
    emb[NEEDLE, 0] = CODE
    emb[PROBE, 1] = CODE
    g = torch.Generator().manual_seed(seed + 1)
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        p = "l%d.mix." % i
        if layer["type"] == "attention":
            H, G, dim = m["heads"], m["kv_heads"], m["dim"]
            at = dim - 1
            if "kv_from" not in m:
                t[p + "k"][at, :] = 0.0
                t[p + "k"][at, 0] = 1.0
                t[p + "v"][:, 0] = 0.25 * torch.sign(t[p + "v"][:, 1])
            for h in range(H // G):
                t[p + "q"][h * dim + at, :] = 0.0
                t[p + "q"][h * dim + at, 1] = strength / (m["scale"] * width)
            t[p + "sink"] = 2.0 + 0.5 * torch.randn(H, generator=g)
        elif layer["type"] == "latent_attention":
            H, dim, r, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["q_rank"], m["kv_rank"]
            at = dim - 1
            t[p + "dkv"][0, :] = 0.0
            t[p + "dkv"][0, 0] = 1.0
            t[p + "dkv.norm"][0] = 1.0
            t[p + "dq"][0, :] = 0.0
            t[p + "dq"][0, 1] = 1.0
            t[p + "dq.norm"][0] = 1.0
            t[p + "uv"][:, 0] = 0.25 * torch.sign(t[p + "uv"][:, 1])
            for h in range(H):
                t[p + "uk"][h * dim + at, :] = 0.0
                t[p + "uk"][h * dim + at, 0] = 1.0
                t[p + "uq"][h * (dim + r) + at, :] = 0.0
                t[p + "uq"][h * (dim + r) + at, 0] = strength / (m["scale"] * (qr * kr) ** 0.5)
    # no branch writes into the planted columns: what the planted keys and queries read stays the tokens' own
    for n in list(t):
        if n.endswith(".mix.o") or n.endswith(".mlp.down"):
            t[n][0:2, :] = 0.0
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
