"""A plain, slow implementation of the Vozinex decoder for the tests: whole sequences, no cache, no batching, one
function per mechanism, float64 on the CPU. It shares no code with the package: config.json is read with ``json``,
the weights with the ``safetensors`` package, and every function is the mechanism's formula written out.

Notation: T tokens, width E, H query heads, G key/value heads, d the query/key size of a head, dv the value size,
r the rotated dimensions of a head, W the window, F the first positions a window keeps.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence

import torch


def load_model(model_dir: str, dtype=torch.float64) -> dict:
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    for n in sorted(os.listdir(model_dir)):
        if n.endswith(".safetensors"):
            w.update(load_file(os.path.join(model_dir, n)))
    return {"cfg": cfg, "w": {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}, "dtype": dtype}


# --------------------------------------------------------------------------------------------- mechanisms
def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    """y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b over the last dimension"""
    mu = x.mean(dim=-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(dim=-1, keepdim=True) + eps) * w + b


def projection_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x [T, all heads' elements] / sqrt(mean over the WHOLE row of x^2 + eps) * w: one root mean square for all
    heads of the projection together"""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotate_first_dims(x: torch.Tensor, positions: torch.Tensor, r: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: of every head's first r dimensions, i and i + r/2 form a pair that turns by the angle
    pos * base^(-2i/r); dimensions from r on stay"""
    if r == 0:
        return x
    half = r // 2
    freq = torch.tensor([base ** (-2.0 * i / r) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:r]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., r:]], dim=-1)


def visible(T: int, window: Optional[int], keep_first: int) -> torch.Tensor:
    """[T, T] bool: row i sees column j when j <= i and (no window, or i - j < window, or j < keep_first)"""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def grouped_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, mask: torch.Tensor,
                      hide: Optional[int] = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; query head h reads key/value head h // (H / G);
    softmax((q . k) * scale) over the visible keys. ``hide``: a key position taken out for every row but its own
    (how the tests measure what a dropped key costs)"""
    T, H, _ = q.shape
    G = k.shape[1]
    if hide is not None:
        mask = mask.clone()
        mask[:, hide] = False
        mask[hide, hide] = True
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        sc = (q[:, h] @ k[:, g].T) * scale
        sc = sc.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(sc, dim=-1) @ v[:, g]
    return out


def attention_mixer(w: dict, pre: str, m: dict, eps: float, h: torch.Tensor, hide: Optional[int] = None):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", d)
    q = projection_rms_norm(h @ w[pre + "q"].T, w[pre + "q.norm"], eps).view(T, H, d)
    k = projection_rms_norm(h @ w[pre + "k"].T, w[pre + "k.norm"], eps).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    rot = m.get("rot") or {}
    pos = torch.arange(T)
    q = rotate_first_dims(q, pos, rot.get("dims", 0), rot.get("base", 10000.0))
    k = rotate_first_dims(k, pos, rot.get("dims", 0), rot.get("base", 10000.0))
    mask = m.get("mask") or {}
    vis = visible(T, mask.get("size"), mask.get("keep_first", 0))
    o = grouped_attention(q, k, v, m["scale"], vis, hide)
    return o.reshape(T, H * dv) @ w[pre + "o"].T


def route(z: torch.Tensor, top: int):
    """z [T, E] -> (experts [T, top], weights [T, top]): the top largest, weights = softmax over those alone"""
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.relu(z) ** 2


def moe_feed_forward(w: dict, pre: str, m: dict, h: torch.Tensor, margins: Optional[list] = None) -> torch.Tensor:
    """``margins``: gets, per row, how far the last chosen logit lies above the first one not chosen"""
    top = m["router"]["top"]
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    idx, wt = route(z, top)
    if margins is not None and top < z.shape[-1]:
        srt = torch.sort(z, dim=-1, descending=True).values
        margins.append(srt[:, top - 1] - srt[:, top])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += wt[t, k] * (w[pre + "e%d.down" % e] @ relu_squared(w[pre + "e%d.up" % e] @ h[t]))
    return out


def run_order(cfg: dict) -> List[tuple]:
    """(layer, first run of a further pass) in running order: layers start..stop-1 run `times` times in a row"""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = [(i, False) for i in range(lp["start"])]
    for p in range(lp["times"]):
        order += [(i, p > 0 and i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return order + [(i, False) for i in range(lp["stop"], n)]


def forward(model: dict, tokens: Sequence[int], hide: Optional[int] = None, layers_out: Optional[list] = None,
            margins: Optional[list] = None):
    """logits [T, vocab] of a whole sequence"""
    cfg, w = model["cfg"], model["w"]
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    x = x0.clone()
    for i, again in run_order(cfg):
        if again:
            x = x + x0
        layer, pre = cfg["layers"][i], "l%d." % i
        x = x + attention_mixer(w, pre + "mix.", layer["mixer"], eps,
                                layer_norm(x, w[pre + "norm1"], w[pre + "norm1.b"], eps), hide)
        if layer.get("mlp") is not None:
            x = x + moe_feed_forward(w, pre + "mlp.", layer["mlp"],
                                     layer_norm(x, w[pre + "norm2"], w[pre + "norm2.b"], eps), margins)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
