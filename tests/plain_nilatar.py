"""A plain, slow implementation of the Nilatar decoder, one function per mechanism, for the tests to compare the
engine with. It works on whole sequences on the CPU with PyTorch tensor arithmetic only (float64 by default), keeps
no cache, and shares no code with the package.

Nilatar: ``x = embed[token] * scale``; pre-norm layers ``x += ls1 * mixer(rms(x))`` and, where the layer has a
feed-forward, ``x += ls2 * ff(rms(x))``; a final RMS norm and an untied head. Three mixers:

* ``attention``: grouped-query attention without any position encoding, a sliding window, a learned per-head sink in
  the softmax denominator, a sigmoid output gate read from the mixer's input; a layer may use the keys and values of
  an earlier layer (``kv_from``).
* ``latent_attention``: queries through a normalised low-rank latent; keys and values through a normalised shared
  latent ``c`` plus one rotated key part shared by all heads; interleaved-pair rotation with YaRN-scaled frequencies;
  full causal softmax; the same output gate.
* ``lightning``: per head ``S_t = decay * S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with silu on q, k and v; the heads'
  outputs are RMS-normed together, gated and projected.

The feed-forward is ``W_down (gelu_tanh(W_gate y) * (W_up y))``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional, Sequence

import torch


def load_model(model_dir: str):
    """(the JSON object of config.json, {name: tensor}) of a model folder"""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    for n in sorted(os.listdir(model_dir)):
        if n.endswith(".safetensors"):
            w.update(load_file(os.path.join(model_dir, n)))
    return cfg, w


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotation_table(rot: Mapping, dtype=torch.float64):
    """(frequency of each pair [dims / 2], the factor on cosines and sines) of a rotation described by ``base``,
    ``dims`` and an optional YaRN ``scaling`` (factor, original, fast, slow)"""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor, mult: float) -> torch.Tensor:
    """x [..., T, dims] with dimension 2i paired with 2i + 1; pos [T]"""
    a = pos.to(freq.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(a) * mult, torch.sin(a) * mult
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale: float, window: Optional[int], sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [H, T, d], k [H, T, d], v [H, T, dv] (key/value heads already spread over the query heads); position i sees
    j with 0 <= i - j (< window); ``sink`` [H] adds exp(sink) to the denominator"""
    H, T, _ = q.shape
    s = torch.einsum("hid,hjd->hij", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    s = s.masked_fill(~seen, float("-inf"))
    if sink is not None:
        s = torch.cat([s, sink.to(s.dtype)[:, None, None].expand(H, T, 1)], dim=-1)
    p = torch.softmax(s, dim=-1)
    if sink is not None:
        p = p[..., :T]
    return torch.einsum("hij,hjd->hid", p, v)


def windowed_attention(h, w: Mapping[str, torch.Tensor], m: Mapping, kv=None):
    """the ``attention`` mixer; ``kv`` = (k, v) of the layer whose keys and values this layer uses. Returns (output
    [T, width], (k, v))"""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w["q"].T).view(T, H, d).transpose(0, 1)
    if kv is None:
        k = (h @ w["k"].T).view(T, G, d).transpose(0, 1)
        v = (h @ w["v"].T).view(T, G, dv).transpose(0, 1)
    else:
        k, v = kv
    rep = H // G
    mask = m.get("mask") or {}
    o = softmax_attention(q, k.repeat_interleave(rep, dim=0), v.repeat_interleave(rep, dim=0), float(m["scale"]),
                          mask.get("size"), w["sink"])
    o = o.transpose(0, 1).reshape(T, H * dv) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T, (k, v)


def latent_attention(h, w: Mapping[str, torch.Tensor], m: Mapping, eps: float):
    T = h.shape[0]
    H, d, r, dv, kr = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T)
    freq, mult = rotation_table(m["rot"], h.dtype)
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + r).transpose(0, 1)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, freq, mult)
    ckv = h @ w["dkv"].T
    c = rms_norm(ckv[:, :kr], w["dkv.norm"], eps)
    k_rot = rotate_pairs(ckv[:, kr:], pos, freq, mult)                 # [T, r], shared by all heads
    k_plain = (c @ w["uk"].T).view(T, H, d).transpose(0, 1)
    v = (c @ w["uv"].T).view(T, H, dv).transpose(0, 1)
    qq = torch.cat([q_plain, q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot[None].expand(H, T, r)], dim=-1)
    o = softmax_attention(qq, kk, v, float(m["scale"]), None, None)
    o = o.transpose(0, 1).reshape(T, H * dv) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def lightning(h, w: Mapping[str, torch.Tensor], m: Mapping, eps: float):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w["q"].T).view(T, H, d)
    k = silu(h @ w["k"].T).view(T, H, d)
    v = silu(h @ w["v"].T).view(T, H, dv)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.empty(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    y = rms_norm(o.reshape(T, H * dv), w["norm"], eps) * torch.sigmoid(h @ w["g"].T)
    return y @ w["o"].T


def dense_ff(h, w: Mapping[str, torch.Tensor]):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {n[len(prefix):]: t.to(dtype) for n, t in tensors.items() if n.startswith(prefix)}


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float64,
            layers_out: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """logits [T, vocab] of one sequence; ``layers_out`` collects the residual stream after every layer"""
    eps = float(config["norm"]["eps"])
    tok = torch.tensor(list(tokens), dtype=torch.long)
    x = tensors["embed"].to(dtype)[tok] * float(config["embedding"]["scale"])
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = "l%d." % i
        m = layer["mixer"]
        w = _sub(tensors, p + "mix.", dtype)
        h = rms_norm(x, tensors[p + "norm1"].to(dtype), eps)
        kind = layer["type"]
        if kind == "attention":
            y, kept[i] = windowed_attention(h, w, m, kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        elif kind == "latent_attention":
            y = latent_attention(h, w, m, eps)
        elif kind == "lightning":
            y = lightning(h, w, m, eps)
        else:
            raise ValueError("unknown mixer %r" % kind)
        x = x + y * tensors[p + "ls1"].to(dtype)
        if layer.get("mlp") is not None:
            h = rms_norm(x, tensors[p + "norm2"].to(dtype), eps)
            x = x + dense_ff(h, _sub(tensors, p + "mlp.", dtype)) * tensors[p + "ls2"].to(dtype)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, tensors["final.norm"].to(dtype), eps) @ tensors["head"].to(dtype).T
