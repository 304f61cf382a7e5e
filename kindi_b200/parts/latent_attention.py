"""Latent attention: queries, keys and values through low-rank latents; only the shared latent and one rotated key
part per position are cached.

With ``y`` the mixer's input, H heads, per head ``dim`` plain and ``rot_dim`` rotated query/key dimensions, value size
``v_dim``, latent sizes ``q_rank`` and ``kv_rank``:

* ``c_q = rms(W_dq y) * g_q`` and ``q = W_uq c_q``, laid out head by head as ``[dim plain | rot_dim rotated]``;
* ``W_dkv y`` has ``kv_rank + rot_dim`` rows: ``c = rms(first kv_rank) * g_kv`` is the latent, the last ``rot_dim``
  (not normalised) are ONE rotated key part shared by all heads;
* head h: keys ``[W_uk_h c | rotated part]``, values ``W_uv_h c``; score ``(q_plain . k_plain + q_rot . k_rot) * scale``;
  causal softmax; the concatenated heads times ``sigmoid(W_g y)`` (optional gate), then ``W_o``.

What runs is the absorbed form, the same arithmetic re-associated: ``q_plain . (W_uk_h c) = (W_uk_h^T q_plain) . c``
and ``sum_j p_j W_uv_h c_j = W_uv_h (sum_j p_j c_j)``. So the cache holds, per position, ONE key/value head: keys
``[c | rotated part | 0]`` and values ``[c | 0]`` of a size ``D >= kv_rank + rot_dim`` that the attention kernels
take; queries become ``[W_uk_h^T q_plain | rotated q | 0]`` per head (a per-head product); attention is the
library's grouped-query attention with H query heads on one key/value head; the heads' outputs (weighted sums of
latents) go through ``W_uv_h`` (a per-head product, the gate in its epilogue). Prompts, single tokens and cut prompts
are the same code, and nothing is expanded per cached position. The rotation is the mixer's position part (its
frequencies, pairing and factor on cosines and sines: see ``parts/rope.py``), applied by the latent kernels.

Parameters: ``n_heads``, ``head_dim`` (plain), ``rot_dim``, ``v_head_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``eps``,
``position`` (a rotation of ``rot_dim`` dimensions), ``names`` (tensor suffixes: ``dq``, ``dq_norm``, ``uq``, ``dkv``,
``dkv_norm``, ``uk``, ``uv``, ``o``, and ``gate`` or None).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..kernels import attention as A
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, KVNeed, Mixer, StepContext, WeightView

_DEFAULT_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                  "uv": "uv", "o": "o", "gate": None}


class LatentAttention(Mixer):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return (int(spec["n_heads"]), int(spec["head_dim"]), int(spec["rot_dim"]), int(spec["v_head_dim"]),
                int(spec["q_rank"]), int(spec["kv_rank"]))

    @classmethod
    def _cache_dim(cls, spec: PartSpec) -> int:
        """the size of the one cached key/value head: latent and rotated part, widened to a size the tensor-core
        attention kernels take (64, 128) where that is near"""
        _, _, r, _, _, kr = cls._sizes(spec)
        m = kr + r
        return 64 if m <= 64 else 128 if m <= 128 else (m + 7) // 8 * 8

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        H, d, r, dv, qr, kr = cls._sizes(spec)
        n = cls._names(spec)
        out = {n["dq"]: (qr, width), n["dq_norm"]: (qr,), n["uq"]: (H * (d + r), qr), n["dkv"]: (kr + r, width),
               n["dkv_norm"]: (kr,), n["uk"]: (H * d, kr), n["uv"]: (H * dv, kr), n["o"]: (width, H * dv)}
        if n["gate"]:
            out[n["gate"]] = (H * dv, width)
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        n = cls._names(spec)
        return {n["dq_norm"]: "gain", n["dkv_norm"]: "gain"}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        return KVNeed(1, cls._cache_dim(spec), None, 0)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.H, self.d, self.r, self.dv, self.qr, self.kr = self._sizes(spec)
        self.D = self._cache_dim(spec)
        if self.D > 512:
            raise ValueError("latent and rotated part together may have up to 512 elements, found %d"
                             % (self.kr + self.r))
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        pspec: PartSpec = spec["position"]
        self.position = part_class("position", pspec.kind)(pspec, width, weights, dtype=dtype, device=device)
        if self.position.rotary_dim != self.r:
            raise ValueError("the position part rotates %d dimensions, the mixer's rotated part has %d"
                             % (self.position.rotary_dim, self.r))
        if self.r and self.position.pairing != "interleaved":
            raise ValueError("latent attention rotates interleaved pairs; the position part pairs %r"
                             % self.position.pairing)
        n = self._names(spec)
        ws = [weights(n["dq"]), weights(n["dkv"])]
        self.has_gate = bool(n["gate"])
        if self.has_gate:
            ws.append(weights(n["gate"]))
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the down projections of %s are stored in different dtypes" % weights.prefix)
        self.w_down = torch.cat(ws, dim=0).contiguous()          # [q latent | kv latent | rotated part | gate]
        self.g_q, self.g_kv = weights(n["dq_norm"]).contiguous(), weights(n["dkv_norm"]).contiguous()
        self.w_uq = weights(n["uq"])
        # per head: W_uk_h^T as [kv_rank, dim] (rows = outputs of the absorbing product), W_uv_h as stored
        self.w_uk_t = weights(n["uk"]).view(self.H, self.d, self.kr).transpose(1, 2).contiguous()
        self.w_uv = weights(n["uv"]).view(self.H, self.dv, self.kr).contiguous()
        self.w_o = weights(n["o"])

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        H, d, r, dv, qr, kr, D = self.H, self.d, self.r, self.dv, self.qr, self.kr, self.D
        pool, table, n_pages = ctx.cache.kv_view(ctx.entry.cache)
        a = L.rows_or_planes(ctx, y, self.w_down, self.dtype)
        cq = torch.empty((ctx.T, qr), dtype=self.dtype, device=y.device)
        pos = self.position
        K.latent_prep(a, qr, kr, r, self.g_q, self.g_kv, self.eps, pos.inv_freq, pos.mult, ctx.pos, ctx.seq, ctx.slot,
                      cq, D, pool, table, n_pages, ctx.status)
        q = L.linear(ctx, cq, self.w_uq, self.dtype)
        qf = torch.empty((ctx.T, H * D), dtype=self.dtype, device=y.device)
        K.head_gemm(q, d + r, self.w_uk_t, qf, D)
        K.latent_qrope(q, d, r, pos.inv_freq, pos.mult, ctx.pos, qf, kr, D, H)
        att = torch.empty((ctx.T, H * D), dtype=self.dtype, device=y.device)
        A.attention(ctx, qf, att, H, 1, D, self.scale, 0, pool, table, n_pages)
        o = torch.empty((ctx.T, H * dv), dtype=self.dtype, device=y.device)
        K.head_gemm(att, D, self.w_uv, o, dv, gate=a[..., qr + kr + r:] if self.has_gate else None)
        return Branch(L.planes(ctx, o, self.w_o))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_down, self.w_uq, self.w_uk_t, self.w_uv, self.w_o))


register_part("mixer", "latent_attention", LatentAttention)
