"""Causal self-attention with grouped queries over the paged cache.

``q, k, v = W y`` without biases (one product over the concatenated weights, as the reference launches its three
together, ``kindi/nanbeige.py:936-937``); the position encoding rotates q and k; k and v are stored at the row's
position of its sequence's cache; query head h reads key/value head ``h // (n_heads / n_kv_heads)``
(``kindi/nbq.cu:525-633``); scores are ``(q * scale) . k`` with ``scale = 1 / sqrt(head_dim)``
(``kindi/nanbeige.py:684``) unless the spec gives another; softmax and the weighted sum are 32-bit; the output
projection's result is the branch (``kindi/nanbeige.py:707-709``). All sizes are parameters of the part.

Options a spec may give:

* ``window``: a row sees the last ``window`` positions only; ``keep_first``: with a window, it also goes on seeing
  the sequence's first ``keep_first`` positions, at their true positions.
* ``v_head_dim``: values of another size than queries and keys. The cache and the kernels know one head size, so the
  smaller of the two is widened with zero rows in the weights (zero rows of W_q and W_k add nothing to a score, zero
  rows of W_v meet zero columns of W_o): the arithmetic is the model's, the cache holds the wider size.
* ``qk_norm`` (``{"eps", "q", "k"}``): before the rotation the query projection and the key projection are each divided
  by their root mean square over the WHOLE projection (all heads at once) and multiplied by the gains named ``q``
  and ``k`` (one per element of the projection).
* ``names``: the tensors' suffixes (``q``, ``k``, ``v``, ``o``).
* ``sink`` (a tensor suffix, ``[n_heads]``): a learned score per head that joins the softmax denominator as
  ``exp(sink_h)``; it has no key and no value and is not scaled.
* ``gate`` (a tensor suffix, ``[n_heads * v_head_dim, width]``): the concatenated heads are multiplied by
  ``sigmoid(W_g y)`` before the output projection; the gate's projection rides in the QKV product.
* ``shares_kv``: the layer has no key and value projections (no tensors for them); its schedule entry names the cache
  entry whose keys and values it attends to (``reads_cache_of``).
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..kernels import attention as A
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, KVNeed, Mixer, StepContext, WeightView

_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight"}


def _pad_heads(w: torch.Tensor, n: int, have: int, want: int) -> torch.Tensor:
    """[n * have, ...] -> [n * want, ...]: every head's rows followed by zero rows"""
    if have == want:
        return w
    out = torch.zeros((n, want) + tuple(w.shape[1:]), dtype=w.dtype, device=w.device)
    out[:, :have] = w.view((n, have) + tuple(w.shape[1:]))
    return out.view((n * want,) + tuple(w.shape[1:]))


class CausalSelfAttention(Mixer):
    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["n_heads"]), int(spec["n_kv_heads"]), int(spec["head_dim"])

    @classmethod
    def _v_dim(cls, spec: PartSpec) -> int:
        return int(spec.get("v_head_dim") or spec["head_dim"])

    @classmethod
    def _cache_dim(cls, spec: PartSpec) -> int:
        """the one head size the cache and the kernels see: the model's when keys and values agree; else the larger
        of the two, widened to a size the tensor-core attention kernels take (64, 128) where that is near"""
        hd, vd = int(spec["head_dim"]), cls._v_dim(spec)
        if hd == vd:
            return hd
        m = max(hd, vd)
        return 64 if m <= 64 else 128 if m <= 128 else (m + 7) // 8 * 8

    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        nh, nkv, hd = cls._sizes(spec)
        vd = cls._v_dim(spec)
        n = cls._names(spec)
        out = {n["q"]: (nh * hd, width), n["o"]: (width, nh * vd)}
        if not spec.get("shares_kv"):
            out[n["k"]] = (nkv * hd, width)
            out[n["v"]] = (nkv * vd, width)
        if spec.get("sink"):
            out[spec["sink"]] = (nh,)
        if spec.get("gate"):
            out[spec["gate"]] = (nh * vd, width)
        qkn = spec.get("qk_norm")
        if qkn:
            out[qkn["q"]] = (nh * hd,)
            out[qkn["k"]] = (nkv * hd,)
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        qkn = spec.get("qk_norm")
        return {qkn["q"]: "gain", qkn["k"]: "gain"} if qkn else {}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        nh, nkv, hd = cls._sizes(spec)
        window = spec.get("window")
        # (``cache_window``: what the cache keeps when other layers with other windows read this layer's keys and
        # values; "all": every position)
        kept = spec.get("cache_window")
        kept = window if kept is None else None if kept == "all" else kept
        return KVNeed(nkv, cls._cache_dim(spec), kept, int(spec.get("keep_first") or 0) if window and kept else 0)

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.nh, self.nkv, self.qk_dim = self._sizes(spec)
        self.v_dim = self._v_dim(spec)
        self.hd = self._cache_dim(spec)
        if self.nh % self.nkv:
            raise ValueError("n_heads %d is not a multiple of n_kv_heads %d" % (self.nh, self.nkv))
        if self.hd > 512:
            raise ValueError("head sizes up to 512 are supported, found %d" % self.hd)
        self.window = int(spec.get("window") or 0)
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        if self.keep_first < 0:
            raise ValueError("keep_first must not be negative, found %d" % self.keep_first)
        self.scale = float(spec.get("scale") or 1.0 / math.sqrt(self.qk_dim))
        pspec: PartSpec = spec["position"]
        self.position = part_class("position", pspec.kind)(pspec, width, weights, dtype=dtype, device=device)
        rot = self.position.rotation()
        if rot is not None and rot[1] > self.qk_dim:
            raise ValueError("rotary_dim %d exceeds head_dim %d" % (rot[1], self.qk_dim))
        n = self._names(spec)
        self.shares_kv = bool(spec.get("shares_kv"))
        if self.shares_kv and spec.get("qk_norm"):
            raise ValueError("a layer without key and value projections cannot normalise a key projection")
        ws = [_pad_heads(weights(n["q"]), self.nh, self.qk_dim, self.hd)]
        if not self.shares_kv:
            ws += [_pad_heads(weights(n["k"]), self.nkv, self.qk_dim, self.hd),
                   _pad_heads(weights(n["v"]), self.nkv, self.v_dim, self.hd)]
        # the gate's projection is one more block of rows of the joined product, laid out like the heads' outputs
        self.n_main = sum(w.shape[0] for w in ws)
        self.has_gate = bool(spec.get("gate"))
        if self.has_gate:
            ws.append(_pad_heads(weights(spec["gate"]), self.nh, self.v_dim, self.hd))
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v weights of %s are stored in different dtypes" % weights.prefix)
        self.wqkv = torch.cat(ws, dim=0).contiguous()
        self.sink = weights(spec["sink"]).to(torch.float32).contiguous() if spec.get("sink") else None
        wo = weights(n["o"])
        if self.v_dim != self.hd:
            wo = _pad_heads(wo.t().contiguous(), self.nh, self.v_dim, self.hd).t().contiguous()
        self.wo = wo
        self.qk_norm = None
        qkn = spec.get("qk_norm")
        if qkn:
            # (gains of the zero rows are zero too; the mean of squares is taken over the model's own element count)
            self.qk_norm = (_pad_heads(weights(qkn["q"]), self.nh, self.qk_dim, self.hd).contiguous(),
                            _pad_heads(weights(qkn["k"]), self.nkv, self.qk_dim, self.hd).contiguous(),
                            float(qkn["eps"]), self.nh * self.qk_dim, self.nkv * self.qk_dim)

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        entry = ctx.entry
        reads_other = entry is not None and entry.reads_cache_of is not None
        n_q = nh * hd
        if self.shares_kv and not reads_other:
            raise ValueError("a layer without key and value projections must read another entry's cache")
        if self.sink is not None or self.has_gate:
            return self._forward_sink_gate(ctx, y, reads_other)
        if reads_other and self.qk_norm is None:
            qkv = L.rows_or_planes(ctx, y, self.wqkv[:n_q], self.dtype)
            pool, table, n_pages = ctx.cache.kv_view(entry.reads_cache_of)
            store_kv = 0
        else:
            qkv = L.rows_or_planes(ctx, y, self.wqkv, self.dtype)
            pool, table, n_pages = ctx.cache.kv_view(entry.reads_cache_of if reads_other else entry.cache)
            store_kv = 0 if reads_other else nkv
        att = torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        plain = self.qk_norm is None and not self.keep_first
        if plain and not reads_other and A.attention_from_planes(ctx, qkv, att, nh, nkv, hd, self.scale, self.window,
                                                                 self.position.rotation(), pool, table, n_pages):
            # a small decode step of the serving kernels: the attention kernel summed the planes, rotated and stored
            return Branch(L.planes(ctx, att, self.wo))
        # the position encoding sums 32-bit planes, encodes and writes the queries out as rows (rows are encoded in
        # place) and stores keys and values; then attention over the cache
        q = qkv if qkv.dim() == 2 else torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        if self.qk_norm is None:
            self.position.encode_and_store(ctx, qkv, q, nh, store_kv, hd, pool, table, n_pages)
        else:
            self.position.encode_and_store(ctx, qkv, q, nh, store_kv, hd, pool, table, n_pages, qk_norm=self.qk_norm)
        A.attention(ctx, q, att, nh, nkv, hd, self.scale, self.window, pool, table, n_pages,
                    keep_first=self.keep_first)
        return Branch(L.planes(ctx, att, self.wo))

    def _forward_sink_gate(self, ctx: StepContext, y: torch.Tensor, reads_other: bool) -> Branch:
        """the same steps for a layer with a sink in its softmax or a gate on its output: one product for
        [q | k | v | gate] (a layer that reads another entry's cache: [q | gate]), encode and store, attention with the
        sink, the gate inside the attention kernel where it takes one, else by a kernel of its own"""
        nh, nkv, hd = self.nh, self.nkv, self.hd
        entry = ctx.entry
        n_q = nh * hd
        if reads_other and not self.shares_kv and self.qk_norm is None:
            # its own key and value rows are not needed: the product runs over the query and gate rows only
            w = torch.cat([self.wqkv[:n_q], self.wqkv[self.n_main:]], dim=0) if self.has_gate else self.wqkv[:n_q]
            if getattr(self, "_w_reads", None) is None:
                self._w_reads = w.contiguous()
            w, n_main = self._w_reads, n_q
        else:
            w, n_main = self.wqkv, self.n_main
        qkv = L.rows_or_planes(ctx, y, w, self.dtype)
        pool, table, n_pages = ctx.cache.kv_view(entry.reads_cache_of if reads_other else entry.cache)
        store_kv = 0 if reads_other else nkv
        att = torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        q = qkv if qkv.dim() == 2 else torch.empty((ctx.T, n_q), dtype=self.dtype, device=y.device)
        main = qkv[..., :n_main]
        if self.qk_norm is None:
            self.position.encode_and_store(ctx, main, q, nh, store_kv, hd, pool, table, n_pages)
        else:
            self.position.encode_and_store(ctx, main, q, nh, store_kv, hd, pool, table, n_pages, qk_norm=self.qk_norm)
        gate = qkv[..., n_main:] if self.has_gate else None
        fused = A.attention(ctx, q, att, nh, nkv, hd, self.scale, self.window, pool, table, n_pages,
                            keep_first=self.keep_first, sink=self.sink, gate=gate)
        if gate is not None and not fused:
            K.gate_mul(att, gate, att)
        return Branch(L.planes(ctx, att, self.wo))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.wqkv, self.wo))


register_part("mixer", "attention", CausalSelfAttention)
