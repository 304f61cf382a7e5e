"""Linear attention with a decay per head: a recurrent mixer whose cache is a fixed-size state.

``q = silu(W_q y)``, ``k = silu(W_k y)`` (H heads of ``head_dim``), ``v = silu(W_v y)`` (H heads of ``v_head_dim``).
Per head the state ``S`` (``head_dim x v_head_dim``, 32-bit, zero when a sequence starts) follows
``S_t = decay_h * S_(t-1) + k_t v_t^T`` and the head's output is ``o_t = S_t^T q_t``, with no other scale. The
concatenated heads are RMS-normed together (gain ``norm``), multiplied by ``sigmoid(W_g y)`` and projected by ``W_o``.

The four projections are one product. The recurrence, the norm and the gate are 32-bit; the state lives in the
cache's per-slot state storage (``[H, v_head_dim, head_dim]`` per sequence), is read at the start of a sequence's rows
of a step and written back after them, so prompts, single tokens and cut prompts are the same code and the same
sums. ``decay`` (H numbers), the sizes, ``eps`` and the tensors' suffixes (``names``: ``q``, ``k``, ``v``, ``gate``,
``o``, ``norm``) are parameters of the part.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from ..kernels import linear as L
from .base import Branch, Mixer, StateNeed, StepContext, WeightView

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm"}


class DecayLinearAttention(Mixer):
    CHUNK = 64                  # tokens of a run in the form for long prompts

    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["n_heads"]), int(spec["head_dim"]), int(spec["v_head_dim"])

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        H, d, dv = cls._sizes(spec)
        n = cls._names(spec)
        return {n["q"]: (H * d, width), n["k"]: (H * d, width), n["v"]: (H * dv, width), n["gate"]: (H * dv, width),
                n["o"]: (width, H * dv), n["norm"]: (H * dv,)}

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        return {cls._names(spec)["norm"]: "gain"}

    @classmethod
    def cache_need(cls, spec: PartSpec, width: int):
        H, d, dv = cls._sizes(spec)
        return StateNeed((H, dv, d))

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.H, self.d, self.dv = self._sizes(spec)
        if self.d > 256:
            raise ValueError("linear attention supports key sizes up to 256, found %d" % self.d)
        decay = [float(x) for x in spec["decay"]]
        if len(decay) != self.H:
            raise ValueError("decay has %d entries for %d heads" % (len(decay), self.H))
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        self.eps = float(spec["eps"])
        n = self._names(spec)
        ws = [weights(n["q"]), weights(n["k"]), weights(n["v"]), weights(n["gate"])]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("the projections of %s are stored in different dtypes" % weights.prefix)
        self.w_in = torch.cat(ws, dim=0).contiguous()            # [q | k | v | gate]
        self.g_norm = weights(n["norm"]).contiguous()
        self.w_o = weights(n["o"])

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        H, d, dv = self.H, self.d, self.dv
        a = L.rows_or_planes(ctx, y, self.w_in, self.dtype)
        # (padding rows of a recorded step belong to no sequence and are not written by the recurrence)
        o = (torch.zeros if ctx.graph else torch.empty)((ctx.T, H * dv), dtype=torch.float32, device=y.device)
        # prompts of the serving path: a sequence's runs of tokens side by side (32-bit sums that differ from the
        # token-by-token kernel's by rounding); single tokens, short steps and the true 32-bit path: token by token
        chunk = 0
        if ctx.fast and not ctx.decode and ctx.max_q > self.CHUNK:
            chunk = self.CHUNK if ctx.max_q <= 32 * self.CHUNK else 2 * self.CHUNK if ctx.max_q <= 128 * self.CHUNK \
                else 4 * self.CHUNK
        K.decay_scan(a, ctx.B, H, d, dv, self.decay, ctx.q_start, ctx.slot, ctx.cache.state_view(ctx.entry.cache), o,
                     chunk=chunk, max_rows=ctx.max_q)
        yn = torch.empty((ctx.T, H * dv), dtype=self.dtype, device=y.device)
        K.gated_rmsnorm(o, self.g_norm, self.eps, a[..., 2 * H * d + H * dv:], yn)
        return Branch(L.planes(ctx, yn, self.w_o))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
