"""SwiGLU feed-forward: ``h = silu(Wg y) * (Wu y)``, branch ``= Wd h``; no biases.

Gate and up run as one product over the concatenated weights (the reference's fused gate/up launch,
``kindi/nanbeige.py:710-716``), ``silu(g) * u = g / (1 + exp(-g)) * u`` in 32-bit (``kindi/nbq.cu:461-467``), then
the down product (``kindi/nanbeige.py:718``). The intermediate size is a parameter of the part, and so are the gate's
activation (``activation``: ``silu``, the default, or ``gelu_tanh``: ``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``)
and the tensors' suffixes (``names``: ``gate``, ``up``, ``down``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import linear as L
from .base import Branch, FeedForward, StepContext, WeightView


_DEFAULT_NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}


class SwiGLU(FeedForward):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        f = int(spec["intermediate"])
        n = cls._names(spec)
        return {n["gate"]: (f, width), n["up"]: (f, width), n["down"]: (width, f)}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.f = int(spec["intermediate"])
        self.act = str(spec.get("activation") or "silu")
        if self.act not in ("silu", "gelu_tanh"):
            raise ValueError("a gated feed-forward's activation is silu or gelu_tanh, found %r" % self.act)
        n = self._names(spec)
        g, u = weights(n["gate"]), weights(n["up"])
        if g.dtype != u.dtype:
            raise ValueError("gate and up weights of %s are stored in different dtypes" % weights.prefix)
        # gate and up rows are put together in the order the products' SwiGLU epilogues want (the kernels' choice)
        self.wgu, self.group = L.join_gate_up(g, u)
        self.wd = weights(n["down"])

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        h = L.gate_up_swiglu(ctx, y, self.wgu, self.group, self.f, self.dtype, self.act)
        return Branch(L.planes(ctx, h, self.wd))

    def bytes_read(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.wgu, self.wd))


register_part("feed_forward", "swiglu", SwiGLU)
