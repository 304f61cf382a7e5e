"""Mixture-of-experts feed-forward: a router picks ``top_k`` of ``n_experts`` small feed-forwards for every row.

Router: ``z = W_r y + b_r`` with 32-bit accumulation (``y`` in the run dtype); the ``top_k`` experts with the largest
``z`` are chosen and weighted by the softmax over the chosen values only. Expert: ``W_down act(W_up y)``, no biases,
no gate; ``act`` is a parameter (``relu2``: the square of relu; ``silu``; ``gelu_tanh``; ``none``). The branch is the
weighted sum of the chosen experts' outputs: it is returned as ``top_k`` 32-bit planes (plane k holds each row's k-th
expert, already weighted), which the next norm adds in order, so every row's sum has the same order in every batch.

All rows of a step go through the experts as grouped products over (row, pick) pairs sorted by expert; the sort
happens on the device, so the part can be recorded. Sizes, the activation, whether the router has a bias and the
tensors' suffixes (``router``, ``router_bias``, ``up`` and ``down`` with ``%d`` for the expert) are parameters.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..config.registry import register_part
from ..config.spec import PartSpec
from ..kernels import lib as K
from ..kernels import moe as M
from .base import Branch, FeedForward, StepContext, WeightView

_DEFAULT_NAMES = {"router": "router.weight", "router_bias": "router.bias", "up": "experts.%d.up_proj.weight",
                  "down": "experts.%d.down_proj.weight"}


class MixtureOfExperts(FeedForward):
    @classmethod
    def _names(cls, spec: PartSpec):
        n = dict(_DEFAULT_NAMES)
        n.update(spec.get("names") or {})
        return n

    @classmethod
    def _sizes(cls, spec: PartSpec):
        return int(spec["n_experts"]), int(spec["top_k"]), int(spec["intermediate"])

    @classmethod
    def tensor_shapes(cls, spec: PartSpec, width: int) -> Dict[str, Tuple[int, ...]]:
        E, top, f = cls._sizes(spec)
        n = cls._names(spec)
        out = {n["router"]: (E, width)}
        if spec.get("router_bias", True):
            out[n["router_bias"]] = (E,)
        for e in range(E):
            out[n["up"] % e] = (f, width)
            out[n["down"] % e] = (width, f)
        return out

    @classmethod
    def tensor_init(cls, spec: PartSpec, width: int) -> Dict[str, str]:
        return {cls._names(spec)["router_bias"]: "zero"} if spec.get("router_bias", True) else {}

    def __init__(self, spec, width, weights: WeightView, *, dtype, device):
        super().__init__(spec, width, weights, dtype=dtype, device=device)
        self.E, self.top, self.f = self._sizes(spec)
        if not (1 <= self.top <= self.E):
            raise ValueError("top_k %d must lie between 1 and n_experts %d" % (self.top, self.E))
        self.act = str(spec.get("activation", "relu2"))
        if self.act not in K.ACT:
            raise ValueError("unknown activation %r; known: %s" % (self.act, ", ".join(sorted(K.ACT))))
        n = self._names(spec)
        self.wr = weights(n["router"])
        self.br = weights(n["router_bias"]).to(torch.float32).contiguous() if spec.get("router_bias", True) else None
        ups = [weights(n["up"] % e) for e in range(self.E)]
        downs = [weights(n["down"] % e) for e in range(self.E)]
        if len({w.dtype for w in ups + downs}) != 1:
            raise ValueError("the expert weights of %s are stored in different dtypes" % weights.prefix)
        self.wup = torch.stack(ups).contiguous()            # [E, f, width]
        self.wdown = torch.stack(downs).contiguous()        # [E, width, f]

    def forward(self, ctx: StepContext, y: torch.Tensor) -> Branch:
        return Branch(M.feed_forward(ctx, y, self.wr, self.br, self.wup, self.wdown, self.top, self.act, self.dtype))

    def bytes_read(self) -> int:
        """the router and, of the experts, the share a single row reads (a large step reads up to all of them)"""
        per_expert = (self.wup.numel() + self.wdown.numel()) // self.E * self.wup.element_size()
        return self.wr.numel() * self.wr.element_size() + self.top * per_expert


register_part("feed_forward", "moe", MixtureOfExperts)
