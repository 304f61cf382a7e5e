"""A mixture-of-experts feed-forward as launches: the router, the pick, and the choice of kernels for the two grouped
products."""
from __future__ import annotations

from typing import Optional

import torch

from . import lib as K
from . import linear as L


def feed_forward(ctx, y: torch.Tensor, wr: torch.Tensor, br: Optional[torch.Tensor], wup: torch.Tensor,
                 wdown: torch.Tensor, top: int, act: str, dtype: torch.dtype) -> torch.Tensor:
    """32-bit planes ``[top, T, width]`` whose sum in order is the feed-forward's output: router logits ``y wr^T + br``
    with 32-bit accumulation, the ``top`` largest per row weighted by the softmax over those alone, plane k of a row =
    its k-th weight times ``W_down[e] act(W_up[e] y)``"""
    logits = L.linear(ctx, y, wr, torch.float32)
    idx, wts = K.moe_topk(logits, br, top)
    return experts(ctx, y, idx, wts, wup, wdown, top, act, dtype)


def experts(ctx, y: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, wup: torch.Tensor, wdown: torch.Tensor,
            top: int, act: str, dtype: torch.dtype) -> torch.Tensor:
    """32-bit planes ``[top, T, width]``: plane k holds ``wts[t, k] * W_down[e] act(W_up[e] y[t])`` for ``e = idx[t,
    k]``. ``wup`` ``[E, F, width]``, ``wdown`` ``[E, width, F]``"""
    T, width = y.shape
    E, F, _ = wup.shape
    if ctx.fast:
        from . import fast
        planes = fast.moe_experts(ctx, y, idx, wts, wup, wdown, top, act)
        if planes is not None:
            return planes
    plan = K.moe_plan(idx, E, K.moe_gemm_tile())
    h = torch.empty((T * top, F), dtype=dtype, device=y.device)
    K.moe_gemm_up(y, wup, plan, top, act, h)
    planes = torch.empty((top, T, width), dtype=torch.float32, device=y.device)
    K.moe_gemm_down(h, wdown, plan, wts, top, planes)
    return planes
