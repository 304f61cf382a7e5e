"""The experts of a mixture-of-experts feed-forward: the choice of kernels for the two grouped products."""
from __future__ import annotations

import torch

from . import lib as K


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
