"""Sequential unroll of ``cell.step``: the evaluation path and the numerical ground truth
behind every agreement check (reference ``solvers/sequential.py:24-120``).  Plain PyTorch;
it shares one ``W_x`` GEMM over all time steps."""

from __future__ import annotations

import torch
from torch import Tensor, nn

from .cells import zero_state


def sequential_apply(cell: nn.Module, x: Tensor, h0: Tensor | None = None, *, step=None,
                     cu_seqlens: Tensor | None = None) -> Tensor:
    if cu_seqlens is not None:
        raise NotImplementedError("packed cu_seqlens batches are not covered yet")
    batch, time, _ = x.shape
    if time < 1:
        raise ValueError(f"sequential_apply needs time >= 1, got {time}")
    h = h0 if h0 is not None else zero_state(cell, batch, x)
    wx_all = cell.W_x(x) if step is None and hasattr(cell, "W_x") else None
    step_fn = step or cell.step
    outs = []
    for t in range(time):
        h = step_fn(h, x[:, t]) if wx_all is None else step_fn(h, x[:, t], wx=wx_all[:, t])
        outs.append(h)
    return torch.stack(outs, dim=1)
