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
        # packed (1, N, d_in): every sequence unrolled on its own from its own h0 row
        from .ops import validate_cu_seqlens

        if x.shape[0] != 1:
            raise ValueError(f"cu_seqlens packs x with batch=1, got batch={x.shape[0]}")
        cs = validate_cu_seqlens(cu_seqlens, x.shape[1])
        if h0 is not None and h0.shape[0] != len(cs) - 1:
            raise ValueError(f"h0 batch {h0.shape[0]} != n_seq {len(cs) - 1}")
        return torch.cat([sequential_apply(cell, x[:, a:b], None if h0 is None else h0[i:i + 1], step=step)
                          for i, (a, b) in enumerate(zip(cs[:-1], cs[1:]))], dim=1)
    batch, time, _ = x.shape
    if time < 1:
        raise ValueError(f"sequential_apply needs time >= 1, got {time}")
    h = h0 if h0 is not None else zero_state(cell, batch, x)
    wx_all = None
    if step is None and hasattr(cell, "W_x"):
        project = getattr(cell, "project_wx", None)  # reference solvers/sequential.py:70
        wx_all = project(x) if callable(project) else cell.W_x(x)
    if step is None and time == 1 and wx_all is not None and not torch.is_grad_enabled():
        # T = 1 without a graph: the one-launch decode kernel (reference solvers/sequential.py:77-81)
        from .decode import can_decode_step, decode_step

        if can_decode_step(cell, wx_all):
            return decode_step(cell, h, wx=wx_all[:, 0]).unsqueeze(1)
    step_fn = step or cell.step
    outs = []
    for t in range(time):
        h = step_fn(h, x[:, t]) if wx_all is None else step_fn(h, x[:, t], wx=wx_all[:, t])
        outs.append(h)
    return torch.stack(outs, dim=1)
