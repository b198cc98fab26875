"""``ParaRNN``: sequence wrapper that trains with the parallel Newton solve and evaluates with
the sequential unroll (reference ``layers/para_rnn.py:187-288``)."""

from __future__ import annotations

import copy

import torch
from torch import Tensor, nn

from .config import NewtonConfig, NewtonStats
from .newton import newton_apply
from .sequential import sequential_apply


class ParaRNN(nn.Module):
    def __init__(self, cell: nn.Module, *, config: NewtonConfig | None = None, num_layers: int = 1,
                 batch_first: bool = True, output_hidden: bool = True):
        super().__init__()
        if num_layers < 1:
            raise ValueError("num_layers must be >= 1")
        if num_layers > 1 and cell.d_in != cell.d_h:
            raise ValueError("stacking needs d_in == d_h")
        self.cells = nn.ModuleList([cell] + [copy.deepcopy(cell) for _ in range(num_layers - 1)])
        for extra in self.cells[1:]:
            extra.reset_parameters()
        self.config = config or NewtonConfig()
        self.batch_first = batch_first
        self.output_hidden = output_hidden
        self.last_stats: NewtonStats | None = None

    @property
    def cell(self) -> nn.Module:
        return self.cells[0]

    def forward(self, x: Tensor, h0: Tensor | None = None) -> Tensor:
        if not self.batch_first:
            x = x.transpose(0, 1)
        out = x
        for i, cell in enumerate(self.cells):
            h0_i = h0 if (h0 is not None and i == 0) else None
            slot = getattr(cell, "hidden_slot", None)
            hidden = slot is not None and (self.output_hidden or i + 1 < len(self.cells))
            if self.training:
                stats = NewtonStats()
                # the hidden slot straight from the solve: its backward takes the (B,T,d) cotangent
                out = newton_apply(cell, out, self.config, h0=h0_i, stats=stats,
                                   output_slot=slot if hidden else None)
                self.last_stats = stats
            else:
                states = sequential_apply(cell, out, h0_i)
                out = states[:, :, slot] if hidden else states
        if not self.batch_first:
            out = out.transpose(0, 1)
        return out
