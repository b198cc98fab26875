"""``decode_step``: one recurrent step (T = 1) in one CUDA launch -- the serving-side
counterpart of the training path (reference ``kernels/decode.py:55-216``).

Same call signature and rules as the reference: ``wx`` is an optional precomputed ``W_x(x)``,
``out=`` reuses a buffer (CUDA graphs, decode loops), ``block_table`` indexes a pool-shaped
``state`` / ``out`` and updates the named rows in place.  The kernel clamps the recurrent
parameters itself, so a step captured in a CUDA graph launches the GEMM and this one kernel and
allocates nothing.  Cells without a kernel here (``ParaGRU(mix='head')``), CPU tensors and calls
with gradients enabled run the cell's own PyTorch ``step``, as in the reference.
"""

from __future__ import annotations

import ctypes

import torch
from torch import Tensor, nn

from . import _lib as L
from .cells import cell_kind

_CELL = {"gru_diag": L.CELL_GRU_DIAG, "nlru": L.CELL_NLRU, "slstm_diag": L.CELL_SLSTM_DIAG,
         "titans": L.CELL_TITANS, "cfc": L.CELL_CFC}


def can_decode_step(cell: nn.Module, ref: Tensor) -> bool:
    """Whether ``decode_step`` runs the CUDA kernel for this cell on ``ref``'s device and dtype."""
    if not ref.is_cuda or ref.dtype not in (torch.float32, torch.bfloat16):
        return False
    try:
        return cell_kind(cell) in _CELL
    except TypeError:
        return False


def _squeeze_time(wx: Tensor) -> Tensor:
    if wx.dim() == 3:
        if wx.shape[1] != 1:
            raise ValueError(f"decode_step wx time dim must be 1, got {tuple(wx.shape)}")
        return wx[:, 0]
    if wx.dim() != 2:
        raise ValueError(f"decode_step wx needs (B, G*d_h), got {tuple(wx.shape)}")
    return wx


def decode_wx(cell: nn.Module, x: Tensor, *, out: Tensor | None = None) -> Tensor:
    """``W_x(x)`` for one step, optionally into a preallocated ``(batch, G*d_h)`` buffer."""
    lin = getattr(cell, "W_x", None)
    if lin is None:
        raise TypeError(f"decode_wx needs cell.W_x; got {type(cell).__name__}")
    x2 = _squeeze_time(x) if x.dim() == 3 else x
    project = getattr(cell, "project_wx", None)
    if callable(project):  # ParaCfC: (f, c, dt, b), not a single linear map
        y = project(x2)
        if out is None:
            return y
        out.copy_(y)
        return out
    if out is None:
        return lin(x2)
    torch.mm(x2, lin.weight.t(), out=out)
    if lin.bias is not None:
        out.add_(lin.bias)
    return out


def _raw_params(cell: nn.Module, kind: str, dtype) -> Tensor:
    if kind == "gru_diag":
        p = torch.stack([cell.a_z, cell.a_r, cell.a_n])
    elif kind in ("nlru", "cfc"):
        p = cell.u[None]
    elif kind == "titans":
        p = torch.stack([cell.u, cell.r])
    else:
        p = cell.R
    return p.detach().to(dtype).contiguous()


def decode_step(cell: nn.Module, state: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None,
                out: Tensor | None = None, block_table: Tensor | None = None) -> Tensor:
    """One sequential recurrent step.  Returns the next state (``out`` when given; the pool itself
    when ``block_table`` is given without ``out``)."""
    ref = wx if wx is not None else x
    if ref is None:
        raise ValueError("decode_step needs x or wx (precomputed W_x(x))")
    if not (can_decode_step(cell, ref) and not torch.is_grad_enabled()):
        if block_table is not None:
            raise RuntimeError("block_table requires the CUDA decode_step kernel")
        y = cell.step(state, x, wx=wx)
        if out is None:
            return y
        out.copy_(y)
        return out
    kind = cell_kind(cell)
    if wx is None:
        wx = decode_wx(cell, x)
    wx = _squeeze_time(wx)
    capturing = torch.cuda.is_current_stream_capturing()
    if capturing:
        if not state.is_contiguous() or not wx.is_contiguous():
            raise RuntimeError("decode_step CUDA graph needs contiguous state and wx")
        if out is None and block_table is None:
            raise RuntimeError("decode_step CUDA graph needs out= (or block_table in-place)")
    elif not state.is_contiguous():
        state = state.contiguous()
    if not wx.is_contiguous():
        wx = wx.contiguous()
    if wx.dtype != state.dtype:
        raise ValueError("decode_step state and wx must have the same dtype")
    bt = None
    if block_table is None:
        if out is None:
            out = torch.empty_like(state)
        elif out.shape != state.shape:
            raise ValueError(f"decode_step out shape {tuple(out.shape)} != state {tuple(state.shape)}")
        batch = int(state.shape[0])
    else:
        bt = block_table.to(device=state.device, dtype=torch.int32).contiguous()
        if bt.dim() != 1:
            raise ValueError(f"block_table must be 1-D (B,), got {tuple(bt.shape)}")
        batch = int(bt.numel())
        if out is None:
            out = state
        elif out.shape != state.shape:
            raise ValueError("block_table decode writes pool-shaped out "
                             f"(same as state {tuple(state.shape)}), got {tuple(out.shape)}")
    if out.dtype != state.dtype or out.device != state.device or not out.is_contiguous():
        raise ValueError("decode_step out must be contiguous and match state dtype and device")
    if wx.shape[0] != batch:
        raise ValueError(f"decode_step wx batch {wx.shape[0]} != {batch}")
    d = int(cell.d_h)
    cap = getattr(cell, "max_recurrent_norm", None)
    # the parameter pack is rebuilt per call outside a capture; inside one the cached pack is used
    pack = getattr(cell, "_prb_decode_pack", None)
    if pack is None or not capturing or pack.dtype != state.dtype or pack.device != state.device:
        pack = _raw_params(cell, kind, state.dtype)
        cell._prb_decode_pack = pack
    code = L.PRB_F32 if state.dtype == torch.float32 else L.PRB_BF16
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())  # noqa: E731
    with torch.cuda.device(state.device):
        rc = L.lib().prb_decode_step(_CELL[kind], p(state), p(wx), p(pack), -1.0 if cap is None else float(cap),
                                     p(bt), p(out), batch, d, code, float(getattr(cell, "eps", 1e-6)),
                                     ctypes.c_void_p(torch.cuda.current_stream(state.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(f"decode_step: {L.error_string(rc)} (code {rc})")
    return out
