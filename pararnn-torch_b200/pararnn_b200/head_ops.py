"""Operators for ``ParaGRU(mix='head')`` (per-head dense recurrence).

Mirrors ``pararnn::newton_gru_head_fused`` / ``pararnn::reverse_gru_head_factor`` and
``gru_head_recurrence_vjp`` of the reference (reference ``kernels/custom_ops.py:311-434``,
``kernels/vjp_gru.py:656-810``).  ``d_head`` must be 8, 16, 32 or 64."""

from __future__ import annotations

import torch
from torch import Tensor

from . import _lib as L
from .ops import (DeviceStats, _check_cuda, _check_iters, _dtype_code, _ptr, _raise,
                  _same, _stream, _workspace)


def _head_shape(wx: Tensor, a_z: Tensor):
    if wx.dim() != 3 or wx.shape[-1] % 3:
        raise ValueError(f"wx must be (B, T, 3*d), got {tuple(wx.shape)}")
    B, T, d3 = wx.shape
    d = d3 // 3
    if a_z.dim() != 3 or a_z.shape[1] != a_z.shape[2] or a_z.shape[0] * a_z.shape[1] != d:
        raise ValueError(f"A_* must be (n_heads, d_head, d_head) with n_heads*d_head = {d}, got {tuple(a_z.shape)}")
    H, dh = a_z.shape[0], a_z.shape[1]
    if dh not in (8, 16, 32, 64):
        raise TypeError(f"the CUDA backend covers d_head in (8, 16, 32, 64), got {dh}")
    return B, T, d, H


def newton_gru_head_fused(wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor, h0: Tensor | None = None,
                          cu_seqlens: Tensor | None = None, *, max_iters: int, omega: float = 1.0,
                          stats: DeviceStats | None = None, want_residual: bool = True) -> Tensor:
    """Fused Newton for ``ParaGRU(mix='head')``: ``wx (B,T,3d)`` -> ``H (B,T,d)`` in ``wx.dtype``."""
    if cu_seqlens is not None:
        # same rule as the reference's dispatcher (kernels/custom_ops.py:323-328)
        raise TypeError("ParaGRU(mix='head') takes rectangular batches only: pad the packed sequences")
    dev = _check_cuda(wx, a_z, a_r, a_n, h0)
    _check_iters(max_iters)
    B, T, d, H = _head_shape(wx, a_z)
    for p in (a_r, a_n):
        if tuple(p.shape) != tuple(a_z.shape):
            raise ValueError("A_z, A_r, A_n must have the same shape")
    if h0 is not None and tuple(h0.shape) != (B, d):
        raise ValueError(f"h0 must be ({B}, {d}), got {tuple(h0.shape)}")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    az, ar, an, h0c = _same(a_z, wx), _same(a_r, wx), _same(a_n, wx), _same(h0, wx)
    out = torch.empty(B, T, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(lib.prb_gru_head_workspace_bytes(B, T, d, H, int(max_iters)), dev)
        rc = lib.prb_newton_gru_head_fused(_ptr(wx_c), _ptr(az), _ptr(ar), _ptr(an), _ptr(h0c), _ptr(out),
                                           B, T, d, H, code, int(max_iters), float(omega),
                                           int(want_residual), _ptr(ws), ws.numel(), _ptr(st.buf),
                                           _stream(dev))
    _raise(rc, "newton_gru_head_fused")
    return out


def gru_head_reverse_vjp(states: Tensor, wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor,
                         grad_states: Tensor, h0: Tensor | None = None, mu_out: Tensor | None = None):
    """Reverse walk with the factorised ``J^T`` fused with the gate part of the packed VJP.
    Returns ``(g_wx, g_Az, g_Ar, g_An, g_h0)``; the ``A`` gradients are fp32 ``(H, dh, dh)``
    outer-product sums accumulated by the same kernel (no clip mask applied)."""
    dev = _check_cuda(states, wx, a_z, a_r, a_n, grad_states, h0)
    B, T, d, H = _head_shape(wx, a_z)
    dh = d // H
    if tuple(states.shape) != (B, T, d) or tuple(grad_states.shape) != (B, T, d):
        raise ValueError("states / grad_states must be (B, T, d)")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    st = states.detach().to(wx.dtype).contiguous()
    gs = grad_states.detach().to(wx.dtype).contiguous()
    az, ar, an, h0c = _same(a_z, wx), _same(a_r, wx), _same(a_n, wx), _same(h0, wx)
    g_wx = torch.empty_like(wx_c)
    g_a = torch.empty(3, H, dh, dh, dtype=torch.float32, device=dev)
    g_h0 = torch.empty(B, d, dtype=torch.float32, device=dev)
    sb = DeviceStats(dev, 0)
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(lib.prb_gru_head_workspace_bytes(B, T, d, H, 0), dev)
        rc = lib.prb_bwd_gru_head(_ptr(st), _ptr(wx_c), _ptr(az), _ptr(ar), _ptr(an), _ptr(h0c), _ptr(gs),
                                  _ptr(g_wx), _ptr(g_a), _ptr(g_h0), _ptr(mu_out), B, T, d, H, code, _ptr(ws),
                                  ws.numel(),
                                  _ptr(sb.buf), _stream(dev))
    _raise(rc, "gru_head_reverse_vjp")
    g_az, g_ar, g_an = g_a.unbind(0)
    return g_wx, g_az, g_ar, g_an, g_h0
