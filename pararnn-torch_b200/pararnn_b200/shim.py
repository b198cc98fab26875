"""Route the UNMODIFIED reference package through this backend.

``install()`` replaces two functions of an imported ``pararnn`` package:

* ``pararnn.kernels.fused_newton.fused_newton`` (reference ``kernels/fused_newton.py:29-389``), the
  dispatcher behind ``scan_backend="fused"``: the fused Newton forward of ``ParaGRU`` (diag and
  head), ``ParaNLRU`` and ``ParaSLSTM(mix='diag')`` then runs on this library's kernels;
* ``pararnn.solvers.newton._eq26_vjp`` (reference ``solvers/newton/__init__.py:765-866``), the
  backward of ``_NewtonFixedPoint``: reverse scan, packed cell VJP and the ``W_x`` GEMMs.

Everything else of the reference stays in charge: ``newton_apply``, configuration, the Picard
retry ladder, ``_fill_stats`` and its divergence gate, the autograd Function.  Cells, knobs or
backends this library does not cover fall through to the reference's own functions.
``uninstall()`` restores them.  The reference's cell objects are used as they are: they expose the
same ``clipped_*`` accessors, ``W_x``, ``eps`` and ``max_recurrent_norm`` this package reads.
"""

from __future__ import annotations

import importlib

import torch

_saved = None


def _kind(cell) -> str | None:
    name, mix = type(cell).__name__, getattr(cell, "mix", "diag")
    if name == "ParaGRU":
        return "gru_diag" if mix == "diag" else ("gru_head" if mix == "head" else None)
    if name == "ParaNLRU":
        return "nlru"
    if name == "ParaTitans":
        return "titans"
    if name == "ParaCfC" and getattr(cell, "gate_mix", "input") == "input":
        return "cfc"
    if name == "ParaLSTM":
        return "lstm"
    if name == "ParaSLSTM" and mix == "diag":
        return "slstm_diag"
    return None


def _head_ok(cell) -> bool:
    return int(cell.d_h // cell.n_heads) in (8, 16, 32, 64)


def install():
    """Patch the imported reference package; returns nothing, idempotent."""
    global _saved
    if _saved is not None:
        return
    fn_mod = importlib.import_module("pararnn.kernels.fused_newton")
    newton_mod = importlib.import_module("pararnn.solvers.newton")
    ref_fused, ref_eq26 = fn_mod.fused_newton, newton_mod._eq26_vjp
    from . import head_ops, ops
    from .newton import _backward, input_affine

    def fused_newton(cell, wx, *, max_iters, omega, h0, log_coords=False, picard_iters=0, scan_tile="assoc",
                     fused_time_loop=False, fused_window_len=None, cu_seqlens=None, block_table=None,
                     early_exit_atol=None, residual_fn=None, iters_done_out=None):
        kind = _kind(cell)
        plain = (not log_coords and scan_tile == "assoc" and not fused_time_loop and fused_window_len is None
                 and residual_fn is None and wx.dtype in (torch.float32, torch.bfloat16))
        if kind is None or not plain or (kind == "gru_head" and not _head_ok(cell)):
            return ref_fused(cell, wx, max_iters=max_iters, omega=omega, h0=h0, log_coords=log_coords,
                             picard_iters=picard_iters, scan_tile=scan_tile, fused_time_loop=fused_time_loop,
                             fused_window_len=fused_window_len, cu_seqlens=cu_seqlens, block_table=block_table,
                             early_exit_atol=early_exit_atol, residual_fn=residual_fn,
                             iters_done_out=iters_done_out)
        if kind == "gru_diag":
            return ops.newton_gru_fused(wx, *cell.clipped_a(), h0, cu_seqlens, block_table, max_iters=max_iters,
                                        omega=omega, want_residual=False)
        if kind == "nlru":
            return ops.newton_nlru_fused(wx, cell.clipped_u(), h0, cu_seqlens, block_table, max_iters=max_iters,
                                         omega=omega, want_residual=False)
        if kind == "cfc":
            return ops.newton_cfc_fused(wx, cell.clipped_u(), h0, cu_seqlens, block_table, max_iters=max_iters,
                                        omega=omega, want_residual=False)
        if kind == "lstm":
            return ops.newton_lstm_fused(wx, *cell.clipped_recurrent(), h0, cu_seqlens, block_table,
                                         max_iters=max_iters, omega=omega, want_residual=False)
        if kind == "titans":
            return ops.newton_titans_fused(wx, cell.clipped_u(), cell.clipped_r(), h0, cu_seqlens, block_table,
                                           max_iters=max_iters, omega=omega, want_residual=False)
        if kind == "slstm_diag":
            return ops.newton_slstm_fused(wx, cell.clipped_r(), h0, None, block_table, max_iters=max_iters,
                                          omega=omega, eps=float(cell.eps), picard_iters=int(picard_iters or 0),
                                          want_residual=False, cu_seqlens=cu_seqlens)
        return head_ops.newton_gru_head_fused(wx, *cell.clipped_a_head(), h0, cu_seqlens, max_iters=max_iters,
                                              omega=omega, want_residual=False)

    def eq26_vjp(cell, states, x, partial, *, backend="eager", jacobian="auto", jac_structure=None, h0=None,
                 cu_seqlens=None):
        kind = _kind(cell)
        ours = (kind is not None and backend in ("fused", "triton") and jacobian in ("auto", "analytic")
                and jac_structure is None and states.is_cuda
                and states.dtype in (torch.float32, torch.bfloat16)
                and not (kind == "gru_head" and (cu_seqlens is not None or not _head_ok(cell))))
        if not ours:
            return ref_eq26(cell, states, x, partial, backend=backend, jacobian=jacobian,
                            jac_structure=jac_structure, h0=h0, cu_seqlens=cu_seqlens)
        with torch.no_grad():
            wx = input_affine(cell, x)
            grad_x, g_h0, grads = _backward(cell, kind, states, x.detach(), wx, partial, h0, None, cu_seqlens)
        aligned = []
        for name, p in cell.named_parameters():
            g = grads.get(name)
            aligned.append(g if (g is not None and p.requires_grad) else None)
        grad_h0 = None if (h0 is None or g_h0 is None) else g_h0.to(h0.dtype)
        return grad_x, tuple(aligned), grad_h0

    fn_mod.fused_newton = fused_newton
    newton_mod._eq26_vjp = eq26_vjp
    _saved = (fn_mod, ref_fused, newton_mod, ref_eq26)


def uninstall():
    global _saved
    if _saved is None:
        return
    fn_mod, ref_fused, newton_mod, ref_eq26 = _saved
    fn_mod.fused_newton = ref_fused
    newton_mod._eq26_vjp = ref_eq26
    _saved = None
