"""``newton_apply``: whole-trajectory Newton solve with the CUDA backend, and its
autograd contract.

Mirror of the reference driver (reference ``solvers/newton/__init__.py:212-324`` for the
entry point, ``:91-190`` for the autograd Function, ``:582-636`` for the residual gate,
``solvers/newton/picard.py:105-158`` for the Picard retry ladder, ``solvers/vjp.py`` for the
gradient packing).  Differences that a caller can observe:

* there is one backend.  ``scan_backend`` ``"auto"`` and ``"fused"`` select the CUDA kernels,
  ``"context_parallel"`` the time-sharded multi-GPU driver; ``"eager"`` and ``"triton"``
  raise, because this package ships neither a PyTorch nor a Triton solver;
* ``NewtonStats.residual_history`` is always filled (the kernels evaluate ``max|F|`` of every
  iterate on the device), and reading it costs one small device-to-host copy per forward;
* backward is one fused launch (reverse scan + packed VJP) followed by the two ``W_x`` GEMMs.
"""

from __future__ import annotations

import logging
import math
from dataclasses import replace

import torch
from torch import Tensor, nn

from . import ops
from .cells import cell_kind
from .config import (
    RESIDUAL_WARN,
    NewtonConfig,
    NewtonDivergenceError,
    NewtonStats,
    resolve_max_iters,
    slstm_auto_picard,
    slstm_picard_next,
    validate_config,
)

log = logging.getLogger("pararnn_b200.newton")


# --------------------------------------------------------------------------- resolution

def _resolve(cell: nn.Module, x: Tensor, config: NewtonConfig) -> tuple[NewtonConfig, str]:
    validate_config(config)
    kind = cell_kind(cell)
    if x.dim() != 3:
        raise ValueError(f"x must be (batch, time, d_in), got {tuple(x.shape)}")
    cfg = replace(config, max_iters=resolve_max_iters(config, x.shape[1]))
    if cfg.scan_backend in ("eager", "triton"):
        raise TypeError(
            f"scan_backend={cfg.scan_backend!r} is not available: pararnn_b200 has a single CUDA "
            "backend (use 'auto' or 'fused'; 'context_parallel' for time-sharded multi-GPU)")
    if cfg.scan_backend == "auto":
        cfg = replace(cfg, scan_backend="fused")
    if cfg.jacobian == "autograd":
        raise TypeError("the CUDA backend uses the analytic Jacobian of the built-in cells")
    if cfg.coords != "native":
        raise TypeError("coords='log' is not covered by the CUDA backend")
    if cfg.scan_tile != "assoc" or cfg.fused_time_loop or cfg.fused_window_len is not None:
        raise TypeError("scan_tile / fused_time_loop / fused_window_len ablations are not available")
    if cfg.newton_backtrack:
        raise TypeError("newton_backtrack is ParaM2RNN only")
    if kind == "slstm_diag":
        auto = cfg.picard_iters is None
        if auto:
            cfg = replace(cfg, picard_iters=slstm_auto_picard(x.shape[1]))
        if cfg.picard_adapt is None:
            cfg = replace(cfg, picard_adapt=auto)
    else:
        if cfg.picard_iters:
            raise TypeError(
                f"NewtonConfig(picard_iters=) is ParaSLSTM only (got {type(cell).__name__})")
        cfg = replace(cfg, picard_iters=0, picard_adapt=False)
    if not x.is_cuda:
        raise RuntimeError(
            "pararnn_b200.newton_apply needs CUDA tensors: this backend has no CPU solver "
            "(sequential_apply is the CPU-capable evaluation path)")
    return cfg, kind


def _recurrent_params(cell: nn.Module, kind: str):
    if kind == "gru_diag":
        return tuple(cell.clipped_a())
    if kind == "gru_head":
        return tuple(cell.clipped_a_head())
    if kind == "nlru":
        return (cell.clipped_u(),)
    if kind == "titans":
        return (cell.clipped_u(), cell.clipped_r())
    if kind == "cfc":
        return (cell.clipped_u(),)
    if kind == "lstm":
        return tuple(cell.clipped_recurrent())
    return (cell.clipped_r(),)


# --------------------------------------------------------------------------- forward

def input_affine(cell: nn.Module, x: Tensor) -> Tensor:
    """Input projection of the solve: ``cell.project_wx(x)`` where the cell packs more than
    ``W_x(x)`` (ParaCfC adds the time step and the time bias), else ``cell.W_x(x)`` (reference
    ``solvers/newton/__init__.py:959-967``)."""
    project = getattr(cell, "project_wx", None)
    return project(x) if callable(project) else cell.W_x(x)


def _solve_window(cell, kind, wx, h0, cfg, dstats, want_residual, cu_seqlens=None, block_table=None):
    rec = _recurrent_params(cell, kind)
    K = int(cfg.max_iters)
    if kind == "gru_diag":
        return ops.newton_gru_fused(wx, *rec, h0, cu_seqlens, block_table, max_iters=K, omega=cfg.omega,
                                    stats=dstats, want_residual=want_residual)
    if kind == "nlru":
        return ops.newton_nlru_fused(wx, rec[0], h0, cu_seqlens, block_table, max_iters=K, omega=cfg.omega,
                                     stats=dstats, want_residual=want_residual)
    if kind == "cfc":
        return ops.newton_cfc_fused(wx, rec[0], h0, cu_seqlens, block_table, max_iters=K, omega=cfg.omega,
                                    stats=dstats, want_residual=want_residual)
    if kind == "lstm":
        return ops.newton_lstm_fused(wx, *rec, h0, cu_seqlens, block_table, max_iters=K, omega=cfg.omega,
                                     stats=dstats, want_residual=want_residual)
    if kind == "titans":
        return ops.newton_titans_fused(wx, rec[0], rec[1], h0, cu_seqlens, block_table, max_iters=K,
                                       omega=cfg.omega, stats=dstats, want_residual=want_residual)
    if kind == "slstm_diag":
        return ops.newton_slstm_fused(wx, rec[0], h0, None, block_table, max_iters=K, omega=cfg.omega,
                                      eps=float(cell.eps), picard_iters=int(cfg.picard_iters or 0),
                                      stats=dstats, want_residual=want_residual, cu_seqlens=cu_seqlens)
    if cu_seqlens is not None or block_table is not None:
        raise TypeError("ParaGRU(mix='head') takes rectangular batches with a dense h0 only")
    from . import head_ops

    return head_ops.newton_gru_head_fused(wx, *rec, h0, max_iters=K, omega=cfg.omega, stats=dstats,
                                          want_residual=want_residual)


def _gate(cell, x, cfg, res, iters, hist, stats, status):
    """Fill ``stats`` and apply the divergence gate (reference ``_fill_stats``)."""
    if status != 0:
        raise RuntimeError(
            "pararnn_b200: a bounded device-side wait ran out during the scan "
            f"(status {status}); the result is not valid")
    if stats is not None:
        stats.max_residual = res
        stats.iters = iters
        stats.scan_backend = cfg.scan_backend
        stats.picard_iters = int(cfg.picard_iters or 0)
        stats.residual_history = tuple(hist)
    cap = cfg.residual_fail
    extra = {
        "max_residual": res, "residual_fail": cap, "iters": iters, "seq_len": int(x.shape[1]),
        "batch": int(x.shape[0]), "cell": type(cell).__name__,
        "picard_iters": int(cfg.picard_iters or 0), "scan_backend": cfg.scan_backend,
        "residual_history": tuple(hist)[-8:],
    }
    if cap is not None and (not math.isfinite(res) or res > cap):
        log.error("newton_diverged", extra=extra)
        raise NewtonDivergenceError(
            f"Newton residual {res:.3e} after {iters} iters exceeds residual_fail={cap:g} "
            f"(seq_len={x.shape[1]}, picard={int(cfg.picard_iters or 0)}, "
            f"history={tuple(hist)[-8:]!r}). For ParaSLSTM raise picard_iters.")
    if res > RESIDUAL_WARN and log.isEnabledFor(logging.WARNING):
        log.warning("newton_residual_high", extra=extra)


def _emulated_iters(hist, cfg) -> int:
    """Number of residual evaluations the eager loop would report: it stops at the first
    iterate whose residual is below ``residual_atol`` (reference ``__init__.py:526-533``).
    Only used with ``fused_early_exit``; the kernels always run all K passes."""
    if cfg.fused_early_exit and cfg.residual_atol is not None:
        for k, r in enumerate(hist):
            if r < cfg.residual_atol:
                return k + 1
    return int(cfg.max_iters)


def _forward_once(cell, kind, x, cfg, h0, stats, wx=None, cu_seqlens=None, block_table=None):
    """One full solve (all windows); returns ``(states, wx)``.  Reads the device statistics
    only when somebody consumes them."""
    if wx is None:
        wx = input_affine(cell, x)
    need_stats = stats is not None or cfg.residual_fail is not None
    K = int(cfg.max_iters)
    if cfg.chunk_len is None:
        ds = ops.DeviceStats(x.device, K)
        states = _solve_window(cell, kind, wx, h0, cfg, ds, need_stats, cu_seqlens, block_table)
        if need_stats:
            hist, res, status = ds.read()
            ops.check_pending_backward()
            _gate(cell, x, cfg, res, _emulated_iters(hist, cfg), hist, stats, status)
        return states, wx
    # windowed solve: the last state of a window is the next window's h0
    # (reference _newton_chunked, __init__.py:552-579)
    length = int(cfg.chunk_len)
    parts, carry, blocks = [], h0, []
    for t0 in range(0, x.shape[1], length):
        ds = ops.DeviceStats(x.device, K)
        piece = _solve_window(cell, kind, wx[:, t0:t0 + length], carry, cfg, ds, need_stats)
        parts.append(piece)
        blocks.append(ds)
        carry = piece[:, -1]
    states = torch.cat(parts, dim=1)
    if need_stats:
        ops.check_pending_backward()
        res, iters, status = 0.0, 0, 0
        for ds in blocks:
            hist, r, st = ds.read()
            res = r if (r != r or r > res) else res
            iters += _emulated_iters(hist, cfg)
            status |= st
        _gate(cell, x, cfg, res, iters, (), stats, status)
    return states, wx


def _forward(cell, kind, x, cfg, h0, stats, cu_seqlens=None, block_table=None):
    if not (cfg.picard_adapt and kind == "slstm_diag"):
        return _forward_once(cell, kind, x, cfg, h0, stats, cu_seqlens=cu_seqlens, block_table=block_table)
    # Picard retry ladder: re-run at the next rung while the residual is outside the basin
    cur = cfg
    wx = None
    while True:
        st = stats if stats is not None else NewtonStats()
        states, wx = _forward_once(cell, kind, x, replace(cur, residual_fail=None), h0, st, wx=wx,
                                   cu_seqlens=cu_seqlens, block_table=block_table)
        res = st.max_residual
        nxt = slstm_picard_next(int(cur.picard_iters or 0))
        retry = (not math.isfinite(res)
                 or (cfg.picard_retry_atol is not None and res > cfg.picard_retry_atol)
                 or (cfg.residual_fail is not None and res > cfg.residual_fail))
        if retry and nxt is not None:
            log.info("picard_adapt", extra={"from_p": int(cur.picard_iters or 0), "to_p": nxt,
                                            "max_residual": res, "seq_len": int(x.shape[1])})
            cur = replace(cur, picard_iters=nxt)
            continue
        if cfg.residual_fail is not None and (not math.isfinite(res) or res > cfg.residual_fail):
            _gate(cell, x, replace(cur, residual_fail=cfg.residual_fail), res, st.iters,
                  st.residual_history, st, 0)
        return states, wx


# --------------------------------------------------------------------------- backward

def _clip_mask(raw: Tensor, cap) -> Tensor | None:
    return None if cap is None else (raw.abs() <= cap)


_BIAS = "__bias__"  # key of the kernel-side sum of g_wx in the dict `_reverse_window` returns


def _reverse_window(cell, kind, states, wx, grad_states, h0, grad_slot=None):
    rec = _recurrent_params(cell, kind)
    if kind == "gru_diag":
        g_wx, gz, gr, gn, g_h0, gb = ops.gru_reverse_vjp(states, wx, *rec, grad_states, h0, want_bias=True)
        return g_wx, {"a_z": gz, "a_r": gr, "a_n": gn, _BIAS: gb}, g_h0
    if kind == "nlru":
        g_wx, gu, g_h0, gb = ops.nlru_reverse_vjp(states, wx, rec[0], grad_states, h0, want_bias=True)
        return g_wx, {"u": gu, _BIAS: gb}, g_h0
    if kind == "cfc":
        g_wx, gu, g_h0, gb = ops.cfc_reverse_vjp(states, wx, rec[0], grad_states, h0, want_bias=True)
        return g_wx, {"u": gu, _BIAS: gb}, g_h0
    if kind == "lstm":
        g_wx, gp, g_h0 = ops.lstm_reverse_vjp(states, wx, *rec, grad_states, h0)
        return g_wx, {n: gp[i] for i, n in enumerate(("a_f", "a_z", "a_o", "c_f", "c_o"))}, g_h0
    if kind == "titans":
        g_wx, gu, gr, g_h0, gb = ops.titans_reverse_vjp(states, wx, rec[0], rec[1], grad_states, h0,
                                                        want_bias=True)
        return g_wx, {"u": gu, "r": gr, _BIAS: gb}, g_h0
    if kind == "slstm_diag":
        g_wx, gr, g_h0, g_bias = ops.slstm_reverse_vjp(states, wx, rec[0], grad_states, h0, float(cell.eps),
                                                       grad_slot=grad_slot, want_bias=True)
        return g_wx, {"R": gr, _BIAS: g_bias}, g_h0
    from . import head_ops

    g_wx, gz, gr, gn, g_h0 = head_ops.gru_head_reverse_vjp(states, wx, *rec, grad_states, h0)
    return g_wx, {"A_z": gz, "A_r": gr, "A_n": gn}, g_h0


def _backward(cell, kind, states, x, wx, grad_states, h0, chunk_len, cu_seqlens=None, grad_slot=None):
    """``(grad_x, grad_h0, {name: grad})`` — eq. 2.6 + packed VJP + the W_x GEMMs.
    ``grad_slot``: ``grad_states`` is the ``(B,T,d)`` cotangent of that state slot alone."""
    if grad_slot is not None and (cu_seqlens is not None or chunk_len is not None or kind != "slstm_diag"):
        # only the one-window sLSTM kernel takes the compact cotangent
        full = torch.zeros_like(states)
        full[:, :, grad_slot] = grad_states
        grad_states, grad_slot = full, None
    if cu_seqlens is not None:
        # packed sequences: independent reverse scans, grad_h0 (S, ...) row by row
        cs = ops.validate_cu_seqlens(cu_seqlens, x.shape[1])
        g_wx = torch.empty_like(wx)
        rec_grads, heads = {}, []
        for i in range(len(cs) - 1):
            lo, hi = cs[i], cs[i + 1]
            g_piece, rg, head = _reverse_window(cell, kind, states[:, lo:hi], wx[:, lo:hi],
                                                grad_states[:, lo:hi], None if h0 is None else h0[i:i + 1])
            g_wx[:, lo:hi] = g_piece
            heads.append(head)
            for k, v in rg.items():
                rec_grads[k] = v if k not in rec_grads else rec_grads[k] + v
        g_h0 = torch.cat(heads, dim=0)
    elif chunk_len is None:
        g_wx, rec_grads, g_h0 = _reverse_window(cell, kind, states, wx, grad_states, h0, grad_slot)
    else:
        # same windows as the forward, walked backwards; grad_h0 of window i+1 is added to
        # the cotangent of the last step of window i (reference _eq26_vjp_chunked)
        length, time = int(chunk_len), x.shape[1]
        g_wx = torch.empty_like(wx)
        rec_grads, carry = {}, None
        for t0 in reversed(range(0, time, length)):
            t1 = min(t0 + length, time)
            gw = grad_states[:, t0:t1]
            if carry is not None:
                gw = gw.clone()
                gw[:, -1] += carry.to(gw.dtype)
            h0_w = h0 if t0 == 0 else states[:, t0 - 1]
            g_piece, rg, carry = _reverse_window(cell, kind, states[:, t0:t1], wx[:, t0:t1], gw, h0_w)
            g_wx[:, t0:t1] = g_piece
            for k, v in rg.items():
                rec_grads[k] = v if k not in rec_grads else rec_grads[k] + v
        g_h0 = carry
    cap = getattr(cell, "max_recurrent_norm", None)
    named = dict(cell.named_parameters())
    grads = {}
    bias_sum = rec_grads.pop(_BIAS, None)
    for name, g in rec_grads.items():
        raw = named[name]
        g = g.reshape(raw.shape)
        mask = _clip_mask(raw.detach(), cap)
        if mask is not None:
            g = g * mask
        grads[name] = g.to(raw.dtype)
    if kind == "cfc":
        grad_x, lin_grads = _cfc_input_grads(cell, x, g_wx, bias_sum)
        grads.update(lin_grads)
        return grad_x, g_h0, grads
    lin = cell.W_x
    gy = g_wx.reshape(-1, g_wx.shape[-1])
    xx = x.reshape(-1, x.shape[-1])
    grad_x = (gy @ lin.weight.detach().to(gy.dtype)).reshape(x.shape)
    grads["W_x.weight"] = (gy.t() @ xx.to(gy.dtype)).to(lin.weight.dtype)
    if lin.bias is not None:
        # the sLSTM reverse kernel accumulates the sum of g_wx itself; the other cells sum here
        grads["W_x.bias"] = (gy.sum(0) if bias_sum is None else bias_sum).to(lin.bias.dtype)
    return grad_x, g_h0, grads


def _cfc_input_grads(cell, x, g_wx, bias_sum=None):
    """Gradients of ``project_wx``: ``g_wx (B,T,4d)`` holds the grads of ``(f, c, dt, b)``.
    ``(f, c)`` go through ``W_x``, ``b`` through ``W_b``, both on the features; the time step
    gets the channel sum of its block where the clamp was inactive (reference
    ``solvers/vjp.py:180-211``)."""
    from .cells import CFC_DT_EPS

    d = cell.d_h
    feat = x[..., :-1].reshape(-1, x.shape[-1] - 1)
    g = g_wx.reshape(-1, 4 * d)
    g_fc, g_dt, g_b = g[:, :2 * d], g[:, 2 * d:3 * d], g[:, 3 * d:]
    wx_w, wb_w = cell.W_x.weight.detach().to(g.dtype), cell.W_b.weight.detach().to(g.dtype)
    grad_feat = g_fc @ wx_w + g_b @ wb_w
    grad_dt = g_dt.sum(-1, keepdim=True) * (x[..., -1:].reshape(-1, 1) >= CFC_DT_EPS).to(g.dtype)
    grad_x = torch.cat((grad_feat, grad_dt), dim=-1).reshape(x.shape)
    featc = feat.to(g.dtype)
    grads = {"W_x.weight": (g_fc.t() @ featc).to(cell.W_x.weight.dtype),
             "W_b.weight": (g_b.t() @ featc).to(cell.W_b.weight.dtype)}
    # bias_sum: the reverse kernel's own per-gate sums of g_wx, (4d,) in the order (f, c, dt, b)
    if cell.W_x.bias is not None:
        grads["W_x.bias"] = (g_fc.sum(0) if bias_sum is None else bias_sum[:2 * d]).to(cell.W_x.bias.dtype)
    if cell.W_b.bias is not None:
        grads["W_b.bias"] = (g_b.sum(0) if bias_sum is None else bias_sum[3 * d:]).to(cell.W_b.bias.dtype)
    return grad_x, grads


class _NewtonFixedPoint(torch.autograd.Function):
    """Forward = Newton solve without a graph; backward = implicit-function gradient
    (one reverse scan with J^T, then the cell VJP), returned as
    ``(grad_x, grad_h0, *param_grads)`` in ``cell.named_parameters()`` order."""

    @staticmethod
    def forward(ctx, cell, kind, cfg, stats, has_h0, cu_seqlens, out_slot, x_in, h0_in, *params):
        del params
        h0 = h0_in if has_h0 else None
        with torch.no_grad():
            states, wx = _forward(cell, kind, x_in, cfg, h0, stats, cu_seqlens=cu_seqlens)
        ctx.cell, ctx.kind, ctx.cfg, ctx.has_h0, ctx.cu_seqlens = cell, kind, cfg, has_h0, cu_seqlens
        ctx.out_slot = out_slot
        if cfg.recompute:
            ctx.save_for_backward(x_in, h0_in)
        else:
            ctx.save_for_backward(x_in, h0_in, states, wx)
        # one slot only: a view of the trajectory; the backward then receives its (B,T,d) cotangent
        return states if out_slot is None else states.select(2, out_slot)

    @staticmethod
    def backward(ctx, grad_states):
        cell, kind, cfg = ctx.cell, ctx.kind, ctx.cfg
        if cfg.recompute:
            x_in, h0_in = ctx.saved_tensors
            h0 = h0_in if ctx.has_h0 else None
            with torch.no_grad():
                states, wx = _forward(cell, kind, x_in, replace(cfg, residual_fail=None,
                                                                 picard_adapt=False), h0, None,
                                      cu_seqlens=ctx.cu_seqlens)
        else:
            x_in, h0_in, states, wx = ctx.saved_tensors
            h0 = h0_in if ctx.has_h0 else None
        with torch.no_grad():
            grad_x, g_h0, grads = _backward(cell, kind, states, x_in.detach(), wx,
                                            grad_states, h0, cfg.chunk_len, ctx.cu_seqlens, ctx.out_slot)
        out_params = []
        for name, p in cell.named_parameters():
            g = grads.get(name)
            out_params.append(g if (g is not None and p.requires_grad) else None)
        if not x_in.requires_grad:
            grad_x = None
        grad_h0 = None
        if ctx.has_h0 and h0_in.requires_grad and g_h0 is not None:
            grad_h0 = g_h0.to(h0_in.dtype)
        return (None, None, None, None, None, None, None, grad_x, grad_h0, *out_params)


def newton_apply(cell: nn.Module, x: Tensor, config: NewtonConfig | None = None, *,
                 h0: Tensor | None = None, stats: NewtonStats | None = None,
                 cu_seqlens: Tensor | None = None, block_table: Tensor | None = None,
                 output_slot: int | None = None) -> Tensor:
    """Solve ``F(H) = 0`` for the whole trajectory with Newton + chained scans on the GPU.

    Same call signature and return layout as the reference's ``newton_apply``:
    ``x (B, T, d_in)`` -> ``H (B, T, *state)`` (``(B,T,d)`` for GRU / NLRU, ``(B,T,4,d)`` for
    sLSTM).  Raises ``NewtonDivergenceError`` when the final ``max|F|`` is non-finite or above
    ``config.residual_fail``.

    ``cu_seqlens`` ``(S+1,)``: ``x`` is a packed ``(1, N, d_in)`` batch of S sequences, each its
    own scan starting from ``h0[s]`` (``h0`` is ``(S, *state)``), differentiable.  ``block_table``
    ``(B,)`` or ``(S,)``: ``h0`` is a pool ``(C, *state)`` and sequence ``i`` starts from
    ``h0[block_table[i]]``; inference only, as in the reference
    (``solvers/newton/__init__.py:286-304``).

    ``output_slot`` (not in the reference; multi-slot cells only): return ``H[:, :, output_slot]``
    ``(B,T,d)`` instead of all slots.  Same values as slicing the full result, but the backward
    takes the ``(B,T,d)`` cotangent as it is instead of a zero-filled ``(B,T,S,d)`` array;
    ``ParaRNN`` uses it for the hidden slot."""
    cfg, kind = _resolve(cell, x, config or NewtonConfig())
    if output_slot is not None:
        slots = int(getattr(cell, "state_slots", 1))
        if slots == 1 or not 0 <= int(output_slot) < slots:
            raise ValueError(f"output_slot={output_slot} needs a cell with state slots, 0 <= slot < {slots}")
        output_slot = int(output_slot)
    if cu_seqlens is not None or block_table is not None:
        if kind == "gru_head":
            raise TypeError("ParaGRU(mix='head') takes rectangular batches with a dense h0 only")
        if cfg.chunk_len is not None:
            raise ValueError("chunk_len cannot be combined with cu_seqlens / block_table")
        if cfg.scan_backend == "context_parallel":
            raise ValueError("cu_seqlens / block_table cannot be combined with scan_backend='context_parallel'")
    if cu_seqlens is not None and x.shape[0] != 1:
        raise ValueError(f"cu_seqlens packs x with batch=1, got batch={x.shape[0]}")
    if cfg.scan_backend == "context_parallel":
        from .seq_shard import newton_apply_sharded

        H = newton_apply_sharded(cell, kind, x, cfg, h0=h0, stats=stats)
        return H if output_slot is None else H[:, :, output_slot]
    if torch.is_autocast_enabled("cuda"):
        ctx_mgr = torch.autocast(device_type="cuda", enabled=False)
    else:
        import contextlib

        ctx_mgr = contextlib.nullcontext()
    params = tuple(cell.parameters())
    has_h0 = h0 is not None
    needs_grad = torch.is_grad_enabled() and (
        x.requires_grad or (has_h0 and h0.requires_grad) or any(p.requires_grad for p in params))
    if block_table is not None and needs_grad:
        raise RuntimeError("block_table newton is inference-only")
    with ctx_mgr:
        if not needs_grad:
            with torch.no_grad():
                H = _forward(cell, kind, x, cfg, h0, stats, cu_seqlens=cu_seqlens, block_table=block_table)[0]
                return H if output_slot is None else H[:, :, output_slot]
        h0_leaf = h0 if has_h0 else x.new_zeros(())
        return _NewtonFixedPoint.apply(cell, kind, cfg, stats, has_h0, cu_seqlens, output_slot, x, h0_leaf,
                                       *params)
