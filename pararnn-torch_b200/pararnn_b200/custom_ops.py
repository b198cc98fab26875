"""``torch.library`` registration of the CUDA backend's operators.

The reference registers its fused ops as ``pararnn::newton_*_fused`` with ``register_fake`` meta
kernels so that Dynamo treats them as opaque calls (reference ``kernels/custom_ops.py:146-540``).
This module does the same under the namespace ``pararnn_b200::`` -- a different namespace, so the
reference can be imported in the same process -- with IDENTICAL argument lists, so a shim can map
one onto the other.  As in the reference the fused ops are not differentiable: gradients flow
through ``newton_apply`` (eq. 2.6), never through these ops.

Registered:

* ``pararnn_b200::newton_gru_fused``, ``::newton_nlru_fused``, ``::newton_cfc_fused``,
  ``::newton_titans_fused``, ``::newton_lstm_fused``, ``::newton_slstm_fused``,
  ``::newton_gru_head_fused``  (reference
  ``custom_ops.py:146-188, 191-227, 230-266, 269-308, 437-483, 486-540, 311-386``);
* ``pararnn_b200::reverse_gru_head_factor``  (reference ``custom_ops.py:389-434``);
* ``pararnn_b200::reverse_gru_vjp``, ``::reverse_nlru_vjp``, ``::reverse_slstm_vjp``,
  ``::reverse_gru_head_vjp``: the reverse scan fused with the packed VJP.  The reference has these
  as a scan op plus plain functions (``solvers/scan.py:126-203``, ``kernels/vjp_*.py``); here each
  is one op.

One difference in behaviour: the reference's ``newton_slstm_fused`` is called with a ``states``
guess produced by ``slstm_picard_init``; here ``states=None`` makes the op run the frozen-gate warm
start itself, with the number of Picard passes taken from ``set_default_picard_iters`` (the op
signature has no such argument; ``ops.newton_slstm_fused`` takes it explicitly).
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import head_ops, ops

_picard_default = 0


def set_default_picard_iters(n: int) -> None:
    """Picard passes run by ``pararnn_b200::newton_slstm_fused`` when no ``states`` guess is given."""
    global _picard_default
    if n < 0:
        raise ValueError("picard iterations must be >= 0")
    _picard_default = int(n)


# ------------------------------------------------------------------------------------ forward

@torch.library.custom_op("pararnn_b200::newton_gru_fused", mutates_args=())
def newton_gru_fused(wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor, h0: Tensor | None = None,
                     cu_seqlens: Tensor | None = None, block_table: Tensor | None = None, *,
                     max_iters: int, omega: float) -> Tensor:
    return ops.newton_gru_fused(wx, a_z, a_r, a_n, h0, cu_seqlens, block_table, max_iters=max_iters,
                                omega=omega, want_residual=False)


@newton_gru_fused.register_fake
def _(wx, a_z, a_r, a_n, h0=None, cu_seqlens=None, block_table=None, *, max_iters, omega):
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, int(a_z.numel()))


@torch.library.custom_op("pararnn_b200::newton_nlru_fused", mutates_args=())
def newton_nlru_fused(wx: Tensor, u: Tensor, h0: Tensor | None = None, cu_seqlens: Tensor | None = None,
                      block_table: Tensor | None = None, *, max_iters: int, omega: float) -> Tensor:
    return ops.newton_nlru_fused(wx, u, h0, cu_seqlens, block_table, max_iters=max_iters, omega=omega,
                                 want_residual=False)


@newton_nlru_fused.register_fake
def _(wx, u, h0=None, cu_seqlens=None, block_table=None, *, max_iters, omega):
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, int(u.numel()))


@torch.library.custom_op("pararnn_b200::newton_cfc_fused", mutates_args=())
def newton_cfc_fused(wx: Tensor, u: Tensor, h0: Tensor | None = None, cu_seqlens: Tensor | None = None,
                     block_table: Tensor | None = None, *, max_iters: int, omega: float) -> Tensor:
    return ops.newton_cfc_fused(wx, u, h0, cu_seqlens, block_table, max_iters=max_iters, omega=omega,
                                want_residual=False)


@newton_cfc_fused.register_fake
def _(wx, u, h0=None, cu_seqlens=None, block_table=None, *, max_iters, omega):
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, int(u.numel()))


@torch.library.custom_op("pararnn_b200::newton_titans_fused", mutates_args=())
def newton_titans_fused(wx: Tensor, u: Tensor, r: Tensor, h0: Tensor | None = None,
                        cu_seqlens: Tensor | None = None, block_table: Tensor | None = None, *,
                        max_iters: int, omega: float) -> Tensor:
    return ops.newton_titans_fused(wx, u, r, h0, cu_seqlens, block_table, max_iters=max_iters, omega=omega,
                                   want_residual=False)


@newton_titans_fused.register_fake
def _(wx, u, r, h0=None, cu_seqlens=None, block_table=None, *, max_iters, omega):
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, int(u.numel()))


@torch.library.custom_op("pararnn_b200::newton_lstm_fused", mutates_args=())
def newton_lstm_fused(wx: Tensor, a_f: Tensor, a_z: Tensor, a_o: Tensor, c_f: Tensor, c_o: Tensor,
                      h0: Tensor | None = None, block_table: Tensor | None = None, *, max_iters: int,
                      omega: float) -> Tensor:
    return ops.newton_lstm_fused(wx, a_f, a_z, a_o, c_f, c_o, h0, None, block_table, max_iters=max_iters,
                                 omega=omega, want_residual=False)


@newton_lstm_fused.register_fake
def _(wx, a_f, a_z, a_o, c_f, c_o, h0=None, block_table=None, *, max_iters, omega):
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, 2, int(a_f.numel()))


@torch.library.custom_op("pararnn_b200::newton_slstm_fused", mutates_args=())
def newton_slstm_fused(wx: Tensor, r: Tensor, h0: Tensor | None = None, states: Tensor | None = None,
                       block_table: Tensor | None = None, *, max_iters: int, omega: float, eps: float,
                       log_coords: bool = False, scan_tile: str = "assoc", time_loop: bool = False,
                       window_len: int = 0) -> Tensor:
    return ops.newton_slstm_fused(wx, r, h0, states, block_table, max_iters=max_iters, omega=omega, eps=eps,
                                  log_coords=log_coords, scan_tile=scan_tile, time_loop=time_loop,
                                  window_len=window_len, picard_iters=_picard_default, want_residual=False)


@newton_slstm_fused.register_fake
def _(wx, r, h0=None, states=None, block_table=None, *, max_iters, omega, eps, log_coords=False,
      scan_tile="assoc", time_loop=False, window_len=0):
    if states is not None:
        return torch.empty_like(states)
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, 4, int(r.shape[-1]))


@torch.library.custom_op("pararnn_b200::newton_gru_head_fused", mutates_args=())
def newton_gru_head_fused(wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor, h0: Tensor | None = None,
                          cu_seqlens: Tensor | None = None, *, max_iters: int, omega: float) -> Tensor:
    return head_ops.newton_gru_head_fused(wx, a_z, a_r, a_n, h0, cu_seqlens, max_iters=max_iters, omega=omega,
                                          want_residual=False)


@newton_gru_head_fused.register_fake
def _(wx, a_z, a_r, a_n, h0=None, cu_seqlens=None, *, max_iters, omega):
    batch, time, _ = wx.shape
    return wx.new_empty(batch, time, int(a_z.shape[0] * a_z.shape[-1]))


# ------------------------------------------------------------------------------------ backward

@torch.library.custom_op("pararnn_b200::reverse_gru_head_factor", mutates_args=())
def reverse_gru_head_factor(h_prev: Tensor, wx: Tensor, partial: Tensor, a_z: Tensor, a_r: Tensor,
                            a_n: Tensor) -> Tensor:
    """``mu_t = J_{t+1}^T mu_{t+1} + g_t`` with the factorised head Jacobian; ``h_prev`` is the
    trajectory shifted right by one step (``h_prev[:, 0]`` is the initial state)."""
    # J_t depends on h_{t-1} only, so the (unused) last state can be anything
    states = torch.cat([h_prev[:, 1:], h_prev[:, -1:]], dim=1)
    mu = torch.empty(partial.shape, dtype=torch.float32, device=partial.device)
    head_ops.gru_head_reverse_vjp(states, wx, a_z, a_r, a_n, partial, h_prev[:, 0], mu_out=mu)
    return mu.to(partial.dtype)


@reverse_gru_head_factor.register_fake
def _(h_prev, wx, partial, a_z, a_r, a_n):
    return torch.empty_like(partial)


@torch.library.custom_op("pararnn_b200::reverse_gru_vjp", mutates_args=())
def reverse_gru_vjp(states: Tensor, wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor, grad_states: Tensor,
                    h0: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    g_wx, gz, gr, gn, g_h0 = ops.gru_reverse_vjp(states, wx, a_z, a_r, a_n, grad_states, h0)
    return g_wx, gz.clone(), gr.clone(), gn.clone(), g_h0


@reverse_gru_vjp.register_fake
def _(states, wx, a_z, a_r, a_n, grad_states, h0=None):
    d = int(a_z.numel())
    f32 = dict(dtype=torch.float32, device=wx.device)
    return (torch.empty_like(wx), torch.empty(d, **f32), torch.empty(d, **f32), torch.empty(d, **f32),
            torch.empty(wx.shape[0], d, **f32))


@torch.library.custom_op("pararnn_b200::reverse_nlru_vjp", mutates_args=())
def reverse_nlru_vjp(states: Tensor, wx: Tensor, u: Tensor, grad_states: Tensor,
                     h0: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor]:
    g_wx, gu, g_h0 = ops.nlru_reverse_vjp(states, wx, u, grad_states, h0)
    return g_wx, gu.clone(), g_h0


@reverse_nlru_vjp.register_fake
def _(states, wx, u, grad_states, h0=None):
    d = int(u.numel())
    f32 = dict(dtype=torch.float32, device=wx.device)
    return torch.empty_like(wx), torch.empty(d, **f32), torch.empty(wx.shape[0], d, **f32)


@torch.library.custom_op("pararnn_b200::reverse_slstm_vjp", mutates_args=())
def reverse_slstm_vjp(states: Tensor, wx: Tensor, r: Tensor, grad_states: Tensor, h0: Tensor | None = None,
                      eps: float = 1e-6) -> tuple[Tensor, Tensor, Tensor]:
    return ops.slstm_reverse_vjp(states, wx, r, grad_states, h0, eps)


@reverse_slstm_vjp.register_fake
def _(states, wx, r, grad_states, h0=None, eps=1e-6):
    d = int(r.shape[-1])
    f32 = dict(dtype=torch.float32, device=wx.device)
    return torch.empty_like(wx), torch.empty(4, d, **f32), torch.empty(wx.shape[0], 4, d, **f32)


@torch.library.custom_op("pararnn_b200::reverse_gru_head_vjp", mutates_args=())
def reverse_gru_head_vjp(states: Tensor, wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor, grad_states: Tensor,
                         h0: Tensor | None = None) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    g_wx, gz, gr, gn, g_h0 = head_ops.gru_head_reverse_vjp(states, wx, a_z, a_r, a_n, grad_states, h0)
    return g_wx, gz.clone(), gr.clone(), gn.clone(), g_h0


@reverse_gru_head_vjp.register_fake
def _(states, wx, a_z, a_r, a_n, grad_states, h0=None):
    f32 = dict(dtype=torch.float32, device=wx.device)
    d = int(a_z.shape[0] * a_z.shape[-1])
    return (torch.empty_like(wx), torch.empty(a_z.shape, **f32), torch.empty(a_z.shape, **f32),
            torch.empty(a_z.shape, **f32), torch.empty(wx.shape[0], d, **f32))


OP_NAMES = ("newton_gru_fused", "newton_nlru_fused", "newton_cfc_fused", "newton_titans_fused", "newton_lstm_fused", "newton_slstm_fused",
            "newton_gru_head_fused",
            "reverse_gru_head_factor", "reverse_gru_vjp", "reverse_nlru_vjp", "reverse_slstm_vjp",
            "reverse_gru_head_vjp")
