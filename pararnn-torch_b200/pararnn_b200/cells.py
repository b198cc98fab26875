"""Cells covered by the CUDA backend: parameters, clamps and the one-step map.

Constructor arguments, parameter names, shapes, initialisation and clamp rules
follow the reference cells (reference ``cells/para_gru.py``, ``cells/para_nlru.py``,
``cells/para_slstm.py``, ``cells/para_titans.py``), so a ``state_dict`` moves between the two libraries.
``step`` is plain PyTorch and is what ``sequential_apply`` unrolls (evaluation and
agreement checks); the training path never calls it.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor, nn

SLSTM_CELL, SLSTM_NORMALIZER, SLSTM_STABILIZER, SLSTM_HIDDEN = 0, 1, 2, 3
_UNSET = object()


def _sizes(input_size, hidden_size, d_in, d_h):
    input_size = d_in if input_size is None else input_size
    hidden_size = d_h if hidden_size is None else hidden_size
    if input_size is None or hidden_size is None:
        raise ValueError("input_size and hidden_size (or d_in / d_h) are required")
    return int(input_size), int(hidden_size)


def _xavier_gaussian_vec_(t: Tensor) -> None:
    n = max(t.numel(), 1)
    nn.init.normal_(t, mean=0.0, std=math.sqrt(2.0 / (n + n)))


def _clamp(p: Tensor, cap: float | None) -> Tensor:
    return p if cap is None else p.clamp(-cap, cap)


class ParaGRU(nn.Module):
    """GRU with diagonal (``mix='diag'``) or per-head dense (``mix='head'``) recurrence."""

    def __init__(self, input_size=None, hidden_size=None, *, d_in=None, d_h=None, mix="diag",
                 n_heads=None, max_recurrent_norm=_UNSET, device=None, dtype=None):
        super().__init__()
        if mix not in ("diag", "head"):
            raise ValueError(f"mix must be 'diag' or 'head', got {mix!r}")
        input_size, hidden_size = _sizes(input_size, hidden_size, d_in, d_h)
        kw = {"device": device, "dtype": dtype}
        if max_recurrent_norm is _UNSET:
            max_recurrent_norm = None if mix == "head" else 0.5
        self.input_size = self.d_in = input_size
        self.hidden_size = self.d_h = hidden_size
        self.state_slots = 1
        self.mix = mix
        self.jac_structure = "diag" if mix == "diag" else "head"
        self.max_recurrent_norm = max_recurrent_norm
        self.n_heads = n_heads
        self.d_head = None
        self.W_x = nn.Linear(input_size, 3 * hidden_size, bias=True, **kw)
        if mix == "diag":
            if n_heads is not None:
                raise ValueError("n_heads is only for mix='head'")
            self.a_z = nn.Parameter(torch.empty(hidden_size, **kw))
            self.a_r = nn.Parameter(torch.empty(hidden_size, **kw))
            self.a_n = nn.Parameter(torch.empty(hidden_size, **kw))
        else:
            if n_heads is None or n_heads < 1 or hidden_size % n_heads:
                raise ValueError(
                    f"mix='head' needs n_heads that divides hidden_size={hidden_size}, got {n_heads!r}")
            self.d_head = hidden_size // n_heads
            shape = (n_heads, self.d_head, self.d_head)
            self.A_z = nn.Parameter(torch.empty(*shape, **kw))
            self.A_r = nn.Parameter(torch.empty(*shape, **kw))
            self.A_n = nn.Parameter(torch.empty(*shape, **kw))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.W_x.weight, a=math.sqrt(5))
        nn.init.zeros_(self.W_x.bias)
        if self.mix == "diag":
            for p in (self.a_z, self.a_r, self.a_n):
                _xavier_gaussian_vec_(p)
            return
        for A in (self.A_z, self.A_r, self.A_n):
            for hd in range(self.n_heads):
                w = torch.empty(self.d_head, self.d_head, dtype=torch.float32, device=A.device)
                nn.init.orthogonal_(w, gain=0.25)
                A.data[hd].copy_(w.to(A.dtype))

    def clipped_a(self):
        if self.mix != "diag":
            raise TypeError("clipped_a is for mix='diag'")
        cap = self.max_recurrent_norm
        return _clamp(self.a_z, cap), _clamp(self.a_r, cap), _clamp(self.a_n, cap)

    def clipped_a_head(self):
        if self.mix != "head":
            raise TypeError("clipped_a_head is for mix='head'")
        cap = self.max_recurrent_norm
        return _clamp(self.A_z, cap), _clamp(self.A_r, cap), _clamp(self.A_n, cap)

    def step(self, h_prev: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None) -> Tensor:
        if wx is None:
            if x is None:
                raise ValueError("ParaGRU.step needs x or wx")
            wx = self.W_x(x)
        zx, rx, nx = wx.chunk(3, dim=-1)
        if self.mix == "diag":
            a_z, a_r, a_n = self.clipped_a()
            z = torch.sigmoid(a_z * h_prev + zx)
            r = torch.sigmoid(a_r * h_prev + rx)
            n = torch.tanh(a_n * (h_prev * r) + nx)
            return torch.lerp(h_prev, n, z)
        A_z, A_r, A_n = self.clipped_a_head()
        pre = h_prev.shape[:-1]
        H, dh = self.n_heads, self.d_head

        def heads(t):
            return t.reshape(*pre, H, dh)

        def mixh(v, A):
            return torch.matmul(v.unsqueeze(-2), A).squeeze(-2)

        hv = heads(h_prev)
        z = torch.sigmoid(mixh(hv, A_z) + heads(zx))
        r = torch.sigmoid(mixh(hv, A_r) + heads(rx))
        n = torch.tanh(mixh(hv * r, A_n) + heads(nx))
        return torch.lerp(hv, n, z).reshape(*pre, self.d_h)


class ParaNLRU(nn.Module):
    """``h_t = a_t h_{t-1} + (1-a_t) tanh(c_x + u h_{t-1})`` with ``a_t = sigmoid(a_x)``."""

    def __init__(self, input_size=None, hidden_size=None, *, d_in=None, d_h=None,
                 max_recurrent_norm=_UNSET, device=None, dtype=None):
        super().__init__()
        input_size, hidden_size = _sizes(input_size, hidden_size, d_in, d_h)
        kw = {"device": device, "dtype": dtype}
        self.input_size = self.d_in = input_size
        self.hidden_size = self.d_h = hidden_size
        self.state_slots = 1
        self.mix = "diag"
        self.jac_structure = "diag"
        self.max_recurrent_norm = 0.5 if max_recurrent_norm is _UNSET else max_recurrent_norm
        self.u = nn.Parameter(torch.empty(hidden_size, **kw))
        self.W_x = nn.Linear(input_size, 2 * hidden_size, bias=True, **kw)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.W_x.weight, a=math.sqrt(5))
        nn.init.zeros_(self.W_x.bias)
        _xavier_gaussian_vec_(self.u)

    def clipped_u(self) -> Tensor:
        return _clamp(self.u, self.max_recurrent_norm)

    def step(self, h_prev: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None) -> Tensor:
        if wx is None:
            if x is None:
                raise ValueError("ParaNLRU.step needs x or wx")
            wx = self.W_x(x)
        ax, cx = wx.chunk(2, dim=-1)
        a = torch.sigmoid(ax)
        n = torch.tanh(cx + self.clipped_u() * h_prev)
        return a * h_prev + (1.0 - a) * n


LSTM_CELL, LSTM_HIDDEN = 0, 1


class ParaLSTM(nn.Module):
    """Coupled input-forget LSTM with peepholes and diagonal recurrence (reference
    ``cells/para_lstm.py``): state ``(..., 2, d_h)`` with slots ``(c, h)``, ``(f_x, z_x, o_x) = W_x(x)``,

        f = sigmoid(a_f h + c_f c + f_x);  z = tanh(a_z h + z_x);  c' = f c + (1 - f) z
        o = sigmoid(a_o h + c_o c' + o_x); h' = o tanh(c')

    All five recurrent vectors are clamped to ``max_recurrent_norm``."""

    def __init__(self, input_size=None, hidden_size=None, *, d_in=None, d_h=None,
                 max_recurrent_norm=_UNSET, device=None, dtype=None):
        super().__init__()
        input_size, hidden_size = _sizes(input_size, hidden_size, d_in, d_h)
        kw = {"device": device, "dtype": dtype}
        self.input_size = self.d_in = input_size
        self.hidden_size = self.d_h = hidden_size
        self.state_slots = 2
        self.hidden_slot = LSTM_HIDDEN
        self.mix = "diag"
        self.jac_structure = "block2"
        self.max_recurrent_norm = 0.5 if max_recurrent_norm is _UNSET else max_recurrent_norm
        for name in ("a_f", "a_z", "a_o", "c_f", "c_o"):
            setattr(self, name, nn.Parameter(torch.empty(hidden_size, **kw)))
        self.W_x = nn.Linear(input_size, 3 * hidden_size, bias=True, **kw)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for p in (self.a_f, self.a_z, self.a_o, self.c_f, self.c_o):
            _xavier_gaussian_vec_(p)
        nn.init.kaiming_uniform_(self.W_x.weight, a=math.sqrt(5))
        nn.init.zeros_(self.W_x.bias)

    def clipped_recurrent(self):
        cap = self.max_recurrent_norm
        return tuple(_clamp(p, cap) for p in (self.a_f, self.a_z, self.a_o, self.c_f, self.c_o))

    def step(self, state_prev: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None) -> Tensor:
        c_prev, h_prev = state_prev[..., LSTM_CELL, :], state_prev[..., LSTM_HIDDEN, :]
        a_f, a_z, a_o, c_f, c_o = self.clipped_recurrent()
        if wx is None:
            if x is None:
                raise ValueError("ParaLSTM.step needs x or wx")
            wx = self.W_x(x)
        fx, zx, ox = wx.chunk(3, dim=-1)
        f = torch.sigmoid(a_f * h_prev + c_f * c_prev + fx)
        z = torch.tanh(a_z * h_prev + zx)
        c = f * c_prev + (1.0 - f) * z
        o = torch.sigmoid(a_o * h_prev + c_o * c + ox)
        return torch.stack((c, o * torch.tanh(c)), dim=-2)


class ParaTitans(nn.Module):
    """Titans-style memory cell with a channelwise-diagonal Jacobian (reference
    ``cells/para_titans.py``): ``(alpha_pre, theta_pre, k, v, n_pre) = W_x(x)``,

        h_t = (1 - sigmoid(alpha_pre)) h_{t-1} - softplus(theta_pre) (h_{t-1} k - v) k
              + u tanh(n_pre + r h_{t-1}),

    with diagonal gains ``u``, ``r`` clamped to ``max_recurrent_norm``."""

    def __init__(self, input_size=None, hidden_size=None, *, d_in=None, d_h=None,
                 max_recurrent_norm=_UNSET, device=None, dtype=None):
        super().__init__()
        input_size, hidden_size = _sizes(input_size, hidden_size, d_in, d_h)
        kw = {"device": device, "dtype": dtype}
        self.input_size = self.d_in = input_size
        self.hidden_size = self.d_h = hidden_size
        self.state_slots = 1
        self.mix = "diag"
        self.jac_structure = "diag"
        self.max_recurrent_norm = 0.5 if max_recurrent_norm is _UNSET else max_recurrent_norm
        self.u = nn.Parameter(torch.empty(hidden_size, **kw))
        self.r = nn.Parameter(torch.empty(hidden_size, **kw))
        self.W_x = nn.Linear(input_size, 5 * hidden_size, bias=True, **kw)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.W_x.weight, a=math.sqrt(5))
        nn.init.zeros_(self.W_x.bias)
        with torch.no_grad():  # softplus(-1) ~ 0.31 keeps |theta k^2| modest
            self.W_x.bias[self.d_h: 2 * self.d_h].fill_(-1.0)
        _xavier_gaussian_vec_(self.u)
        _xavier_gaussian_vec_(self.r)

    def clipped_u(self) -> Tensor:
        return _clamp(self.u, self.max_recurrent_norm)

    def clipped_r(self) -> Tensor:
        return _clamp(self.r, self.max_recurrent_norm)

    def step(self, h_prev: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None) -> Tensor:
        if wx is None:
            if x is None:
                raise ValueError("ParaTitans.step needs x or wx")
            wx = self.W_x(x)
        alpha_pre, theta_pre, k, v, n_pre = wx.chunk(5, dim=-1)
        alpha = torch.sigmoid(alpha_pre)
        theta = torch.nn.functional.softplus(theta_pre)
        grad = (h_prev * k - v) * k
        n = torch.tanh(n_pre + self.clipped_r() * h_prev)
        return (1.0 - alpha) * h_prev - theta * grad + self.clipped_u() * n


CFC_DT_EPS = 1e-4


def split_cfc_input(x: Tensor) -> tuple[Tensor, Tensor]:
    """``x[..., :-1]`` are the features, ``x[..., -1:]`` the time step, clamped from below
    (reference ``cells/para_cfc.py:57-60``)."""
    if x.shape[-1] < 2:
        raise ValueError(f"ParaCfC needs d_in >= 2 (features + time step), got {x.shape[-1]}")
    return x[..., :-1], x[..., -1:].clamp_min(CFC_DT_EPS)


class ParaCfC(nn.Module):
    """Closed-form continuous-time cell with irregular time steps (reference
    ``cells/para_cfc.py``).  The last channel of ``x`` is the time step ``dt``:

        a_t = sigmoid(-(softplus(f_t) dt_t + b_t)),   (f_t, c_t) = W_x(feat_t),  b_t = W_b(feat_t)
        h_t = a_t h_{t-1} + (1 - a_t) tanh(c_t + u h_{t-1})

    ``project_wx`` packs ``(f, c, dt, b)`` as the ``(…, 4 d_h)`` input of the fused solve.  Only
    ``gate_mix='input'`` (the reference's fused and packed-VJP case) is covered."""

    def __init__(self, input_size=None, hidden_size=None, *, d_in=None, d_h=None, gate_mix="input",
                 time_bias_init=-3.0, max_recurrent_norm=_UNSET, device=None, dtype=None):
        super().__init__()
        input_size, hidden_size = _sizes(input_size, hidden_size, d_in, d_h)
        if input_size < 2:
            raise ValueError(f"ParaCfC d_in must be >= 2, got {input_size}")
        if gate_mix != "input":
            raise ValueError("this backend covers ParaCfC(gate_mix='input') only")
        kw = {"device": device, "dtype": dtype}
        self.input_size = self.d_in = input_size
        self.hidden_size = self.d_h = hidden_size
        self.feature_size = input_size - 1
        self.state_slots = 1
        self.mix = "diag"
        self.gate_mix = gate_mix
        self.jac_structure = "diag"
        self.max_recurrent_norm = 0.5 if max_recurrent_norm is _UNSET else max_recurrent_norm
        self.time_bias_init = float(time_bias_init)
        self.u = nn.Parameter(torch.empty(hidden_size, **kw))
        self.register_parameter("v", None)
        self.W_x = nn.Linear(self.feature_size, 2 * hidden_size, bias=True, **kw)
        self.W_b = nn.Linear(self.feature_size, hidden_size, bias=True, **kw)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.W_x.weight, a=math.sqrt(5))
        nn.init.zeros_(self.W_x.bias)
        _xavier_gaussian_vec_(self.u)
        # zero weight and bias -3: the gate starts near sigmoid(3) ~ 0.95 for dt -> 0
        nn.init.zeros_(self.W_b.weight)
        nn.init.constant_(self.W_b.bias, self.time_bias_init)

    def clipped_u(self) -> Tensor:
        return _clamp(self.u, self.max_recurrent_norm)

    def project_wx(self, x: Tensor) -> Tensor:
        feat, dt = split_cfc_input(x)
        return torch.cat((self.W_x(feat), dt.expand(*feat.shape[:-1], self.d_h), self.W_b(feat)), dim=-1)

    def step(self, h_prev: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None) -> Tensor:
        if wx is None:
            if x is None:
                raise ValueError("ParaCfC.step needs x or wx")
            wx = self.project_wx(x)
        if wx.shape[-1] != 4 * self.d_h:
            raise ValueError(f"ParaCfC wx last dim must be 4*d_h={4 * self.d_h}, got {wx.shape[-1]}")
        f_pre, cx, dt, b = wx.chunk(4, dim=-1)
        a = torch.sigmoid(-(torch.nn.functional.softplus(f_pre) * dt + b))
        n = torch.tanh(cx + self.clipped_u() * h_prev)
        return a * h_prev + (1.0 - a) * n


class ParaSLSTM(nn.Module):
    """Stabilised sLSTM with channelwise recurrence ``R (4, d)``; state slots ``(c, n, m, h)``."""

    def __init__(self, input_size=None, hidden_size=None, *, d_in=None, d_h=None, mix="diag",
                 n_heads=None, max_recurrent_norm=0.5, eps=1e-6, device=None, dtype=None):
        super().__init__()
        if mix != "diag":
            raise ValueError("this backend covers ParaSLSTM(mix='diag') only")
        if n_heads is not None:
            raise ValueError("n_heads is only for mix='head'")
        input_size, hidden_size = _sizes(input_size, hidden_size, d_in, d_h)
        kw = {"device": device, "dtype": dtype}
        self.input_size = self.d_in = input_size
        self.hidden_size = self.d_h = hidden_size
        self.state_slots = 4
        self.hidden_slot = SLSTM_HIDDEN
        self.mix = mix
        self.jac_structure = "block4"
        self.max_recurrent_norm = max_recurrent_norm
        self.eps = eps
        self.n_heads = None
        self.W_x = nn.Linear(input_size, 4 * hidden_size, bias=True, **kw)
        self.R = nn.Parameter(torch.empty(4, hidden_size, **kw))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.W_x.weight, a=math.sqrt(5))
        nn.init.zeros_(self.W_x.bias)
        _xavier_gaussian_vec_(self.R)

    def clipped_r(self) -> Tensor:
        return _clamp(self.R, self.max_recurrent_norm)

    def step(self, state_prev: Tensor, x: Tensor | None = None, *, wx: Tensor | None = None) -> Tensor:
        if wx is None:
            wx = self.W_x(x)
        c, n, m, h = state_prev.unbind(dim=-2)
        r = self.clipped_r()
        z_i, z_f, z_z, z_o = (wx + (r * h.unsqueeze(-2)).reshape(*h.shape[:-1], 4 * self.d_h)).chunk(4, dim=-1)
        left = z_f + m
        m_new = torch.maximum(left, z_i)
        i_t = torch.exp(z_i - m_new)
        f_t = torch.exp(left - m_new)
        n_new = f_t * n + i_t
        c_new = f_t * c + i_t * torch.tanh(z_z)
        h_new = torch.sigmoid(z_o) * (c_new / (n_new + self.eps))
        return torch.stack((c_new, n_new, m_new, h_new), dim=-2)


def cell_kind(cell: nn.Module) -> str:
    """Classify a cell by name and ``mix`` so that cells of the reference library are
    accepted as well as the ones defined here."""
    name = type(cell).__name__
    mix = getattr(cell, "mix", "diag")
    if name == "ParaGRU":
        return "gru_diag" if mix == "diag" else "gru_head"
    if name == "ParaNLRU":
        return "nlru"
    if name == "ParaTitans":
        return "titans"
    if name == "ParaCfC":
        if getattr(cell, "gate_mix", "input") != "input":
            raise TypeError("the CUDA backend covers ParaCfC(gate_mix='input') only")
        return "cfc"
    if name == "ParaLSTM":
        return "lstm"
    if name == "ParaSLSTM" and mix == "diag":
        return "slstm_diag"
    raise TypeError(
        f"the CUDA backend covers ParaGRU (diag, head), ParaNLRU, ParaTitans, ParaCfC, ParaLSTM and ParaSLSTM(mix='diag'); "
        f"got {name}(mix={mix!r})")


def zero_state(cell: nn.Module, batch: int, like: Tensor) -> Tensor:
    slots = int(getattr(cell, "state_slots", 1))
    if slots == 1:
        return like.new_zeros(batch, cell.d_h)
    return like.new_zeros(batch, slots, cell.d_h)
