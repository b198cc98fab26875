"""ctypes front end of the CPU oracle (``pararnn_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU arm of ``bench.py``.  The product package never imports it.

The C file is compiled twice, once with ``REAL=float`` (matches the fp32
arithmetic of the reference's eager path) and once with ``REAL=double`` (ground
truth for error measurements).  ``build()`` writes ``liboracle_f32.so`` and
``liboracle_f64.so`` next to this file.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "pararnn_oracle.c")

GRU_DIAG, NLRU, SLSTM_DIAG, GRU_HEAD, TITANS, LSTM, CFC = 0, 1, 2, 3, 4, 5, 6
KIND = {"gru_diag": GRU_DIAG, "nlru": NLRU, "slstm_diag": SLSTM_DIAG, "gru_head": GRU_HEAD, "titans": TITANS,
        "lstm": LSTM, "cfc": CFC}
GATES = {GRU_DIAG: 3, NLRU: 2, SLSTM_DIAG: 4, GRU_HEAD: 3, TITANS: 5, LSTM: 3, CFC: 4}
SLOTS = {GRU_DIAG: 1, NLRU: 1, SLSTM_DIAG: 4, GRU_HEAD: 1, TITANS: 1, LSTM: 2, CFC: 1}


def _lib_path(prec: str) -> str:
    return os.path.join(HERE, f"liboracle_{prec}.so")


def build(force: bool = False) -> None:
    """Compile both precisions with gcc (OpenMP, no fast-math)."""
    for prec, real in (("f32", "float"), ("f64", "double")):
        out = _lib_path(prec)
        if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(SRC):
            continue
        cmd = [
            "gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
            f"-DREAL={real}", SRC, "-o", out, "-lm",
        ]
        subprocess.run(cmd, check=True)


_libs: dict[str, ctypes.CDLL] = {}


def _lib(prec: str) -> ctypes.CDLL:
    if prec not in _libs:
        build()
        lib = ctypes.CDLL(_lib_path(prec))
        real = ctypes.c_float if prec == "f32" else ctypes.c_double
        lib.oracle_residual.restype = real
        lib.oracle_newton.restype = real
        _libs[prec] = lib
    return _libs[prec]


def _np_dtype(prec: str):
    return np.float32 if prec == "f32" else np.float64


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _prep(a, dt):
    return None if a is None else np.ascontiguousarray(np.asarray(a), dtype=dt)


def pack_params(kind: int, params) -> np.ndarray:
    """Concatenate the (already clamped) recurrent parameters in the C layout."""
    if isinstance(params, np.ndarray):
        return params
    return np.concatenate([np.asarray(p).reshape(-1) for p in params])


@dataclass
class NewtonResult:
    states: np.ndarray
    iters: int
    max_residual: float
    history: tuple


def _shape(kind, wx, n_heads):
    B, T, GD = wx.shape
    d = GD // GATES[kind]
    return B, T, d


def sequential(kind, wx, params, h0=None, *, n_heads=1, eps=1e-6, prec="f32"):
    dt = _np_dtype(prec)
    wx = _prep(wx, dt)
    params = _prep(pack_params(kind, params), dt)
    h0 = _prep(h0, dt)
    B, T, d = _shape(kind, wx, n_heads)
    S = SLOTS[kind]
    out = np.empty((B, T, S, d) if S > 1 else (B, T, d), dtype=dt)
    real = ctypes.c_float if prec == "f32" else ctypes.c_double
    _lib(prec).oracle_sequential(
        ctypes.c_int(kind), _ptr(wx), _ptr(params), _ptr(h0), B, T, d, n_heads, real(eps), _ptr(out)
    )
    return out


def guess(kind, wx, params, h0=None, *, n_heads=1, picard=0, eps=1e-6, prec="f32"):
    dt = _np_dtype(prec)
    wx = _prep(wx, dt)
    params = _prep(pack_params(kind, params), dt)
    h0 = _prep(h0, dt)
    B, T, d = _shape(kind, wx, n_heads)
    S = SLOTS[kind]
    out = np.empty((B, T, S, d) if S > 1 else (B, T, d), dtype=dt)
    real = ctypes.c_float if prec == "f32" else ctypes.c_double
    _lib(prec).oracle_guess(
        ctypes.c_int(kind), _ptr(wx), _ptr(params), _ptr(h0), B, T, d, n_heads, picard, real(eps),
        _ptr(out),
    )
    return out


def residual(kind, wx, params, states, h0=None, *, n_heads=1, eps=1e-6, prec="f32"):
    dt = _np_dtype(prec)
    wx = _prep(wx, dt)
    params = _prep(pack_params(kind, params), dt)
    h0 = _prep(h0, dt)
    states = _prep(states, dt)
    B, T, d = _shape(kind, wx, n_heads)
    real = ctypes.c_float if prec == "f32" else ctypes.c_double
    return float(
        _lib(prec).oracle_residual(
            ctypes.c_int(kind), _ptr(wx), _ptr(params), _ptr(h0), B, T, d, n_heads, real(eps),
            _ptr(states),
        )
    )


def newton(kind, wx, params, h0=None, *, n_heads=1, max_iters=3, picard=0, omega=1.0, eps=1e-6,
           early_atol=None, prec="f32") -> NewtonResult:
    """Eager Newton+scan.  ``early_atol=None`` runs exactly ``max_iters`` passes."""
    dt = _np_dtype(prec)
    wx = _prep(wx, dt)
    params = _prep(pack_params(kind, params), dt)
    h0 = _prep(h0, dt)
    B, T, d = _shape(kind, wx, n_heads)
    S = SLOTS[kind]
    out = np.empty((B, T, S, d) if S > 1 else (B, T, d), dtype=dt)
    hist = np.zeros(max(max_iters, 1), dtype=dt)
    iters = ctypes.c_int(0)
    real = ctypes.c_float if prec == "f32" else ctypes.c_double
    res = _lib(prec).oracle_newton(
        ctypes.c_int(kind), _ptr(wx), _ptr(params), _ptr(h0), B, T, d, n_heads, max_iters, picard,
        real(omega), real(eps), real(-1.0 if early_atol is None else early_atol), _ptr(out),
        _ptr(hist), ctypes.byref(iters),
    )
    n_hist = iters.value if early_atol is not None else max_iters
    return NewtonResult(out, iters.value, float(res), tuple(float(v) for v in hist[:n_hist]))


def backward(kind, states, wx, params, grad_states, h0=None, *, n_heads=1, eps=1e-6, prec="f32",
             want_mu=False):
    """Eq. 2.6 reverse scan + packed VJP.  Returns (g_wx, g_params, g_h0[, mu])."""
    dt = _np_dtype(prec)
    wx = _prep(wx, dt)
    params = _prep(pack_params(kind, params), dt)
    h0 = _prep(h0, dt)
    states = _prep(states, dt)
    grad_states = _prep(grad_states, dt)
    B, T, d = _shape(kind, wx, n_heads)
    S = SLOTS[kind]
    g_wx = np.empty_like(wx)
    g_params = np.zeros_like(params)
    g_h0 = np.empty((B, S, d) if S > 1 else (B, d), dtype=dt)
    mu = np.empty_like(states) if want_mu else None
    real = ctypes.c_float if prec == "f32" else ctypes.c_double
    _lib(prec).oracle_backward(
        ctypes.c_int(kind), _ptr(states), _ptr(wx), _ptr(params), _ptr(h0), _ptr(grad_states), B, T,
        d, n_heads, real(eps), _ptr(g_wx), _ptr(g_params), _ptr(g_h0), _ptr(mu),
    )
    if want_mu:
        return g_wx, g_params, g_h0, mu
    return g_wx, g_params, g_h0


# ---- packed batches (cu_seqlens): every sequence is its own scan from its own h0 row, nothing
# crosses a segment head (reference layout.py:93-138, prepend_state_ragged).  wx is (1, N, G*d).

def _segments(cu_seqlens, T):
    cs = [int(v) for v in np.asarray(cu_seqlens).reshape(-1)]
    assert cs[0] == 0 and cs[-1] == T and all(b > a for a, b in zip(cs[:-1], cs[1:])), cs
    return list(zip(cs[:-1], cs[1:]))


def _row(h0, i):
    return None if h0 is None else np.ascontiguousarray(np.asarray(h0)[i:i + 1])


def sequential_packed(kind, wx, params, h0, cu_seqlens, **kw):
    segs = _segments(cu_seqlens, wx.shape[1])
    return np.concatenate([sequential(kind, np.ascontiguousarray(wx[:, a:b]), params, _row(h0, i), **kw)
                           for i, (a, b) in enumerate(segs)], axis=1)


def newton_packed(kind, wx, params, h0, cu_seqlens, **kw) -> NewtonResult:
    """The reference evaluates one residual maximum over the whole pack per iteration, so the
    per-segment histories are merged with max."""
    segs = _segments(cu_seqlens, wx.shape[1])
    parts = [newton(kind, np.ascontiguousarray(wx[:, a:b]), params, _row(h0, i), **kw)
             for i, (a, b) in enumerate(segs)]
    n = max(len(p.history) for p in parts)
    hist = tuple(max(p.history[k] for p in parts if len(p.history) > k) for k in range(n))
    return NewtonResult(np.concatenate([p.states for p in parts], axis=1), max(p.iters for p in parts),
                        max(p.max_residual for p in parts), hist)


def backward_packed(kind, states, wx, params, grad_states, h0, cu_seqlens, **kw):
    segs = _segments(cu_seqlens, wx.shape[1])
    g_wx, g_par, heads = [], None, []
    for i, (a, b) in enumerate(segs):
        gw, gp, gh = backward(kind, np.ascontiguousarray(states[:, a:b]), np.ascontiguousarray(wx[:, a:b]),
                              params, np.ascontiguousarray(grad_states[:, a:b]), _row(h0, i), **kw)
        g_wx.append(gw)
        heads.append(gh)
        g_par = gp if g_par is None else g_par + gp
    return np.concatenate(g_wx, axis=1), g_par, np.concatenate(heads, axis=0)


def time_shard_bounds(T: int, world: int, rank: int) -> tuple[int, int]:
    s, e = ctypes.c_int(0), ctypes.c_int(0)
    _lib("f32").oracle_time_shard_bounds(T, world, rank, ctypes.byref(s), ctypes.byref(e))
    return s.value, e.value


if __name__ == "__main__":
    build(force=True)
    print("built", _lib_path("f32"), _lib_path("f64"))
