"""Helpers to load the golden fixtures produced by tests/golden/make_golden.py."""

import glob
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_names(prefix=""):
    return sorted(
        os.path.splitext(os.path.basename(p))[0]
        for p in glob.glob(os.path.join(GOLDEN_DIR, f"{prefix}*.npz"))
    )


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"), allow_pickle=False)
    g = {k: z[k] for k in z.files}
    g["cell"] = str(g["cell"])
    g["K"] = int(g["K"])
    g["P"] = int(g["P"])
    g["iters"] = int(g["iters"])
    g["omega"] = float(g["omega"])
    g["eps"] = float(g.get("eps", 1e-6))
    g["n_heads"] = int(g.get("n_heads", 1))
    g.setdefault("h0", None)
    g.setdefault("cu_seqlens", None)
    return g


def oracle_calls(g):
    """(sequential, newton, backward) of the oracle for a fixture: the packed variants when the
    fixture carries ``cu_seqlens``."""
    from functools import partial

    from oracle import oracle

    if g["cu_seqlens"] is None:
        return oracle.sequential, oracle.newton, oracle.backward
    cs = g["cu_seqlens"]
    return (lambda kind, wx, params, h0, **kw: oracle.sequential_packed(kind, wx, params, h0, cs, **kw),
            lambda kind, wx, params, h0, **kw: oracle.newton_packed(kind, wx, params, h0, cs, **kw),
            lambda kind, st, wx, params, G, h0, **kw: oracle.backward_packed(kind, st, wx, params, G, h0, cs, **kw))


def linear_grads(g_wx, x, W):
    """grad_x, grad_W, grad_b of y = x W^T + b given grad_y (reference solvers/vjp.py:109-120)."""
    gy = g_wx.reshape(-1, g_wx.shape[-1]).astype(np.float64)
    xx = x.reshape(-1, x.shape[-1]).astype(np.float64)
    return (gy @ W.astype(np.float64)).reshape(x.shape), gy.T @ xx, gy.sum(0)


def cfc_input_grads(g_wx, x, W, W_b):
    """Gradients of ParaCfC's ``project_wx`` given the grads of ``(f, c, dt, b)`` (reference
    ``solvers/vjp.py:180-211``): ``(grad_x, grad_W, grad_b, grad_W_b, grad_b_b)``."""
    d = W_b.shape[0]
    g = g_wx.reshape(-1, 4 * d).astype(np.float64)
    feat = x[..., :-1].reshape(-1, x.shape[-1] - 1).astype(np.float64)
    g_fc, g_dt, g_b = g[:, :2 * d], g[:, 2 * d:3 * d], g[:, 3 * d:]
    grad_feat = g_fc @ W.astype(np.float64) + g_b @ W_b.astype(np.float64)
    grad_dt = g_dt.sum(-1, keepdims=True) * (x[..., -1:].reshape(-1, 1) >= 1e-4)
    grad_x = np.concatenate([grad_feat, grad_dt], axis=-1).reshape(x.shape)
    return grad_x, g_fc.T @ feat, g_fc.sum(0), g_b.T @ feat, g_b.sum(0)


def clip_mask(raw, cap):
    if cap < 0:
        return np.ones_like(raw)
    return (np.abs(raw) <= cap).astype(raw.dtype)
