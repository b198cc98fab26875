"""Helpers shared by the GPU parity tests: seeded problems and oracle calls."""

import numpy as np
import torch

from oracle import oracle

GATES = {"gru_diag": 3, "nlru": 2, "slstm_diag": 4, "gru_head": 3, "titans": 5, "lstm": 3, "cfc": 4}


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def make_problem(kind, B, T, d, seed, *, h0=False, x_scale=1.0, bias_f=0.0, rec_scale=1.0, n_heads=1):
    """Seeded synthetic (wx, params, h0) at the op boundary, fp32 numpy."""
    rng = np.random.default_rng(seed)
    G = GATES[kind]
    wx = (x_scale * rng.standard_normal((B, T, G * d))).astype(np.float32)
    if kind == "gru_diag":
        params = np.clip(rec_scale * 0.3 * rng.standard_normal((3, d)), -0.5, 0.5).astype(np.float32)
    elif kind == "nlru":
        a0 = rng.uniform(0.9, 0.999, size=d)
        wx[..., :d] += np.log(a0 / (1 - a0)).astype(np.float32)
        params = np.clip(rec_scale * 0.3 * rng.standard_normal((1, d)), -0.5, 0.5).astype(np.float32)
    elif kind == "lstm":
        params = np.clip(rec_scale * 0.3 * rng.standard_normal((5, d)), -0.5, 0.5).astype(np.float32)
    elif kind == "cfc":
        # gates (f, c, dt, b): one positive time step per (row, step) broadcast over the channels,
        # time bias around the cell's initialisation
        dt = rng.uniform(1e-4, 2.0, size=(B, T, 1)).astype(np.float32)
        wx[..., 2 * d:3 * d] = dt
        wx[..., 3 * d:] = 0.5 * wx[..., 3 * d:] - 1.0
        params = np.clip(rec_scale * 0.3 * rng.standard_normal((1, d)), -0.5, 0.5).astype(np.float32)
    elif kind == "titans":
        wx[..., d:2 * d] -= 1.0  # softplus(theta_pre) ~ 0.3, as the cell's bias initialisation
        wx[..., 2 * d:4 * d] *= 0.5
        params = np.clip(rec_scale * 0.3 * rng.standard_normal((2, d)), -0.5, 0.5).astype(np.float32)
    elif kind == "slstm_diag":
        wx[..., d:2 * d] += bias_f
        params = np.clip(rec_scale * 0.3 * rng.standard_normal((4, d)), -0.5, 0.5).astype(np.float32)
    else:
        dh = d // n_heads
        mats = []
        for _ in range(3 * n_heads):
            q, _r = np.linalg.qr(rng.standard_normal((dh, dh)))
            mats.append(0.9 * rec_scale * q)
        params = np.stack(mats).reshape(3, n_heads, dh, dh).astype(np.float32)
    h0_arr = None
    if h0:
        if kind == "lstm":
            h0_arr = (0.5 * rng.standard_normal((B, 2, d))).astype(np.float32)
        elif kind == "slstm_diag":
            h0_arr = np.stack([0.3 * rng.standard_normal((B, d)), rng.uniform(0.5, 1.5, (B, d)),
                               0.2 * rng.standard_normal((B, d)), 0.3 * rng.standard_normal((B, d))],
                              axis=1).astype(np.float32)
        else:
            h0_arr = (0.5 * rng.standard_normal((B, d))).astype(np.float32)
    return wx, params, h0_arr


def dev(a, dtype=torch.float32):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype)


def rel_err(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(got - want).max() / max(1e-30, np.abs(want).max()))
