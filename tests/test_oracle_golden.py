"""Pin the CPU oracle against vectors produced by the reference's own eager path."""

import numpy as np
import pytest

from golden_util import cfc_input_grads, clip_mask, golden_names, linear_grads, load_golden, oracle_calls
from oracle import oracle

NAMES = golden_names()


def test_fixtures_present():
    assert len(NAMES) >= 23


@pytest.mark.parametrize("name", NAMES)
def test_sequential_matches_reference(name):
    g = load_golden(name)
    kind = oracle.KIND[g["cell"]]
    H = oracle_calls(g)[0](kind, g["wx"], g["params"], g["h0"], n_heads=g["n_heads"], eps=g["eps"])
    scale = max(1.0, float(np.abs(g["H_seq"]).max()))
    assert np.abs(H - g["H_seq"]).max() <= 2e-6 * scale


@pytest.mark.parametrize("name", NAMES)
def test_newton_matches_reference_eager(name):
    g = load_golden(name)
    kind = oracle.KIND[g["cell"]]
    r = oracle_calls(g)[1](kind, g["wx"], g["params"], g["h0"], n_heads=g["n_heads"], max_iters=g["K"],
                      picard=g["P"], omega=g["omega"], eps=g["eps"],
                      early_atol=1e-30 if g["iters"] < g["K"] else None)
    assert r.iters == g["iters"]
    scale = max(1.0, float(np.abs(g["H"]).max()))
    # Newton amplifies rounding when an iterate is far from converged: scale by the
    # largest residual the reference itself saw.
    amp = max(1.0, float(np.max(g["history"])) if len(g["history"]) else 1.0)
    assert np.abs(r.states - g["H"]).max() <= 5e-6 * scale * amp
    np.testing.assert_allclose(np.asarray(r.history), g["history"], rtol=2e-3, atol=2e-6 * scale)
    assert abs(r.max_residual - float(g["max_residual"])) <= 2e-3 * abs(float(g["max_residual"])) + 4e-6 * scale


@pytest.mark.parametrize("name", NAMES)
def test_backward_matches_reference_autograd(name):
    g = load_golden(name)
    kind = oracle.KIND[g["cell"]]
    g_wx, g_params, g_h0 = oracle_calls(g)[2](kind, g["H"], g["wx"], g["params"], g["G"], g["h0"],
                                              n_heads=g["n_heads"], eps=g["eps"])
    if g["cell"] == "cfc":
        gx, gW, gb, gWb, gbb = cfc_input_grads(g_wx, g["x"], g["W"], g["W_b"])
        pairs = ((gx, g["g_x"]), (gW, g["g_W"]), (gb, g["g_b"]), (gWb, g["g_W_b"]), (gbb, g["g_b_b"]))
    else:
        gx, gW, gb = linear_grads(g_wx, g["x"], g["W"])
        pairs = ((gx, g["g_x"]), (gW, g["g_W"]), (gb, g["g_b"]))
    for got, want in pairs:
        tol = 2e-5 * max(1.0, float(np.abs(want).max()))
        assert np.abs(got - want).max() <= tol
    gp = g_params.reshape(g["raw_params"].shape) * clip_mask(g["raw_params"], float(g["cap"]))
    tol = 2e-5 * max(1.0, float(np.abs(g["g_params"]).max()))
    assert np.abs(gp - g["g_params"]).max() <= tol
    if g["h0"] is not None:
        tol = 2e-5 * max(1.0, float(np.abs(g["g_h0"]).max()))
        assert np.abs(g_h0 - g["g_h0"]).max() <= tol


@pytest.mark.parametrize("name", NAMES)
def test_f64_build_agrees_with_f32(name):
    g = load_golden(name)
    kind = oracle.KIND[g["cell"]]
    seq = oracle_calls(g)[0]
    a = seq(kind, g["wx"], g["params"], g["h0"], n_heads=g["n_heads"], eps=g["eps"])
    b = seq(kind, g["wx"], g["params"], g["h0"], n_heads=g["n_heads"], eps=g["eps"], prec="f64")
    scale = max(1.0, float(np.abs(b).max()))
    assert np.abs(a - b).max() <= 5e-5 * scale


def test_time_shard_bounds():
    # reference solvers/seq_parallel.py:126-138: remainder on the last rank
    assert [oracle.time_shard_bounds(17, 4, r) for r in range(4)] == [(0, 4), (4, 8), (8, 12), (12, 17)]
    assert oracle.time_shard_bounds(16, 1, 0) == (0, 16)
