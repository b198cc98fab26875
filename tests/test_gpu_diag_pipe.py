"""The GRU-diag / NLRU parity tests once more, forced onto the pipelined persistent kernels
(kernel family forced through prb_debug_set), plus shapes chosen for that family: channel counts TMA can address
(d a multiple of 4 in fp32, of 8 in bf16), sequence lengths around the 64-step round, a ragged
last channel block.  Shapes TMA cannot address fall back to the look-back kernels."""

import numpy as np
import pytest
import torch

from gpu_util import bf16_round, dev, make_problem, rel_err
from oracle import oracle
from test_gpu_diag import *  # noqa: F401,F403
from test_gpu_diag import _bwd, _fwd, pytestmark  # noqa: F401


@pytest.fixture(autouse=True)
def _force_pipelined_kernels(prb_options):
    prb_options("kernel_family", "pipe")


PIPE_SHAPES = [(1, 1, 32), (2, 63, 64), (1, 64, 40), (3, 65, 96), (2, 128, 36), (1, 1000, 64), (4, 4097, 72)]


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
@pytest.mark.parametrize("B,T,d", PIPE_SHAPES)
@pytest.mark.parametrize("K", [1, 2, 4])
def test_pipe_forward_vs_oracle_fp32(kind, B, T, d, K):
    wx, params, h0 = make_problem(kind, B, T, d, seed=B * 77 + T + d, h0=(T % 2 == 1))
    want = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=K)
    H, hist, res = _fwd(kind, wx, params, h0, K)
    amp = max(1.0, max(want.history))
    assert np.abs(H - want.states).max() <= 1e-5 * amp
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=5e-3, atol=2e-6)
    assert abs(res - want.max_residual) <= 5e-3 * want.max_residual + 2e-6


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
@pytest.mark.parametrize("B,T,d", PIPE_SHAPES)
def test_pipe_backward_vs_oracle_fp32(kind, B, T, d):
    wx, params, h0 = make_problem(kind, B, T, d, seed=B + T + d, h0=(T % 2 == 0))
    H = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=6).states
    G = np.random.default_rng(3).standard_normal(H.shape).astype(np.float32)
    want = oracle.backward(oracle.KIND[kind], H, wx, params, G, h0)
    got = _bwd(kind, H, wx, params, G, h0)
    assert rel_err(got[0], want[0]) <= 2e-5
    assert rel_err(got[1], np.asarray(want[1]).reshape(got[1].shape)) <= 2e-5
    if h0 is not None:
        assert rel_err(got[2], want[2]) <= 2e-5


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
def test_pipe_bf16_matches_lookback_family(kind, prb_options):
    """Two independent implementations on the same bf16 problem."""
    wx, params, h0 = make_problem(kind, 2, 777, 64, seed=9, h0=True)
    wx, params, h0 = bf16_round(wx), bf16_round(params), bf16_round(h0)
    a, _, _ = _fwd(kind, wx, params, h0, 2, dtype=torch.bfloat16)
    prb_options("kernel_family", "lookback")
    b, _, _ = _fwd(kind, wx, params, h0, 2, dtype=torch.bfloat16)
    assert rel_err(a, b) <= 1e-2


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
@pytest.mark.parametrize("B,T,d,h0", [(1, 1, 32, False), (2, 63, 64, True), (3, 1000, 96, True), (2, 4099, 40, False)])
@pytest.mark.parametrize("K", [1, 2, 3, 4, 5])
def test_fused_iterations_equal_separate_passes(kind, B, T, d, h0, K, prb_options):
    """All K Newton iterations in one sweep against K launches: the same arithmetic in the same
    order, so states, residual history and final residual agree to the last bit (K = 5 exceeds
    the fused kernel's limit and takes the separate passes either way)."""
    prb_options("kernel_family", "pipe")
    wx, params, h0a = make_problem(kind, B, T, d, seed=K + T, h0=h0)
    a = _fwd(kind, wx, params, h0a, K)
    prb_options("newton_fused", 0)
    b = _fwd(kind, wx, params, h0a, K)
    assert np.array_equal(a[0], b[0])
    assert list(a[1]) == list(b[1]) and a[2] == b[2]
    wxq, pq = bf16_round(wx), bf16_round(params)
    h0q = None if h0a is None else bf16_round(h0a)
    prb_options("newton_fused", 1)
    a = _fwd(kind, wxq, pq, h0q, K, dtype=torch.bfloat16)
    prb_options("newton_fused", 0)
    b = _fwd(kind, wxq, pq, h0q, K, dtype=torch.bfloat16)
    assert np.array_equal(a[0], b[0]) and list(a[1]) == list(b[1]) and a[2] == b[2]
