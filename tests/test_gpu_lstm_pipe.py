"""The ParaLSTM parity tests once more, forced onto the pipelined persistent kernels (all Newton
iterations in one sweep, pipelined reverse sweep); shapes TMA cannot address fall back to the
look-back kernels.  Plus: the two families against each other on larger shapes and bf16 I/O."""

import numpy as np
import pytest
import torch

from gpu_util import bf16_round, dev, make_problem, rel_err
from oracle import oracle
from test_gpu_lstm import *  # noqa: F401,F403
from test_gpu_lstm import _fwd, pytestmark  # noqa: F401


@pytest.fixture(autouse=True)
def _force_pipelined_kernels(prb_options):
    prb_options("kernel_family", "pipe")


@pytest.mark.parametrize("B,T,d,h0", [(1, 1, 32, False), (2, 63, 64, True), (3, 1000, 96, True), (2, 4099, 40, False),
                                      (16, 2050, 128, True)])
@pytest.mark.parametrize("K", [1, 2, 4, 5])
def test_fused_iterations_match_the_lookback_passes(B, T, d, h0, K, prb_options):
    """Two independent implementations (K = 5 exceeds the fused sweep's limit and runs the look-back
    passes either way); the oracle is the referee."""
    wx, params, h0a = make_problem("lstm", B, T, d, seed=K + T, h0=h0)
    want = oracle.newton(oracle.LSTM, wx, params, h0a, max_iters=K)
    a = _fwd(wx, params, h0a, K)
    prb_options("kernel_family", "lookback")
    b = _fwd(wx, params, h0a, K)
    amp = max(1.0, max(want.history))
    for got in (a, b):
        assert np.abs(got[0] - want.states).max() <= 1e-5 * amp
        np.testing.assert_allclose(got[1], np.asarray(want.history), rtol=1e-2, atol=2e-6)
        assert abs(got[2] - want.max_residual) <= 1e-2 * want.max_residual + 4e-6
    assert np.abs(a[0] - b[0]).max() <= 4e-6 * amp


@pytest.mark.parametrize("B,T,d,h0", [(1, 1, 32, False), (2, 63, 64, True), (3, 1000, 96, True), (16, 2050, 128, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pipelined_reverse_sweep_matches_oracle_and_lookback(B, T, d, h0, dtype, prb_options):
    from pararnn_b200 import ops

    wx, params, h0a = make_problem("lstm", B, T, d, seed=T + d, h0=h0)
    if dtype == torch.bfloat16:
        wx, params, h0a = bf16_round(wx), bf16_round(params), (None if h0a is None else bf16_round(h0a))
    H = oracle.sequential(oracle.LSTM, wx, params, h0a)
    G = np.random.default_rng(1).standard_normal(H.shape).astype(np.float32)
    if dtype == torch.bfloat16:
        H, G = bf16_round(H), bf16_round(G)
    want = oracle.backward(oracle.LSTM, H, wx, params, G, h0a, prec="f64")
    tol = 5e-5 if dtype == torch.float32 else 2e-2

    def run():
        out = ops.lstm_reverse_vjp(dev(H, dtype), dev(wx, dtype), *[dev(p, dtype) for p in params], dev(G, dtype),
                                   dev(h0a, dtype))
        return [o.float().cpu().numpy() for o in out]

    a = run()
    prb_options("kernel_family", "lookback")
    b = run()
    for got in (a, b):
        assert rel_err(got[0], want[0]) <= tol
        assert rel_err(got[1].reshape(-1), np.asarray(want[1]).reshape(-1)) <= 2 * tol
        assert rel_err(got[2], want[2]) <= tol
