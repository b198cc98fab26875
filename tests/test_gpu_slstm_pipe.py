"""The sLSTM parity tests once more, forced onto the warp-pipelined persistent kernels
(kernel family forced through prb_debug_set); passes that have no pipelined variant fall back to the other families."""

import pytest

from test_gpu_slstm import *  # noqa: F401,F403
from test_gpu_slstm import pytestmark  # noqa: F401


@pytest.fixture(autouse=True)
def _force_pipelined_kernels(prb_options):
    prb_options("kernel_family", "pipe")


# ---- the fused sweep (all Picard passes in one launch) against the per-pass kernels
import numpy as np  # noqa: E402
import torch  # noqa: E402

from gpu_util import dev, make_problem  # noqa: E402


@pytest.mark.parametrize("P", [0, 1, 3, 5])
@pytest.mark.parametrize("B,T,d,h0", [(1, 1, 32, False), (2, 57, 64, True), (2, 1000, 96, True),
                                      (1, 4099, 40, False)])
def test_fused_picard_sweep_equals_separate_passes(P, B, T, d, h0, prb_options):
    from pararnn_b200 import ops

    wx, r, h0a = make_problem("slstm_diag", B, T, d, seed=P + T, h0=h0, x_scale=0.7, bias_f=2.0, rec_scale=2.0)

    def guess():
        return ops.newton_slstm_fused(dev(wx), dev(r), dev(h0a), None, max_iters=0, picard_iters=P,
                                      want_residual=False).float().cpu().numpy()

    fused = guess()
    prb_options("picard_fused", 0)
    separate = guess()
    for slot in range(4):
        scale = max(1.0, float(np.abs(separate[:, :, slot]).max()))
        assert np.abs(fused[:, :, slot] - separate[:, :, slot]).max() <= 1e-6 * scale, slot


def test_seven_passes_fall_back_to_separate_kernels():
    from oracle import oracle
    from pararnn_b200 import ops

    wx, r, _ = make_problem("slstm_diag", 2, 300, 64, seed=3, x_scale=0.7, bias_f=2.0, rec_scale=2.0)
    want = oracle.guess(oracle.SLSTM_DIAG, wx, r, None, picard=6)
    got = ops.newton_slstm_fused(dev(wx), dev(r), None, None, max_iters=0, picard_iters=6,
                                 want_residual=False).float().cpu().numpy()
    for slot in range(4):
        scale = max(1.0, float(np.abs(want[:, :, slot]).max()))
        # a guess, not a fixed point: chained summaries and the reference's cumsum / cummax form
        # round differently, a little more with every pass
        assert np.abs(got[:, :, slot] - want[:, :, slot]).max() <= 1e-4 * scale


@pytest.mark.parametrize("K", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("B,T,d,h0", [(1, 1, 32, False), (2, 57, 64, True), (2, 1000, 96, True),
                                      (1, 4099, 40, False)])
def test_fused_newton_sweep_equals_separate_passes(K, B, T, d, h0, prb_options):
    """K = 5 exceeds what one sweep takes and runs the separate passes in both cases."""
    from pararnn_b200 import ops

    wx, r, h0a = make_problem("slstm_diag", B, T, d, seed=K + T, h0=h0, x_scale=0.5, bias_f=3.0)

    def solve():
        st = ops.DeviceStats("cuda", K)
        H = ops.newton_slstm_fused(dev(wx), dev(r), dev(h0a), None, max_iters=K, picard_iters=2, stats=st)
        hist, res, status = st.read()
        assert status == 0
        return H.float().cpu().numpy(), np.asarray(hist), res

    fused, hist_f, res_f = solve()
    prb_options("newton_fused", 0)
    separate, hist_s, res_s = solve()
    amp = max(1.0, float(hist_s.max()))
    for slot in range(4):
        scale = max(1.0, float(np.abs(separate[:, :, slot]).max()))
        assert np.abs(fused[:, :, slot] - separate[:, :, slot]).max() <= 2e-6 * scale * amp, slot
    np.testing.assert_allclose(hist_f, hist_s, rtol=1e-3, atol=1e-6)
    assert abs(res_f - res_s) <= 1e-3 * res_s + 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_sweeps_with_damping_eps_and_h0(dtype, prb_options):
    """omega != 1, a non-default eps, a start state and both I/O dtypes through the fused sweeps,
    against the separate passes (fp32: also against the oracle)."""
    from gpu_util import bf16_round
    from oracle import oracle
    from pararnn_b200 import ops

    wx, r, h0a = make_problem("slstm_diag", 3, 777, 64, seed=21, h0=True, x_scale=0.5, bias_f=3.0)
    if dtype == torch.bfloat16:
        wx, r, h0a = bf16_round(wx), bf16_round(r), bf16_round(h0a)

    def solve():
        st = ops.DeviceStats("cuda", 3)
        H = ops.newton_slstm_fused(dev(wx, dtype), dev(r, dtype), dev(h0a, dtype), None, max_iters=3,
                                   omega=0.8, eps=1e-4, picard_iters=4, stats=st)
        hist, res, status = st.read()
        assert status == 0
        return H.float().cpu().numpy(), np.asarray(hist), res

    fused, hist_f, res_f = solve()
    prb_options("newton_fused", 0)
    prb_options("picard_fused", 0)
    separate, hist_s, res_s = solve()
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    for slot in range(4):
        scale = max(1.0, float(np.abs(separate[:, :, slot]).max()))
        assert np.abs(fused[:, :, slot] - separate[:, :, slot]).max() <= tol * scale, slot
    np.testing.assert_allclose(hist_f, hist_s, rtol=2e-3, atol=1e-6)
    if dtype == torch.float32:
        want = oracle.newton(oracle.SLSTM_DIAG, wx, r, h0a, max_iters=3, picard=4, omega=0.8, eps=1e-4)
        amp = max(1.0, max(want.history))
        assert np.abs(fused[:, :, 3] - want.states[:, :, 3]).max() <= 1e-5 * amp
        # the histories sit at the fp32 floor of the stabiliser slot (|m| ~ 2e3: one ulp = 2.4e-4)
        np.testing.assert_allclose(hist_f, np.asarray(want.history), rtol=1e-2, atol=5e-4)
