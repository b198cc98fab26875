"""GPU parity at the full benchmark sizes.

The oracle cannot finish a full-size problem in seconds, but the diagonal cells are independent
per channel and the head cell per (batch row, head): the oracle therefore solves a 32-channel
(or one-head) slice of the SAME inputs at the full sequence length, and the matching slice of the
GPU result is compared with it.  Whole-tensor checks complete the picture: the residual the solve
reports, monotone Newton histories, finiteness, and equality of two independent code paths
(time-sharded versus single sweep) over every element.

Tolerances: fp32 1e-5 max-abs scaled by max(1, |state|); bf16 2e-2 relative."""

import numpy as np
import pytest
import torch

from gpu_util import rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu

BF16_RTOL = 2e-2


def _randn(shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return (scale * torch.randn(shape, device="cuda", generator=g)).to(dtype)


def _np(t):
    return t.float().cpu().numpy()


def _gate_slice(wx, G, d, c0, n):
    """Columns c0..c0+n of each of the G gates of a gate-major (B,T,G*d) array."""
    idx = torch.cat([torch.arange(g * d + c0, g * d + c0 + n) for g in range(G)]).to(wx.device)
    return wx.index_select(2, idx)


def _slstm_problem(B, T, d, seed, dtype):
    wx = _randn((B, T, 4 * d), seed, 0.5)
    wx[..., d:2 * d] += 3.0
    r = (0.3 * _randn((4, d), seed + 1)).clamp(-0.5, 0.5)
    return wx.to(dtype), r.to(dtype)


@pytest.mark.parametrize("c0", [0, 480, 992])
def test_c2_slstm_bf16_slice_matches_oracle(c0):
    """ParaSLSTM diag bf16, B=8, T=16384, d=1024, K=2, P=5: forward and backward."""
    from pararnn_b200 import ops

    B, T, d, n = 8, 16384, 1024, 32
    wx, r = _slstm_problem(B, T, d, 11, torch.bfloat16)
    st = ops.DeviceStats("cuda", 2)
    H = ops.newton_slstm_fused(wx, r, None, None, max_iters=2, picard_iters=5, stats=st)
    hist, res, status = st.read()
    assert status == 0
    assert bool(torch.isfinite(H.float()).all())
    # with the forget bias the stabiliser m grows to ~5e4, where one fp32 ulp is 2^-8: that is the
    # floor of max|F| for this problem, reached by the warm start already
    ulp_m = float(H[:, :, 2].float().abs().max()) * 2.0 ** -23
    assert hist[1] <= hist[0] and res <= 1e-3 + 4 * ulp_m

    wx_s, r_s = _np(_gate_slice(wx, 4, d, c0, n)), _np(r[:, c0:c0 + n])
    want = oracle.newton(oracle.SLSTM_DIAG, wx_s, r_s, None, max_iters=2, picard=5)
    got = _np(H[:, :, :, c0:c0 + n])
    for slot in range(4):
        assert rel_err(got[:, :, slot], want.states[:, :, slot]) <= BF16_RTOL, slot

    G = _randn((B, T, 4, d), 12, 1.0, torch.bfloat16)
    g_wx, g_r, _ = ops.slstm_reverse_vjp(H, wx, r, G, None)
    assert bool(torch.isfinite(g_wx.float()).all())
    w_wx, w_r, _ = oracle.backward(oracle.SLSTM_DIAG, got, wx_s, r_s, _np(G[:, :, :, c0:c0 + n]), None)
    assert rel_err(_np(_gate_slice(g_wx, 4, d, c0, n)), w_wx) <= BF16_RTOL
    assert rel_err(_np(g_r[:, c0:c0 + n]), w_r.reshape(4, -1)) <= 2e-3


def test_c2_sharded_equals_single_sweep_everywhere():
    """Two independent code paths over the full C2 tensor: 4 time shards (aggregate sweeps,
    carry folds, apply sweeps) against the single persistent sweep."""
    from pararnn_b200 import ops
    from pararnn_b200.seq_shard import emulate_sharded

    B, T, d = 8, 16384, 1024
    wx, r = _slstm_problem(B, T, d, 13, torch.bfloat16)
    one = ops.newton_slstm_fused(wx, r, None, None, max_iters=2, picard_iters=5)
    many, _ = emulate_sharded("slstm_diag", wx, (r,), world=4, K=2, P=5)
    for slot in range(4):
        a, b = many[:, :, slot].float(), one[:, :, slot].float()
        assert float((a - b).abs().max() / b.abs().max()) <= BF16_RTOL, slot


def test_c4_long_sequence_slice_and_shards():
    """ParaSLSTM diag bf16, B=1, T=131072, d=2048, K=2, P=5 on one GPU and as 8 time shards."""
    from pararnn_b200 import ops
    from pararnn_b200.seq_shard import emulate_sharded

    B, T, d, n, c0 = 1, 131072, 2048, 32, 1056
    wx, r = _slstm_problem(B, T, d, 14, torch.bfloat16)
    st = ops.DeviceStats("cuda", 2)
    one = ops.newton_slstm_fused(wx, r, None, None, max_iters=2, picard_iters=5, stats=st)
    assert st.read()[2] == 0
    wx_s, r_s = _np(_gate_slice(wx, 4, d, c0, n)), _np(r[:, c0:c0 + n])
    want = oracle.newton(oracle.SLSTM_DIAG, wx_s, r_s, None, max_iters=2, picard=5)
    got = _np(one[:, :, :, c0:c0 + n])
    for slot in range(4):
        assert rel_err(got[:, :, slot], want.states[:, :, slot]) <= BF16_RTOL, slot
    many, _ = emulate_sharded("slstm_diag", wx, (r,), world=8, K=2, P=5)
    for slot in range(4):
        a, b = many[:, :, slot].float(), one[:, :, slot].float()
        assert float((a - b).abs().max() / b.abs().max()) <= BF16_RTOL, slot


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_c3_gru_head_slice_matches_oracle(dtype):
    """ParaGRU head, 8 heads x 64, B=16, T=4096, K=3: one head of all rows against the oracle."""
    from pararnn_b200 import head_ops, ops

    B, T, H, dh, head = 16, 4096, 8, 64, 5
    d = H * dh
    wx = _randn((B, T, 3 * d), 21).to(dtype)
    rng = np.random.default_rng(22)
    A = np.stack([0.9 * np.linalg.qr(rng.standard_normal((dh, dh)))[0] for _ in range(3 * H)])
    A = torch.from_numpy(A.reshape(3, H, dh, dh).astype(np.float32)).cuda().to(dtype)
    st = ops.DeviceStats("cuda", 3)
    Hs = head_ops.newton_gru_head_fused(wx, A[0], A[1], A[2], None, max_iters=3, stats=st)
    hist, res, status = st.read()
    assert status == 0 and hist[2] < hist[1] < hist[0]

    wx_s = _np(_gate_slice(wx, 3, d, head * dh, dh))
    A_s = _np(A[:, head:head + 1])
    want = oracle.newton(oracle.GRU_HEAD, wx_s, A_s, None, n_heads=1, max_iters=3)
    got = _np(Hs[:, :, head * dh:(head + 1) * dh])
    if dtype == torch.float32:
        assert np.abs(got - want.states).max() <= 1e-5 * max(1.0, max(want.history))
    else:
        assert rel_err(got, want.states) <= BF16_RTOL

    G = _randn((B, T, d), 23).to(dtype)
    g_wx, g_az, g_ar, g_an, _ = head_ops.gru_head_reverse_vjp(Hs, wx, A[0], A[1], A[2], G, None)
    w_wx, w_A, _ = oracle.backward(oracle.GRU_HEAD, got, wx_s, A_s, _np(G[:, :, head * dh:(head + 1) * dh]),
                                   None, n_heads=1)
    tol = 5e-5 if dtype == torch.float32 else BF16_RTOL
    assert rel_err(_np(_gate_slice(g_wx, 3, d, head * dh, dh)), w_wx) <= tol
    w_A = np.asarray(w_A).reshape(3, dh, dh)
    for k, g_a in enumerate((g_az, g_ar, g_an)):
        assert rel_err(_np(g_a[head]), w_A[k]) <= (2e-4 if dtype == torch.float32 else 5e-3), k


def test_c5_nlru_layer_slice_matches_oracle():
    """One layer of the 12-layer NLRU stack: d=768, bf16, B=4, T=8192, K=2."""
    from pararnn_b200 import ops

    B, T, d, n, c0 = 4, 8192, 768, 32, 704
    wx = _randn((B, T, 2 * d), 31)
    a0 = torch.rand(d, device="cuda") * 0.099 + 0.9
    wx[..., :d] += torch.log(a0 / (1 - a0))
    wx = wx.to(torch.bfloat16)
    u = (0.3 * _randn((d,), 32)).clamp(-0.5, 0.5).to(torch.bfloat16)
    st = ops.DeviceStats("cuda", 2)
    H = ops.newton_nlru_fused(wx, u, None, max_iters=2, stats=st)
    assert st.read()[2] == 0
    wx_s, u_s = _np(_gate_slice(wx, 2, d, c0, n)), _np(u[c0:c0 + n]).reshape(1, -1)
    want = oracle.newton(oracle.NLRU, wx_s, u_s, None, max_iters=2)
    got = _np(H[:, :, c0:c0 + n])
    assert rel_err(got, want.states) <= BF16_RTOL
    G = _randn((B, T, d), 33).to(torch.bfloat16)
    g_wx, g_u, _ = ops.nlru_reverse_vjp(H, wx, u, G, None)
    w_wx, w_u, _ = oracle.backward(oracle.NLRU, got, wx_s, u_s, _np(G[:, :, c0:c0 + n]), None)
    assert rel_err(_np(_gate_slice(g_wx, 2, d, c0, n)), w_wx) <= BF16_RTOL
    assert rel_err(_np(g_u.reshape(-1)[c0:c0 + n]), np.asarray(w_u).reshape(-1)) <= 2e-3


def test_c1_gru_diag_fp32_full_problem():
    """ParaGRU diag fp32, B=2, T=1024, d=64, K=3: small enough for the oracle in full."""
    from gpu_util import dev, make_problem
    from pararnn_b200 import ops

    wx, a, _ = make_problem("gru_diag", 2, 1024, 64, seed=0)
    want = oracle.newton(oracle.GRU_DIAG, wx, a, None, max_iters=3)
    st = ops.DeviceStats("cuda", 3)
    H = ops.newton_gru_fused(dev(wx), dev(a[0]), dev(a[1]), dev(a[2]), None, max_iters=3, stats=st)
    hist, res, status = st.read()
    assert status == 0
    assert np.abs(_np(H) - want.states).max() <= 1e-5 * max(1.0, max(want.history))
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=2e-2, atol=4e-6)
