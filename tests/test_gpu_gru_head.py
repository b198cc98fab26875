"""GPU parity of ParaGRU(mix='head') through the C ABI: fused Newton (skewed pipeline over the
iterations), reverse walk with J^T, packed VJP."""

import numpy as np
import pytest
import torch

from golden_util import golden_names, load_golden
from gpu_util import bf16_round, dev, make_problem, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu


def _fwd(wx, A, h0, K, omega=1.0, dtype=torch.float32):
    from pararnn_b200 import head_ops, ops

    st = ops.DeviceStats("cuda", K)
    H = head_ops.newton_gru_head_fused(dev(wx, dtype), dev(A[0], dtype), dev(A[1], dtype), dev(A[2], dtype),
                                       dev(h0, dtype), max_iters=K, omega=omega, stats=st)
    hist, res, status = st.read()
    assert status == 0
    return H.float().cpu().numpy(), hist, res


def _bwd(H, wx, A, G, h0, dtype=torch.float32):
    from pararnn_b200 import head_ops

    out = head_ops.gru_head_reverse_vjp(dev(H, dtype), dev(wx, dtype), dev(A[0], dtype), dev(A[1], dtype),
                                        dev(A[2], dtype), dev(G, dtype), dev(h0, dtype))
    g_wx, gz, gr, gn, g_h0 = out
    return g_wx.float().cpu().numpy(), torch.stack([gz, gr, gn]).cpu().numpy(), g_h0.cpu().numpy()


@pytest.mark.parametrize("name", golden_names("gru_head"))
def test_forward_and_backward_match_reference_golden(name):
    g = load_golden(name)
    H, hist, res = _fwd(g["wx"], g["params"], g["h0"], g["K"], g["omega"])
    assert np.abs(H - g["H"]).max() <= 1e-5
    np.testing.assert_allclose(np.asarray(hist), g["history"], rtol=5e-3, atol=2e-6)
    assert abs(res - float(g["max_residual"])) <= 5e-3 * float(g["max_residual"]) + 2e-6
    w_wx, w_p, w_h0 = oracle.backward(oracle.GRU_HEAD, g["H"], g["wx"], g["params"], g["G"], g["h0"],
                                      n_heads=g["n_heads"])
    g_wx, g_p, g_h0 = _bwd(g["H"], g["wx"], g["params"], g["G"], g["h0"])
    assert rel_err(g_wx, w_wx) <= 2e-5
    assert rel_err(g_p.reshape(-1), w_p.reshape(-1)) <= 5e-5
    assert rel_err(g_p, g["g_params"]) <= 5e-5
    if g["h0"] is not None:
        assert rel_err(g_h0, w_h0) <= 2e-5 and rel_err(g_h0, g["g_h0"]) <= 5e-5


@pytest.mark.parametrize("B,T,H,dh,K", [(1, 1, 1, 8, 2), (2, 3, 2, 16, 3), (2, 65, 2, 32, 3), (2, 300, 2, 64, 3),
                                        (1, 1000, 4, 64, 3), (2, 200, 1, 64, 5), (1, 150, 2, 64, 0),
                                        (1, 150, 2, 64, 1), (2, 120, 2, 16, 7)])
def test_forward_seeded_vs_oracle_fp32(B, T, H, dh, K):
    wx, A, h0 = make_problem("gru_head", B, T, H * dh, seed=T + dh, h0=(T % 2 == 1), n_heads=H)
    want = oracle.newton(oracle.GRU_HEAD, wx, A, h0, n_heads=H, max_iters=K)
    got, hist, res = _fwd(wx, A, h0, K)
    amp = max(1.0, max(want.history) if want.history else 1.0)
    assert np.abs(got - want.states).max() <= 1e-5 * amp
    if K:
        np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=5e-3, atol=2e-6)
    assert abs(res - want.max_residual) <= 5e-3 * want.max_residual + 2e-6


@pytest.mark.parametrize("B,T,H,dh", [(1, 1, 1, 8), (2, 65, 2, 32), (2, 400, 2, 64)])
def test_backward_seeded_vs_oracle_fp32(B, T, H, dh):
    wx, A, h0 = make_problem("gru_head", B, T, H * dh, seed=T, h0=(T % 2 == 1), n_heads=H)
    Hs = oracle.sequential(oracle.GRU_HEAD, wx, A, h0, n_heads=H)
    G = np.random.default_rng(T).standard_normal(Hs.shape).astype(np.float32)
    w_wx, w_p, w_h0 = oracle.backward(oracle.GRU_HEAD, Hs, wx, A, G, h0, n_heads=H, prec="f64")
    g_wx, g_p, g_h0 = _bwd(Hs, wx, A, G, h0)
    assert rel_err(g_wx, w_wx) <= 5e-5
    assert rel_err(g_p.reshape(-1), w_p.reshape(-1)) <= 1e-4
    assert rel_err(g_h0, w_h0) <= 5e-5


def test_bf16_io_within_relative_tolerance():
    H, dh = 2, 64
    wx, A, h0 = make_problem("gru_head", 2, 512, H * dh, seed=3, n_heads=H)
    wx, A = bf16_round(wx), bf16_round(A)
    want = oracle.newton(oracle.GRU_HEAD, wx, A, None, n_heads=H, max_iters=3)
    got, hist, _ = _fwd(wx, A, None, 3, dtype=torch.bfloat16)
    assert rel_err(got, want.states) <= 2e-2


def test_newton_apply_head_cell_autograd():
    import pararnn_b200 as prb

    torch.manual_seed(0)
    cell = prb.ParaGRU(64, 128, mix="head", n_heads=2).cuda()
    x = torch.randn(2, 200, 64, device="cuda", requires_grad=True)
    st = prb.NewtonStats()
    Hs = prb.newton_apply(cell, x, prb.NewtonConfig(max_iters=3), stats=st)
    assert st.iters == 3 and st.max_residual < 1e-4
    Hs.square().sum().backward()
    ref = prb.sequential_apply(cell, x.detach())
    assert (Hs - ref).abs().max() < 1e-4
    # gradients against BPTT through the sequential unroll
    cell2 = prb.ParaGRU(64, 128, mix="head", n_heads=2).cuda()
    cell2.load_state_dict(cell.state_dict())
    x2 = x.detach().clone().requires_grad_(True)
    prb.sequential_apply(cell2, x2).square().sum().backward()
    assert rel_err(x.grad.cpu().numpy(), x2.grad.cpu().numpy()) <= 1e-3
    assert rel_err(cell.A_n.grad.cpu().numpy(), cell2.A_n.grad.cpu().numpy()) <= 1e-3
    assert rel_err(cell.W_x.weight.grad.cpu().numpy(), cell2.W_x.weight.grad.cpu().numpy()) <= 1e-3
