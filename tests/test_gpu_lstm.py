"""ParaLSTM (CIFG peephole LSTM, 2x2 block Jacobian per channel) against the reference-generated
goldens and the oracle: forward Newton, residual history, reverse scan + packed VJP."""

import numpy as np
import pytest
import torch

from golden_util import golden_names, load_golden
from gpu_util import bf16_round, dev, make_problem, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu

RECT = [n for n in golden_names("lstm") if "packed" not in n]


def _fwd(wx, params, h0, K, omega=1.0, dtype=torch.float32):
    from pararnn_b200 import ops

    st = ops.DeviceStats("cuda", K)
    H = ops.newton_lstm_fused(dev(wx, dtype), *[dev(p, dtype) for p in params], dev(h0, dtype), max_iters=K,
                              omega=omega, stats=st)
    hist, res, status = st.read()
    assert status == 0
    return H.float().cpu().numpy(), np.asarray(hist), res


def test_fixtures_present():
    assert len(RECT) == 2


@pytest.mark.parametrize("name", RECT)
def test_forward_and_backward_match_reference_golden(name):
    from pararnn_b200 import ops

    g = load_golden(name)
    H, hist, res = _fwd(g["wx"], g["params"], g["h0"], g["K"], g["omega"])
    amp = max(1.0, float(np.max(g["history"])))
    assert np.abs(H - g["H"]).max() <= 1e-5 * amp
    np.testing.assert_allclose(hist, g["history"], rtol=5e-3, atol=2e-6)
    assert abs(res - float(g["max_residual"])) <= 5e-3 * float(g["max_residual"]) + 2e-6
    want_wx, want_p, want_h0 = oracle.backward(oracle.LSTM, g["H"], g["wx"], g["params"], g["G"], g["h0"])
    g_wx, gp, g_h0 = ops.lstm_reverse_vjp(dev(g["H"]), dev(g["wx"]), *[dev(p) for p in g["params"]], dev(g["G"]),
                                          dev(g["h0"]))
    assert rel_err(g_wx.cpu().numpy(), want_wx) <= 2e-5
    assert rel_err(gp.cpu().numpy().reshape(-1), want_p.reshape(-1)) <= 2e-5
    if g["h0"] is not None:
        assert rel_err(g_h0.cpu().numpy(), g["g_h0"]) <= 5e-5


@pytest.mark.parametrize("B,T,d", [(1, 1, 1), (2, 31, 33), (3, 32, 64), (2, 33, 40), (1, 1000, 70), (2, 4097, 32)])
@pytest.mark.parametrize("K", [0, 1, 3, 5])
def test_forward_seeded_vs_oracle_fp32(B, T, d, K):
    wx, params, h0 = make_problem("lstm", B, T, d, seed=B * 100 + T + d, h0=(T % 2 == 1))
    want = oracle.newton(oracle.LSTM, wx, params, h0, max_iters=K) if K else None
    H, hist, res = _fwd(wx, params, h0, K)
    if K == 0:
        g0 = oracle.guess(oracle.LSTM, wx, params, h0)
        assert np.abs(H - g0).max() <= 2e-6
        assert abs(res - oracle.residual(oracle.LSTM, wx, params, g0, h0)) <= 1e-5
        return
    amp = max(1.0, max(want.history))
    assert np.abs(H - want.states).max() <= 1e-5 * amp
    np.testing.assert_allclose(hist, np.asarray(want.history), rtol=1e-2, atol=2e-6)


@pytest.mark.parametrize("B,T,d", [(1, 1, 32), (2, 63, 40), (2, 1025, 64)])
def test_backward_seeded_vs_oracle(B, T, d):
    from pararnn_b200 import ops

    wx, params, h0 = make_problem("lstm", B, T, d, seed=T + d, h0=(T % 2 == 1))
    H = oracle.sequential(oracle.LSTM, wx, params, h0)
    G = np.random.default_rng(1).standard_normal(H.shape).astype(np.float32)
    want_wx, want_p, want_h0 = oracle.backward(oracle.LSTM, H, wx, params, G, h0, prec="f64")
    g_wx, gp, g_h0 = ops.lstm_reverse_vjp(dev(H), dev(wx), *[dev(p) for p in params], dev(G), dev(h0))
    assert rel_err(g_wx.cpu().numpy(), want_wx) <= 5e-5
    assert rel_err(gp.cpu().numpy().reshape(-1), want_p.reshape(-1)) <= 1e-4
    assert rel_err(g_h0.cpu().numpy(), want_h0) <= 5e-5


def test_bf16_io_within_relative_tolerance():
    wx, params, h0 = make_problem("lstm", 2, 2048, 96, seed=9, h0=True)
    wx, params, h0 = bf16_round(wx), bf16_round(params), bf16_round(h0)
    want = oracle.newton(oracle.LSTM, wx, params, h0, max_iters=3)
    H, _, _ = _fwd(wx, params, h0, 3, dtype=torch.bfloat16)
    assert rel_err(H, want.states) <= 2e-2


def test_output_slot_on_the_two_slot_cell_equals_slicing():
    """ParaLSTM has no compact-cotangent kernel: output_slot goes through the zero-filled array."""
    import pararnn_b200 as prb

    torch.manual_seed(0)
    cell = prb.ParaLSTM(16, 24).cuda()
    x = torch.randn(2, 150, 16, device="cuda", requires_grad=True)
    cfg = prb.NewtonConfig(max_iters=3)
    G = torch.randn(2, 150, 24, device="cuda")

    def grads(sliced):
        x.grad = None
        cell.zero_grad(set_to_none=True)
        out = prb.newton_apply(cell, x, cfg)[:, :, 1] if sliced else prb.newton_apply(cell, x, cfg, output_slot=1)
        (out * G).sum().backward()
        return [out.detach().clone(), x.grad.clone()] + [p.grad.clone() for p in cell.parameters()]

    for u, v in zip(grads(True), grads(False)):
        assert torch.equal(u, v)
    rnn = prb.ParaRNN(cell, config=cfg).train()
    assert rnn(x.detach()).shape == (2, 150, 24)
