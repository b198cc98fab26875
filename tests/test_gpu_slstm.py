"""GPU parity of ParaSLSTM(mix='diag') through the C ABI: Picard warm start, 4x4 Newton,
residual gate, reverse scan + packed VJP.

fp32: the hidden slot within 1e-5 max-abs; slots c, n, m within 1e-6 of max|slot| scaled by the
largest Newton residual on the way (rounding is amplified while an iterate is far from the
fixed point).  bf16: 2e-2 relative against the fp32 oracle on bf16-rounded inputs."""

import numpy as np
import pytest
import torch

from golden_util import golden_names, load_golden
from gpu_util import bf16_round, dev, make_problem, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu

FP32_ATOL_H = 1e-5
FP32_RTOL_SLOT = 1e-6
BF16_RTOL = 2e-2


def _fwd(wx, r, h0, K, P, omega=1.0, eps=1e-6, dtype=torch.float32, guess=None):
    from pararnn_b200 import ops

    st = ops.DeviceStats("cuda", K)
    H = ops.newton_slstm_fused(dev(wx, dtype), dev(r, dtype), dev(h0, dtype), dev(guess, dtype),
                               max_iters=K, omega=omega, eps=eps, picard_iters=P, stats=st)
    hist, res, status = st.read()
    assert status == 0
    return H.float().cpu().numpy(), hist, res


# the packed (cu_seqlens) fixtures have their own test file
RECT = [n for n in golden_names("slstm") if "packed" not in n]


def _check_states(H, want, amp):
    for slot, name in enumerate("cnmh"):
        err = np.abs(H[:, :, slot] - want[:, :, slot]).max()
        if name == "h":
            assert err <= FP32_ATOL_H * amp, (name, err)
        else:
            scale = max(1.0, np.abs(want[:, :, slot]).max())
            assert err <= 4 * FP32_RTOL_SLOT * scale * amp + 2e-6, (name, err)


@pytest.mark.parametrize("name", RECT)
def test_forward_matches_reference_golden(name):
    g = load_golden(name)
    H, hist, res = _fwd(g["wx"], g["params"], g["h0"], g["K"], g["P"], g["omega"], g["eps"])
    amp = max(1.0, float(np.max(g["history"])))
    _check_states(H, g["H"], amp)
    scale = max(1.0, float(np.abs(g["H"]).max()))
    np.testing.assert_allclose(np.asarray(hist), g["history"], rtol=1e-2, atol=4e-6 * scale)
    assert abs(res - float(g["max_residual"])) <= 1e-2 * float(g["max_residual"]) + 4e-6 * scale * amp


@pytest.mark.parametrize("name", RECT)
def test_backward_matches_reference_golden(name):
    from pararnn_b200 import ops

    g = load_golden(name)
    want_wx, want_p, want_h0 = oracle.backward(oracle.SLSTM_DIAG, g["H"], g["wx"], g["params"], g["G"],
                                               g["h0"], eps=g["eps"])
    g_wx, gp, g_h0 = ops.slstm_reverse_vjp(dev(g["H"]), dev(g["wx"]), dev(g["params"]), dev(g["G"]),
                                           dev(g["h0"]), g["eps"])
    assert rel_err(g_wx.cpu().numpy(), want_wx) <= 2e-5
    assert rel_err(gp.cpu().numpy(), want_p.reshape(4, -1)) <= 2e-5
    if g["h0"] is not None:
        assert rel_err(g_h0.cpu().numpy(), want_h0) <= 2e-5
        assert rel_err(g_h0.cpu().numpy(), g["g_h0"]) <= 5e-5


@pytest.mark.parametrize("P", [0, 1, 3])
def test_picard_guess_matches_oracle(P):
    wx, r, h0 = make_problem("slstm_diag", 2, 300, 40, seed=P, h0=True, rec_scale=2.0)
    want = oracle.guess(oracle.SLSTM_DIAG, wx, r, h0, picard=P)
    H, _, _ = _fwd(wx, r, h0, 0, P)
    # the warm start is a guess, not a fixed point: the chained (a, b, N, C) summaries and the
    # reference's cumsum / cummax formulation round differently over hundreds of steps
    for slot in range(4):
        scale = max(1.0, np.abs(want[:, :, slot]).max())
        assert np.abs(H[:, :, slot] - want[:, :, slot]).max() <= 3e-5 * scale


SHAPES = [(1, 1, 1), (2, 2, 5), (1, 31, 33), (2, 32, 32), (3, 33, 31), (2, 127, 70), (2, 129, 64),
          (1, 1000, 96), (2, 4096, 40)]


@pytest.mark.parametrize("B,T,d", SHAPES)
def test_forward_seeded_vs_oracle_fp32(B, T, d):
    # short sequences: a stress setting where Newton does the work; long sequences: a milder
    # one (the stress setting leaves the Newton basin beyond a few hundred steps)
    stress = T <= 129
    wx, r, h0 = make_problem("slstm_diag", B, T, d, seed=B * 1000 + T + d, h0=(T % 2 == 1),
                             x_scale=0.7 if stress else 0.6, rec_scale=1.5 if stress else 1.2,
                             bias_f=0.0 if stress else 1.0)
    P = 2 if stress else 3
    want = oracle.newton(oracle.SLSTM_DIAG, wx, r, h0, max_iters=3, picard=P)
    H, hist, res = _fwd(wx, r, h0, 3, P)
    amp = max(1.0, max(want.history))
    _check_states(H, want.states, amp)
    scale = max(1.0, float(np.abs(want.states).max()))
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=2e-2, atol=4e-6 * scale * amp)


def test_forget_bias_config_shape_family():
    """Inputs of the headline configuration family (x*0.5, forget bias +3, P=5, K=2)."""
    wx, r, h0 = make_problem("slstm_diag", 2, 8192, 64, seed=1, x_scale=0.5, bias_f=3.0)
    want = oracle.newton(oracle.SLSTM_DIAG, wx, r, None, max_iters=2, picard=5)
    seq = oracle.sequential(oracle.SLSTM_DIAG, wx, r, None)
    H, hist, res = _fwd(wx, r, None, 2, 5)
    assert np.abs(H[:, :, 3] - want.states[:, :, 3]).max() <= FP32_ATOL_H
    assert np.abs(H[:, :, 3] - seq[:, :, 3]).max() <= FP32_ATOL_H
    for slot in range(3):
        scale = np.abs(seq[:, :, slot]).max()
        assert np.abs(H[:, :, slot] - seq[:, :, slot]).max() <= 4e-6 * scale
    # the residual is limited by one ulp of the stabiliser m
    ulp_m = np.spacing(np.float32(np.abs(seq[:, :, 2]).max()))
    assert res <= 4 * ulp_m and want.max_residual <= 4 * ulp_m


def test_states_guess_argument_replaces_picard():
    wx, r, h0 = make_problem("slstm_diag", 2, 200, 24, seed=4, x_scale=0.5, bias_f=1.0)
    guess = oracle.guess(oracle.SLSTM_DIAG, wx, r, None, picard=1)
    a, ha, _ = _fwd(wx, r, None, 3, 1)
    b, hb, _ = _fwd(wx, r, None, 3, 0, guess=guess)
    assert ha[-1] < 1e-3 and hb[-1] < 1e-3
    assert np.abs(a[:, :, 3] - b[:, :, 3]).max() <= 1e-5
    assert np.abs(a - b).max() <= 4e-6 * np.abs(a).max()


@pytest.mark.parametrize("B,T,d", [(1, 1, 3), (2, 33, 31), (2, 513, 70), (1, 3000, 64)])
def test_backward_seeded_vs_oracle_fp32(B, T, d):
    from pararnn_b200 import ops

    wx, r, h0 = make_problem("slstm_diag", B, T, d, seed=T + d, h0=(T % 2 == 1), x_scale=0.7, rec_scale=1.5)
    H = oracle.sequential(oracle.SLSTM_DIAG, wx, r, h0)
    G = np.random.default_rng(T).standard_normal(H.shape).astype(np.float32)
    want_wx, want_p, want_h0 = oracle.backward(oracle.SLSTM_DIAG, H, wx, r, G, h0, prec="f64")
    g_wx, gp, g_h0 = ops.slstm_reverse_vjp(dev(H), dev(wx), dev(r), dev(G), dev(h0))
    assert rel_err(g_wx.cpu().numpy(), want_wx) <= 5e-5
    assert rel_err(gp.cpu().numpy(), want_p.reshape(4, -1)) <= 1e-4
    assert rel_err(g_h0.cpu().numpy(), want_h0) <= 5e-5


def test_bf16_io_within_relative_tolerance():
    from pararnn_b200 import ops

    wx, r, h0 = make_problem("slstm_diag", 2, 2048, 96, seed=9, x_scale=0.5, bias_f=3.0)
    wx, r = bf16_round(wx), bf16_round(r)
    want = oracle.newton(oracle.SLSTM_DIAG, wx, r, None, max_iters=2, picard=5)
    H, hist, res = _fwd(wx, r, None, 2, 5, dtype=torch.bfloat16)
    for slot in range(4):
        assert rel_err(H[:, :, slot], want.states[:, :, slot]) <= BF16_RTOL
    Hq = bf16_round(want.states)
    G = bf16_round(np.random.default_rng(1).standard_normal(Hq.shape))
    G[:, :, :3] = 0  # the sequence wrapper only differentiates the hidden slot
    want_wx, want_p, _ = oracle.backward(oracle.SLSTM_DIAG, Hq, wx, r, G, None)
    g_wx, gp, _ = ops.slstm_reverse_vjp(dev(Hq, torch.bfloat16), dev(wx, torch.bfloat16),
                                        dev(r, torch.bfloat16), dev(G, torch.bfloat16))
    assert rel_err(g_wx.float().cpu().numpy(), want_wx) <= BF16_RTOL
    assert rel_err(gp.cpu().numpy(), want_p.reshape(4, -1)) <= BF16_RTOL


def test_divergence_is_reported_not_hidden():
    wx, r, h0 = make_problem("slstm_diag", 1, 64, 8, seed=2)
    wx[0, 10, 2] = np.inf
    _, hist, res = _fwd(wx, r, None, 2, 1)
    assert not np.isfinite(res)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,d,h0,slot", [(1, 1, 32, False, 3), (2, 65, 40, True, 3), (2, 1000, 96, True, 0),
                                            (1, 4099, 64, False, 3), (3, 513, 32, True, 2)])
def test_one_slot_cotangent_and_bias_sum(B, T, d, h0, slot, dtype):
    """grad_slot: the (B,T,d) cotangent of one state slot gives what the zero-filled (B,T,4,d)
    array gives; want_bias: the kernel's own sum of g_wx over batch and time."""
    from pararnn_b200 import ops

    wx, r, h0a = make_problem("slstm_diag", B, T, d, seed=T + d, h0=h0, x_scale=0.7, bias_f=2.0)
    if dtype == torch.bfloat16:
        wx, r, h0a = bf16_round(wx), bf16_round(r), (None if h0a is None else bf16_round(h0a))
    H = oracle.sequential(oracle.SLSTM_DIAG, wx, r, h0a)
    g1 = np.random.default_rng(T).standard_normal((B, T, d)).astype(np.float32)
    full = np.zeros((B, T, 4, d), np.float32)
    full[:, :, slot] = g1
    a = ops.slstm_reverse_vjp(dev(H, dtype), dev(wx, dtype), dev(r, dtype), dev(full, dtype), dev(h0a, dtype))
    b = ops.slstm_reverse_vjp(dev(H, dtype), dev(wx, dtype), dev(r, dtype), dev(g1, dtype), dev(h0a, dtype),
                              grad_slot=slot, want_bias=True)
    for u, v in zip(a, b[:3]):
        if slot == 3:
            assert torch.equal(u, v)  # same kernel family: the three absent terms are exact zeros
        else:
            # slots other than the hidden one are served by the look-back kernels, whatever family
            # the full cotangent ran on: same values up to the order of the fp32 sums
            tol = 2e-5 if dtype == torch.float32 else 1e-2
            assert float((u.float() - v.float()).abs().max()) <= tol * max(1.0, float(u.float().abs().max()))
    want_bias = a[0].double().sum((0, 1))
    tol = 2e-5 if dtype == torch.float32 else 1e-2  # bf16: g_wx is rounded on store, the kernel's sum is not
    assert float((b[3].double() - want_bias).abs().max()) <= tol * max(1.0, float(want_bias.abs().max()))
    with pytest.raises(ValueError):
        ops.slstm_reverse_vjp(dev(H, dtype), dev(wx, dtype), dev(r, dtype), dev(full, dtype), dev(h0a, dtype),
                              grad_slot=3)


@pytest.mark.parametrize("chunk_len", [None, 128])
def test_output_slot_equals_slicing_the_states(chunk_len):
    import pararnn_b200 as prb

    torch.manual_seed(0)
    cell = prb.ParaSLSTM(24, 32).cuda()
    with torch.no_grad():
        cell.W_x.bias[32:64] = 1.0
    x = (0.6 * torch.randn(2, 300, 24, device="cuda")).requires_grad_(True)
    h0 = torch.zeros(2, 4, 32, device="cuda")
    h0[:, 1] = 1.0
    h0.requires_grad_(True)
    cfg = prb.NewtonConfig(max_iters=3, picard_iters=3, picard_adapt=False, chunk_len=chunk_len)
    G = torch.randn(2, 300, 32, device="cuda")

    def grads(sliced):
        for t in (x, h0):
            t.grad = None
        cell.zero_grad(set_to_none=True)
        out = (prb.newton_apply(cell, x, cfg, h0=h0)[:, :, 3] if sliced
               else prb.newton_apply(cell, x, cfg, h0=h0, output_slot=3))
        (out * G).sum().backward()
        return [out.detach().clone(), x.grad.clone(), h0.grad.clone()] + [p.grad.clone() for p in cell.parameters()]

    a, b = grads(True), grads(False)
    assert torch.equal(a[0], b[0])
    names = ["out", "x", "h0"] + [n for n, _ in cell.named_parameters()]
    for n, u, v in zip(names, a, b):
        # W_x.bias: summed by the kernel in fp32 instead of by a reduction over the stored g_wx
        assert float((u - v).abs().max()) <= 2e-5 * max(1.0, float(u.abs().max())), n
    with pytest.raises(ValueError):
        prb.newton_apply(prb.ParaGRU(8, 8).cuda(), torch.randn(1, 4, 8, device="cuda"), output_slot=0)
    with pytest.raises(ValueError):
        prb.newton_apply(cell, x, cfg, output_slot=4)


def test_para_rnn_layer_outputs_the_hidden_slot_with_gradients():
    import pararnn_b200 as prb

    torch.manual_seed(1)
    rnn = prb.ParaRNN(prb.ParaSLSTM(32, 32).cuda(), config=prb.NewtonConfig(max_iters=3), num_layers=2).train()
    x = (0.5 * torch.randn(2, 200, 32, device="cuda")).requires_grad_(True)
    y = rnn(x)
    assert y.shape == (2, 200, 32)
    y.square().sum().backward()
    want = prb.sequential_apply(rnn.cells[1], prb.sequential_apply(rnn.cells[0], x.detach())[:, :, 3])[:, :, 3]
    assert float((y.detach() - want).abs().max()) <= 1e-4
    assert x.grad is not None and all(p.grad is not None for p in rnn.parameters())
