"""GPU parity of the scalar-diagonal cells (ParaGRU diag, ParaNLRU, ParaTitans, ParaCfC), through the C ABI.

fp32 tolerance: 1e-5 max-abs on the hidden trajectory against the reference's eager path
(golden fixtures) and against the CPU oracle on seeded inputs.  bf16 tolerance: 2e-2 relative
against the fp32 oracle run on bf16-rounded inputs."""

import numpy as np
import pytest
import torch

from golden_util import golden_names, load_golden
from gpu_util import bf16_round, dev, make_problem, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu

FP32_ATOL = 1e-5
BF16_RTOL = 2e-2


# the packed (cu_seqlens) fixtures have their own test file
RECT = [n for n in golden_names("gru_diag") + golden_names("nlru") + golden_names("titans") + golden_names("cfc")
        if "packed" not in n]


def _fwd(kind, wx, params, h0, K, omega=1.0, dtype=torch.float32):
    from pararnn_b200 import ops

    st = ops.DeviceStats("cuda", K)
    if kind == "gru_diag":
        H = ops.newton_gru_fused(dev(wx, dtype), dev(params[0], dtype), dev(params[1], dtype),
                                 dev(params[2], dtype), dev(h0, dtype), max_iters=K, omega=omega, stats=st)
    elif kind == "titans":
        H = ops.newton_titans_fused(dev(wx, dtype), dev(params[0], dtype), dev(params[1], dtype), dev(h0, dtype),
                                    max_iters=K, omega=omega, stats=st)
    elif kind == "cfc":
        H = ops.newton_cfc_fused(dev(wx, dtype), dev(params[0], dtype), dev(h0, dtype), max_iters=K,
                                 omega=omega, stats=st)
    else:
        H = ops.newton_nlru_fused(dev(wx, dtype), dev(params[0], dtype), dev(h0, dtype), max_iters=K,
                                  omega=omega, stats=st)
    hist, res, status = st.read()
    assert status == 0
    return H.float().cpu().numpy(), hist, res


def _bwd(kind, H, wx, params, G, h0, dtype=torch.float32):
    from pararnn_b200 import ops

    if kind == "gru_diag":
        g_wx, gz, gr, gn, g_h0 = ops.gru_reverse_vjp(dev(H, dtype), dev(wx, dtype), dev(params[0], dtype),
                                                     dev(params[1], dtype), dev(params[2], dtype),
                                                     dev(G, dtype), dev(h0, dtype))
        gp = torch.stack([gz, gr, gn])
    elif kind == "titans":
        g_wx, gu, gr, g_h0 = ops.titans_reverse_vjp(dev(H, dtype), dev(wx, dtype), dev(params[0], dtype),
                                                    dev(params[1], dtype), dev(G, dtype), dev(h0, dtype))
        gp = torch.stack([gu, gr])
    else:
        fn = ops.cfc_reverse_vjp if kind == "cfc" else ops.nlru_reverse_vjp
        g_wx, gu, g_h0 = fn(dev(H, dtype), dev(wx, dtype), dev(params[0], dtype), dev(G, dtype), dev(h0, dtype))
        gp = gu[None]
    return g_wx.float().cpu().numpy(), gp.cpu().numpy(), g_h0.cpu().numpy()


@pytest.mark.parametrize("name", RECT)
def test_forward_matches_reference_golden(name):
    g = load_golden(name)
    H, hist, res = _fwd(g["cell"], g["wx"], g["params"], g["h0"], g["K"], g["omega"])
    amp = max(1.0, float(np.max(g["history"])) if len(g["history"]) else 1.0)
    assert np.abs(H - g["H"]).max() <= FP32_ATOL * amp
    n = len(g["history"])
    np.testing.assert_allclose(np.asarray(hist[:n]), g["history"], rtol=5e-3, atol=2e-6)
    assert abs(res - float(g["max_residual"])) <= 5e-3 * float(g["max_residual"]) + 2e-6


@pytest.mark.parametrize("name", RECT)
def test_backward_matches_reference_golden(name):
    g = load_golden(name)
    kind = oracle.KIND[g["cell"]]
    want_wx, want_p, want_h0 = oracle.backward(kind, g["H"], g["wx"], g["params"], g["G"], g["h0"])
    g_wx, gp, g_h0 = _bwd(g["cell"], g["H"], g["wx"], g["params"], g["G"], g["h0"])
    assert np.abs(g_wx - want_wx).max() <= 2e-5 * max(1.0, np.abs(want_wx).max())
    assert np.abs(gp - want_p.reshape(gp.shape)).max() <= 2e-5 * max(1.0, np.abs(want_p).max())
    if g["h0"] is not None:
        assert np.abs(g_h0 - want_h0).max() <= 2e-5 * max(1.0, np.abs(want_h0).max())
        assert np.abs(g_h0 - g["g_h0"]).max() <= 2e-5 * max(1.0, np.abs(g["g_h0"]).max())


SHAPES = [(1, 1, 1), (2, 2, 5), (1, 63, 33), (2, 64, 32), (3, 65, 31), (2, 127, 70), (2, 129, 64),
          (1, 1000, 96), (2, 4096, 40)]


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
@pytest.mark.parametrize("B,T,d", SHAPES)
@pytest.mark.parametrize("K", [1, 3])
def test_forward_seeded_vs_oracle_fp32(kind, B, T, d, K):
    wx, params, h0 = make_problem(kind, B, T, d, seed=B * 1000 + T + d, h0=(T % 2 == 1))
    want = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=K)
    H, hist, res = _fwd(kind, wx, params, h0, K)
    amp = max(1.0, max(want.history))
    assert np.abs(H - want.states).max() <= FP32_ATOL * amp
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=5e-3, atol=2e-6)
    assert abs(res - want.max_residual) <= 5e-3 * want.max_residual + 2e-6


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
def test_k0_returns_guess_and_k2_matches(kind):
    wx, params, h0 = make_problem(kind, 2, 200, 48, seed=5, h0=True)
    g0 = oracle.guess(oracle.KIND[kind], wx, params, h0)
    H, _, res = _fwd(kind, wx, params, h0, 0)
    assert np.abs(H - g0).max() <= 2e-6
    assert abs(res - oracle.residual(oracle.KIND[kind], wx, params, g0, h0)) <= 1e-5
    want = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=2)
    H2, _, _ = _fwd(kind, wx, params, h0, 2)
    assert np.abs(H2 - want.states).max() <= FP32_ATOL * max(1.0, max(want.history))


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
@pytest.mark.parametrize("B,T,d", [(1, 1, 3), (2, 65, 31), (2, 513, 70), (1, 3000, 64)])
def test_backward_seeded_vs_oracle_fp32(kind, B, T, d):
    wx, params, h0 = make_problem(kind, B, T, d, seed=T + d, h0=(T % 2 == 1))
    H = oracle.sequential(oracle.KIND[kind], wx, params, h0)
    G = np.random.default_rng(T).standard_normal(H.shape).astype(np.float32)
    want_wx, want_p, want_h0 = oracle.backward(oracle.KIND[kind], H, wx, params, G, h0, prec="f64")
    g_wx, gp, g_h0 = _bwd(kind, H, wx, params, G, h0)
    assert rel_err(g_wx, want_wx) <= 2e-5
    assert rel_err(gp, want_p.reshape(gp.shape)) <= 5e-5
    assert rel_err(g_h0, want_h0) <= 2e-5


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
def test_bf16_io_within_relative_tolerance(kind):
    wx, params, h0 = make_problem(kind, 2, 2048, 96, seed=9, h0=True)
    wx, params, h0 = bf16_round(wx), bf16_round(params), bf16_round(h0)
    want = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=3)
    H, hist, res = _fwd(kind, wx, params, h0, 3, dtype=torch.bfloat16)
    assert rel_err(H, want.states) <= BF16_RTOL
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=2e-2, atol=1e-5)
    Hq = bf16_round(want.states)
    G = bf16_round(np.random.default_rng(1).standard_normal(Hq.shape))
    want_wx, want_p, want_h0 = oracle.backward(oracle.KIND[kind], Hq, wx, params, G, h0)
    g_wx, gp, g_h0 = _bwd(kind, Hq, wx, params, G, h0, dtype=torch.bfloat16)
    assert rel_err(g_wx, want_wx) <= BF16_RTOL
    assert rel_err(gp, want_p.reshape(gp.shape)) <= BF16_RTOL
    assert rel_err(g_h0, want_h0) <= BF16_RTOL


def test_vjp_is_bitwise_deterministic():
    wx, params, h0 = make_problem("gru_diag", 2, 777, 50, seed=3)
    H = oracle.sequential(oracle.GRU_DIAG, wx, params, h0)
    G = np.random.default_rng(0).standard_normal(H.shape).astype(np.float32)
    a = _bwd("gru_diag", H, wx, params, G, h0)
    b = _bwd("gru_diag", H, wx, params, G, h0)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_nan_input_propagates_to_residual():
    wx, params, h0 = make_problem("nlru", 1, 100, 16, seed=2)
    wx[0, 50, 3] = np.nan
    _, hist, res = _fwd("nlru", wx, params, h0, 2)
    assert np.isnan(res) and np.isnan(hist[0])


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "titans", "cfc"])
@pytest.mark.parametrize("B,T,d", [(1, 1, 3), (2, 65, 31), (3, 1000, 64), (2, 4097, 96)])
def test_bias_sum_from_the_reverse_kernel(kind, B, T, d, prb_options):
    """want_bias: the kernel's own per-gate sum of g_wx over batch and time, on both kernel families;
    the other results are unchanged by asking for it."""
    from pararnn_b200 import ops

    wx, params, h0 = make_problem(kind, B, T, d, seed=T + d, h0=True)
    H = oracle.sequential(oracle.KIND[kind], wx, params, h0)
    G = np.random.default_rng(T).standard_normal(H.shape).astype(np.float32)
    fn = {"gru_diag": ops.gru_reverse_vjp, "nlru": ops.nlru_reverse_vjp, "titans": ops.titans_reverse_vjp,
          "cfc": ops.cfc_reverse_vjp}[kind]
    for family in ("auto", "lookback"):
        if family == "lookback":
            prb_options("kernel_family", "lookback")
        plain = fn(dev(H), dev(wx), *[dev(p) for p in params], dev(G), dev(h0))
        withb = fn(dev(H), dev(wx), *[dev(p) for p in params], dev(G), dev(h0), want_bias=True)
        assert len(withb) == len(plain) + 1
        for u, v in zip(plain, withb):
            assert torch.equal(u, v)
        want = plain[0].double().sum((0, 1))
        assert float((withb[-1].double() - want).abs().max()) <= 2e-5 * max(1.0, float(want.abs().max()))
