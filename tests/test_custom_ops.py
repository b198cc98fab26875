"""torch.library registration: every op of the backend is visible under ``torch.ops.pararnn_b200``
and has a meta kernel that gives the output shapes and dtypes without touching a device."""

import pytest
import torch

import pararnn_b200  # noqa: F401  (registers the ops)
from pararnn_b200 import custom_ops


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, dtype=dtype, device="meta")


def test_ops_are_registered_with_the_reference_argument_lists():
    ns = torch.ops.pararnn_b200
    for name in custom_ops.OP_NAMES:
        assert hasattr(ns, name), name
    schema = str(ns.newton_gru_fused.default._schema)
    for arg in ("Tensor wx", "Tensor a_z", "Tensor a_r", "Tensor a_n", "Tensor? h0", "Tensor? cu_seqlens",
                "Tensor? block_table", "max_iters", "float omega"):
        assert arg in schema, (arg, schema)
    schema = str(ns.newton_slstm_fused.default._schema)
    for arg in ("Tensor wx", "Tensor r", "Tensor? h0", "Tensor? states", "Tensor? block_table", "max_iters",
                "float omega", "float eps", "bool log_coords", "str scan_tile", "bool time_loop", "window_len"):
        assert arg in schema, (arg, schema)
    schema = str(ns.newton_gru_head_fused.default._schema)
    assert "Tensor? cu_seqlens" in schema and "block_table" not in schema
    schema = str(ns.reverse_gru_head_factor.default._schema)
    for arg in ("Tensor h_prev", "Tensor wx", "Tensor partial", "Tensor a_z", "Tensor a_r", "Tensor a_n"):
        assert arg in schema


def test_fake_kernels_on_meta_tensors():
    ns = torch.ops.pararnn_b200
    B, T, d, H = 3, 50, 64, 4
    out = ns.newton_gru_fused(_meta(B, T, 3 * d), _meta(d), _meta(d), _meta(d), max_iters=3, omega=1.0)
    assert out.shape == (B, T, d) and out.dtype == torch.bfloat16 and out.device.type == "meta"
    out = ns.newton_nlru_fused(_meta(B, T, 2 * d), _meta(d), _meta(B, d), max_iters=2, omega=0.9)
    assert out.shape == (B, T, d)
    out = ns.newton_slstm_fused(_meta(B, T, 4 * d), _meta(4, d), max_iters=2, omega=1.0, eps=1e-6)
    assert out.shape == (B, T, 4, d)
    guess = _meta(B, T, 4, d, dtype=torch.float32)
    out = ns.newton_slstm_fused(_meta(B, T, 4 * d, dtype=torch.float32), _meta(4, d), None, guess,
                                max_iters=2, omega=1.0, eps=1e-6)
    assert out.shape == guess.shape and out.dtype == torch.float32
    A = _meta(H, d // H, d // H)
    out = ns.newton_gru_head_fused(_meta(B, T, 3 * d), A, A, A, max_iters=3, omega=1.0)
    assert out.shape == (B, T, d)
    mu = ns.reverse_gru_head_factor(_meta(B, T, d), _meta(B, T, 3 * d), _meta(B, T, d), A, A, A)
    assert mu.shape == (B, T, d)
    g_wx, gz, gr, gn, g_h0 = ns.reverse_gru_vjp(_meta(B, T, d), _meta(B, T, 3 * d), _meta(d), _meta(d), _meta(d),
                                                _meta(B, T, d))
    assert g_wx.shape == (B, T, 3 * d) and gz.shape == (d,) and gz.dtype == torch.float32 and g_h0.shape == (B, d)
    g_wx, gu, g_h0 = ns.reverse_nlru_vjp(_meta(B, T, d), _meta(B, T, 2 * d), _meta(d), _meta(B, T, d))
    assert g_wx.shape == (B, T, 2 * d) and gu.shape == (d,)
    g_wx, g_r, g_h0 = ns.reverse_slstm_vjp(_meta(B, T, 4, d), _meta(B, T, 4 * d), _meta(4, d), _meta(B, T, 4, d))
    assert g_wx.shape == (B, T, 4 * d) and g_r.shape == (4, d) and g_h0.shape == (B, 4, d)
    g_wx, gz, gr, gn, g_h0 = ns.reverse_gru_head_vjp(_meta(B, T, d), _meta(B, T, 3 * d), A, A, A, _meta(B, T, d))
    assert gz.shape == A.shape and g_h0.shape == (B, d)


def test_ops_refuse_cpu_tensors():
    # no CPU kernel behind the ops: a real CPU tensor raises instead of computing somewhere else
    with pytest.raises(RuntimeError):
        torch.ops.pararnn_b200.newton_nlru_fused(torch.zeros(1, 4, 8), torch.zeros(4), max_iters=1, omega=1.0)


@pytest.mark.gpu
def test_ops_run_on_the_gpu_and_match_the_python_operators():
    from gpu_util import dev, make_problem
    from pararnn_b200 import head_ops, ops

    ns = torch.ops.pararnn_b200
    wx, params, h0 = make_problem("gru_diag", 2, 300, 40, seed=1, h0=True)
    a = ns.newton_gru_fused(dev(wx), *[dev(p) for p in params], dev(h0), max_iters=3, omega=1.0)
    b = ops.newton_gru_fused(dev(wx), *[dev(p) for p in params], dev(h0), max_iters=3)
    assert torch.equal(a, b)
    wx, r, _ = make_problem("slstm_diag", 2, 200, 32, seed=2)
    custom_ops.set_default_picard_iters(2)
    try:
        a = ns.newton_slstm_fused(dev(wx), dev(r), max_iters=2, omega=1.0, eps=1e-6)
    finally:
        custom_ops.set_default_picard_iters(0)
    assert torch.equal(a, ops.newton_slstm_fused(dev(wx), dev(r), max_iters=2, picard_iters=2))
    # reverse_gru_head_factor returns the adjoint mu of eq. 2.6: compare with the oracle's
    import numpy as np

    from oracle import oracle

    wx, A, h0 = make_problem("gru_head", 2, 64, 32, seed=3, h0=True, n_heads=2)
    H = oracle.sequential(oracle.GRU_HEAD, wx, A, h0, n_heads=2)
    G = np.random.default_rng(0).standard_normal(H.shape).astype(np.float32)
    _, _, _, mu = oracle.backward(oracle.GRU_HEAD, H, wx, A, G, h0, n_heads=2, want_mu=True)
    h_prev = np.concatenate([h0[:, None], H[:, :-1]], axis=1)
    got = ns.reverse_gru_head_factor(dev(h_prev), dev(wx), dev(G), dev(A[0]), dev(A[1]), dev(A[2]))
    assert np.abs(got.cpu().numpy() - mu).max() <= 2e-5 * max(1.0, np.abs(mu).max())
