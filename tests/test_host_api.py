"""Host-side mirror of the reference interface: configuration, cells, sequential unroll."""

import numpy as np
import pytest
import torch

import pararnn_b200 as prb
from golden_util import golden_names, load_golden
from oracle import oracle
from pararnn_b200.config import resolve_max_iters, validate_config


def _cell_from_golden(g):
    d = g["params"].shape[-1] if g["cell"] != "gru_head" else g["W"].shape[0] // 3
    d_in = g["W"].shape[1]
    if g["cell"] == "gru_diag":
        cell = prb.ParaGRU(d_in, d)
        names = ("a_z", "a_r", "a_n")
    elif g["cell"] == "gru_head":
        cell = prb.ParaGRU(d_in, d, mix="head", n_heads=g["n_heads"])
        names = ("A_z", "A_r", "A_n")
    elif g["cell"] == "nlru":
        cell = prb.ParaNLRU(d_in, d)
        names = ("u",)
    elif g["cell"] == "titans":
        cell = prb.ParaTitans(d_in, d)
        names = ("u", "r")
    elif g["cell"] == "lstm":
        cell = prb.ParaLSTM(d_in, d)
        names = ("a_f", "a_z", "a_o", "c_f", "c_o")
    elif g["cell"] == "cfc":
        d_in += 1  # the last input channel is the time step, not a feature of W_x
        cell = prb.ParaCfC(d_in, d)
        names = ("u",)
        with torch.no_grad():
            cell.W_b.weight.copy_(torch.from_numpy(g["W_b"]))
            cell.W_b.bias.copy_(torch.from_numpy(g["b_b"]))
    else:
        cell = prb.ParaSLSTM(d_in, d, eps=g["eps"])
        names = ("R",)
    with torch.no_grad():
        cell.W_x.weight.copy_(torch.from_numpy(g["W"]))
        cell.W_x.bias.copy_(torch.from_numpy(g["b"]))
        if names == ("R",):
            cell.R.copy_(torch.from_numpy(g["raw_params"]))
        else:
            for n, v in zip(names, g["raw_params"]):
                getattr(cell, n).copy_(torch.from_numpy(v))
    return cell


@pytest.mark.parametrize("name", golden_names())
def test_sequential_apply_matches_reference(name):
    g = load_golden(name)
    cell = _cell_from_golden(g)
    h0 = None if g["h0"] is None else torch.from_numpy(g["h0"])
    cs = None if g["cu_seqlens"] is None else torch.from_numpy(g["cu_seqlens"])
    with torch.no_grad():
        H = prb.sequential_apply(cell, torch.from_numpy(g["x"]), h0, cu_seqlens=cs).numpy()
    scale = max(1.0, float(np.abs(g["H_seq"]).max()))
    assert np.abs(H - g["H_seq"]).max() <= 2e-6 * scale


def test_parameter_order_is_the_autograd_contract():
    assert [n for n, _ in prb.ParaGRU(4, 8).named_parameters()] == ["a_z", "a_r", "a_n", "W_x.weight", "W_x.bias"]
    assert [n for n, _ in prb.ParaGRU(4, 8, mix="head", n_heads=2).named_parameters()] == [
        "A_z", "A_r", "A_n", "W_x.weight", "W_x.bias"]
    assert [n for n, _ in prb.ParaNLRU(4, 8).named_parameters()] == ["u", "W_x.weight", "W_x.bias"]
    assert [n for n, _ in prb.ParaSLSTM(4, 8).named_parameters()] == ["R", "W_x.weight", "W_x.bias"]
    assert [n for n, _ in prb.ParaCfC(4, 8).named_parameters()] == ["u", "W_x.weight", "W_x.bias", "W_b.weight",
                                                                    "W_b.bias"]


def test_config_validation_errors():
    for bad in (dict(scan_backend="nope"), dict(jacobian="x"), dict(coords="polar"), dict(chunk_len=0),
                dict(max_iters=-1), dict(picard_iters=-2), dict(residual_fail=-1.0),
                dict(newton_iters_by_t={64: 2}), dict(scan_tile="zig"),
                dict(fused_window_len=64), dict(fused_early_exit=True, residual_atol=None)):
        with pytest.raises(ValueError):
            validate_config(prb.NewtonConfig(**bad))
    validate_config(prb.NewtonConfig())
    validate_config(prb.compile_safe_config())


def test_resolve_max_iters_and_picard_ladder():
    assert resolve_max_iters(prb.NewtonConfig(max_iters=None), 4096) == 3
    cfg = prb.NewtonConfig(max_iters=None, newton_iters_by_t={64: 2, 1024: 3, 4096: 4})
    assert [resolve_max_iters(cfg, t) for t in (64, 1000, 1024, 5000)] == [2, 2, 3, 4]
    assert [prb.slstm_auto_picard(t) for t in (1, 64, 65, 2048, 2049)] == [1, 1, 3, 3, 5]
    assert [prb.slstm_picard_next(p) for p in (0, 1, 3, 5)] == [1, 3, 5, None]


def test_newton_apply_has_no_cpu_path():
    cell = prb.ParaGRU(4, 8)
    with pytest.raises(RuntimeError, match="no CPU solver"):
        prb.newton_apply(cell, torch.randn(2, 5, 4))
    with pytest.raises(TypeError, match="single CUDA"):
        prb.newton_apply(cell, torch.randn(2, 5, 4), prb.NewtonConfig(scan_backend="eager"))
    with pytest.raises(TypeError):
        prb.newton_apply(cell, torch.randn(2, 5, 4), prb.NewtonConfig(picard_iters=2))


def test_ops_reject_cpu_tensors():
    from pararnn_b200 import ops

    with pytest.raises(RuntimeError, match="CUDA"):
        ops.newton_nlru_fused(torch.randn(1, 4, 8), torch.randn(4), max_iters=1)


def test_oracle_early_stop_counts_residual_evaluations():
    g = load_golden("gru_diag_k3")
    r = oracle.newton(oracle.GRU_DIAG, g["wx"], g["params"], max_iters=8, early_atol=1e-5)
    assert r.iters < 8 and r.history[-1] < 1e-5 and all(h >= 1e-5 for h in r.history[:-1])


def test_cfc_input_gradients_match_autograd_through_project_wx():
    """The hand-written gradients of ParaCfC's input projection (two linear maps on the features,
    the clamped time step broadcast over the channels) against autograd, on the CPU."""
    from pararnn_b200.newton import _cfc_input_grads

    torch.manual_seed(0)
    cell = prb.ParaCfC(7, 5).double()
    with torch.no_grad():
        cell.W_b.weight.normal_(0.0, 0.3)
    x = torch.randn(2, 9, 7, dtype=torch.float64)
    x[..., -1] = torch.rand(2, 9, dtype=torch.float64)
    x[0, ::3, -1] = 0.0  # below the clamp: no gradient reaches the raw time step there
    x.requires_grad_(True)
    g_wx = torch.randn(2, 9, 20, dtype=torch.float64)
    (cell.project_wx(x) * g_wx).sum().backward()
    with torch.no_grad():
        grad_x, grads = _cfc_input_grads(cell, x.detach(), g_wx)
    assert torch.allclose(grad_x, x.grad, atol=1e-12)
    for name in ("W_x.weight", "W_x.bias", "W_b.weight", "W_b.bias"):
        want = dict(cell.named_parameters())[name].grad
        assert torch.allclose(grads[name], want, atol=1e-12), name
    # with the kernel's per-gate sums of g_wx given, the two bias gradients are slices of them
    bias_sum = g_wx.reshape(-1, 20).sum(0)
    with torch.no_grad():
        _, grads2 = _cfc_input_grads(cell, x.detach(), g_wx, bias_sum)
    assert torch.allclose(grads2["W_x.bias"], cell.W_x.bias.grad, atol=1e-12)
    assert torch.allclose(grads2["W_b.bias"], cell.W_b.bias.grad, atol=1e-12)


def test_input_affine_uses_project_wx_when_the_cell_has_one():
    from pararnn_b200.newton import input_affine

    torch.manual_seed(1)
    gru, cfc = prb.ParaGRU(6, 4), prb.ParaCfC(6, 4)
    x = torch.randn(2, 3, 6)
    assert torch.equal(input_affine(gru, x), gru.W_x(x))
    wx = input_affine(cfc, x)
    assert wx.shape == (2, 3, 16)
    assert torch.equal(wx[..., 8:12], x[..., -1:].clamp_min(1e-4).expand(2, 3, 4))
    with pytest.raises(ValueError):
        prb.ParaCfC(1, 4)
    with pytest.raises(ValueError):
        prb.ParaCfC(6, 4, gate_mix="diag_h")
