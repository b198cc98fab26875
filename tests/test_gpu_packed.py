"""Packed batches (``cu_seqlens``) and paged initial states (``block_table``) through the
operators and through ``newton_apply``: every sequence of the pack is its own scan, so the result
must equal the oracle run sequence by sequence (and the reference's own packed eager solve, which
the ``*_packed_*`` golden fixtures hold)."""

import numpy as np
import pytest
import torch

import pararnn_b200 as prb
from golden_util import golden_names, load_golden, oracle_calls
from gpu_util import dev, make_problem, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu

PACKED = [n for n in golden_names() if "packed" in n]


def _fwd(kind, wx, params, h0, cs, K, P=0, eps=1e-6):
    from pararnn_b200 import ops

    st = ops.DeviceStats("cuda", K)
    csd = torch.tensor(cs, device="cuda")
    if kind == "gru_diag":
        H = ops.newton_gru_fused(dev(wx), *[dev(p) for p in params], dev(h0), csd, max_iters=K, stats=st)
    elif kind == "nlru":
        H = ops.newton_nlru_fused(dev(wx), dev(params[0]), dev(h0), csd, max_iters=K, stats=st)
    elif kind == "titans":
        H = ops.newton_titans_fused(dev(wx), dev(params[0]), dev(params[1]), dev(h0), csd, max_iters=K, stats=st)
    elif kind == "cfc":
        H = ops.newton_cfc_fused(dev(wx), dev(params[0]), dev(h0), csd, max_iters=K, stats=st)
    elif kind == "lstm":
        H = ops.newton_lstm_fused(dev(wx), *[dev(p) for p in params], dev(h0), csd, max_iters=K, stats=st)
    else:
        H = ops.newton_slstm_fused(dev(wx), dev(params), dev(h0), max_iters=K, picard_iters=P, eps=eps,
                                   stats=st, cu_seqlens=csd)
    hist, res, status = st.read()
    assert status == 0
    return H.cpu().numpy(), np.asarray(hist), res


def test_fixtures_present():
    assert len(PACKED) == 6


@pytest.mark.parametrize("name", PACKED)
def test_packed_forward_matches_reference_golden(name):
    g = load_golden(name)
    H, hist, res = _fwd(g["cell"], g["wx"], g["params"], g["h0"], list(g["cu_seqlens"]), g["K"], g["P"], g["eps"])
    amp = max(1.0, float(np.max(g["history"])))
    scale = max(1.0, float(np.abs(g["H"]).max()))
    assert np.abs(H - g["H"]).max() <= 1e-5 * amp * scale
    np.testing.assert_allclose(hist, g["history"], rtol=1e-2, atol=4e-6 * scale)
    assert abs(res - float(g["max_residual"])) <= 1e-2 * float(g["max_residual"]) + 4e-6 * scale * amp


@pytest.mark.parametrize("kind,P", [("gru_diag", 0), ("nlru", 0), ("titans", 0), ("cfc", 0), ("lstm", 0),
                                    ("slstm_diag", 2)])
@pytest.mark.parametrize("cs", [[0, 1, 2, 3], [0, 300, 301, 1000], [0, 64, 128, 129, 700]])
def test_packed_matches_oracle_forward_and_backward(kind, P, cs):
    d, K = 40, 2
    N, S = cs[-1], len(cs) - 1
    wx, params, _ = make_problem(kind, 1, N, d, seed=N + S, x_scale=0.6, bias_f=1.0)
    _, _, h0 = make_problem(kind, S, 1, d, seed=5, h0=True)
    want = oracle.newton_packed(oracle.KIND[kind], wx, params, h0, cs, max_iters=K, picard=P)
    H, hist, res = _fwd(kind, wx, params, h0, cs, K, P)
    amp = max(1.0, max(want.history))
    scale = max(1.0, float(np.abs(want.states).max()))
    assert np.abs(H - want.states).max() <= 1e-5 * amp * scale
    np.testing.assert_allclose(hist, np.asarray(want.history), rtol=2e-2, atol=4e-6 * scale)
    # backward through newton_apply: grads of a packed call = grads of the per-sequence calls
    torch.manual_seed(3)
    cls = {"gru_diag": prb.ParaGRU, "nlru": prb.ParaNLRU, "titans": prb.ParaTitans, "cfc": prb.ParaCfC,
           "lstm": prb.ParaLSTM,
           "slstm_diag": prb.ParaSLSTM}[kind]
    cell = cls(24, d).cuda()
    x = torch.randn(1, N, 24, device="cuda")
    if kind == "cfc":
        x[..., -1] = 2.0 * torch.rand(1, N, device="cuda")  # time steps; a few below the clamp
        x[:, ::5, -1] = 0.0
    x.requires_grad_(True)
    h0t = dev(h0).requires_grad_(True)
    cfg = prb.NewtonConfig(max_iters=3, picard_iters=P if kind == "slstm_diag" else None, picard_adapt=False)
    G = torch.randn(1, N, *({"slstm_diag": (4, d), "lstm": (2, d)}.get(kind, (d,))), device="cuda")
    Hp = prb.newton_apply(cell, x, cfg, h0=h0t, cu_seqlens=torch.tensor(cs, device="cuda"))
    (Hp * G).sum().backward()
    got = [x.grad.clone(), h0t.grad.clone()] + [p.grad.clone() for p in cell.parameters()]
    x.grad = None
    h0t.grad = None
    cell.zero_grad(set_to_none=True)
    loss = 0
    for i, (a, b) in enumerate(zip(cs[:-1], cs[1:])):
        Hs = prb.newton_apply(cell, x[:, a:b], cfg, h0=h0t[i:i + 1])
        # not bit-equal: the W_x GEMM of a slice may round differently from the GEMM of the pack
        assert torch.allclose(Hs, Hp[:, a:b], atol=5e-6, rtol=1e-5)
        loss = loss + (Hs * G[:, a:b]).sum()
    loss.backward()
    want_g = [x.grad, h0t.grad] + [p.grad for p in cell.parameters()]
    for a, b in zip(got, want_g):
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) <= 2e-5


@pytest.mark.parametrize("kind", ["gru_diag", "nlru", "slstm_diag"])
def test_block_table_selects_pool_rows(kind):
    from pararnn_b200 import ops

    B, T, d = 3, 200, 32
    wx, params, _ = make_problem(kind, B, T, d, seed=2)
    _, _, pool = make_problem(kind, 7, 1, d, seed=9, h0=True)
    table = torch.tensor([5, 0, 5], device="cuda", dtype=torch.int32)
    dense = pool[[5, 0, 5]]
    if kind == "gru_diag":
        a = ops.newton_gru_fused(dev(wx), *[dev(p) for p in params], dev(pool), None, table, max_iters=2)
        b = ops.newton_gru_fused(dev(wx), *[dev(p) for p in params], dev(dense), max_iters=2)
    elif kind == "nlru":
        a = ops.newton_nlru_fused(dev(wx), dev(params[0]), dev(pool), None, table, max_iters=2)
        b = ops.newton_nlru_fused(dev(wx), dev(params[0]), dev(dense), max_iters=2)
    else:
        a = ops.newton_slstm_fused(dev(wx), dev(params), dev(pool), None, table, max_iters=2, picard_iters=1)
        b = ops.newton_slstm_fused(dev(wx), dev(params), dev(dense), max_iters=2, picard_iters=1)
    assert torch.equal(a, b)
    with pytest.raises(ValueError, match="outside pool capacity"):
        ops.gather_h0(dev(pool), torch.tensor([0, 1, 9], device="cuda"), 3, tuple(pool.shape[1:]))


def test_newton_apply_block_table_is_inference_only_and_packed_checks():
    cell = prb.ParaGRU(8, 16).cuda()
    x = torch.randn(2, 10, 8, device="cuda")
    pool = torch.randn(4, 16, device="cuda")
    table = torch.tensor([3, 1], device="cuda")
    with pytest.raises(RuntimeError, match="inference-only"):
        prb.newton_apply(cell, x, prb.NewtonConfig(max_iters=2), h0=pool, block_table=table)
    with torch.no_grad():
        a = prb.newton_apply(cell, x, prb.NewtonConfig(max_iters=2), h0=pool, block_table=table)
        b = prb.newton_apply(cell, x, prb.NewtonConfig(max_iters=2), h0=pool[[3, 1]])
    assert torch.equal(a, b)
    with pytest.raises(ValueError, match="batch=1"):
        prb.newton_apply(cell, x, cu_seqlens=torch.tensor([0, 4, 10], device="cuda"))
    with torch.no_grad(), pytest.raises(ValueError, match="strictly increasing"):
        prb.newton_apply(cell, x[:1], cu_seqlens=torch.tensor([0, 4, 4, 10], device="cuda"))
    head = prb.ParaGRU(16, 16, mix="head", n_heads=2).cuda()
    with torch.no_grad(), pytest.raises(TypeError):
        prb.newton_apply(head, torch.randn(1, 10, 16, device="cuda"),
                         cu_seqlens=torch.tensor([0, 4, 10], device="cuda"))
