"""The most literal drop-in test: the UNMODIFIED reference package drives this backend.

With a copy of the reference under ``oracle/_ref`` (``python oracle/make_ref.py``, git-ignored),
the reference is imported next to ``pararnn_b200``, ``pararnn_b200.shim.install()`` swaps its fused
forward dispatcher and its eq.-2.6 backward for this library's kernels, and the reference's own
``newton_apply(scan_backend="fused")`` + ``backward()`` must agree with the reference's own
``scan_backend="eager"`` on the same CUDA tensors.  Skipped when ``oracle/_ref`` is absent."""

import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(os.path.dirname(HERE), "oracle", "_ref")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "pararnn")),
                                 reason="no copy of the reference under oracle/_ref")]


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, REF)
    try:
        import logging

        import pararnn

        logging.getLogger("pararnn").setLevel(logging.CRITICAL)
        from pararnn_b200 import shim

        shim.install()
        yield pararnn
        shim.uninstall()
    finally:
        sys.path.remove(REF)


def _cells(p):
    torch.manual_seed(0)
    gru = p.ParaGRU(24, 32)
    nlru = p.ParaNLRU(24, 32)
    with torch.no_grad():
        a0 = torch.empty(32).uniform_(0.9, 0.999)
        nlru.W_x.bias[:32] = torch.log(a0 / (1 - a0))
    slstm = p.ParaSLSTM(24, 32, mix="diag")
    with torch.no_grad():
        slstm.W_x.bias[32:64] = 1.0
    head = p.ParaGRU(32, 32, mix="head", n_heads=2)
    with torch.no_grad():
        for A in (head.A_z, head.A_r, head.A_n):
            for hd in range(2):
                torch.nn.init.orthogonal_(A[hd], gain=0.9)
    c1 = p.ParaGRU(64, 64)
    torch.nn.init.xavier_uniform_(c1.W_x.weight)
    titans, lstm, cfc = p.ParaTitans(24, 32), p.ParaLSTM(24, 32), p.ParaCfC(24, 32)
    with torch.no_grad():
        cfc.W_b.weight.normal_(0.0, 0.3)
    return {"titans": (titans, (2, 180, 24), 3, None), "lstm": (lstm, (2, 160, 24), 3, None),
            "cfc": (cfc, (2, 170, 24), 3, None),
            "gru_diag": (gru, (2, 200, 24), 3, None), "nlru": (nlru, (2, 300, 24), 3, None),
            "slstm_diag": (slstm, (2, 150, 24), 3, 3), "gru_head": (head, (2, 100, 32), 3, None),
            "c1_gru_diag_B2_T1024_d64": (c1, (2, 1024, 64), 3, None)}


@pytest.mark.parametrize("name", ["gru_diag", "nlru", "slstm_diag", "gru_head", "titans", "lstm", "cfc",
                                  "c1_gru_diag_B2_T1024_d64"])
@pytest.mark.parametrize("with_h0", [False, True])
def test_reference_newton_apply_through_this_backend(ref, name, with_h0):
    p = ref
    cell, shape, K, P = _cells(p)[name]
    cell = cell.cuda()
    torch.manual_seed(1)
    x0 = torch.randn(*shape, device="cuda") * (0.6 if name == "slstm_diag" else 1.0)
    if name == "cfc":
        x0[..., -1] = 2.0 * torch.rand(shape[:2], device="cuda")  # the last channel is the time step
    slots = {"slstm_diag": 4, "lstm": 2}.get(name)
    state_shape = (shape[0], cell.d_h) if slots is None else (shape[0], slots, cell.d_h)
    h00 = None
    if with_h0:
        h00 = 0.3 * torch.randn(*state_shape, device="cuda")
        if name == "slstm_diag":
            h00[:, 1] = h00[:, 1].abs() + 0.5
    results = {}
    for backend in ("eager", "fused"):
        cell.zero_grad(set_to_none=True)
        x = x0.clone().requires_grad_(True)
        h0 = None if h00 is None else h00.clone().requires_grad_(True)
        st = p.NewtonStats()
        cfg = p.NewtonConfig(max_iters=K, scan_backend=backend, picard_iters=P, picard_adapt=False,
                             residual_atol=None, residual_fail=None)
        H = p.newton_apply(cell, x, cfg, h0=h0, stats=st)
        G = torch.randn(H.shape, device="cuda", generator=torch.Generator("cuda").manual_seed(5))
        (H * G).sum().backward()
        results[backend] = dict(H=H.detach(), gx=x.grad, gh0=None if h0 is None else h0.grad,
                                gp={n: q.grad for n, q in cell.named_parameters()}, res=st.max_residual,
                                backend=st.scan_backend)
    a, b = results["eager"], results["fused"]
    assert b["backend"] == "fused"
    scale = max(1.0, float(a["H"].abs().max()))
    assert float((a["H"] - b["H"]).abs().max()) <= 2e-5 * scale
    assert abs(a["res"] - b["res"]) <= 1e-2 * abs(a["res"]) + 1e-5 * scale

    def close(u, v, what):
        tol = 5e-4 * max(1.0, float(u.abs().max()))
        assert float((u - v).abs().max()) <= tol, what

    close(a["gx"], b["gx"], "grad_x")
    if with_h0:
        close(a["gh0"], b["gh0"], "grad_h0")
    for n in a["gp"]:
        close(a["gp"][n], b["gp"][n], n)


def test_unsupported_cells_fall_through_to_the_reference(ref):
    p = ref
    if not hasattr(p, "ParaLSTM"):
        pytest.skip("reference without ParaLSTM")
    torch.manual_seed(0)
    cell = p.ParaLSTM(8, 16).cuda()
    x = torch.randn(1, 20, 8, device="cuda")
    cfg = p.NewtonConfig(max_iters=2, scan_backend="eager")
    with torch.no_grad():
        H = p.newton_apply(cell, x, cfg)
    assert torch.isfinite(H).all()
