"""Generate the golden vectors in this directory from the reference itself.

Run in a container that has the reference checked out (it is imported, never
copied):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference/src

For every case the script builds the reference cell, runs the reference's eager
Newton+scan path (``scan_backend="eager"``), its sequential unroll and a backward
pass with a fixed random cotangent, and stores inputs and outputs in one ``.npz``
per case.  The fixtures pin the CPU oracle (``oracle/``) and, through it, the CUDA
kernels.  They are deliberately tiny (a few tens of KB each).
"""

from __future__ import annotations

import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def run_case(name, cell, x, *, K, P=None, h0=None, omega=1.0, cu_seqlens=None):
    from pararnn import NewtonConfig, NewtonStats, newton_apply, sequential_apply

    torch.manual_seed(1234)
    cell.zero_grad(set_to_none=True)
    x = x.clone().requires_grad_(True)
    if h0 is not None:
        h0 = h0.clone().requires_grad_(True)
    st = NewtonStats()
    cfg = NewtonConfig(
        max_iters=K, scan_backend="eager", picard_iters=P, picard_adapt=False, omega=omega,
        residual_atol=1e-30, residual_fail=None,
    )
    cs = None if cu_seqlens is None else torch.tensor(cu_seqlens, dtype=torch.long)
    H = newton_apply(cell, x, cfg, h0=h0, stats=st, cu_seqlens=cs)
    G = torch.randn_like(H)
    (H * G).sum().backward()
    with torch.no_grad():
        if cs is None:
            H_seq = sequential_apply(cell, x.detach(), None if h0 is None else h0.detach())
        else:  # packed: every sequence unrolled on its own from its own h0 row
            H_seq = torch.cat([sequential_apply(cell, x.detach()[:, a:b],
                                                None if h0 is None else h0.detach()[i:i + 1])
                               for i, (a, b) in enumerate(zip(cu_seqlens[:-1], cu_seqlens[1:]))], dim=1)
        project = getattr(cell, "project_wx", None)  # ParaCfC packs (f, c, dt, b)
        wx = project(x.detach()) if callable(project) else cell.W_x(x.detach())
    out = {
        "x": _np(x), "wx": _np(wx), "W": _np(cell.W_x.weight), "b": _np(cell.W_x.bias),
        "H": _np(H), "H_seq": _np(H_seq), "G": _np(G),
        "iters": np.int64(st.iters), "max_residual": np.float64(st.max_residual),
        "history": np.asarray(st.residual_history, dtype=np.float64),
        "K": np.int64(K), "P": np.int64(int(cfg.picard_iters or 0) if P is None else P),
        "omega": np.float64(omega),
        "g_x": _np(x.grad), "g_W": _np(cell.W_x.weight.grad), "g_b": _np(cell.W_x.bias.grad),
    }
    if h0 is not None:
        out["h0"] = _np(h0)
        out["g_h0"] = _np(h0.grad)
    if cs is not None:
        out["cu_seqlens"] = np.asarray(cu_seqlens, dtype=np.int64)
    kind = type(cell).__name__
    if kind == "ParaGRU" and cell.mix == "diag":
        az, ar, an = cell.clipped_a()
        out["params"] = np.stack([_np(az), _np(ar), _np(an)])
        out["raw_params"] = np.stack([_np(cell.a_z), _np(cell.a_r), _np(cell.a_n)])
        out["g_params"] = np.stack([_np(cell.a_z.grad), _np(cell.a_r.grad), _np(cell.a_n.grad)])
        out["cell"] = "gru_diag"
    elif kind == "ParaGRU":
        az, ar, an = cell.clipped_a_head()
        out["params"] = np.stack([_np(az), _np(ar), _np(an)])
        out["raw_params"] = np.stack([_np(cell.A_z), _np(cell.A_r), _np(cell.A_n)])
        out["g_params"] = np.stack([_np(cell.A_z.grad), _np(cell.A_r.grad), _np(cell.A_n.grad)])
        out["n_heads"] = np.int64(cell.n_heads)
        out["cell"] = "gru_head"
    elif kind == "ParaNLRU":
        out["params"] = _np(cell.clipped_u())[None]
        out["raw_params"] = _np(cell.u)[None]
        out["g_params"] = _np(cell.u.grad)[None]
        out["cell"] = "nlru"
    elif kind == "ParaLSTM":
        names = ("a_f", "a_z", "a_o", "c_f", "c_o")
        out["params"] = np.stack([_np(p) for p in cell.clipped_recurrent()])
        out["raw_params"] = np.stack([_np(getattr(cell, n)) for n in names])
        out["g_params"] = np.stack([_np(getattr(cell, n).grad) for n in names])
        out["cell"] = "lstm"
    elif kind == "ParaTitans":
        out["params"] = np.stack([_np(cell.clipped_u()), _np(cell.clipped_r())])
        out["raw_params"] = np.stack([_np(cell.u), _np(cell.r)])
        out["g_params"] = np.stack([_np(cell.u.grad), _np(cell.r.grad)])
        out["cell"] = "titans"
    elif kind == "ParaCfC":
        out["params"] = _np(cell.clipped_u())[None]
        out["raw_params"] = _np(cell.u)[None]
        out["g_params"] = _np(cell.u.grad)[None]
        out["W_b"], out["b_b"] = _np(cell.W_b.weight), _np(cell.W_b.bias)
        out["g_W_b"], out["g_b_b"] = _np(cell.W_b.weight.grad), _np(cell.W_b.bias.grad)
        out["cell"] = "cfc"
    elif kind == "ParaSLSTM":
        out["params"] = _np(cell.clipped_r())
        out["raw_params"] = _np(cell.R)
        out["g_params"] = _np(cell.R.grad)
        out["eps"] = np.float64(cell.eps)
        out["cell"] = "slstm_diag"
    else:
        raise TypeError(kind)
    out["cap"] = np.float64(-1.0 if cell.max_recurrent_norm is None else cell.max_recurrent_norm)
    path = os.path.join(HERE, f"{name}.npz")
    np.savez_compressed(path, **out)
    print(f"{name}: iters={st.iters} hist={tuple(f'{v:.3e}' for v in st.residual_history)} "
          f"res={st.max_residual:.3e} |H-Hseq|={float((H.detach()-H_seq).abs().max()):.3e} "
          f"-> {os.path.getsize(path)/1024:.1f} KB")


def main():
    ref_src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PARARNN_REFERENCE_SRC")
    if not ref_src:
        raise SystemExit("usage: make_golden.py /path/to/reference/src")
    sys.path.insert(0, ref_src)
    warnings.filterwarnings("ignore")
    import logging

    logging.disable(logging.CRITICAL)
    from pararnn import ParaCfC, ParaGRU, ParaLSTM, ParaNLRU, ParaSLSTM, ParaTitans

    torch.set_num_threads(4)

    # --- ParaGRU diag (shape family of the CPU-runnable baseline config) ---
    torch.manual_seed(0)
    cell = ParaGRU(12, 16)
    with torch.no_grad():
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
        cell.a_z.mul_(3.0)  # some entries reach the +-0.5 clamp
    run_case("gru_diag_k3", cell, torch.randn(2, 64, 12), K=3)
    run_case("gru_diag_k2_h0", cell, torch.randn(3, 33, 12), K=2, h0=0.5 * torch.randn(3, 16))
    run_case("gru_diag_t1", cell, torch.randn(2, 1, 12), K=2)

    # --- ParaNLRU ---
    torch.manual_seed(4)
    cell = ParaNLRU(10, 12)
    with torch.no_grad():
        a0 = torch.empty(12).uniform_(0.9, 0.999)
        cell.W_x.bias[:12] = torch.log(a0 / (1 - a0))
        cell.u.mul_(4.0)
    run_case("nlru_k2", cell, torch.randn(2, 96, 10), K=2)
    run_case("nlru_k3_h0_omega", cell, torch.randn(2, 47, 10), K=3, h0=torch.randn(2, 12), omega=0.9)

    # --- ParaSLSTM diag ---
    torch.manual_seed(1)
    cell = ParaSLSTM(8, 8, mix="diag")
    with torch.no_grad():
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
        cell.W_x.bias[8:16] = 3.0
    run_case("slstm_bias3_p5_k2", cell, 0.5 * torch.randn(2, 80, 8), K=2, P=5)
    # stress: Newton has to work (no forget bias, x scale 1, R at the clamp, few Picard passes)
    torch.manual_seed(11)
    cell = ParaSLSTM(8, 8, mix="diag")
    with torch.no_grad():
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
        cell.R.copy_(torch.where(torch.rand(4, 8) > 0.5, 0.7, -0.7))  # clamped to +-0.5
    run_case("slstm_stress_p0_k4", cell, 0.6 * torch.randn(2, 32, 8), K=4, P=0)
    run_case("slstm_stress_p1_k3_h0", cell, torch.randn(2, 40, 8), K=3, P=1,
             h0=torch.stack([0.3 * torch.randn(2, 8), torch.rand(2, 8) + 0.5,
                             0.2 * torch.randn(2, 8), 0.3 * torch.randn(2, 8)], dim=1))
    run_case("slstm_stress_p3_k1", cell, torch.randn(1, 129, 8), K=1, P=3)

    # --- ParaGRU head ---
    torch.manual_seed(2)
    cell = ParaGRU(16, 16, mix="head", n_heads=2)
    with torch.no_grad():
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
        for A in (cell.A_z, cell.A_r, cell.A_n):
            for hd in range(2):
                torch.nn.init.orthogonal_(A[hd], gain=0.9)
    run_case("gru_head_k3", cell, torch.randn(2, 48, 16), K=3)
    run_case("gru_head_k2_h0", cell, torch.randn(2, 17, 16), K=2, h0=0.5 * torch.randn(2, 16))

    # --- packed batches (cu_seqlens): ragged sequences, one of length 1, own h0 per sequence ---
    torch.manual_seed(20)
    cell = ParaGRU(12, 16)
    with torch.no_grad():
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
    run_case("gru_diag_packed_k3_h0", cell, torch.randn(1, 61, 12), K=3, h0=0.5 * torch.randn(4, 16),
             cu_seqlens=[0, 7, 8, 40, 61])
    torch.manual_seed(21)
    cell = ParaNLRU(10, 12)
    with torch.no_grad():
        a0 = torch.empty(12).uniform_(0.9, 0.999)
        cell.W_x.bias[:12] = torch.log(a0 / (1 - a0))
    run_case("nlru_packed_k2", cell, torch.randn(1, 50, 10), K=2, cu_seqlens=[0, 1, 20, 50])
    torch.manual_seed(22)
    cell = ParaSLSTM(8, 8, mix="diag")
    with torch.no_grad():
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
        cell.W_x.bias[8:16] = 1.0
    run_case("slstm_packed_p2_k2_h0", cell, 0.6 * torch.randn(1, 45, 8), K=2, P=2,
             h0=torch.stack([0.3 * torch.randn(3, 8), torch.rand(3, 8) + 0.5,
                             0.2 * torch.randn(3, 8), 0.3 * torch.randn(3, 8)], dim=1),
             cu_seqlens=[0, 16, 17, 45])

    # --- ParaTitans (scalar-diagonal memory cell) ---
    torch.manual_seed(30)
    cell_t = ParaTitans(10, 12)
    with torch.no_grad():
        cell_t.u.mul_(5.0)  # some entries reach the +-0.5 clamp
        cell_t.r.mul_(5.0)
    run_case("titans_k3", cell_t, torch.randn(2, 70, 10), K=3)
    run_case("titans_k2_h0_omega", cell_t, torch.randn(2, 41, 10), K=2, h0=0.5 * torch.randn(2, 12), omega=0.9)
    run_case("titans_packed_k3_h0", cell_t, torch.randn(1, 37, 10), K=3, h0=0.5 * torch.randn(3, 12),
             cu_seqlens=[0, 1, 15, 37])

    # --- ParaLSTM (CIFG peephole LSTM, state (c, h), 2x2 block Jacobian) ---
    torch.manual_seed(40)
    cell_l = ParaLSTM(10, 12)
    with torch.no_grad():
        for p in (cell_l.a_f, cell_l.a_z, cell_l.a_o, cell_l.c_f, cell_l.c_o):
            p.mul_(4.0)  # some entries reach the +-0.5 clamp
    run_case("lstm_k3", cell_l, torch.randn(2, 72, 10), K=3)
    run_case("lstm_k2_h0_omega", cell_l, torch.randn(2, 35, 10), K=2, h0=0.5 * torch.randn(2, 2, 12), omega=0.9)
    run_case("lstm_packed_k3_h0", cell_l, torch.randn(1, 40, 10), K=3, h0=0.5 * torch.randn(3, 2, 12),
             cu_seqlens=[0, 9, 10, 40])

    # --- ParaCfC (irregular time steps in the last input channel, gate_mix='input') ---
    torch.manual_seed(50)
    cell_c = ParaCfC(11, 12)
    with torch.no_grad():
        cell_c.u.mul_(5.0)  # some entries reach the +-0.5 clamp
        cell_c.W_b.weight.normal_(0.0, 0.3)  # the default zero weight would leave b constant
        cell_c.W_b.bias.fill_(-1.0)

    def cfc_x(b, t):
        x = torch.randn(b, t, 11)
        x[..., -1] = 2.0 * torch.rand(b, t)  # time steps
        x[:, ::7, -1] = 0.0  # below the clamp: dt = 1e-4 and no gradient to dt
        return x

    run_case("cfc_k3", cell_c, cfc_x(2, 66), K=3)
    run_case("cfc_k2_h0_omega", cell_c, cfc_x(2, 39), K=2, h0=0.5 * torch.randn(2, 12), omega=0.9)
    run_case("cfc_packed_k3_h0", cell_c, cfc_x(1, 38), K=3, h0=0.5 * torch.randn(3, 12), cu_seqlens=[0, 1, 14, 38])


if __name__ == "__main__":
    main()
