"""``decode_step`` (T = 1, one launch) against the cells' own PyTorch ``step``: dense batch, ``out=``,
pool + ``block_table`` updated in place, and a decode loop captured in a CUDA graph."""

import pytest
import torch

import pararnn_b200 as prb

pytestmark = pytest.mark.gpu


def _cell(kind, d_in=24, d=96):
    torch.manual_seed(0)
    cell = {"gru": prb.ParaGRU, "nlru": prb.ParaNLRU, "slstm": prb.ParaSLSTM}[kind](d_in, d).cuda()
    with torch.no_grad():  # push some recurrent weights past the clamp so the in-kernel clamp matters
        for name in ("a_z", "a_r", "a_n", "u", "R"):
            if hasattr(cell, name):
                getattr(cell, name).mul_(6.0)
    return cell.eval()


def _state(kind, B, d, dtype=torch.float32):
    if kind == "slstm":
        s = 0.3 * torch.randn(B, 4, d, device="cuda")
        s[:, 1] = s[:, 1].abs() + 0.5
        return s.to(dtype)
    return (0.5 * torch.randn(B, d, device="cuda")).to(dtype)


@pytest.mark.parametrize("kind", ["gru", "nlru", "slstm"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_step_matches_cell_step(kind, dtype):
    cell = _cell(kind).to(dtype)
    B, d = 5, 96
    state = _state(kind, B, d, dtype)
    x = torch.randn(B, 24, device="cuda", dtype=dtype)
    with torch.no_grad():
        assert prb.can_decode_step(cell, x)
        want = cell.float().step(state.float(), x.float())
        cell.to(dtype)
        got = prb.decode_step(cell, state, x)
        tol = 2e-6 if dtype == torch.float32 else 3e-2
        assert float((got.float() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
        # out= and precomputed wx, (B, 1, d_in) input
        out = torch.empty_like(state)
        wx = prb.decode_wx(cell, x[:, None])
        assert prb.decode_step(cell, state, wx=wx, out=out) is out
        assert torch.equal(out, got)
        # sequential_apply with T = 1 takes the same kernel
        assert torch.equal(prb.sequential_apply(cell, x[:, None], state)[:, 0], got)


@pytest.mark.parametrize("kind", ["gru", "slstm"])
def test_block_table_updates_pool_rows_in_place(kind):
    cell = _cell(kind)
    d = 96
    pool = _state(kind, 9, d)
    before = pool.clone()
    table = torch.tensor([7, 2, 4], device="cuda")
    x = torch.randn(3, 24, device="cuda")
    with torch.no_grad():
        want = cell.step(before[table], x)
        ret = prb.decode_step(cell, pool, x, block_table=table)
    assert ret is pool
    assert float((pool[table] - want).abs().max()) <= 2e-6 * max(1.0, float(want.abs().max()))
    untouched = [i for i in range(9) if i not in (7, 2, 4)]
    assert torch.equal(pool[untouched], before[untouched])
    with pytest.raises(RuntimeError):
        prb.decode_step(cell.cpu(), before.cpu(), x.cpu(), block_table=table.cpu())


def test_decode_loop_in_a_cuda_graph():
    cell = _cell("slstm")
    B, d, steps = 4, 96, 16
    xs = torch.randn(steps, B, 24, device="cuda")
    x_static = torch.zeros(B, 24, device="cuda")
    wx_static = torch.zeros(B, 4 * d, device="cuda")
    state = [torch.zeros(B, 4, d, device="cuda"), torch.zeros(B, 4, d, device="cuda")]
    with torch.no_grad():
        prb.decode_step(cell, state[0], wx=prb.decode_wx(cell, x_static, out=wx_static), out=state[1])  # warm up
        state[0].zero_()
        state[1].zero_()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):  # two steps per replay: state 0 -> 1 -> 0
            prb.decode_step(cell, state[0], wx=prb.decode_wx(cell, x_static, out=wx_static), out=state[1])
            prb.decode_step(cell, state[1], wx=wx_static, out=state[0])
        state[0].zero_()
        state[1].zero_()
        want = torch.zeros(B, 4, d, device="cuda")
        for t in range(steps):
            x_static.copy_(xs[t])
            g.replay()
            want = cell.step(cell.step(want, xs[t]), xs[t])
    assert float((state[0] - want).abs().max()) <= 1e-5 * max(1.0, float(want.abs().max()))
