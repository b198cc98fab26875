"""Time-sharded solve on ONE GPU: the programs of 2-4 virtual ranks run in lockstep in one
process (no kernel waits on another rank), and the result must match the unsharded kernels."""

import numpy as np
import pytest
import torch

from gpu_util import dev, make_problem, rel_err
from oracle import oracle

pytestmark = pytest.mark.gpu


def _rec(kind, params):
    if kind == "slstm_diag":
        return (dev(params),)
    return tuple(dev(p) for p in params)


@pytest.mark.parametrize("kind,K,P", [("gru_diag", 3, 0), ("nlru", 2, 0), ("slstm_diag", 2, 3)])
@pytest.mark.parametrize("world,T", [(2, 257), (3, 100), (4, 1024)])
@pytest.mark.parametrize("path", ["lookback", "pipe"])
def test_sharded_matches_oracle(kind, K, P, world, T, path, prb_options):
    from pararnn_b200.seq_shard import _bits_to_stats, emulate_sharded

    prb_options("kernel_family", path)
    B, d = 2, 40
    wx, params, h0 = make_problem(kind, B, T, d, seed=T + world, h0=True, x_scale=0.6, bias_f=1.0)
    want = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=K, picard=P)
    G = np.random.default_rng(1).standard_normal(want.states.shape).astype(np.float32)
    states, bits, grads = emulate_sharded(kind, dev(wx), _rec(kind, params), world=world, K=K, P=P,
                                          h0=dev(h0), grad_states=dev(G))
    H = states.cpu().numpy()
    amp = max(1.0, max(want.history))
    scale = max(1.0, float(np.abs(want.states).max()))
    assert np.abs(H - want.states).max() <= 1e-5 * amp * scale
    hist, final, status = _bits_to_stats(bits, K)
    assert status == 0
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=2e-2, atol=4e-6 * scale)
    assert abs(final - want.max_residual) <= 2e-2 * want.max_residual + 4e-6 * scale * amp
    # backward at the sharded trajectory
    w_wx, w_p, w_h0 = oracle.backward(oracle.KIND[kind], H, wx, params, G, h0)
    g_wx, g_p, g_h0 = grads
    assert rel_err(g_wx.cpu().numpy(), w_wx) <= 5e-5
    assert rel_err(g_p.cpu().numpy().reshape(-1), w_p.reshape(-1)) <= 1e-4
    assert rel_err(g_h0.cpu().numpy().reshape(w_h0.shape), w_h0) <= 5e-5


def test_sharded_equals_unsharded_bf16():
    from pararnn_b200 import ops
    from pararnn_b200.seq_shard import emulate_sharded

    wx, r, _ = make_problem("slstm_diag", 2, 2048, 64, seed=5, x_scale=0.5, bias_f=3.0)
    wxd, rd = dev(wx, torch.bfloat16), dev(r, torch.bfloat16)
    one = ops.newton_slstm_fused(wxd, rd, None, None, max_iters=2, picard_iters=5)
    many, _ = emulate_sharded("slstm_diag", wxd, (rd,), world=4, K=2, P=5)
    assert rel_err(many[:, :, 3].float().cpu().numpy(), one[:, :, 3].float().cpu().numpy()) <= 2e-2


@pytest.mark.parametrize("kind,K,P", [("slstm_diag", 2, 3), ("gru_diag", 3, 0), ("nlru", 2, 0)])
def test_unequal_shards_match_oracle(kind, K, P, prb_options):
    """The first rank sweeps once per pass, the others twice, so a balanced split gives the first
    rank a longer shard; the programs make no assumption on shard lengths."""
    from pararnn_b200.seq_shard import _bits_to_stats, emulate_sharded

    prb_options("kernel_family", "pipe")
    B, T, d = 2, 1000, 64
    bounds = [(0, 470), (470, 730), (730, 731), (731, 1000)]
    wx, params, h0 = make_problem(kind, B, T, d, seed=17, h0=True, x_scale=0.6, bias_f=1.0)
    want = oracle.newton(oracle.KIND[kind], wx, params, h0, max_iters=K, picard=P)
    G = np.random.default_rng(2).standard_normal(want.states.shape).astype(np.float32)
    states, bits, grads = emulate_sharded(kind, dev(wx), _rec(kind, params), world=4, K=K, P=P, h0=dev(h0),
                                          grad_states=dev(G), bounds=bounds)
    amp = max(1.0, max(want.history))
    scale = max(1.0, float(np.abs(want.states).max()))
    assert np.abs(states.cpu().numpy() - want.states).max() <= 1e-5 * amp * scale
    assert _bits_to_stats(bits, K)[2] == 0
    want_g = oracle.backward(oracle.KIND[kind], states.cpu().numpy(), wx, params, G, h0)
    assert rel_err(grads[0].cpu().numpy(), want_g[0]) <= 5e-5
    assert rel_err(grads[1].cpu().numpy().reshape(-1), np.asarray(want_g[1]).reshape(-1)) <= 1e-4


@pytest.mark.parametrize("world,segments,T", [(1, 3, 1000), (2, 2, 777), (3, 5, 2050), (2, 4, 131)])
def test_time_segments_match_oracle(world, segments, T, prb_options):
    """ParaSLSTM passes with the shard of every rank cut into time segments that are swept by
    different thread blocks (aggregate sweep, device-side fold, apply sweep with per-segment
    carries): same result as the oracle's unsharded solve, forward and backward."""
    from pararnn_b200.seq_shard import _bits_to_stats, emulate_sharded

    prb_options("kernel_family", "pipe")
    B, d, K, P = 2, 64, 2, 3
    wx, params, h0 = make_problem("slstm_diag", B, T, d, seed=T + segments, h0=True, x_scale=0.6, bias_f=1.0)
    want = oracle.newton(oracle.SLSTM_DIAG, wx, params, h0, max_iters=K, picard=P)
    G = np.random.default_rng(4).standard_normal(want.states.shape).astype(np.float32)
    states, bits, grads = emulate_sharded("slstm_diag", dev(wx), (dev(params),), world=world, K=K, P=P,
                                          h0=dev(h0), grad_states=dev(G), segments=segments)
    amp = max(1.0, max(want.history))
    scale = max(1.0, float(np.abs(want.states).max()))
    assert np.abs(states.cpu().numpy() - want.states).max() <= 1e-5 * amp * scale
    hist, final, status = _bits_to_stats(bits, K)
    assert status == 0
    np.testing.assert_allclose(np.asarray(hist), np.asarray(want.history), rtol=2e-2, atol=4e-6 * scale)
    want_g = oracle.backward(oracle.SLSTM_DIAG, states.cpu().numpy(), wx, params, G, h0)
    assert rel_err(grads[0].cpu().numpy(), want_g[0]) <= 5e-5
    assert rel_err(grads[1].cpu().numpy().reshape(-1), np.asarray(want_g[1]).reshape(-1)) <= 1e-4
    assert rel_err(grads[2].cpu().numpy().reshape(want_g[2].shape), want_g[2]) <= 5e-5


def test_segment_plan_and_argument_checks():
    import ctypes

    from pararnn_b200 import _lib

    lib = _lib.lib()
    n, ln = ctypes.c_int(0), ctypes.c_int(0)
    # few chains, long shard: several segments that tile T exactly once
    assert lib.prb_plan_segments(_lib.CELL_SLSTM_DIAG, _lib.PRB_BF16, 1, 16384, 2048, ctypes.byref(n),
                                 ctypes.byref(ln)) == 0
    assert n.value > 1 and (n.value - 1) * ln.value < 16384 <= n.value * ln.value
    # enough chains to fill the GPU: one segment
    assert lib.prb_plan_segments(_lib.CELL_SLSTM_DIAG, _lib.PRB_BF16, 8, 16384, 2048, ctypes.byref(n),
                                 ctypes.byref(ln)) == 0
    assert (n.value, ln.value) == (1, 16384)
    # a segment layout that does not cover T is refused before anything is launched
    one = torch.zeros(64, device="cuda")
    p = ctypes.c_void_p(one.data_ptr())
    rc = lib.prb_slstm_newton_pass(p, p, p, None, None, p, None, None, 0, 3, 100, 1, 1000, 32, _lib.PRB_F32, 1.0,
                                   1e-6, p, 256, p, 0, None)
    assert rc == -1


def test_graphed_step_replays_with_new_inputs(prb_options):
    """The forward + backward programs captured into a CUDA graph (one-rank NCCL group, three time
    segments so that the device-side folds are part of it): a replay after new inputs were written
    into the static buffers gives what the eager programs give for those inputs."""
    import socket

    import torch.distributed as dist

    from pararnn_b200.seq_shard import DistComm, GraphedShardedStep, emulate_sharded

    prb_options("kernel_family", "pipe")
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                            device_id=torch.device("cuda", 0))
    try:
        B, T, d, K, P = 2, 700, 64, 2, 2
        wx1, r, _ = make_problem("slstm_diag", B, T, d, seed=1, x_scale=0.6, bias_f=1.0)
        wx2, _, _ = make_problem("slstm_diag", B, T, d, seed=2, x_scale=0.6, bias_f=1.0)
        G1 = np.random.default_rng(5).standard_normal((B, T, 4, d)).astype(np.float32)
        G2 = np.random.default_rng(6).standard_normal((B, T, 4, d)).astype(np.float32)
        wx_s, G_s = dev(wx1), dev(G1)
        gs = GraphedShardedStep("slstm_diag", wx_s, (dev(r),), G_s, DistComm(), K=K, P=P, segments=3)
        assert gs.ops.n_seg == 3
        for wx, G in ((wx1, G1), (wx2, G2), (wx1, G1)):
            gs.wx.copy_(dev(wx))
            gs.grad_states.copy_(dev(G))
            gs.replay()
            torch.cuda.synchronize()
            states, _, grads = emulate_sharded("slstm_diag", dev(wx), (dev(r),), world=1, K=K, P=P,
                                               grad_states=dev(G), segments=3)
            assert torch.equal(gs.states, states)
            assert torch.equal(gs.g_wx, grads[0]) and torch.equal(gs.g_params, grads[1])
    finally:
        dist.destroy_process_group()
