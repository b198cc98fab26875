"""World-size-2 and -3 gloo runs (CPU processes) of the time-sharded driver: same generator
programs and the same DistComm as on GPUs, with a CPU stand-in for the local kernels; the
gathered result must equal the oracle's unsharded solve."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, out_dir, first_weight, kind="gru_diag", K=3, P=0):
    sys.path[:0] = [HERE, os.path.dirname(HERE), os.path.join(os.path.dirname(HERE), "pararnn-torch_b200")]
    import torch.distributed as dist

    from cpu_shard_ops import CpuShardOps
    from gpu_util import make_problem
    from pararnn_b200.seq_shard import (DistComm, backward_program, balanced_shard_bounds, drive,
                                        forward_program, time_shard_bounds)

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        wx, params, h0 = _problem(kind, T)
        s, e = (time_shard_bounds(T, rank, world) if first_weight is None
                else balanced_shard_bounds(T, rank, world, first_weight))
        comm = DistComm()
        rec = [torch.from_numpy(p) for p in params] if kind == "gru_diag" else [torch.from_numpy(params)]
        ops = CpuShardOps(kind, torch.from_numpy(wx[:, s:e]), rec, 1e-6, 1.0)
        res = drive(forward_program(ops, rank, world, K, P, torch.from_numpy(h0).double()), comm)
        shape = (2, T, 6) if kind == "gru_diag" else (2, T, 4, 6)
        G = torch.from_numpy(np.random.default_rng(3).standard_normal(shape).astype(np.float32))
        g_wx, g_par, head = drive(backward_program(ops, rank, world, res.states, G[:, s:e], res.halo), comm)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), H=res.states.numpy(), bits=res.stats_bits.numpy(),
                 g_wx=g_wx.numpy(), g_par=g_par.numpy(), head=head.numpy())
    finally:
        dist.destroy_process_group()


def _problem(kind, T):
    from gpu_util import make_problem

    if kind == "gru_diag":
        return make_problem("gru_diag", 2, T, 6, seed=7, h0=True)
    return make_problem("slstm_diag", 2, T, 6, seed=11, h0=True, x_scale=0.6, bias_f=1.0)


@pytest.mark.parametrize("world,T,P,K", [(2, 19, 2, 2), (3, 25, 1, 1), (3, 7, 3, 2)])
def test_sharded_slstm_over_gloo(world, T, P, K, tmp_path):
    """The sLSTM protocol across real processes: Picard gather slots that also ship the output-gate
    pre-activation of the rank's last step, halos derived from the folded carries, 4x4 maps."""
    from oracle import oracle
    from pararnn_b200.seq_shard import _bits_to_stats

    mp.spawn(_worker, args=(world, _free_port(), T, str(tmp_path), None, "slstm_diag", K, P), nprocs=world,
             join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    wx, params, h0 = _problem("slstm_diag", T)
    want = oracle.newton(oracle.SLSTM_DIAG, wx, params, h0, max_iters=K, picard=P)
    H = np.concatenate([p["H"] for p in parts], axis=1)
    amp = max(1.0, max(want.history))
    scale = max(1.0, float(np.abs(want.states).max()))
    assert np.abs(H - want.states).max() <= 2e-5 * amp * scale
    for p in parts:
        hist, final, status = _bits_to_stats(torch.from_numpy(p["bits"]), K)
        np.testing.assert_allclose(hist, want.history, rtol=2e-2, atol=4e-6 * scale)
        assert status == 0
    G = np.random.default_rng(3).standard_normal((2, T, 4, 6)).astype(np.float32)
    w_wx, w_p, w_h0 = oracle.backward(oracle.SLSTM_DIAG, H.astype(np.float32), wx, params, G, h0)
    g_wx = np.concatenate([p["g_wx"] for p in parts], axis=1)
    assert np.abs(g_wx - w_wx).max() <= 1e-4 * max(1.0, np.abs(w_wx).max())
    for p in parts:
        assert np.abs(p["g_par"].reshape(-1) - w_p.reshape(-1)).max() <= 1e-4 * max(1, np.abs(w_p).max())
    assert np.abs(parts[0]["head"].reshape(w_h0.shape) - w_h0).max() <= 1e-4 * max(1.0, np.abs(w_h0).max())


@pytest.mark.parametrize("world,T,first_weight", [(2, 17, None), (3, 20, None), (3, 23, 2.0)])
def test_sharded_driver_over_gloo(world, T, first_weight, tmp_path):
    from gpu_util import make_problem
    from oracle import oracle
    from pararnn_b200.seq_shard import _bits_to_stats

    mp.spawn(_worker, args=(world, _free_port(), T, str(tmp_path), first_weight), nprocs=world, join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    wx, params, h0 = _problem("gru_diag", T)
    want = oracle.newton(oracle.GRU_DIAG, wx, params, h0, max_iters=3)
    H = np.concatenate([p["H"] for p in parts], axis=1)
    assert np.abs(H - want.states).max() <= 2e-5
    for p in parts:  # every rank sees the reduced statistics
        hist, final, status = _bits_to_stats(torch.from_numpy(p["bits"]), 3)
        np.testing.assert_allclose(hist, want.history, rtol=1e-3, atol=1e-6)
        assert status == 0 and abs(final - want.max_residual) <= 1e-3 * want.max_residual + 1e-6
    G = np.random.default_rng(3).standard_normal((2, T, 6)).astype(np.float32)
    w_wx, w_p, w_h0 = oracle.backward(oracle.GRU_DIAG, H, wx, params, G, h0)
    assert np.abs(np.concatenate([p["g_wx"] for p in parts], axis=1) - w_wx).max() <= 1e-4
    for p in parts:
        assert np.abs(p["g_par"].reshape(-1) - w_p.reshape(-1)).max() <= 1e-4 * max(1, np.abs(w_p).max())
    assert np.abs(parts[0]["head"][:, 0] - w_h0).max() <= 1e-4


def test_time_shard_bounds_match_reference_convention():
    from pararnn_b200.seq_shard import time_shard_bounds

    assert [time_shard_bounds(17, r, 4) for r in range(4)] == [(0, 4), (4, 8), (8, 12), (12, 17)]
    with pytest.raises(ValueError):
        time_shard_bounds(8, 4, 4)


def test_balanced_shard_bounds():
    from pararnn_b200.seq_shard import balanced_shard_bounds

    b = [balanced_shard_bounds(32768, r, 2, 1.8, 64) for r in range(2)]
    assert b == [(0, 21120), (21120, 32768)]
    b = [balanced_shard_bounds(23, r, 3, 2.0) for r in range(3)]
    assert b == [(0, 13), (13, 18), (18, 23)]
    assert balanced_shard_bounds(100, 0, 1) == (0, 100)
    for world in (2, 4, 8):
        bs = [balanced_shard_bounds(16384 * world, r, world, 1.8, 64) for r in range(world)]
        assert bs[0][0] == 0 and bs[-1][1] == 16384 * world
        assert all(bs[i][1] == bs[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        balanced_shard_bounds(10, 3, 3)
