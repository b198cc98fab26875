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


def _worker(rank, world, port, T, out_dir, first_weight):
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
        wx, params, h0 = make_problem("gru_diag", 2, T, 6, seed=7, h0=True)
        s, e = (time_shard_bounds(T, rank, world) if first_weight is None
                else balanced_shard_bounds(T, rank, world, first_weight))
        comm = DistComm()
        ops = CpuShardOps("gru_diag", torch.from_numpy(wx[:, s:e]), [torch.from_numpy(p) for p in params],
                          1e-6, 1.0)
        res = drive(forward_program(ops, rank, world, 3, 0, torch.from_numpy(h0)), comm)
        G = torch.from_numpy(np.random.default_rng(3).standard_normal((2, T, 6)).astype(np.float32))
        g_wx, g_par, head = drive(backward_program(ops, rank, world, res.states, G[:, s:e], res.halo), comm)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), H=res.states.numpy(), bits=res.stats_bits.numpy(),
                 g_wx=g_wx.numpy(), g_par=g_par.numpy(), head=head.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,first_weight", [(2, 17, None), (3, 20, None), (3, 23, 2.0)])
def test_sharded_driver_over_gloo(world, T, first_weight, tmp_path):
    from gpu_util import make_problem
    from oracle import oracle
    from pararnn_b200.seq_shard import _bits_to_stats

    mp.spawn(_worker, args=(world, _free_port(), T, str(tmp_path), first_weight), nprocs=world, join=True)
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    wx, params, h0 = make_problem("gru_diag", 2, T, 6, seed=7, h0=True)
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
