"""A bounded device-side wait that runs out: the call returns, the status word says so, and the
public API turns it into an exception.  Only the look-back kernels are driven into their
time-out here (they poll flags in global memory and have no asynchronous copy in flight); the
wait limit is lowered through the library's test hook, nothing is made to hang."""

import numpy as np
import pytest
import torch

from gpu_util import dev, make_problem

pytestmark = pytest.mark.gpu


def test_lookback_wait_runs_out_and_is_reported(prb_options):
    from pararnn_b200 import ops

    prb_options("kernel_family", "lookback")
    prb_options("spin_limit", 1)  # give up at the first poll that finds the predecessor unfinished
    wx, params, _ = make_problem("gru_diag", 4, 65536, 32, seed=3)
    st = ops.DeviceStats("cuda", 2)
    H = ops.newton_gru_fused(dev(wx), *[dev(p) for p in params], None, max_iters=2, stats=st)
    torch.cuda.synchronize()  # the launch terminates
    assert H.shape == (4, 65536, 32)
    assert st.read()[2] == 1
    # the same problem with the default limit is fine
    prb_options("spin_limit", 0)
    st2 = ops.DeviceStats("cuda", 2)
    ops.newton_gru_fused(dev(wx), *[dev(p) for p in params], None, max_iters=2, stats=st2)
    assert st2.read()[2] == 0


def test_newton_apply_raises_on_device_timeout(prb_options):
    import pararnn_b200 as prb

    prb_options("kernel_family", "lookback")
    prb_options("spin_limit", 1)
    torch.manual_seed(0)
    cell = prb.ParaGRU(32, 32).cuda()
    x = torch.randn(4, 65536, 32, device="cuda")
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        prb.newton_apply(cell, x, prb.NewtonConfig(max_iters=2), stats=prb.NewtonStats())


def test_backward_timeout_is_reported_by_the_next_forward(prb_options):
    import pararnn_b200 as prb

    prb_options("kernel_family", "lookback")
    torch.manual_seed(0)
    cell = prb.ParaGRU(32, 32).cuda()
    x = torch.randn(4, 65536, 32, device="cuda", requires_grad=True)
    H = prb.newton_apply(cell, x, prb.NewtonConfig(max_iters=2))
    prb_options("spin_limit", 1)
    H.sum().backward()  # the reverse scan times out; nothing raises inside autograd
    prb_options("spin_limit", 0)
    with pytest.raises(RuntimeError, match="reverse scan"):
        prb.newton_apply(cell, x.detach(), prb.NewtonConfig(max_iters=2), stats=prb.NewtonStats())
    # the pending report is consumed: the next call is clean
    prb.newton_apply(cell, x.detach(), prb.NewtonConfig(max_iters=2), stats=prb.NewtonStats())
