"""`prb_bwd_nlru_static`: the NLRU backward entry point for callers that cannot allocate.

Some hosts of this library may not touch the device allocator where they call it (a service
loop that must not block on an allocator, a plugin inside a process that owns all device memory,
a job with a memory budget fixed at start-up).  For them the library carries its own fixed
scratch.  The entry point must give the same gradients as `prb_bwd_nlru`, call after call, even
though every call reuses the same scratch bytes and finds the previous call's leftovers in them.

The file name sorts last on purpose: with `-x` every other test has run before this one.
"""

import ctypes

import numpy as np
import pytest
import torch

from gpu_util import dev, make_problem
from oracle import oracle

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _static_call(lib, H, wx, u, G, h0, B, T, d, dtype_code):
    from pararnn_b200 import ops

    g_wx = torch.full_like(wx, float("nan"))
    g_u = torch.full((1, d), float("nan"), dtype=torch.float32, device="cuda")
    g_h0 = torch.full((B, d), float("nan"), dtype=torch.float32, device="cuda")
    st = ops.DeviceStats("cuda", 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.prb_bwd_nlru_static(_p(H), _p(wx), _p(u), _p(h0), _p(G), _p(g_wx), _p(g_u), _p(g_h0),
                                 B, T, d, dtype_code, _p(st.buf), stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    assert st.read()[2] == 0
    return g_wx, g_u[0], g_h0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_matches_workspace_entry_twice(dtype):
    from pararnn_b200 import _lib, ops

    lib = _lib.lib()
    code = _lib.PRB_F32 if dtype == torch.float32 else _lib.PRB_BF16
    results = []
    # two different problems back to back: the second call finds the first call's flags,
    # aggregates and partial sums in the shared scratch
    for seed, (B, T, d) in ((3, (2, 700, 72)), (4, (3, 333, 40))):
        wx_np, par, h0_np = make_problem("nlru", B, T, d, seed=seed, h0=True)
        H_np = oracle.sequential(oracle.NLRU, wx_np, par, h0_np)
        G_np = np.random.default_rng(seed).standard_normal(H_np.shape).astype(np.float32)
        H, wx, u, G, h0 = dev(H_np, dtype), dev(wx_np, dtype), dev(par[0], dtype), dev(G_np, dtype), dev(h0_np, dtype)
        want = ops.nlru_reverse_vjp(H, wx, u, G, h0)
        got = _static_call(lib, H, wx, u, G, h0, B, T, d, code)
        results.append((want, got))
    for want, got in results:
        for a, b in zip(want, got):
            # same kernels, same order of operations: the tolerance of the other backward tests
            # (2e-5 relative in fp32, 2e-2 in bf16) is met with room to spare
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            scale = max(1.0, float(a.float().abs().max()))
            assert float((a.float() - b.float()).abs().max()) <= tol * scale


def test_static_scratch_entry_rejects_what_does_not_fit():
    from pararnn_b200 import _lib

    lib = _lib.lib()
    cap = lib.prb_static_scratch_bytes()
    assert cap == 8 << 20
    B, T, d = 8, 1 << 20, 4096
    assert lib.prb_bwd_workspace_bytes(_lib.CELL_NLRU, _lib.PRB_F32, B, T, d, 1) > cap
    one = torch.zeros(16, device="cuda")
    rc = lib.prb_bwd_nlru_static(_p(one), _p(one), _p(one), None, _p(one), _p(one), _p(one), None,
                                 B, T, d, _lib.PRB_F32, _p(one), None)
    assert rc == -5
    assert "capacity" in lib.prb_error_string(rc).decode()
