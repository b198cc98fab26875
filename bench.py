#!/usr/bin/env python
"""Benchmark of the Newton+scan training hot path (forward + packed-VJP backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): ParaSLSTM mix='diag', bf16 I/O with fp32 scan state, B=8, T=16384,
d=1024, picard_iters=5, max_iters=2, one forward + one backward per step, synthetic
inputs x ~ 0.5*N(0,1), Xavier-uniform W_x, forget-gate bias +3, seed 1.  With N > 1 the
sequence is sharded along time over N ranks (one process per GPU, NCCL) with T = 16384*N,
so per-GPU work is fixed (weak scaling) and N = 8 is the T = 131072 case.

`value` is tokens/s at the op boundary (gate pre-activations resident in HBM -> states,
cotangent -> gradients of the pre-activations and of R), timed with CUDA events.
`e2e` is the same metric through the `ParaRNN` layer + autograd with host-resident inputs,
including the three W_x GEMMs and the host<->device copies (with a GEMM / scan / rest breakdown).
`roofline` is computed on the bytes the dominant launch really moves; the figure the
separate passes it replaces would need is reported beside it under its own name.
`parity` compares a 32-channel slice of this run's own result with the CPU oracle.
`sustained` repeats the step back to back for at least three seconds.
With N > 1 the timed step is one CUDA graph per rank (kernels, folds, NCCL all-gathers;
the same programs issued from Python are `eager_ms_per_step`), and the line also carries
`c4_strong` (B=1, T=131072, d=2048 sharded over the N ranks against the same shape on one
GPU) and `c5_sharded` (12 x ParaNLRU stack).  `--workload c1|c3|c5|lstm` time the secondary
configurations, `--workload ref_fused` the reference's own GPU paths next to this backend.
The CPU arm (`--impl reference`, and `cpu_baseline` at N = 1) times the C restatement of
the reference's eager algorithm (oracle/) on the host cores.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "pararnn-torch_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

B, T_PER_GPU, D, K_NEWTON, P_PICARD = 8, 16384, 1024, 2, 5
DEFAULT_T = T_PER_GPU
SEED = 1
# algorithmic bytes per (token, channel): bf16 I/O (a=2), fp32 work state (w=4), G=S=4
BYTES_PICARD_MID = 4 * 2 + 4 + 4          # read wx + h, write h
BYTES_PICARD_PHASE = 12 + 4 * 16 + 28     # the six separate passes of the warm start (P = 5)
BYTES_PICARD_SWEEP = 4 * 2 + 16           # what the fused sweep has to move: read wx, write state
BYTES_NEWTON_MID = 4 * 2 + 16 + 16        # read wx + state, write state
BYTES_NEWTON_LAST = 4 * 2 + 16 + 4 * 2    # read wx + state, write the I/O-dtype state
BYTES_NEWTON_PHASE = 40 + 32 + 16         # K = 2 separate passes and the separate residual gate
BYTES_NEWTON_SWEEP = 4 * 2 + 16 + 4 * 2   # what the fused sweep has to move
BYTES_BWD = 4 * 2 + 4 * 2 + 4 * 2 + 4 * 2  # read states, wx, cotangent; write g_wx
BYTES_STEP = 224                          # all passes of one forward + backward
# DRAM bytes per (token, channel) of each kernel as ncu counted them in an earlier capture of the
# same kernels at a quarter of this sequence length (traffic grows in proportion to the units);
# NOT measured by this run: a run under a profiler is never a bench run
NCU_TRAFFIC_PER_UNIT = {"slstm_picard_pipe_kernel": 15.44, "slstm_newton_pipe_kernel": 39.02,
                        "slstm_bwd_pipe_kernel": 31.37,
                        "slstm_picard_fused_kernel": 22.44, "slstm_newton_fused_kernel": 31.53}
# issue-slot utilisation of the fused sweeps in the same capture (they are bound by it, not by HBM)
NCU_ISSUE_ACTIVE = {"slstm_picard_fused_kernel": 0.61, "slstm_newton_fused_kernel": 0.72}
PARITY_TOL = 2e-2     # bf16 I/O against the fp32 oracle on bf16-rounded inputs, relative to max|.|
PARITY_CH = 32
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled every
    5 ms from a thread (read-only queries), or `nvidia-smi -lms 100` when NVML is not importable."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.sm, self.mx, self.seen, self._stop, self._thread = [], [], set(), False, None

    def _poll_nvml(self, nv, handle):
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                "sw_power_cap": 0x4}
        while not self._stop:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                self.seen.update(n for n, b in bits.items() if mask & b)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].strip().isdigit():
                    phys = int(ids[self.index])
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self._thread = threading.Thread(target=self._poll_nvml, args=(nv, handle), daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self._thread is not None:
            self._stop = True
            self._thread.join(timeout=1)
            reasons = [n for n in self.NAMES if n in self.seen]
            return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                    "sm_max_mhz": max(self.mx) if self.mx else None, "reasons": reasons,
                    "samples": len(self.sm), "source": "nvml"}
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        reasons = [n for i, n in enumerate(self.NAMES)
                   if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm),
                "source": "nvidia-smi"}


def make_inputs(t_len: int, seed: int):
    """Synthetic layer inputs and parameters (CPU tensors), fp32 master copies."""
    import torch

    g = torch.Generator().manual_seed(SEED)
    gx = torch.Generator().manual_seed(seed)
    x = 0.5 * torch.randn(B, t_len, D, generator=gx)
    bound = (6.0 / (D + 4 * D)) ** 0.5
    W = (torch.rand(4 * D, D, generator=g) * 2 - 1) * bound
    bias = torch.zeros(4 * D)
    bias[D:2 * D] = 3.0
    R = (torch.randn(4, D, generator=g) * (1.0 / (4 * D)) ** 0.5).clamp(-0.5, 0.5)
    return x, W, bias, R


# ----------------------------------------------------------------------------- CPU arm

def cpu_step(sample, threads):
    """One forward + backward of the oracle on one batch row; returns seconds."""
    import numpy as np

    from oracle import oracle

    wx, r, G = sample
    os.environ["OMP_NUM_THREADS"] = str(threads)
    t0 = time.perf_counter()
    res = oracle.newton(oracle.SLSTM_DIAG, wx, r, None, max_iters=K_NEWTON, picard=P_PICARD)
    oracle.backward(oracle.SLSTM_DIAG, res.states, wx, r, G, None)
    return time.perf_counter() - t0, res


def cpu_sample():
    import numpy as np
    import torch

    x, W, bias, R = make_inputs(T_PER_GPU, SEED)
    xb = x[:1].bfloat16().float()
    wx = (xb.reshape(-1, D) @ W.bfloat16().float().t() + bias).reshape(1, T_PER_GPU, 4 * D)
    wx = wx.bfloat16().float().numpy()
    r = R.bfloat16().float().numpy()
    G = np.zeros((1, T_PER_GPU, 4, D), dtype=np.float32)
    G[:, :, 3] = 1.0
    return wx, r, G


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.build()
    threads = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(threads)
    sample = cpu_sample()
    for _ in range(args.warmup):
        cpu_step(sample, threads)
    times = [cpu_step(sample, threads)[0] for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = T_PER_GPU / sec  # one batch row per step
    line = {
        "impl": "reference", "metric": "newton_scan_fwd_bwd_tokens_per_s", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        # the CPU arm always times the same one-row, T = T_PER_GPU sample, whatever N is
        "config": dict(workload_config(1), timed_sample="1 batch row, T=%d" % T_PER_GPU,
                       requested_gpus=args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": "1 of 8 batch rows per step (rows are independent), full T=16384, "
                                   "d=1024, fp32 arithmetic on bf16-rounded inputs"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(n):
    return {"workload": f"ParaSLSTM mix=diag fwd+bwd, B={B}, T={T_PER_GPU * n}, d={D}, bf16 I/O + fp32 "
                        f"scan state, picard_iters={P_PICARD}, max_iters={K_NEWTON}, seed {SEED}",
            "global_batch": B, "seq_len": T_PER_GPU * n, "d_model": D,
            "parallelism": "single GPU" if n == 1 else f"time-sharded x{n} (NCCL carry exchange)",
            "l2": "inputs (>= 1 GB per pass) are larger than the 126 MB L2; no flush needed"}


# ----------------------------------------------------------------------------- GPU arm

def slice_parity(wx_rows, r, H_rows, gwx_rows, d, K, P, eps=1e-6):
    """Max relative error of this run's own result against the CPU oracle on a slice: one batch
    row, the first PARITY_CH channels, the whole sequence.  `wx_rows` (T, 4, C), `H_rows`
    (T, 4, C), `gwx_rows` (T, 4, C) are that slice (any float dtype, CPU or GPU), `r` (4, C).
    The cotangent is 1 on the hidden slot, 0 elsewhere (what the bench's loss produces)."""
    import numpy as np

    from oracle import oracle

    wx_np = wx_rows.float().cpu().numpy()
    T, _, C = wx_np.shape
    wx_np = np.ascontiguousarray(wx_np.reshape(1, T, 4 * C))
    r_np = np.ascontiguousarray(r.float().cpu().numpy())
    want = oracle.newton(oracle.SLSTM_DIAG, wx_np, r_np, None, max_iters=K, picard=P, eps=eps)
    got_H = H_rows.float().cpu().numpy().reshape(1, T, 4, C)
    G = np.zeros((1, T, 4, C), dtype=np.float32)
    G[:, :, 3] = 1.0
    want_g, _, _ = oracle.backward(oracle.SLSTM_DIAG, got_H, wx_np, r_np, G, None, eps=eps)
    got_g = gwx_rows.float().cpu().numpy().reshape(1, T, 4 * C)
    rel_h = float(np.abs(got_H[:, :, 3] - want.states[:, :, 3]).max() / max(1e-30, np.abs(want.states[:, :, 3]).max()))
    rel_g = float(np.abs(got_g - want_g).max() / max(1e-30, np.abs(want_g).max()))
    return {"max_rel_h": rel_h, "max_rel_gwx": rel_g, "tol": PARITY_TOL, "ok": bool(rel_h <= PARITY_TOL and rel_g <= PARITY_TOL),
            "slice": f"batch row 0, channels 0..{C - 1}, all {T} steps, against the fp32 CPU oracle on the same "
                     "bf16-rounded inputs", "oracle_residual_history": [float(v) for v in want.history]}


def gate_slice(t, d, n_ch=PARITY_CH):
    """(T, 4, n_ch) slice of a (T, 4*d) gate-major row or of a (T, 4, d) state row."""
    T = t.shape[0]
    return t.reshape(T, 4, d)[:, :, :n_ch]


def sustained_run(step, device_index, seconds=3.0):
    """The step back to back for at least `seconds`: what it costs once the burst clock is gone."""
    import torch

    sampler = ClockSampler(device_index)
    sampler.start()
    n, total = 0, 0.0
    chunk = 50
    t_start = time.perf_counter()
    while time.perf_counter() - t_start < seconds:
        total += time_region(step, chunk, None)
        n += chunk
    clocks = sampler.stop()
    ms = total / n * 1e3
    mhz = clocks.get("sm_mhz")
    return {"ms_per_step": ms, "steps": n, "seconds": total, "sm_mhz_median": mhz,
            "ms_times_mhz": (ms * mhz) if mhz else None, "reasons": clocks.get("reasons")}


def time_region(fn, steps, stream_sync, barrier=None):
    import torch

    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1) / 1e3


def kernel_rooflines(wx, r32, states32, states_io, G_io, peak):
    """Average launch duration of each scan kernel in isolation, CUDA events on the launch stream."""
    import torch

    from pararnn_b200 import _lib as L
    from pararnn_b200 import ops

    lib = L.lib()
    dev = wx.device
    ws = torch.empty(lib.prb_pass_workspace_bytes(L.CELL_SLSTM_DIAG, B, T_PER_GPU, D),
                     dtype=torch.uint8, device=dev)
    st = ops.DeviceStats(dev, K_NEWTON)
    stream = ops._stream(dev)
    hbuf = torch.empty(B, T_PER_GPU, D, dtype=torch.float32, device=dev)
    hbuf2 = torch.empty_like(hbuf)
    sout = torch.empty_like(states32)
    states_out = torch.empty_like(states_io)
    g_wx = torch.empty_like(wx)
    g_r = torch.empty(4, D, dtype=torch.float32, device=dev)
    g_h0 = torch.empty(B, 4, D, dtype=torch.float32, device=dev)
    P = ops._ptr
    hbuf.copy_(states32[:, :, 3])

    def picard():
        rc = lib.prb_slstm_picard_pass(P(wx), P(r32), P(hbuf), None, None, P(hbuf2), None, None, None, 0,
                                       1, T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1e-6, P(ws), ws.numel(), P(st.buf), stream)
        assert rc == 0, rc

    def picard_sweep():
        rc = lib.prb_slstm_picard_sweep(P(wx), P(r32), None, None, P(sout), None, P_PICARD + 1, B, T_PER_GPU, D,
                                        L.PRB_BF16, 1e-6, P(ws), ws.numel(), P(st.buf), stream)
        assert rc == 0, rc

    def newton_sweep():
        rc = lib.prb_slstm_newton_sweep(P(wx), P(r32), P(states32), None, P(states_out), K_NEWTON, 1, B,
                                        T_PER_GPU, D, L.PRB_BF16, 1.0, 1e-6, P(ws), ws.numel(), P(st.buf),
                                        stream)
        assert rc == 0, rc

    def newton_last():
        rc = lib.prb_slstm_newton_pass(P(wx), P(r32), P(states32), None, None, P(states_out), None, None, 1, 1,
                                       T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1.0, 1e-6, P(ws), ws.numel(), P(st.buf),
                                       1, stream)
        assert rc == 0, rc

    def newton():
        rc = lib.prb_slstm_newton_pass(P(wx), P(r32), P(states32), None, None, P(sout), None, None, 0, 1,
                                       T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1.0, 1e-6, P(ws), ws.numel(), P(st.buf),
                                       0, stream)
        assert rc == 0, rc

    def bwd():
        rc = lib.prb_slstm_bwd_pass(P(states_io), P(wx), P(r32), None, None, P(G_io), P(g_wx), P(g_r),
                                    P(g_h0), None, 0, 1, T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1e-6, P(ws), ws.numel(),
                                    P(st.buf), stream)
        assert rc == 0, rc

    agg_n = torch.empty(1, B, 20, D, dtype=torch.float32, device=dev)
    agg_p = torch.empty(1, B, 4, D, dtype=torch.float32, device=dev)

    def newton_agg():
        rc = lib.prb_slstm_newton_pass(P(wx), P(r32), P(states32), None, None, None, None, P(agg_n), 2, 1,
                                       T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1.0, 1e-6, P(ws), ws.numel(),
                                       P(st.buf), 0, stream)
        assert rc == 0, rc

    def picard_agg():
        rc = lib.prb_slstm_picard_pass(P(wx), P(r32), P(hbuf), None, None, None, None, None, P(agg_p), 2,
                                       1, T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1e-6, P(ws), ws.numel(),
                                       P(st.buf), stream)
        assert rc == 0, rc

    def bwd_agg():
        rc = lib.prb_slstm_bwd_pass(P(states_io), P(wx), P(r32), None, None, P(G_io), None, None, None,
                                    P(agg_n), 2, 1, T_PER_GPU, B, T_PER_GPU, D, L.PRB_BF16, 1e-6, P(ws),
                                    ws.numel(), P(st.buf), stream)
        assert rc == 0, rc

    n_units = B * T_PER_GPU * D
    out = {}
    # One training step = 1 fused Picard sweep + 1 fused Newton sweep (K iterations and the final
    # residual) + 1 backward launch.  The per-pass kernels (used by the time-sharded path) are
    # timed too, with launches_per_step 0.
    for name, fn, nbytes, per_step in (("slstm_picard_fused_kernel", picard_sweep, BYTES_PICARD_SWEEP, 1),
                                       ("slstm_newton_fused_kernel", newton_sweep, BYTES_NEWTON_SWEEP, 1),
                                       ("slstm_bwd_pipe_kernel", bwd, BYTES_BWD, 1),
                                       ("slstm_picard_pipe_kernel", picard, BYTES_PICARD_MID, 0),
                                       ("slstm_newton_pipe_kernel", newton, BYTES_NEWTON_MID, 0),
                                       ("slstm_newton_pipe_kernel_last", newton_last, BYTES_NEWTON_LAST, 0),
                                       # aggregate-only sweeps of the time-sharded path: inputs only
                                       ("slstm_picard_agg_seg_kernel", picard_agg, 4 * 2 + 4, 0),
                                       ("slstm_newton_agg_seg_kernel", newton_agg, 4 * 2 + 16, 0),
                                       ("slstm_bwd_agg_seg_kernel", bwd_agg, 4 * 2 * 3, 0)):
        for _ in range(3):
            fn()
        sec = time_region(fn, 10, None) / 10
        gbs = n_units * nbytes / sec / 1e9
        out[name] = {"ms_per_launch": sec * 1e3, "achieved": gbs, "frac": gbs / peak,
                     "launches_per_step": per_step, "algorithmic_bytes_per_launch": n_units * nbytes}
        if fn is picard_sweep or fn is newton_sweep:
            # the same work as the separate passes of the per-pass accounting (104 B per
            # token-channel for the six Picard passes, 88 B for two Newton passes and the residual
            # gate); the sweeps are bound by instruction issue, not by HBM
            phase = BYTES_PICARD_PHASE if fn is picard_sweep else BYTES_NEWTON_PHASE
            out[name]["bound"] = "issue"
            out[name]["separate_passes_bytes"] = n_units * phase
            out[name]["achieved_vs_separate_passes"] = n_units * phase / sec / 1e9
    return out


def run_gpu_single(args):
    import torch

    from pararnn_b200 import ops
    import pararnn_b200 as prb

    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    peak, peak_kind = measured_peaks()
    x, W, bias, R = make_inputs(T_PER_GPU, SEED)
    cell = prb.ParaSLSTM(D, D).to(dev)
    with torch.no_grad():
        cell.W_x.weight.copy_(W)
        cell.W_x.bias.copy_(bias)
        cell.R.copy_(R)
    cell = cell.bfloat16()
    x_host = x.bfloat16().pin_memory()
    x_dev = x_host.to(dev)
    with torch.no_grad():
        wx = cell.W_x(x_dev).contiguous()
    r_io = cell.clipped_r().detach()
    G_io = torch.zeros(B, T_PER_GPU, 4, D, dtype=torch.bfloat16, device=dev)
    G_io[:, :, 3] = 1.0
    stats = ops.DeviceStats(dev, K_NEWTON)
    keep = {}

    def step():
        H = ops.newton_slstm_fused(wx, r_io, None, None, max_iters=K_NEWTON, picard_iters=P_PICARD,
                                   stats=stats, want_residual=True)
        keep["out"] = ops.slstm_reverse_vjp(H, wx, r_io, G_io)
        keep["H"] = H

    for _ in range(max(args.warmup, 3)):
        step()
    # clocks are sampled over all timed regions of this run (step, end-to-end, kernels in isolation)
    sampler = ClockSampler(0)
    sampler.start()
    sec = time_region(step, args.steps, None)
    hist, res, status = stats.read()
    assert status == 0, "chain wait timed out"
    ms = sec / args.steps * 1e3
    tokens = B * T_PER_GPU
    value = tokens / (sec / args.steps)

    # end to end through the public API with host-resident inputs
    cfg = prb.NewtonConfig(max_iters=K_NEWTON, picard_iters=P_PICARD, picard_adapt=False)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    # Input pipeline of the end-to-end step: the pinned host batch of step i+1 is copied on a second
    # stream into the other of two device buffers while step i computes; every step still issues
    # one full host->device copy of its input and one device->host read of its loss.
    copy_stream = torch.cuda.Stream()
    x_bufs = [torch.empty_like(x_dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    for ev in consumed:
        ev.record()
    e2e_state = {"i": 0}

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            x_bufs[i % 2].copy_(x_host, non_blocking=True)
            ready[i % 2].record(copy_stream)

    prefetch(0)

    layer = prb.ParaRNN(cell, config=cfg).train()  # the user-facing call: x -> hidden states

    def e2e_step():
        i = e2e_state["i"]
        torch.cuda.current_stream().wait_event(ready[i % 2])
        prefetch(i + 1)
        xd = x_bufs[i % 2].detach().requires_grad_(True)
        loss = layer(xd).sum(dtype=torch.float32)
        loss.backward()
        consumed[i % 2].record()
        loss_host.copy_(loss.detach(), non_blocking=True)
        cell.zero_grad(set_to_none=True)
        e2e_state["i"] = i + 1

    e2e_breakdown = None
    if args.no_e2e:
        e2e_sec = float("nan")
    else:
        for _ in range(2):
            e2e_step()
        e2e_steps = max(2, min(args.steps, 5))
        e2e_sec = time_region(e2e_step, e2e_steps, None) / e2e_steps
        # where the end-to-end step goes: the three W_x GEMMs timed alone, the scan step from above
        with torch.no_grad():
            gy = torch.randn(B * T_PER_GPU, 4 * D, device=dev, dtype=torch.bfloat16)
            xx = x_dev.reshape(-1, D)
            w_ = cell.W_x.weight.detach()
            gemm_fwd = time_region(lambda: cell.W_x(x_dev), 5, None) / 5
            gemm_bwd = time_region(lambda: (gy @ w_, gy.t() @ xx), 5, None) / 5
            del gy
        e2e_breakdown = {"wx_gemm_fwd_ms": gemm_fwd * 1e3, "wx_gemm_bwd_ms": gemm_bwd * 1e3,
                         "scan_fwd_bwd_ms": ms,
                         "rest_ms": (e2e_sec - gemm_fwd - gemm_bwd) * 1e3 - ms,
                         "rest_is": "loss and its cotangent, dtype/layout copies, host launch gaps, the "
                                    "residual read-back of the solve, contention with the input copy"}

    # per-kernel rooflines
    states_io = keep["H"]
    states32 = states_io.float()
    roofs = kernel_rooflines(wx, r_io.float().contiguous(), states32, states_io, G_io, peak)
    n_units = tokens * D
    # The dominant kernel by time per step.  `achieved` / `frac` are computed on the bytes the
    # launch really moves (its inputs once, its outputs once).  A fused sweep replaces several
    # HBM-bound passes while moving a fraction of their bytes, so its fraction of the HBM peak is
    # low by construction: it is bound by instruction issue (`binding_resource`).  What the
    # separate passes would have needed is kept under `equivalent_per_pass_gbs`.
    total = {k: v["ms_per_launch"] * v["launches_per_step"] for k, v in roofs.items()}
    # the two fused sweeps take the same time to within 2 %: among kernels within 5 % of the longest
    # the one that moves the most bytes is reported, so that the line does not flip between runs
    longest = max(total.values())
    top = max((k for k in total if total[k] >= 0.95 * longest),
              key=lambda k: roofs[k]["algorithmic_bytes_per_launch"])
    per_unit = NCU_TRAFFIC_PER_UNIT.get(top)
    moved_step = (BYTES_PICARD_SWEEP + BYTES_NEWTON_SWEEP + BYTES_BWD) * n_units
    roofline = {"bound": "hbm", "kernel": top, "ms_per_launch": roofs[top]["ms_per_launch"],
                "achieved": roofs[top]["achieved"], "peak": peak, "unit": "GB/s",
                "frac": roofs[top]["achieved"] / peak, "peak_kind": peak_kind,
                "algorithmic_bytes_per_launch": roofs[top]["algorithmic_bytes_per_launch"],
                "traffic": per_unit * n_units if per_unit else None,
                "traffic_source": "ncu capture of the same kernel at T=4096 scaled by the units; not measured "
                                  "by this run",
                "binding_resource": ("instruction issue: %.0f %% of issue slots active in the ncu capture"
                                     % (100 * NCU_ISSUE_ACTIVE[top])) if top in NCU_ISSUE_ACTIVE else "hbm",
                "equivalent_per_pass_gbs": roofs[top].get("achieved_vs_separate_passes"),
                "ms_per_step_by_kernel": {k: v for k, v in total.items() if v > 0}, "kernels": roofs,
                "step": {"bytes_moved": moved_step, "achieved": moved_step / (ms / 1e3) / 1e9,
                         "frac": moved_step / (ms / 1e3) / 1e9 / peak,
                         "per_pass_accounting_bytes": BYTES_STEP * n_units,
                         "equivalent_per_pass_gbs": BYTES_STEP * n_units / (ms / 1e3) / 1e9,
                         "equivalent_per_pass_frac": BYTES_STEP * n_units / (ms / 1e3) / 1e9 / peak,
                         "equivalent_per_pass_frac_of_nominal_8TBs": BYTES_STEP * n_units / (ms / 1e3) / 1e9 / NOMINAL_HBM_GBS,
                         "note": "the three launches of a step move 88 B per token-channel; 224 B is what "
                                 "the nine separate sweeps of the per-pass formulation move"}}

    # parity of THIS run's result (seed-1 inputs of the bench) against the CPU oracle
    g_wx_run = keep["out"][0]
    parity = slice_parity(gate_slice(wx[0], D), r_io[:, :PARITY_CH], gate_slice(keep["H"][0], D),
                          gate_slice(g_wx_run[0], D), D, K_NEWTON, P_PICARD)
    assert parity["ok"], parity

    sustained = None if args.no_sustained else sustained_run(step, 0)

    clocks = sampler.stop()

    # CPU baseline on a bounded sample (rank 0, N = 1 only)
    threads = os.cpu_count() or 1
    if args.no_cpu:
        cpu_value = float("nan")
    else:
        sample = cpu_sample()
        cpu_sec, cpu_res = cpu_step(sample, threads)
        cpu_value = T_PER_GPU / cpu_sec

    line = {
        "metric": "newton_scan_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 scan arithmetic, bf16 I/O",
        "data": "synthetic", "config": workload_config(1), "clocks": clocks,
        "e2e": {"value": tokens / e2e_sec, "unit": "tokens/s",
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": 4,
                "ms_per_step": e2e_sec * 1e3, "breakdown": e2e_breakdown,
                "api": "ParaRNN(ParaSLSTM)(x).sum().backward()",
                "includes": "H2D of x (double-buffered on a copy stream, one copy per step), 3 W_x GEMMs "
                            "(cuBLAS), Newton+scan fwd, reverse scan + VJP, D2H of loss"},
        # per step: fp32 copy of R (x2), Picard sweep, Newton sweep, backward, reduction
        "gpu_launches": 6 * args.steps,
        "roofline": roofline,
        "cpu_baseline": {"value": cpu_value, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": "1 of 8 batch rows (rows are independent), full T=16384, d=1024, "
                                   "fp32 arithmetic on bf16-rounded inputs, one forward+backward"},
        "parity": parity, "sustained": sustained,
        "newton": {"iters": K_NEWTON, "residual_history": list(hist), "max_residual": res,
                   "note": "max_iters is mandated by the configuration; the warm start already lands at "
                           "1e-7 and the Newton iterations move the stabiliser m by one ulp"},
    }
    print(json.dumps(line))


def run_gpu_sharded(args):
    """N ranks, one per GPU: the sequence (T = T_PER_GPU * N) is sharded along time; every scan
    pass exchanges per-shard carries with one NCCL all-gather.  Max over ranks of the
    event-timed region; rank 0 prints the line."""
    import torch
    import torch.distributed as dist

    import pararnn_b200 as prb
    from pararnn_b200.seq_shard import (CudaShardOps, DistComm, GraphedShardedStep, _bits_to_stats,
                                        backward_program, drive, forward_program)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    comm = DistComm()
    peak, peak_kind = measured_peaks()
    # Shard lengths: equal by default.  The first rank sweeps once per pass and the others twice
    # (aggregate, then apply), but the others' apply sweep has to wait for the first rank's sweep
    # anyway (its result is their carry), so a longer first shard buys little
    # (`--first-shard-weight`).  The total stays T_PER_GPU * N.
    from pararnn_b200.seq_shard import balanced_shard_bounds

    t_total = T_PER_GPU * world
    lo, hi = balanced_shard_bounds(t_total, rank, world, args.first_shard_weight, 64)
    t_local = hi - lo
    t_first = balanced_shard_bounds(t_total, 0, world, args.first_shard_weight, 64)[1]
    t_other = (t_total - t_first) // (world - 1)
    x, W, bias, R = make_inputs(max(t_local, T_PER_GPU), SEED + 1000 * rank)
    cell = prb.ParaSLSTM(D, D).to(dev)
    with torch.no_grad():
        cell.W_x.weight.copy_(W)
        cell.W_x.bias.copy_(bias)
        cell.R.copy_(R)
    cell = cell.bfloat16()
    x_host = x[:, :t_local].bfloat16().contiguous().pin_memory()
    x_dev = x_host.to(dev)
    with torch.no_grad():
        wx = cell.W_x(x_dev).contiguous()
        wx_dp = cell.W_x(x[:, :T_PER_GPU].bfloat16().to(dev)).contiguous()
    G_io = torch.zeros(B, t_local, 4, D, dtype=torch.bfloat16, device=dev)
    G_io[:, :, 3] = 1.0
    G_dp = torch.zeros(B, T_PER_GPU, 4, D, dtype=torch.bfloat16, device=dev)
    G_dp[:, :, 3] = 1.0
    rec = (cell.clipped_r().detach(),)
    keep = {}

    def step():
        ops = CudaShardOps("slstm_diag", wx, rec, 1e-6, 1.0)
        res = drive(forward_program(ops, rank, world, K_NEWTON, P_PICARD, None), comm)
        keep["bwd"] = drive(backward_program(ops, rank, world, res.states, G_io, res.halo), comm)
        keep["res"] = res
        keep["launches"] = ops.launches

    def barrier():
        dist.barrier(device_ids=[local])

    for _ in range(max(args.warmup, 3)):
        step()
    eager_sec = _max_over_ranks(dist, dev, time_region(step, args.steps, None, barrier))
    # The timed step: the same programs captured once into a CUDA graph (kernels, device-side
    # folds and the NCCL all-gathers) and replayed, which removes the host's per-launch cost.
    graphed = not args.no_graph
    graph_error = None
    if graphed:
        try:
            gs = GraphedShardedStep("slstm_diag", wx, rec, G_io, comm, K=K_NEWTON, P=P_PICARD)
            for _ in range(3):
                gs.replay()
            timed_step = gs.replay
        except Exception as exc:  # capture refused (library / driver): time the eager step instead
            graph_error, graphed = repr(exc)[:300], False
    if not graphed:
        timed_step = step
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sec = _max_over_ranks(dist, dev, time_region(timed_step, args.steps, None, barrier))
    clocks = sampler.stop() if rank == 0 else None
    if graphed:
        from types import SimpleNamespace

        keep["res"] = SimpleNamespace(states=gs.states, stats_bits=gs.stats_bits)
        keep["bwd"] = (gs.g_wx, gs.g_params, gs.head)
    hist, res_final, status = _bits_to_stats(keep["res"].stats_bits, K_NEWTON)

    # end to end through the public API (host-resident shard of x per rank)
    cfg = prb.NewtonConfig(max_iters=K_NEWTON, picard_iters=P_PICARD, picard_adapt=False,
                           scan_backend="context_parallel")
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    # Input pipeline of the end-to-end step: the pinned host batch of step i+1 is copied on a second
    # stream into the other of two device buffers while step i computes; every step still issues
    # one full host->device copy of its input and one device->host read of its loss.
    copy_stream = torch.cuda.Stream()
    x_bufs = [torch.empty_like(x_dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    for ev in consumed:
        ev.record()
    e2e_state = {"i": 0}

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[i % 2])
            x_bufs[i % 2].copy_(x_host, non_blocking=True)
            ready[i % 2].record(copy_stream)

    prefetch(0)

    layer = prb.ParaRNN(cell, config=cfg).train()  # the user-facing call: x -> hidden states

    def e2e_step():
        i = e2e_state["i"]
        torch.cuda.current_stream().wait_event(ready[i % 2])
        prefetch(i + 1)
        xd = x_bufs[i % 2].detach().requires_grad_(True)
        loss = layer(xd).sum(dtype=torch.float32)
        loss.backward()
        consumed[i % 2].record()
        loss_host.copy_(loss.detach(), non_blocking=True)
        cell.zero_grad(set_to_none=True)
        e2e_state["i"] = i + 1

    # For comparison only: the same GPUs used batch-parallel (every rank solves its own B rows of
    # T_PER_GPU steps with the single-GPU kernels; the only exchange is the all-reduce of grad R).
    # It is not the time-sharded path this line measures and never enters `value`.
    from pararnn_b200 import ops as _ops

    r_io = rec[0]
    dp_stats = _ops.DeviceStats(dev, K_NEWTON)

    def dp_step():
        H = _ops.newton_slstm_fused(wx_dp, r_io, None, None, max_iters=K_NEWTON, picard_iters=P_PICARD,
                                    stats=dp_stats, want_residual=True)
        out = _ops.slstm_reverse_vjp(H, wx_dp, r_io, G_dp)
        dist.all_reduce(out[1])
        keep["dp"] = out

    for _ in range(3):
        dp_step()
    dp_sec = time_region(dp_step, args.steps, None, barrier)
    t = torch.tensor([dp_sec], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dp_sec = float(t.item()) / args.steps

    e2e_sec = float("nan")
    if not args.no_e2e:
        for _ in range(2):
            e2e_step()
        n_e2e = max(2, min(args.steps, 5))
        e2e_sec = time_region(e2e_step, n_e2e, None, barrier) / n_e2e
        t = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
    # parity of this run's own (sharded, NCCL) result: the slice of every rank goes to rank 0,
    # which runs the CPU oracle over the whole T = T_PER_GPU * N sequence of that slice
    sl_wx = gather_time(dist, dev, world, gate_slice(wx[0], D).contiguous())
    sl_H = gather_time(dist, dev, world, gate_slice(keep["res"].states[0], D).contiguous())
    sl_g = gather_time(dist, dev, world, gate_slice(keep["bwd"][0][0], D).contiguous())
    parity = None
    if rank == 0:
        parity = slice_parity(sl_wx, rec[0][:, :PARITY_CH], sl_H, sl_g, D, K_NEWTON, P_PICARD)
        parity["path"] = f"time-sharded over {world} ranks, NCCL carry exchange"
    extra = {}
    # kernels of this library per step, summed over the ranks (rank 0 sweeps once per pass, the others twice)
    n_launch = torch.tensor([keep.get("launches", 0)], dtype=torch.int64, device=dev)
    dist.all_reduce(n_launch)
    if not args.no_extra:
        extra["c4_strong"] = c4_strong_record(args, rank, world, dev, dist, comm, barrier)
        extra["c5_sharded"] = c5_sharded_record(args, rank, world, dev, dist, barrier)
    if rank == 0:
        assert status == 0, "chain wait timed out"
        assert parity["ok"], parity
        ms = sec / args.steps * 1e3
        tokens = B * T_PER_GPU * world
        step_bytes = BYTES_STEP * tokens * D
        line = {
            "metric": "newton_scan_fwd_bwd_tokens_per_s", "value": tokens / (sec / args.steps),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 scan arithmetic, bf16 I/O", "data": "synthetic",
            "config": dict(workload_config(world), shard_lengths=[t_first] + [t_other] * (world - 1),
                           step="CUDA graph replay of the sharded forward + backward programs" if graphed
                           else "programs issued from Python"),
            "eager_ms_per_step": eager_sec / args.steps * 1e3, "graph_error": graph_error,
            "clocks": clocks,
            "e2e": {"value": tokens / e2e_sec, "unit": "tokens/s",
                    "h2d_bytes_per_step": B * t_total * D * 2, "d2h_bytes_per_step": 4 * world,
                    "ms_per_step": e2e_sec * 1e3,
                    "includes": "per rank: H2D of its x shard, 3 W_x GEMMs, sharded Newton+scan fwd and "
                                "reverse scan + VJP with NCCL carry exchange and gradient all-reduce, "
                                "D2H of loss"},
            # kernels of this library per step on rank 0 (sweeps, folds, reductions; counted by the
            # driver object), the same whether issued from Python or replayed from the graph
            "gpu_launches": int(n_launch.item()) * args.steps,
            "roofline": {"bound": "hbm", "kernel": "whole step (all ranks)", "peak": peak * world,
                         "unit": "GB/s", "achieved": step_bytes / (ms / 1e3) / 1e9,
                         "frac": step_bytes / (ms / 1e3) / 1e9 / (peak * world), "peak_kind": peak_kind,
                         "traffic": None,
                         "note": "ranks other than the first sweep each pass twice (aggregate, then apply)"},
            "newton": {"iters": K_NEWTON, "residual_history": list(hist), "max_residual": res_final},
            "parity": parity, **extra,
            "batch_parallel_for_comparison": {
                "value": B * T_PER_GPU * world / dp_sec, "unit": "tokens/s", "ms_per_step": dp_sec * 1e3,
                "workload": f"B={B * world} rows split over the ranks, T={T_PER_GPU}: independent rows, "
                            "fused single-GPU sweeps, all-reduce of grad R only"},
        }
        print(json.dumps(line), flush=True)
    # release the captured graphs (they hold NCCL kernels) before the communicator goes away; a
    # teardown that does not return must not keep the job alive after the line is out
    gs = None
    keep.clear()
    import gc

    gc.collect()
    torch.cuda.synchronize()
    dist.barrier(device_ids=[local])
    guard = threading.Timer(60.0, lambda: os._exit(0))
    guard.daemon = True
    guard.start()
    dist.destroy_process_group()
    guard.cancel()


def gather_time(dist, dev, world, t):
    """Slices (T_local, ...) of all ranks concatenated along time (shards may differ in length)."""
    import torch

    n_local = torch.tensor([t.shape[0]], device=dev)
    sizes = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(sizes, n_local)
    n_max = max(int(v.item()) for v in sizes)
    pad = torch.zeros(n_max, *t.shape[1:], dtype=t.dtype, device=dev)
    pad[: t.shape[0]] = t
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p_[: int(n.item())] for p_, n in zip(parts, sizes)], dim=0)


def _max_over_ranks(dist, dev, sec):
    import torch

    t = torch.tensor([sec], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def c4_strong_record(args, rank, world, dev, dist, comm, barrier):
    """Strong scaling of the T = 131072 configuration (ParaSLSTM mix='diag', bf16, B=1, d=2048,
    picard_iters=5, max_iters=2, seed 3): the sequence sharded over the N ranks against the SAME
    sequence on one GPU (rank 0, the other ranks idle), both at the op boundary, both checked."""
    import torch

    import pararnn_b200 as prb
    from pararnn_b200 import ops as _ops
    from pararnn_b200.seq_shard import (CudaShardOps, _bits_to_stats, backward_program, drive,
                                        forward_program, time_shard_bounds)

    Bc, Tc, Dc, seed = 1, 131072, 2048, 3
    if args.c4_seq_len:
        Tc = args.c4_seq_len
    g = torch.Generator().manual_seed(seed)
    bound = (6.0 / (Dc + 4 * Dc)) ** 0.5
    W = (torch.rand(4 * Dc, Dc, generator=g) * 2 - 1) * bound
    bias = torch.zeros(4 * Dc)
    bias[Dc:2 * Dc] = 3.0
    R = (torch.randn(4, Dc, generator=g) * (1.0 / (4 * Dc)) ** 0.5).clamp(-0.5, 0.5)
    cell = prb.ParaSLSTM(Dc, Dc).to(dev)
    with torch.no_grad():
        cell.W_x.weight.copy_(W)
        cell.W_x.bias.copy_(bias)
        cell.R.copy_(R)
    cell = cell.bfloat16()
    rec = (cell.clipped_r().detach(),)

    def x_shard(r):
        lo, hi = time_shard_bounds(Tc, r, world)
        gx = torch.Generator(device=dev).manual_seed(seed + 1000 * (r + 1))
        return (0.5 * torch.randn(Bc, hi - lo, Dc, generator=gx, device=dev)).bfloat16()

    with torch.no_grad():
        wx = cell.W_x(x_shard(rank)).contiguous()
    t_local = wx.shape[1]
    G_io = torch.zeros(Bc, t_local, 4, Dc, dtype=torch.bfloat16, device=dev)
    G_io[:, :, 3] = 1.0
    keep = {}

    def step():
        sops = CudaShardOps("slstm_diag", wx, rec, 1e-6, 1.0)
        res = drive(forward_program(sops, rank, world, K_NEWTON, P_PICARD, None), comm)
        keep["bwd"] = drive(backward_program(sops, rank, world, res.states, G_io, res.halo), comm)
        keep["res"], keep["segs"] = res, (sops.n_seg, sops.seg_len)

    n_steps = max(3, min(args.steps, 10))
    for _ in range(3):
        step()
    eager_sec = _max_over_ranks(dist, dev, time_region(step, n_steps, None, barrier)) / n_steps
    sec = eager_sec
    if not args.no_graph:
        from types import SimpleNamespace

        from pararnn_b200.seq_shard import GraphedShardedStep

        keep.pop("res", None)
        keep.pop("bwd", None)
        gs = GraphedShardedStep("slstm_diag", wx, rec, G_io, comm, K=K_NEWTON, P=P_PICARD)
        for _ in range(3):
            gs.replay()
        sec = _max_over_ranks(dist, dev, time_region(gs.replay, n_steps, None, barrier)) / n_steps
        keep["res"] = SimpleNamespace(states=gs.states, stats_bits=gs.stats_bits)
        keep["bwd"] = (gs.g_wx, gs.g_params, gs.head)
        keep["segs"] = (gs.ops.n_seg, gs.ops.seg_len)
    status = _bits_to_stats(keep["res"].stats_bits, K_NEWTON)[2]

    # slices of the sharded result to rank 0
    sl_wx = gather_time(dist, dev, world, gate_slice(wx[0], Dc).contiguous())
    sl_H = gather_time(dist, dev, world, gate_slice(keep["res"].states[0], Dc).contiguous())
    sl_g = gather_time(dist, dev, world, gate_slice(keep["bwd"][0][0], Dc).contiguous())
    record = None
    del keep["res"], keep["bwd"]
    if not args.no_graph:
        del gs
    torch.cuda.empty_cache()
    if rank == 0:
        parity = slice_parity(sl_wx, rec[0][:, :PARITY_CH], sl_H, sl_g, Dc, K_NEWTON, P_PICARD)
        # the same sequence on one GPU: rank 0 rebuilds all shards of x
        with torch.no_grad():
            wx_full = torch.cat([cell.W_x(x_shard(r)) for r in range(world)], dim=1).contiguous()
        G_full = torch.zeros(Bc, Tc, 4, Dc, dtype=torch.bfloat16, device=dev)
        G_full[:, :, 3] = 1.0
        st = _ops.DeviceStats(dev, K_NEWTON)

        def one_gpu():
            H = _ops.newton_slstm_fused(wx_full, rec[0], None, None, max_iters=K_NEWTON, picard_iters=P_PICARD,
                                        stats=st, want_residual=True)
            keep["one"] = (H, _ops.slstm_reverse_vjp(H, wx_full, rec[0], G_full))

        for _ in range(2):
            one_gpu()
        one_sec = time_region(one_gpu, n_steps, None) / n_steps
        H1, (g1, _, _) = keep["one"]
        h_one = gate_slice(H1[0], Dc)[:, 3].float()
        h_sh = sl_H[:, 3].float()
        rel_vs_one = float((h_one - h_sh).abs().max() / h_one.abs().max())
        g_one = gate_slice(g1[0], Dc).float()
        rel_g_vs_one = float((g_one - sl_g.float()).abs().max() / g_one.abs().max())
        units = Bc * Tc * Dc
        record = {
            "workload": f"ParaSLSTM mix=diag fwd+bwd, B={Bc}, T={Tc}, d={Dc}, bf16 I/O, picard_iters={P_PICARD}, "
                        f"max_iters={K_NEWTON}, seed {seed}; op boundary",
            "n_gpus": world, "ms_per_step": sec * 1e3, "tokens_per_s": Bc * Tc / sec,
            "eager_ms_per_step": eager_sec * 1e3,
            "step": "CUDA graph replay" if not args.no_graph else "issued from Python",
            "one_gpu_ms_per_step": one_sec * 1e3, "one_gpu_tokens_per_s": Bc * Tc / one_sec,
            "speedup": one_sec / sec, "segments_per_rank": keep["segs"][0], "segment_steps": keep["segs"][1],
            "status": status, "parity": parity,
            "sharded_vs_one_gpu": {"max_rel_h": rel_vs_one, "max_rel_gwx": rel_g_vs_one},
            "per_pass_accounting_gbs": BYTES_STEP * units / sec / 1e9,
            "timing": "CUDA events, max over ranks; one-GPU time measured on rank 0 in the same run"}
        assert parity["ok"] and status == 0, record
        del keep["one"], wx_full, G_full
    torch.cuda.empty_cache()
    barrier()
    return record


def c5_sharded_record(args, rank, world, dev, dist, barrier):
    """The 12-layer ParaNLRU residual stack (d=768, bf16, B=4, T=8192, max_iters=2, seed 4) with
    the sequence sharded over the N ranks, forward + backward through newton_apply, against the
    same stack on one GPU.  Latency-dominated by construction (1024 steps per rank at N = 8)."""
    import torch

    import pararnn_b200 as prb
    from pararnn_b200.seq_shard import time_shard_bounds

    Bc, Tc, Dc, layers, vocab = 4, 8192, 768, 12, 50304
    torch.manual_seed(4)
    cells = []
    for _ in range(layers):
        c = prb.ParaNLRU(Dc, Dc)
        with torch.no_grad():
            a0 = torch.empty(Dc).uniform_(0.9, 0.999)
            c.W_x.bias[:Dc] = torch.log(a0 / (1 - a0))
        cells.append(c.to(dev, torch.bfloat16))
    emb = (torch.randn(vocab, Dc) * 0.02).to(dev, torch.bfloat16)
    ids = torch.randint(0, vocab, (Bc, Tc)).to(dev)
    norm = torch.nn.RMSNorm(Dc).to(dev, torch.bfloat16)
    lo, hi = time_shard_bounds(Tc, rank, world)
    cfg_sh = prb.NewtonConfig(max_iters=2, scan_backend="context_parallel", residual_fail=None)
    cfg_one = prb.NewtonConfig(max_iters=2, residual_fail=None)
    keep = {}

    def stack(ids_, cfg):
        h = emb[ids_].requires_grad_(True)
        for c in cells:
            h = h + prb.newton_apply(c, norm(h), cfg)
        keep["h"] = h.detach()
        h.float().sum().backward()

    def sharded():
        stack(ids[:, lo:hi], cfg_sh)

    n_steps = max(3, min(args.steps, 10))
    for _ in range(3):
        sharded()
    sec = _max_over_ranks(dist, dev, time_region(sharded, n_steps, None, barrier)) / n_steps
    h_all = gather_time(dist, dev, world, keep["h"][0, :, :PARITY_CH].float().contiguous())
    record = None
    if rank == 0:
        def one_gpu():
            stack(ids, cfg_one)

        for _ in range(3):
            one_gpu()
        one_sec = time_region(one_gpu, n_steps, None) / n_steps
        h_one = keep["h"][0, :, :PARITY_CH].float()
        rel = float((h_all - h_one).abs().max() / h_one.abs().max())
        record = {"workload": f"{layers} x ParaNLRU d={Dc} bf16 B={Bc} T={Tc} K=2 pre-norm residual stack, "
                              "forward + backward through newton_apply (layer boundary)",
                  "n_gpus": world, "ms_per_step": sec * 1e3, "tokens_per_s": Bc * Tc / sec,
                  "one_gpu_ms_per_step": one_sec * 1e3, "one_gpu_tokens_per_s": Bc * Tc / one_sec,
                  "speedup": one_sec / sec, "sharded_vs_one_gpu_max_rel_out": rel, "tol": PARITY_TOL}
        assert rel <= PARITY_TOL, record
    for c in cells:
        c.zero_grad(set_to_none=True)
    barrier()
    return record


def run_reference_gpu(args):
    """`--workload ref_fused`: the REFERENCE's own GPU path (its Triton kernels behind
    scan_backend="fused", and its eager PyTorch path on CUDA) timed on this GPU next to this backend
    on the same tensors -- a secondary comparison, not the `--impl reference` arm (which stays the
    CPU path).  Needs the importable copy of the reference that `oracle/make_ref.py` creates; prints
    one JSON line per case, with the error text where the reference's path does not run."""
    import torch

    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "pararnn")):
        print(json.dumps({"workload": "ref_fused", "unavailable": "no copy of the reference under oracle/_ref"}))
        return
    sys.path.insert(0, ref_dir)
    import logging

    logging.disable(logging.WARNING)
    import pararnn as ref

    import pararnn_b200 as prb

    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)

    def timed(fn, n=5):
        for _ in range(2):
            fn()
        return time_region(fn, n, None) / n

    cases = [("slstm_diag d=1024 bf16 B=1 T=16384 K=2 P=5 (one row of C2)", "slstm", 1024, 1, 16384, torch.bfloat16, 2, 5),
             ("slstm_diag d=1024 fp32 B=1 T=4096 K=2 P=3", "slstm", 1024, 1, 4096, torch.float32, 2, 3),
             ("nlru d=768 bf16 B=4 T=8192 K=2 (one layer of C5)", "nlru", 768, 4, 8192, torch.bfloat16, 2, None),
             ("gru_diag d=64 fp32 B=2 T=1024 K=3 (C1)", "gru", 64, 2, 1024, torch.float32, 3, None)]
    for label, kind, d, Bc, Tc, dtype, K, P in cases:
        torch.manual_seed(1)
        mk = {"slstm": lambda m: m.ParaSLSTM(d, d), "nlru": lambda m: m.ParaNLRU(d, d), "gru": lambda m: m.ParaGRU(d, d)}[kind]
        cell_ref = mk(ref).to(dev)
        if kind == "slstm":
            with torch.no_grad():
                cell_ref.W_x.bias[d:2 * d] = 3.0
        cell_ref = cell_ref.to(dtype)
        cell_ours = mk(prb).to(dev, dtype)
        cell_ours.load_state_dict(cell_ref.state_dict())
        x = ((0.5 if kind == "slstm" else 1.0) * torch.randn(Bc, Tc, d, device=dev)).to(dtype)
        line = {"workload": "ref_fused", "case": label, "tokens": Bc * Tc}

        def run(module, cell, backend):
            cfg = module.NewtonConfig(max_iters=K, scan_backend=backend, picard_iters=P, picard_adapt=False,
                                      residual_atol=None, residual_fail=None)
            xin = x.detach().requires_grad_(True)
            H = module.newton_apply(cell, xin, cfg)
            (H.float().sum() if kind != "slstm" else H[:, :, 3].float().sum()).backward()
            cell.zero_grad(set_to_none=True)
            return H.detach()

        for name, module, cell, backend in (("ours", prb, cell_ours, "fused"),
                                            ("reference_fused_triton", ref, cell_ref, "fused"),
                                            ("reference_eager_cuda", ref, cell_ref, "eager")):
            if name == "reference_eager_cuda" and Bc * Tc * d > 2 ** 24:
                line[name] = "skipped: the eager path materialises the (B,T,S,S,d) Jacobian"
                continue
            try:
                H = run(module, cell, backend)
                sec = timed(lambda: run(module, cell, backend))
                line[name + "_ms"] = sec * 1e3
                if name == "ours":
                    H_ours = H
                else:
                    a = H if kind != "slstm" else H[:, :, 3]
                    b = H_ours if kind != "slstm" else H_ours[:, :, 3]
                    line[name + "_max_rel_vs_ours"] = float((a.float() - b.float()).abs().max() / b.float().abs().max())
            except Exception as exc:
                line[name] = "error: " + repr(exc)[:400]
        print(json.dumps(line), flush=True)


def run_secondary(args):
    """Other BASELINE configurations (one JSON line each): `--workload c1|c3|c5`.
    c1: ParaGRU diag fp32 B=2 T=1024 d=64 K=3; c3: ParaGRU head 8x64 B=16 T=4096 K=3 (fp32 and
    bf16); c5: 12 x ParaNLRU d=768 bf16 B=4 T=8192 K=2 residual stack.  Forward + backward through
    newton_apply (layer boundary: includes the W_x GEMMs), CUDA events, inputs resident in HBM.
    `--seq-len` shortens c3 / c5 for profiling captures."""
    import torch

    import pararnn_b200 as prb

    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    t_c3 = args.seq_len if args.seq_len != DEFAULT_T else 4096
    t_c5 = args.seq_len if args.seq_len != DEFAULT_T else 8192

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        return time_region(fn, args.steps, None) / args.steps

    lines = []
    if args.workload == "c1":
        torch.manual_seed(0)
        cell = prb.ParaGRU(64, 64).to(dev)
        torch.nn.init.xavier_uniform_(cell.W_x.weight)
        x = torch.randn(2, 1024, 64, device=dev, requires_grad=True)
        cfg = prb.NewtonConfig(max_iters=3)

        def step():
            prb.newton_apply(cell, x, cfg).sum().backward()

        sec = timed(step)
        rep = prb.verify_agreement(cell, x.detach(), config=cfg)
        lines.append({"workload": "c1 ParaGRU diag fp32 B=2 T=1024 d=64 K=3", "ms_per_step": sec * 1e3,
                      "tokens_per_s": 2 * 1024 / sec, "agreement_max_abs": rep.max_abs,
                      "newton_iters": rep.newton_iters})
    elif args.workload == "lstm":
        # not a BASELINE configuration: ParaLSTM at C2's shape (or --seq-len), op and layer boundary
        from pararnn_b200 import ops

        t_l = args.seq_len if args.seq_len != DEFAULT_T else 16384
        torch.manual_seed(5)
        cell = prb.ParaLSTM(1024, 1024).to(dev, torch.bfloat16)
        x = (0.5 * torch.randn(8, t_l, 1024, device=dev)).bfloat16().requires_grad_(True)
        cfg = prb.NewtonConfig(max_iters=2)
        with torch.no_grad():
            wx = cell.W_x(x).contiguous()
            rec = [p_.detach() for p_ in cell.clipped_recurrent()]
            G = torch.randn(8, t_l, 2, 1024, device=dev).bfloat16()
            Hs = ops.newton_lstm_fused(wx, *rec, None, max_iters=2)
        fwd = timed(lambda: ops.newton_lstm_fused(wx, *rec, None, max_iters=2))
        bwd = timed(lambda: ops.lstm_reverse_vjp(Hs, wx, *rec, G))

        def step():
            prb.newton_apply(cell, x, cfg, output_slot=1).float().sum().backward()

        sec = timed(step)
        lines.append({"workload": f"ParaLSTM d=1024 bf16 B=8 T={t_l} K=2", "op_fwd_ms": fwd * 1e3,
                      "op_bwd_ms": bwd * 1e3, "op_tokens_per_s": 8 * t_l / (fwd + bwd),
                      "layer_ms_per_step": sec * 1e3})
    elif args.workload == "c3":
        for dtype in (torch.float32, torch.bfloat16):
            torch.manual_seed(2)
            cell = prb.ParaGRU(512, 512, mix="head", n_heads=8)
            with torch.no_grad():
                torch.nn.init.xavier_uniform_(cell.W_x.weight)
                for A in (cell.A_z, cell.A_r, cell.A_n):
                    for hd in range(8):
                        torch.nn.init.orthogonal_(A[hd], gain=0.9)
            cell = cell.to(dev, dtype)
            x = torch.randn(16, t_c3, 512, device=dev, dtype=dtype, requires_grad=True)
            cfg = prb.NewtonConfig(max_iters=3)
            st = prb.NewtonStats()

            def step():
                prb.newton_apply(cell, x, cfg, stats=st).float().sum().backward()

            sec = timed(step)
            lines.append({"workload": f"c3 ParaGRU head 8x64 B=16 T={t_c3} K=3 {str(dtype)[6:]}",
                          "ms_per_step": sec * 1e3, "tokens_per_s": 16 * t_c3 / sec,
                          "residual_history": list(st.residual_history), "max_residual": st.max_residual})
    else:
        torch.manual_seed(4)
        cells = []
        for _ in range(12):
            c = prb.ParaNLRU(768, 768)
            with torch.no_grad():
                a0 = torch.empty(768).uniform_(0.9, 0.999)
                c.W_x.bias[:768] = torch.log(a0 / (1 - a0))
            cells.append(c.to(dev, torch.bfloat16))
        emb = (torch.randn(50304, 768) * 0.02).to(dev, torch.bfloat16)
        ids = torch.randint(0, 50304, (4, t_c5), device=dev)
        # no host reads inside the step (residual gate off), so the whole stack can be captured
        cfg = prb.NewtonConfig(max_iters=2, residual_fail=None)
        norm = torch.nn.RMSNorm(768).to(dev, torch.bfloat16)

        # Three readings of "12-layer residual stack": h <- h + cell(rmsnorm(h)) with a weightless
        # RMS norm (the line's `ms_per_step`), the plain
        # residual h <- h + cell(h) (|cell(h)| < 1, so twelve layers stay bounded), and the
        # pre-norm with torch's learnable-gain RMSNorm, whose gain-gradient kernel alone costs 2 ms.
        def step(mode="prenorm"):
            h = emb[ids].requires_grad_(True)
            for c in cells:
                if mode == "prenorm":
                    u = torch.nn.functional.rms_norm(h, (768,))
                elif mode == "affine":
                    u = norm(h)
                else:
                    u = h
                h = h + prb.newton_apply(c, u, cfg)
            h.float().sum().backward()

        sec = timed(step)
        sec_plain = timed(lambda: step("plain"))
        sec_affine = timed(lambda: step("affine"))
        line = {"workload": f"c5 12 x ParaNLRU d=768 bf16 B=4 T={t_c5} K=2 residual stack, "
                            "h <- h + cell(rmsnorm(h))",
                "ms_per_step": sec * 1e3, "tokens_per_s": 4 * t_c5 / sec,
                "plain_residual_ms_per_step": sec_plain * 1e3,
                "prenorm_learnable_gain_ms_per_step": sec_affine * 1e3}
        # the same step (forward + backward of all 12 layers) captured once into a CUDA graph:
        # ~300 short launches (scan kernels, norms, GEMMs, adds) replayed with one host call
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    for c in cells:
                        c.zero_grad(set_to_none=True)
                    norm.zero_grad(set_to_none=True)
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            for c in cells:
                c.zero_grad(set_to_none=True)
            norm.zero_grad(set_to_none=True)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            gsec = timed(graph.replay)
            line.update({"graph_ms_per_step": gsec * 1e3, "graph_tokens_per_s": 4 * t_c5 / gsec})
        except Exception as exc:  # pragma: no cover
            line["graph_error"] = repr(exc)[:300]
        lines.append(line)
    for ln in lines:
        print(json.dumps(ln))


def main():
    global T_PER_GPU
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--seq-len", type=int, default=T_PER_GPU,
                    help="time steps per GPU (profiling captures use a smaller case)")
    ap.add_argument("--first-shard-weight", type=float, default=1.0,
                    help="N > 1: length of the first time shard relative to the others")
    ap.add_argument("--workload", default="c2", choices=("c2", "c1", "c3", "c5", "lstm", "ref_fused"),
                    help="c2 (default) is the headline line; the others print secondary lines")
    ap.add_argument("--c4-seq-len", type=int, default=0,
                    help="N > 1: sequence length of the c4_strong sub-record (default 131072)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 3-second sustained leg")
    ap.add_argument("--no-graph", action="store_true",
                    help="N > 1: issue the sharded programs from Python instead of replaying a CUDA graph")
    ap.add_argument("--no-extra", action="store_true",
                    help="N > 1: skip the c4_strong and c5_sharded sub-records")
    args = ap.parse_args()
    T_PER_GPU = args.seq_len
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "ref_fused":
        run_reference_gpu(args)
        return
    if args.workload != "c2":
        run_secondary(args)
        return
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_gpu_single(args)
    else:
        run_gpu_sharded(args)


if __name__ == "__main__":
    main()
