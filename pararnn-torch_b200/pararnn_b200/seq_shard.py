"""Time-sharded (sequence-parallel) Newton solve: each rank owns a contiguous time shard of
``x`` / ``wx`` / ``H`` and only per-shard scan carries cross ranks.

Counterpart of the reference's context-parallel scan (reference
``solvers/seq_parallel.py:126-342``), which exists for the scalar monoid only, keeps ``H``
replicated and all-gathers the full update every iteration.  Here every cell and every pass type
is sharded, trajectories stay sharded, and one pass costs one small all-gather:

* the first rank in scan direction knows the carry entering its shard and sweeps once;
* every other rank first runs an aggregate-only sweep (mode 2 of the pass-level C ABI) that
  yields the affine map of its whole shard, the maps are all-gathered, ``prb_fold_carries`` turns
  them into the carry entering the rank, and a second sweep applies it;
* when a rank has fewer (batch row, channel block) chains than its GPU has SMs, its shard is cut
  further into time segments that different thread blocks sweep at the same time (ParaSLSTM
  passes): the same aggregate / carry / apply scheme one level down, folded on the device by
  ``prb_fold_segments`` and ``prb_segment_carries`` with no further collective.

The per-rank algorithm is written as a generator that yields its collectives.  ``DistComm``
fulfils them with ``torch.distributed`` (one process per GPU); ``run_lockstep`` fulfils them for
several ranks inside one process, which is how the multi-rank path is tested on a single GPU and,
with a CPU stand-in for the local kernels, on CPU.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
from torch import Tensor


def time_shard_bounds(time: int, rank: int, world_size: int) -> tuple[int, int]:
    """Contiguous ``[start, end)``; the last rank takes the remainder (reference convention,
    ``solvers/seq_parallel.py:126-138``)."""
    if world_size < 1:
        raise ValueError(f"world_size must be >= 1, got {world_size}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank={rank} outside [0, {world_size})")
    if time < 0:
        raise ValueError(f"time must be >= 0, got {time}")
    base = time // world_size
    if rank < world_size - 1:
        return rank * base, (rank + 1) * base
    return (world_size - 1) * base, time


# ------------------------------------------------------------------------------- comms

def balanced_shard_bounds(time: int, rank: int, world_size: int, first_weight: float = 1.8,
                          multiple: int = 1) -> tuple[int, int]:
    """Contiguous ``[start, end)`` with the first shard ``first_weight`` times as long as each of
    the others (their length a multiple of ``multiple``).  The first rank knows the state entering
    its shard and sweeps once per pass while the others sweep twice (aggregate, then apply); the
    others' apply sweep waits for the first rank's result, so the best weight depends on the ratio
    of the sweep costs and is close to 1 for ParaSLSTM (measured).  ``first_weight=1`` gives equal
    shards with the remainder on the first rank."""
    if world_size < 1 or not 0 <= rank < world_size or time < 0 or first_weight <= 0 or multiple < 1:
        raise ValueError("bad arguments to balanced_shard_bounds")
    if world_size == 1:
        return 0, time
    other = int(time / (first_weight + world_size - 1)) // multiple * multiple
    first = time - (world_size - 1) * other
    if rank == 0:
        return 0, first
    return first + (rank - 1) * other, first + rank * other


class DistComm:
    """Collectives over a ``torch.distributed`` process group."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def gather(self, t: Tensor) -> Tensor:
        flat = t.contiguous().view(-1)
        out = torch.empty(self.world * flat.numel(), dtype=t.dtype, device=t.device)
        self.dist.all_gather_into_tensor(out, flat, group=self.group)
        return out.view(self.world, *t.shape)

    def reduce_max(self, t: Tensor) -> Tensor:
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX, group=self.group)
        return t

    def reduce_sum(self, t: Tensor) -> Tensor:
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM, group=self.group)
        return t


def drive(program, comm: DistComm):
    """Run one rank's program, fulfilling its collectives with ``comm``."""
    try:
        req = next(program)
        while True:
            op, t = req
            res = getattr(comm, op)(t)
            req = program.send(res)
    except StopIteration as stop:
        return stop.value


def run_lockstep(programs):
    """Run the programs of all ranks in one process, in lockstep (single-device emulation)."""
    n = len(programs)
    results, reqs, alive = [None] * n, [None] * n, [True] * n
    for i, p in enumerate(programs):
        try:
            reqs[i] = next(p)
        except StopIteration as stop:
            results[i], alive[i] = stop.value, False
    while any(alive):
        assert all(alive), "ranks disagree on the number of collectives"
        ops = {r[0] for r in reqs}
        assert len(ops) == 1, f"ranks disagree on the collective: {ops}"
        op = ops.pop()
        tensors = [r[1] for r in reqs]
        if op == "gather":
            stacked = torch.stack([t.contiguous() for t in tensors])
            answers = [stacked.clone() for _ in range(n)]
        elif op == "reduce_max":
            m = torch.stack(tensors).amax(0)
            answers = [m.clone() for _ in range(n)]
        elif op == "reduce_sum":
            m = torch.stack(tensors).sum(0)
            answers = [m.clone() for _ in range(n)]
        else:
            raise ValueError(op)
        for i, p in enumerate(programs):
            try:
                reqs[i] = p.send(answers[i])
            except StopIteration as stop:
                results[i], alive[i] = stop.value, False
    return results


# ------------------------------------------------------------------------------- local ops

MONOID = {"affine1": 0, "affine4": 1, "picard": 2}
NV = {"affine1": 2, "affine4": 20, "picard": 4}
NS = {"affine1": 1, "affine4": 4, "picard": 3}


@dataclass
class ShardResult:
    states: Tensor               # local shard of H in the I/O dtype
    halo: Tensor | None          # fp32 state preceding the shard (None on rank 0 without h0)
    stats_bits: Tensor           # int32 view of the statistics block, max-reduced over ranks


class CudaShardOps:
    """Local scan passes of one rank on its GPU, through the pass-level C ABI."""

    def __init__(self, kind: str, wx: Tensor, rec: tuple[Tensor, ...], eps: float, omega: float,
                 segments: int | None = None):
        from . import _lib as L
        from . import ops

        self.L, self.ops, self.lib = L, ops, L.lib()
        self.kind, self.wx, self.eps, self.omega = kind, wx.contiguous(), float(eps), float(omega)
        self.dev = wx.device
        self.code = ops._dtype_code(wx)
        self.B, self.T = wx.shape[:2]
        gates = {"gru_diag": 3, "nlru": 2, "slstm_diag": 4}[kind]
        self.d = wx.shape[2] // gates
        self.cell = {"gru_diag": L.CELL_GRU_DIAG, "nlru": L.CELL_NLRU, "slstm_diag": L.CELL_SLSTM_DIAG}[kind]
        self.slots = 4 if kind == "slstm_diag" else 1
        self.par = torch.stack([p.detach().float().reshape(-1) for p in rec]).contiguous() \
            if kind != "slstm_diag" else rec[0].detach().float().contiguous()
        with torch.cuda.device(self.dev):
            n = self.lib.prb_pass_workspace_bytes(self.cell, self.B, self.T, self.d)
        self.ws = torch.empty(max(n, 256), dtype=torch.uint8, device=self.dev)
        self.stats = ops.DeviceStats(self.dev, L.MAX_ITERS)
        self.monoid = "affine4" if kind == "slstm_diag" else "affine1"
        self.launches = 0  # kernels of this library launched through this object
        # time segments inside this rank's shard: the library's plan, or `segments` pieces (tests)
        self.n_seg, self.seg_len = 1, int(self.T)
        if kind == "slstm_diag":
            if segments is None:
                n, ln = ctypes.c_int(1), ctypes.c_int(int(self.T))
                with torch.cuda.device(self.dev):
                    rc = self.lib.prb_plan_segments(self.cell, self.code, self.B, self.T, self.d,
                                                    ctypes.byref(n), ctypes.byref(ln))
                self._check(rc, "plan_segments")
                self.n_seg, self.seg_len = n.value, ln.value
            elif segments > 1 and self.T >= 64:
                # at least 32 steps per segment (the workspace has one partial row per 32 steps)
                ln = max(32, -(-int(self.T) // int(segments)))
                self.n_seg, self.seg_len = -(-int(self.T) // ln), ln

    # helpers
    def _p(self, t):
        return None if t is None else ctypes.c_void_p(t.data_ptr())

    def _stream(self):
        return self.ops._stream(self.dev)

    def _check(self, rc, what):
        self.ops._raise(rc, what)

    def new_traj(self):
        shape = (self.B, self.T, 4, self.d) if self.slots == 4 else (self.B, self.T, self.d)
        return torch.empty(shape, dtype=torch.float32, device=self.dev)

    def new_out(self):
        shape = (self.B, self.T, 4, self.d) if self.slots == 4 else (self.B, self.T, self.d)
        return torch.empty(shape, dtype=self.wx.dtype, device=self.dev)

    def fold_segments(self, monoid: str, agg: Tensor, reverse: bool) -> Tensor:
        """Map of the whole shard from its segment maps ``(n_seg, B, NV, d)``."""
        out = torch.empty(self.B, NV[monoid], self.d, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.lib.prb_fold_segments(MONOID[monoid], self._p(agg), agg.shape[0], int(reverse),
                                            self._p(out), self.B, self.d, self._stream())
        self._check(rc, "fold_segments")
        self.launches += 1
        return out

    def segment_carries(self, monoid: str, agg: Tensor, reverse: bool, carry0: Tensor | None) -> Tensor:
        """``(n_seg + 1, B, NS, d)``: the carry entering every segment, then the one leaving the shard."""
        n = agg.shape[0]
        out = torch.empty(n + 1, self.B, NS[monoid], self.d, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.lib.prb_segment_carries(MONOID[monoid], self._p(agg), n, int(reverse), self._p(carry0),
                                              self._p(out), self.B, self.d, self._stream())
        self._check(rc, "segment_carries")
        self.launches += 1
        return out

    def fold(self, monoid: str, gathered: Tensor, rank: int, world: int, reverse: bool) -> Tensor:
        out = torch.empty(self.B, NS[monoid], self.d, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.lib.prb_fold_carries(MONOID[monoid], self._p(gathered), rank, world, int(reverse),
                                           self._p(out), self.B, self.d, self._stream())
        self._check(rc, "fold_carries")
        self.launches += 1
        return out

    def shard_carries(self, monoid: str, gathered: Tensor, rank: int, world: int, reverse: bool,
                      agg: Tensor | None, want_h_end: bool = False):
        """``fold`` and ``segment_carries`` in one launch on the gathered slots as they are (the
        map rows first, anything riding along after them).  Returns ``(carry entering the rank,
        carries entering its segments + the one leaving it or None, h_end or None)``; ``h_end`` is
        the hidden value at the previous rank's last step (frozen-gate passes)."""
        n_seg = 1 if agg is None else agg.shape[0]
        carry = torch.empty(self.B, NS[monoid], self.d, dtype=torch.float32, device=self.dev)
        carries = None
        if agg is not None and n_seg > 1:
            carries = torch.empty(n_seg + 1, self.B, NS[monoid], self.d, dtype=torch.float32, device=self.dev)
        h_end = torch.empty(self.B, self.d, dtype=torch.float32, device=self.dev) if want_h_end else None
        with torch.cuda.device(self.dev):
            rc = self.lib.prb_shard_carries(MONOID[monoid], self._p(gathered), gathered.shape[2], rank, world,
                                            int(reverse), self._p(agg), n_seg, self._p(carry), self._p(carries),
                                            float(self.eps), self._p(h_end), self.B, self.d, self._stream())
        self._check(rc, "shard_carries")
        self.launches += 1
        return carry, carries, h_end

    def diag_guess(self, h0):
        out = self.new_traj()
        with torch.cuda.device(self.dev):
            rc = self.lib.prb_diag_guess(self.cell, self._p(self.wx), self._p(self.par), self._p(h0),
                                         self._p(out), self.B, self.T, self.d, self.code, self._stream())
        self._check(rc, "diag_guess")
        self.launches += 1
        return out

    def newton_pass(self, traj, halo, carry, mode, out, hist_slot):
        """mode 0/1: applies ``carry`` (per segment: ``(n_seg, B, NS, d)``) and returns the carry
        leaving the shard; mode 2: returns the segment aggregates ``(n_seg, B, NV, d)``."""
        nv, ns = NV[self.monoid], NS[self.monoid]
        if mode == 2:
            res = torch.empty(self.n_seg, self.B, nv, self.d, dtype=torch.float32, device=self.dev)
        else:
            res = torch.empty(self.B, ns, self.d, dtype=torch.float32, device=self.dev)
        tail = None if mode == 2 else res
        agg = res if mode == 2 else None
        with torch.cuda.device(self.dev):
            if self.kind == "slstm_diag":
                rc = self.lib.prb_slstm_newton_pass(
                    self._p(self.wx), self._p(self.par), self._p(traj), self._p(halo), self._p(carry),
                    self._p(out), self._p(tail), self._p(agg), mode, self.n_seg, self.seg_len, self.B,
                    self.T, self.d, self.code,
                    self.omega, self.eps, self._p(self.ws), self.ws.numel(), self._p(self.stats.buf),
                    hist_slot, self._stream())
            else:
                rc = self.lib.prb_diag_newton_pass(
                    self.cell, self._p(self.wx), self._p(self.par), self._p(traj), self._p(halo),
                    self._p(carry), self._p(out), self._p(tail), self._p(agg), mode, self.B, self.T, self.d,
                    self.code, self.omega, self._p(self.ws), self.ws.numel(), self._p(self.stats.buf),
                    hist_slot, self._stream())
        self._check(rc, "newton_pass")
        self.launches += 1
        return res

    def picard_pass(self, h_prev, h_halo, carry, mode, h_out, state_out):
        if mode == 2:
            res = torch.empty(self.n_seg, self.B, 4, self.d, dtype=torch.float32, device=self.dev)
        else:
            res = torch.empty(self.B, 3, self.d, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.lib.prb_slstm_picard_pass(
                self._p(self.wx), self._p(self.par), self._p(h_prev), self._p(h_halo), self._p(carry),
                self._p(h_out), self._p(state_out), self._p(None if mode == 2 else res),
                self._p(res if mode == 2 else None), mode, self.n_seg, self.seg_len, self.B, self.T, self.d,
                self.code, self.eps,
                self._p(self.ws), self.ws.numel(), self._p(self.stats.buf), self._stream())
        self._check(rc, "picard_pass")
        self.launches += 1
        return res

    def bwd_pass(self, states, grad_states, halo, carry, mode):
        """mode 0: returns (g_wx, g_params, head); mode 2: returns the aggregate."""
        nv, ns = NV[self.monoid], NS[self.monoid]
        npar = self.par.shape[0]
        st = states.to(self.wx.dtype).contiguous()
        gs = grad_states.to(self.wx.dtype).contiguous()
        if mode == 2:
            agg = torch.empty(self.n_seg, self.B, nv, self.d, dtype=torch.float32, device=self.dev)
            g_wx = g_par = head = None
        else:
            agg = None
            g_wx = torch.empty_like(self.wx)
            g_par = torch.empty(npar, self.d, dtype=torch.float32, device=self.dev)
            head = torch.empty(self.B, ns, self.d, dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            if self.kind == "slstm_diag":
                rc = self.lib.prb_slstm_bwd_pass(
                    self._p(st), self._p(self.wx), self._p(self.par), self._p(halo), self._p(carry),
                    self._p(gs), self._p(g_wx), self._p(g_par), self._p(head), self._p(agg), mode, self.n_seg,
                    self.seg_len, self.B, self.T, self.d, self.code, self.eps, self._p(self.ws),
                    self.ws.numel(), self._p(self.stats.buf), self._stream())
            else:
                rc = self.lib.prb_diag_bwd_pass(
                    self.cell, self._p(st), self._p(self.wx), self._p(self.par), self._p(halo),
                    self._p(carry), self._p(gs), self._p(g_wx), self._p(g_par), self._p(head), self._p(agg),
                    mode, self.B, self.T, self.d, self.code, self._p(self.ws), self.ws.numel(),
                    self._p(self.stats.buf), self._stream())
        self._check(rc, "bwd_pass")
        self.launches += 1 if mode == 2 else 2  # the sweep, and the reduction of the parameter partials
        return agg if mode == 2 else (g_wx, g_par, head)

    def stats_bits(self) -> Tensor:
        return self.stats.buf.view(torch.int32)


# ------------------------------------------------------------------------------- programs

def _pad(t: Tensor, nv: int) -> Tensor:
    """Place a (B, ns, d) carry in the first rows of a (B, nv, d) gather slot."""
    if t.shape[1] == nv:
        return t
    out = t.new_zeros(t.shape[0], nv, t.shape[2])
    out[:, : t.shape[1]] = t
    return out


def _sharded_scan(ops, rank, world, reverse, monoid, boundary, sweep, extra=None, want_h_end=False):
    """One sharded scan pass.  ``sweep(True, None)`` returns the aggregates of the rank's time
    segments ``(n_seg, B, NV, d)``; ``sweep(False, carries)`` applies the carries entering the
    segments ``(n_seg, B, NS, d)`` (None = zeros) and returns the carry leaving the shard.
    ``extra`` (B, E, d) rides along in the rank's gather slot.  Yields at most one gather; returns
    ``(carry entering this rank, carry leaving it, gathered slots or None, h_end or None)``;
    ``h_end`` (``want_h_end``, frozen-gate passes, ranks after the first) is the hidden value at
    the previous rank's last step, from the carry and the gate value in the extra row."""
    first = world - 1 if reverse else 0
    n_seg = getattr(ops, "n_seg", 1)
    nv = NV[monoid]
    gathered = None
    if rank == first:
        if n_seg == 1:
            leaving = sweep(False, boundary)
        else:
            agg = sweep(True, None)
            carries = ops.segment_carries(monoid, agg, reverse, boundary)
            sweep(False, carries)
            leaving = carries[n_seg]
        if world > 1:
            slot = _pad(leaving, nv)
            gathered = yield ("gather", slot if extra is None else torch.cat([slot, extra], dim=1))
        return boundary, leaving, gathered, None
    agg = sweep(True, None)
    slot = agg[0] if n_seg == 1 else ops.fold_segments(monoid, agg, reverse)
    gathered = yield ("gather", slot if extra is None else torch.cat([slot, extra], dim=1))
    h_end = None
    if hasattr(ops, "shard_carries"):
        # one launch: fold of the gathered maps, the segment carries and (frozen-gate passes) h_end
        carry, carries, h_end = ops.shard_carries(monoid, gathered, rank, world, reverse,
                                                  agg if n_seg > 1 else None, want_h_end)
        if carries is None:
            carries = carry
    else:
        maps = gathered if extra is None else gathered[:, :, :nv].contiguous()
        carry = ops.fold(monoid, maps, rank, world, reverse)
        carries = carry if n_seg == 1 else ops.segment_carries(monoid, agg, reverse, carry)
        if want_h_end:
            zo_prev = gathered[rank - 1][:, nv]
            h_end = torch.sigmoid(zo_prev) * carry[:, 0] / (carry[:, 1] + ops.eps)
    leaving = sweep(False, carries)
    return carry, leaving, gathered, h_end


def forward_program(ops, rank: int, world: int, K: int, P: int, h0: Tensor | None):
    """Forward solve of one rank.  ``h0`` (fp32, state layout) is used on rank 0 only.
    Returns a ``ShardResult``."""
    kind = ops.kind
    B, d = ops.B, ops.d
    dev = ops.dev

    def prev_rank_last(t_last: Tensor):
        """Exchange the last state of every rank's shard; returns the previous rank's."""
        gathered = yield ("gather", t_last.contiguous())
        return gathered[rank - 1] if rank > 0 else None

    if kind == "slstm_diag":
        # No halo exchange is needed between the frozen-gate passes: the carry entering a rank is
        # the state (c, n, m) at the previous rank's last step, and with that step's output-gate
        # pre-activation (which the previous rank knows BEFORE the pass and ships in its gather
        # slot) the hidden value at that step follows as sigmoid(zo) c / (n + eps).
        h_prev = None
        h_halo = None if (h0 is None or rank > 0) else h0[:, 3].contiguous()
        carry0 = None if h0 is None or rank > 0 else h0[:, :3].contiguous()
        traj = None
        r_o = ops.par[3]
        wx_o_last = ops.wx[:, -1, 3 * d:].float()
        wx_o = ops.wx[:, :, 3 * d:]
        halo = None
        for p in range(P + 1):
            last = p == P
            h_out = None if last else torch.empty(B, ops.T, d, dtype=torch.float32, device=dev)
            state_out = ops.new_traj() if last else None
            if h_prev is None:
                zo_last = wx_o_last
            elif ops.T >= 2:
                zo_last = torch.addcmul(wx_o_last, r_o, h_prev[:, -2])
            else:
                zo_last = wx_o_last + r_o * (h_halo if h_halo is not None else 0.0)
            def sweep(agg_only, carry, h_prev=h_prev, h_halo=h_halo, h_out=h_out, state_out=state_out):
                if agg_only:
                    return ops.picard_pass(h_prev, h_halo, None, 2, None, None)
                return ops.picard_pass(h_prev, h_halo, carry, 0, h_out, state_out)

            carry, _, gathered, h_end = yield from _sharded_scan(
                ops, rank, world, False, "picard", carry0, sweep,
                extra=zo_last[:, None] if world > 1 else None, want_h_end=world > 1)
            if rank > 0:
                # hidden state at the previous rank's last step under the new trajectory
                h_halo = h_end
                if last:
                    halo = torch.cat([carry, h_end[:, None]], dim=1)
            h_prev = h_out
            traj = state_out
        if rank == 0:
            halo = None if h0 is None else h0.contiguous()
    else:
        traj = ops.diag_guess(h0 if rank == 0 else None)
        halo = None
        if world > 1:
            halo = yield from prev_rank_last(traj[:, -1])
        if rank == 0:
            halo = h0

    out = ops.new_out()
    if K == 0:
        out.copy_(traj)
    for k in range(K):
        last = k == K - 1
        dst = out if last else ops.new_traj()

        def sweep(agg_only, carry, traj=traj, halo=halo, dst=dst, last=last, k=k):
            return ops.newton_pass(traj, halo, carry, 2 if agg_only else (1 if last else 0), dst, k)

        carry, _, _, _ = yield from _sharded_scan(ops, rank, world, False, ops.monoid, None, sweep)
        if rank > 0 and carry is not None:
            # the carry entering the shard is the update of the previous rank's last step
            c = carry if ops.slots == 4 else carry[:, 0]
            halo = halo + ops.omega * c
        traj = dst
    # state preceding the shard in the RETURNED trajectory (used by the backward pass): the old
    # halo plus the last update, rounded like the stored output
    halo_out = halo
    if rank > 0 and K > 0 and halo is not None:
        halo_out = halo.to(out.dtype).float()
    if rank == 0:
        halo_out = h0
    bits = ops.stats_bits().clone()
    if world > 1:
        bits = yield ("reduce_max", bits)
    return ShardResult(out, halo_out, bits)


def backward_program(ops, rank: int, world: int, states: Tensor, grad_states: Tensor,
                     halo: Tensor | None):
    """Reverse scan + packed VJP of one rank.  Returns ``(g_wx, g_params, g_h0)`` with the
    parameter gradients already summed over ranks; ``g_h0`` is meaningful on rank 0."""

    def sweep(agg_only, carry):
        if agg_only:
            return ops.bwd_pass(states, grad_states, halo, None, 2)
        sweep.out = ops.bwd_pass(states, grad_states, halo, carry, 0)
        return sweep.out[2]

    yield from _sharded_scan(ops, rank, world, True, ops.monoid, None, sweep)
    g_wx, g_par, head = sweep.out
    if world > 1:
        g_par = yield ("reduce_sum", g_par)
    return g_wx, g_par, head


# ------------------------------------------------------------------------------- graphed step

class GraphedShardedStep:
    """One rank's forward + backward programs captured ONCE into a CUDA graph and replayed.

    A sharded step is a chain of ~20 short sweeps, ~20 tiny fold kernels and ~10 small NCCL
    all-gathers; at 8 ranks each sweep lasts 0.1-0.4 ms, so issuing them from Python (ctypes calls,
    allocations, slicing) costs as much as running them.  The graph holds the kernels of this
    library, the device-side folds and the collectives (NCCL collectives can be captured), so a
    replay costs one launch on the host.  Inputs are static: write the next step's ``wx`` and
    cotangent into ``self.wx`` / ``self.grad_states`` (for example as the ``out=`` of the ``W_x``
    GEMM) and call ``replay()``; results are in ``self.states``, ``self.g_wx``, ``self.g_params``,
    ``self.head``.  Every rank must construct and replay it in step with the others."""

    def __init__(self, kind: str, wx: Tensor, rec, grad_states: Tensor, comm: DistComm, *, K: int, P: int = 0,
                 eps: float = 1e-6, omega: float = 1.0, h0: Tensor | None = None, warmup: int = 2,
                 segments: int | None = None):
        self.wx, self.grad_states, self.comm = wx.contiguous(), grad_states.contiguous(), comm
        self.K, self.P, self.h0 = int(K), int(P), _h0_f32(h0)
        self.ops = CudaShardOps(kind, self.wx, rec, eps, omega, segments=segments)
        side = torch.cuda.Stream(device=wx.device)
        side.wait_stream(torch.cuda.current_stream(wx.device))
        with torch.cuda.stream(side):  # eager runs first: communicators, kernel attributes, allocator
            for _ in range(max(1, warmup)):
                self._run()
        torch.cuda.current_stream(wx.device).wait_stream(side)
        torch.cuda.synchronize(wx.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._run()

    def _run(self):
        self.ops.stats.buf.zero_()
        res = drive(forward_program(self.ops, self.comm.rank, self.comm.world, self.K, self.P, self.h0),
                    self.comm)
        self.g_wx, self.g_params, self.head = drive(
            backward_program(self.ops, self.comm.rank, self.comm.world, res.states, self.grad_states, res.halo),
            self.comm)
        self.states, self.stats_bits = res.states, res.stats_bits

    def replay(self):
        self.graph.replay()


# ------------------------------------------------------------------------------- public entry

def _bits_to_stats(bits: Tensor, K: int):
    import struct

    raw = bits.cpu().numpy().tobytes()
    vals = struct.unpack("<20i", raw[:80])
    as_f = struct.unpack("<17f", raw[:68])
    return tuple(as_f[:K]), as_f[16], vals[17]


def _h0_f32(h0: Tensor | None):
    return None if h0 is None else h0.detach().float().contiguous()


class _ShardedFixedPoint(torch.autograd.Function):
    """Autograd contract of the time-sharded solve: every rank returns the gradient of its own
    shard of ``x``; parameter gradients are summed over ranks (each rank holds the full sum);
    ``grad_h0`` is non-zero on rank 0."""

    @staticmethod
    def forward(ctx, cell, kind, cfg, stats, comm, has_h0, x_in, h0_in, *params):
        from .newton import _gate, _recurrent_params

        del params
        with torch.no_grad():
            wx = cell.W_x(x_in)
            ops = CudaShardOps(kind, wx, _recurrent_params(cell, kind), getattr(cell, "eps", 1e-6),
                               cfg.omega)
            h0 = _h0_f32(h0_in) if has_h0 else None
            res = drive(forward_program(ops, comm.rank, comm.world, int(cfg.max_iters),
                                        int(cfg.picard_iters or 0), h0), comm)
        if stats is not None or cfg.residual_fail is not None:
            hist, final, status = _bits_to_stats(res.stats_bits, int(cfg.max_iters))
            _gate(cell, x_in, cfg, final, int(cfg.max_iters), hist, stats, status)
        ctx.cell, ctx.kind, ctx.cfg, ctx.comm, ctx.has_h0, ctx.ops = cell, kind, cfg, comm, has_h0, ops
        ctx.halo = res.halo
        ctx.save_for_backward(x_in, h0_in, res.states)
        return res.states

    @staticmethod
    def backward(ctx, grad_states):
        from .newton import _clip_mask

        x_in, h0_in, states = ctx.saved_tensors
        cell, comm, ops = ctx.cell, ctx.comm, ctx.ops
        with torch.no_grad():
            g_wx, g_par, head = drive(backward_program(ops, comm.rank, comm.world, states,
                                                       grad_states, ctx.halo), comm)
            names = {"gru_diag": ("a_z", "a_r", "a_n"), "nlru": ("u",), "slstm_diag": ("R",)}[ctx.kind]
            named = dict(cell.named_parameters())
            cap = getattr(cell, "max_recurrent_norm", None)
            grads = {}
            if ctx.kind == "slstm_diag":
                pieces = {"R": g_par}
            else:
                pieces = {n: g_par[i] for i, n in enumerate(names)}
            for n, g in pieces.items():
                raw = named[n]
                g = g.reshape(raw.shape)
                mask = _clip_mask(raw.detach(), cap)
                grads[n] = (g * mask if mask is not None else g).to(raw.dtype)
            lin = cell.W_x
            gy = g_wx.reshape(-1, g_wx.shape[-1])
            xx = x_in.detach().reshape(-1, x_in.shape[-1])
            grad_x = (gy @ lin.weight.detach().to(gy.dtype)).reshape(x_in.shape)
            gw = (gy.t() @ xx.to(gy.dtype)).float()
            gb = gy.float().sum(0)
            if comm.world > 1:
                gw = comm.reduce_sum(gw)
                gb = comm.reduce_sum(gb)
            grads["W_x.weight"] = gw.to(lin.weight.dtype)
            if lin.bias is not None:
                grads["W_x.bias"] = gb.to(lin.bias.dtype)
        out_params = []
        for name, p in cell.named_parameters():
            g = grads.get(name)
            out_params.append(g if (g is not None and p.requires_grad) else None)
        grad_h0 = None
        if ctx.has_h0 and h0_in.requires_grad:
            g0 = head if ops.slots == 4 else head[:, 0]
            grad_h0 = (g0 if comm.rank == 0 else torch.zeros_like(g0)).to(h0_in.dtype)
        if not x_in.requires_grad:
            grad_x = None
        return (None, None, None, None, None, None, grad_x, grad_h0, *out_params)


def newton_apply_sharded(cell, kind: str, x: Tensor, cfg, *, h0: Tensor | None = None, stats=None,
                         group=None) -> Tensor:
    """``newton_apply`` for ``scan_backend="context_parallel"``: ``x`` is THIS rank's time shard
    ``(B, T_local, d_in)`` (shards follow ``time_shard_bounds``), the result is the matching
    shard of ``H``.  ``h0`` is read on rank 0.  Needs an initialised process group."""
    import torch.distributed as dist

    if kind == "gru_head":
        raise TypeError("time sharding of ParaGRU(mix='head') is not available")
    if cfg.chunk_len is not None or cfg.recompute:
        raise ValueError("chunk_len / recompute cannot be combined with scan_backend='context_parallel'")
    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError("scan_backend='context_parallel' needs torch.distributed.init_process_group")
    comm = DistComm(group)
    params = tuple(cell.parameters())
    has_h0 = h0 is not None
    h0_leaf = h0 if has_h0 else x.new_zeros(())
    cfg2 = cfg
    if cfg.picard_adapt:
        from dataclasses import replace

        cfg2 = replace(cfg, picard_adapt=False)  # the retry ladder is a host loop; pin P when sharding
    if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in params)
                                    or (has_h0 and h0.requires_grad)):
        return _ShardedFixedPoint.apply(cell, kind, cfg2, stats, comm, has_h0, x, h0_leaf, *params)
    with torch.no_grad():
        return _ShardedFixedPoint.forward(_Ctx(), cell, kind, cfg2, stats, comm, has_h0, x, h0_leaf)


class _Ctx:
    """Stand-in for the autograd context when no gradient is needed."""

    def save_for_backward(self, *a):
        pass


def emulate_sharded(kind: str, wx: Tensor, rec, *, world: int, K: int, P: int = 0, h0=None,
                    eps: float = 1e-6, omega: float = 1.0, grad_states: Tensor | None = None,
                    ops_factory=None, bounds=None, segments=None):
    """Run the time-sharded programs of ``world`` virtual ranks in one process on one device
    (shards of ``wx`` along time per ``time_shard_bounds``, or the contiguous ``bounds`` given:
    shards need not have equal lengths).  Returns the concatenated states, the statistics bits and,
    when ``grad_states`` is given, ``(g_wx, g_params, g_h0)``."""
    factory = ops_factory or CudaShardOps
    T = wx.shape[1]
    if bounds is None:
        bounds = [time_shard_bounds(T, r, world) for r in range(world)]
    if len(bounds) != world or bounds[0][0] != 0 or bounds[-1][1] != T or any(
            bounds[i][1] != bounds[i + 1][0] for i in range(world - 1)):
        raise ValueError(f"bounds must be {world} contiguous [start, end) pairs covering [0, {T})")
    extra = {} if segments is None else {"segments": segments}
    ops = [factory(kind, wx[:, s:e].contiguous(), rec, eps, omega, **extra) for s, e in bounds]
    res = run_lockstep([forward_program(ops[r], r, world, K, P, _h0_f32(h0)) for r in range(world)])
    states = torch.cat([r.states for r in res], dim=1)
    out = [states, res[0].stats_bits]
    if grad_states is not None:
        back = run_lockstep([
            backward_program(ops[r], r, world, res[r].states, grad_states[:, s:e].contiguous(), res[r].halo)
            for r, (s, e) in enumerate(bounds)])
        out.append((torch.cat([b[0] for b in back], dim=1), back[0][1], back[0][2]))
    return tuple(out)
