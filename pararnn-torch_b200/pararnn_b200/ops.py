"""Operators of the CUDA backend, one per fused op of the reference.

Names, argument order and error behaviour follow the reference's custom ops
(``pararnn::newton_gru_fused`` etc., reference ``kernels/custom_ops.py:146-540``)
and its packed VJP functions (reference ``kernels/vjp_*.py``).  Each function
validates its tensors, allocates outputs and scratch through PyTorch's caching
allocator, and calls the C ABI on the current CUDA stream.  Nothing here computes
on the host, and there is no fallback: without a CUDA device or without the built
library the functions raise.
"""

from __future__ import annotations

import ctypes
import struct

import torch
from torch import Tensor

from . import _lib as L

_DTYPES = {torch.float32: L.PRB_F32, torch.bfloat16: L.PRB_BF16}


def _dtype_code(t: Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(
            f"pararnn_b200 kernels take float32 or bfloat16 tensors, got {t.dtype}"
        ) from None


def _check_cuda(*tensors: Tensor | None) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "pararnn_b200 operators need CUDA tensors (this backend has no CPU path); "
                f"got a tensor on {t.device}"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


def _ptr(t: Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _same(t: Tensor | None, ref: Tensor) -> Tensor | None:
    """Contiguous copy in the I/O dtype of ``ref`` (the reference copies non-contiguous inputs)."""
    if t is None:
        return None
    return t.detach().to(dtype=ref.dtype).contiguous()


def _workspace(nbytes: int, device) -> Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _raise(code: int, what: str) -> None:
    if code == 0:
        return
    msg = f"{what}: {L.error_string(code)} (code {code})"
    if code in (-1, -3, -5):
        raise ValueError(msg)
    raise RuntimeError(msg)


class DeviceStats:
    """Handle on the device-side statistics block of one forward call.  A packed (``cu_seqlens``)
    call solves its segments one after the other; their blocks hang off ``parts`` and ``read``
    merges them (max over segments, NaN wins, as one solve over the packed batch would report)."""

    def __init__(self, device, max_iters: int):
        self.buf = torch.zeros(L.STATS_BYTES, dtype=torch.uint8, device=device)
        self.max_iters = int(max_iters)
        self.parts: list[DeviceStats] = []

    @staticmethod
    def _unpack(raw: bytes):
        hist = struct.unpack(f"<{L.MAX_ITERS}f", raw[: 4 * L.MAX_ITERS])
        final = struct.unpack("<f", raw[4 * L.MAX_ITERS: 4 * L.MAX_ITERS + 4])[0]
        status = struct.unpack("<i", raw[4 * L.MAX_ITERS + 4: 4 * L.MAX_ITERS + 8])[0]
        return hist, final, status

    def read(self) -> tuple[tuple[float, ...], float, int]:
        """One small device-to-host copy: (residual_history, final max|F|, status)."""
        if not self.parts:
            hist, final, status = self._unpack(bytes(self.buf.cpu().numpy().tobytes()))
            return tuple(hist[: self.max_iters]), final, status
        rows = torch.stack([p.buf for p in self.parts]).cpu().numpy()

        def worse(a, b):
            return b if (b != b or (a == a and b > a)) else a

        hist, final, status = [0.0] * L.MAX_ITERS, 0.0, 0
        for row in rows:
            h, f, st = self._unpack(row.tobytes())
            hist = [worse(a, b) for a, b in zip(hist, h)]
            final = worse(final, f)
            status |= st
        return tuple(hist[: self.max_iters]), final, status


# Statistics blocks of reverse-scan calls whose status word nobody has looked at yet.  Reading one
# costs a device-to-host copy, so the backward functions do not do it themselves: the next forward
# that reads its own statistics checks them in the same breath (check_pending_backward).
_pending_backward: list[DeviceStats] = []


def _track_backward(sb: DeviceStats) -> None:
    _pending_backward.append(sb)
    if len(_pending_backward) > 64:
        del _pending_backward[0]


def check_pending_backward() -> None:
    """Raise if a reverse scan issued since the last check ran into a bounded device-side wait
    that gave up (its gradients are not valid).  One small device-to-host copy per device."""
    if not _pending_backward:
        return
    pending, _pending_backward[:] = list(_pending_backward), []
    by_dev: dict = {}
    for sb in pending:
        by_dev.setdefault(sb.buf.device, []).append(sb.buf)
    for bufs in by_dev.values():
        raw = torch.stack(bufs).cpu().numpy()
        for row in raw:
            status = struct.unpack("<i", row.tobytes()[4 * L.MAX_ITERS + 4: 4 * L.MAX_ITERS + 8])[0]
            if status != 0:
                raise RuntimeError(
                    "pararnn_b200: a bounded device-side wait ran out during an earlier reverse scan "
                    f"(status {status}); the gradients of that backward call are not valid")


def validate_cu_seqlens(cu_seqlens: Tensor, time: int) -> list[int]:
    """Exclusive prefix ``(S+1,)`` with ``[0] = 0``, strictly increasing, last ``= time``
    (same checks and messages as the reference's ``layout.validate_cu_seqlens``,
    ``layout.py:93-106``).  Returns the offsets as Python ints (one host read)."""
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2:
        raise ValueError(f"cu_seqlens must be (S+1,), got {tuple(cu_seqlens.shape)}")
    cs = [int(v) for v in cu_seqlens.tolist()]
    if cs[0] != 0:
        raise ValueError(f"cu_seqlens[0] must be 0, got {cs[0]}")
    if cs[-1] != int(time):
        raise ValueError(f"cu_seqlens[-1] must equal time={time}, got {cs[-1]}")
    if any(b <= a for a, b in zip(cs[:-1], cs[1:])):
        raise ValueError("cu_seqlens must be strictly increasing")
    return cs


def gather_h0(h0: Tensor | None, block_table: Tensor | None, rows: int, tail: tuple[int, ...]) -> Tensor | None:
    """Paged initial state: with ``block_table`` (``(rows,)`` slot ids) ``h0`` is a pool
    ``(C, *tail)`` and row ``i`` of the batch starts from ``h0[block_table[i]]`` (reference
    ``kernels/_fused_common.py:106-139``, same checks)."""
    if block_table is None:
        return h0
    if h0 is None:
        raise ValueError("block_table needs h0 as a pool (C, …)")
    if block_table.dim() != 1:
        raise ValueError(f"block_table must be 1-D (B,), got {tuple(block_table.shape)}")
    if int(block_table.numel()) != rows:
        raise ValueError(f"block_table B={int(block_table.numel())} != {rows}")
    if tuple(h0.shape[1:]) != tuple(tail):
        raise ValueError(f"pool h0 tail {tuple(h0.shape[1:])} != {tuple(tail)}")
    if int(h0.shape[0]) < 1:
        raise ValueError("pool h0 is empty")
    bt = block_table.to(device=h0.device, dtype=torch.long)
    mn, mx = int(bt.min().item()), int(bt.max().item())
    if mn < 0 or mx >= int(h0.shape[0]):
        raise ValueError(f"block_table slots [{mn}, {mx}] outside pool capacity {int(h0.shape[0])}")
    return h0.index_select(0, bt)


def _packed(fn, wx: Tensor, h0: Tensor | None, cu_seqlens: Tensor, block_table: Tensor | None,
            tail: tuple[int, ...], stats: "DeviceStats | None", states: Tensor | None = None) -> Tensor:
    """A packed batch ``(1, N, ...)`` of S sequences (``cu_seqlens``): every sequence is its own
    scan with its own initial state ``h0[s]`` and nothing carried over the segment heads
    (reference ``layout.py:121-138``, ``kernels/newton_gru.py:205-236``).  The segments are solved
    one after the other with the rectangular kernels; ``fn(wx_seg, h0_seg, stats_seg, guess_seg)``."""
    if wx.shape[0] != 1:
        raise ValueError(f"cu_seqlens packs x with batch=1, got batch={wx.shape[0]}")
    cs = validate_cu_seqlens(cu_seqlens, wx.shape[1])
    n_seq = len(cs) - 1
    h0 = gather_h0(h0, block_table, n_seq, tail)
    if h0 is not None and h0.shape[0] != n_seq:
        raise ValueError(f"h0 batch {h0.shape[0]} != n_seq {n_seq}")
    outs = []
    for i in range(n_seq):
        st = None
        if stats is not None:
            st = DeviceStats(wx.device, stats.max_iters)
            stats.parts.append(st)
        outs.append(fn(wx[:, cs[i]:cs[i + 1]], None if h0 is None else h0[i:i + 1], st,
                       None if states is None else states[:, cs[i]:cs[i + 1]]))
    return torch.cat(outs, dim=1)


def _check_iters(max_iters: int) -> None:
    if not 0 <= int(max_iters) <= L.MAX_ITERS:
        raise ValueError(f"max_iters must be in [0, {L.MAX_ITERS}], got {max_iters}")


# ---------------------------------------------------------------------------- forward

def newton_gru_fused(wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor, h0: Tensor | None = None,
                     cu_seqlens: Tensor | None = None, block_table: Tensor | None = None, *,
                     max_iters: int, omega: float = 1.0, stats: DeviceStats | None = None,
                     want_residual: bool = True) -> Tensor:
    """Fused Newton for ``ParaGRU(mix='diag')``: ``wx (B,T,3d)`` -> ``H (B,T,d)`` in ``wx.dtype``.
    With ``cu_seqlens`` ``wx`` is a packed ``(1, N, 3d)`` batch and ``h0`` is ``(S, d)``; with
    ``block_table`` ``h0`` is a pool ``(C, d)``."""
    if cu_seqlens is not None:
        if stats is not None:
            stats.parts.clear()
        return _packed(lambda w, h, st, _g: newton_gru_fused(w, a_z, a_r, a_n, h, max_iters=max_iters,
                                                              omega=omega, stats=st,
                                                              want_residual=want_residual),
                       wx, h0, cu_seqlens, block_table, (a_z.numel(),), stats)
    h0 = gather_h0(h0, block_table, wx.shape[0], (a_z.numel(),))
    dev = _check_cuda(wx, a_z, a_r, a_n, h0)
    _check_iters(max_iters)
    if wx.dim() != 3 or wx.shape[-1] % 3:
        raise ValueError(f"wx must be (B, T, 3*d), got {tuple(wx.shape)}")
    B, T, d3 = wx.shape
    d = d3 // 3
    for name, p in (("a_z", a_z), ("a_r", a_r), ("a_n", a_n)):
        if p.numel() != d:
            raise ValueError(f"{name} must have {d} elements, got {tuple(p.shape)}")
    if h0 is not None and tuple(h0.shape) != (B, d):
        raise ValueError(f"h0 must be ({B}, {d}), got {tuple(h0.shape)}")
    if T < 1:
        raise ValueError("time must be >= 1")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    az, ar, an, h0c = _same(a_z, wx), _same(a_r, wx), _same(a_n, wx), _same(h0, wx)
    out = torch.empty(B, T, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        nbytes = lib.prb_newton_workspace_bytes(L.CELL_GRU_DIAG, code, B, T, d, 1, max_iters, 0)
        ws = _workspace(nbytes, dev)
        rc = lib.prb_newton_gru_fused(_ptr(wx_c), _ptr(az), _ptr(ar), _ptr(an), _ptr(h0c), _ptr(out),
                                      B, T, d, code, int(max_iters), float(omega),
                                      int(want_residual), _ptr(ws), ws.numel(), _ptr(st.buf),
                                      _stream(dev))
    _raise(rc, "newton_gru_fused")
    return out


def newton_nlru_fused(wx: Tensor, u: Tensor, h0: Tensor | None = None,
                      cu_seqlens: Tensor | None = None, block_table: Tensor | None = None, *,
                      max_iters: int, omega: float = 1.0, stats: DeviceStats | None = None,
                      want_residual: bool = True) -> Tensor:
    """Fused Newton for ``ParaNLRU``: ``wx (B,T,2d)`` -> ``H (B,T,d)``.  ``cu_seqlens`` /
    ``block_table`` as in ``newton_gru_fused``."""
    if cu_seqlens is not None:
        if stats is not None:
            stats.parts.clear()
        return _packed(lambda w, h, st, _g: newton_nlru_fused(w, u, h, max_iters=max_iters, omega=omega,
                                                               stats=st, want_residual=want_residual),
                       wx, h0, cu_seqlens, block_table, (u.numel(),), stats)
    h0 = gather_h0(h0, block_table, wx.shape[0], (u.numel(),))
    dev = _check_cuda(wx, u, h0)
    _check_iters(max_iters)
    if wx.dim() != 3 or wx.shape[-1] % 2:
        raise ValueError(f"wx must be (B, T, 2*d), got {tuple(wx.shape)}")
    B, T, d2 = wx.shape
    d = d2 // 2
    if u.numel() != d:
        raise ValueError(f"u must have {d} elements, got {tuple(u.shape)}")
    if h0 is not None and tuple(h0.shape) != (B, d):
        raise ValueError(f"h0 must be ({B}, {d}), got {tuple(h0.shape)}")
    if T < 1:
        raise ValueError("time must be >= 1")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    uc, h0c = _same(u, wx), _same(h0, wx)
    out = torch.empty(B, T, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        nbytes = lib.prb_newton_workspace_bytes(L.CELL_NLRU, code, B, T, d, 1, max_iters, 0)
        ws = _workspace(nbytes, dev)
        rc = lib.prb_newton_nlru_fused(_ptr(wx_c), _ptr(uc), _ptr(h0c), _ptr(out), B, T, d, code,
                                       int(max_iters), float(omega), int(want_residual), _ptr(ws),
                                       ws.numel(), _ptr(st.buf), _stream(dev))
    _raise(rc, "newton_nlru_fused")
    return out


def newton_cfc_fused(wx: Tensor, u: Tensor, h0: Tensor | None = None,
                      cu_seqlens: Tensor | None = None, block_table: Tensor | None = None, *,
                      max_iters: int, omega: float = 1.0, stats: DeviceStats | None = None,
                      want_residual: bool = True) -> Tensor:
    """Fused Newton for ``ParaCfC`` (``gate_mix="input"``): ``wx = cell.project_wx(x) (B,T,4d)`` -> ``H (B,T,d)``.  ``cu_seqlens`` /
    ``block_table`` as in ``newton_gru_fused`` (reference ``pararnn::newton_cfc_fused``,
    ``kernels/custom_ops.py:230-266``)."""
    if cu_seqlens is not None:
        if stats is not None:
            stats.parts.clear()
        return _packed(lambda w, h, st, _g: newton_cfc_fused(w, u, h, max_iters=max_iters, omega=omega,
                                                               stats=st, want_residual=want_residual),
                       wx, h0, cu_seqlens, block_table, (u.numel(),), stats)
    h0 = gather_h0(h0, block_table, wx.shape[0], (u.numel(),))
    dev = _check_cuda(wx, u, h0)
    _check_iters(max_iters)
    if wx.dim() != 3 or wx.shape[-1] % 4:
        raise ValueError(f"wx must be (B, T, 4*d), got {tuple(wx.shape)}")
    B, T, d4 = wx.shape
    d = d4 // 4
    if u.numel() != d:
        raise ValueError(f"u must have {d} elements, got {tuple(u.shape)}")
    if h0 is not None and tuple(h0.shape) != (B, d):
        raise ValueError(f"h0 must be ({B}, {d}), got {tuple(h0.shape)}")
    if T < 1:
        raise ValueError("time must be >= 1")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    uc, h0c = _same(u, wx), _same(h0, wx)
    out = torch.empty(B, T, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        nbytes = lib.prb_newton_workspace_bytes(L.CELL_CFC, code, B, T, d, 1, max_iters, 0)
        ws = _workspace(nbytes, dev)
        rc = lib.prb_newton_cfc_fused(_ptr(wx_c), _ptr(uc), _ptr(h0c), _ptr(out), B, T, d, code,
                                       int(max_iters), float(omega), int(want_residual), _ptr(ws),
                                       ws.numel(), _ptr(st.buf), _stream(dev))
    _raise(rc, "newton_cfc_fused")
    return out


def newton_titans_fused(wx: Tensor, u: Tensor, r: Tensor, h0: Tensor | None = None,
                        cu_seqlens: Tensor | None = None, block_table: Tensor | None = None, *,
                        max_iters: int, omega: float = 1.0, stats: DeviceStats | None = None,
                        want_residual: bool = True) -> Tensor:
    """Fused Newton for ``ParaTitans``: ``wx (B,T,5d)`` -> ``H (B,T,d)`` (reference
    ``pararnn::newton_titans_fused``, ``kernels/custom_ops.py:269-308``)."""
    if cu_seqlens is not None:
        if stats is not None:
            stats.parts.clear()
        return _packed(lambda w, h, st, _g: newton_titans_fused(w, u, r, h, max_iters=max_iters, omega=omega,
                                                                 stats=st, want_residual=want_residual),
                       wx, h0, cu_seqlens, block_table, (u.numel(),), stats)
    h0 = gather_h0(h0, block_table, wx.shape[0], (u.numel(),))
    dev = _check_cuda(wx, u, r, h0)
    _check_iters(max_iters)
    if wx.dim() != 3 or wx.shape[-1] % 5:
        raise ValueError(f"wx must be (B, T, 5*d), got {tuple(wx.shape)}")
    B, T, d5 = wx.shape
    d = d5 // 5
    if u.numel() != d or r.numel() != d:
        raise ValueError(f"u and r must have {d} elements, got {tuple(u.shape)} / {tuple(r.shape)}")
    if h0 is not None and tuple(h0.shape) != (B, d):
        raise ValueError(f"h0 must be ({B}, {d}), got {tuple(h0.shape)}")
    if T < 1:
        raise ValueError("time must be >= 1")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    uc, rc_, h0c = _same(u, wx), _same(r, wx), _same(h0, wx)
    out = torch.empty(B, T, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        nbytes = lib.prb_newton_workspace_bytes(L.CELL_TITANS, code, B, T, d, 1, max_iters, 0)
        ws = _workspace(nbytes, dev)
        rc = lib.prb_newton_titans_fused(_ptr(wx_c), _ptr(uc), _ptr(rc_), _ptr(h0c), _ptr(out), B, T, d, code,
                                         int(max_iters), float(omega), int(want_residual), _ptr(ws),
                                         ws.numel(), _ptr(st.buf), _stream(dev))
    _raise(rc, "newton_titans_fused")
    return out


def newton_lstm_fused(wx: Tensor, a_f: Tensor, a_z: Tensor, a_o: Tensor, c_f: Tensor, c_o: Tensor,
                      h0: Tensor | None = None, cu_seqlens: Tensor | None = None,
                      block_table: Tensor | None = None, *, max_iters: int, omega: float = 1.0,
                      stats: DeviceStats | None = None, want_residual: bool = True) -> Tensor:
    """Fused Newton for ``ParaLSTM``: ``wx (B,T,3d)`` -> ``H (B,T,2,d)`` with slots ``(c, h)``
    (reference ``pararnn::newton_lstm_fused``, ``kernels/custom_ops.py:437-483``)."""
    d = a_f.numel()
    if cu_seqlens is not None:
        if stats is not None:
            stats.parts.clear()
        return _packed(lambda w, h, st, _g: newton_lstm_fused(w, a_f, a_z, a_o, c_f, c_o, h, max_iters=max_iters,
                                                               omega=omega, stats=st,
                                                               want_residual=want_residual),
                       wx, h0, cu_seqlens, block_table, (2, d), stats)
    h0 = gather_h0(h0, block_table, wx.shape[0], (2, d))
    dev = _check_cuda(wx, a_f, a_z, a_o, c_f, c_o, h0)
    _check_iters(max_iters)
    if wx.dim() != 3 or wx.shape[-1] != 3 * d:
        raise ValueError(f"wx must be (B, T, 3*d) with d={d}, got {tuple(wx.shape)}")
    B, T, _ = wx.shape
    for name, p in (("a_z", a_z), ("a_o", a_o), ("c_f", c_f), ("c_o", c_o)):
        if p.numel() != d:
            raise ValueError(f"{name} must have {d} elements, got {tuple(p.shape)}")
    if h0 is not None and tuple(h0.shape) != (B, 2, d):
        raise ValueError(f"h0 must be ({B}, 2, {d}), got {tuple(h0.shape)}")
    if T < 1:
        raise ValueError("time must be >= 1")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    pars = [_same(p, wx) for p in (a_f, a_z, a_o, c_f, c_o)]
    h0c = _same(h0, wx)
    out = torch.empty(B, T, 2, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(lib.prb_lstm_workspace_bytes(B, T, d, int(max_iters), 0), dev)
        rc = lib.prb_newton_lstm_fused(_ptr(wx_c), *[_ptr(p) for p in pars], _ptr(h0c), _ptr(out), B, T, d, code,
                                       int(max_iters), float(omega), int(want_residual), _ptr(ws), ws.numel(),
                                       _ptr(st.buf), _stream(dev))
    _raise(rc, "newton_lstm_fused")
    return out


def newton_slstm_fused(wx: Tensor, r: Tensor, h0: Tensor | None = None,
                       states: Tensor | None = None, block_table: Tensor | None = None, *,
                       max_iters: int, omega: float = 1.0, eps: float = 1e-6,
                       log_coords: bool = False, scan_tile: str = "assoc", time_loop: bool = False,
                       window_len: int = 0, picard_iters: int = 0,
                       stats: DeviceStats | None = None, want_residual: bool = True,
                       cu_seqlens: Tensor | None = None) -> Tensor:
    """Fused Newton for ``ParaSLSTM(mix='diag')``: ``wx (B,T,4d)`` -> ``H (B,T,4,d)``.

    ``states`` is an optional initial guess (cloned, never modified).  Without it the
    kernel runs the zero-hidden frozen-gate scan followed by ``picard_iters`` Picard
    passes itself (the reference does this in ``slstm_picard_init`` before calling its op).
    """
    if log_coords:
        raise TypeError("coords='log' is not covered by the CUDA backend")
    if scan_tile != "assoc" or time_loop or window_len:
        raise TypeError("scan_tile / fused_time_loop / fused_window_len ablations are not available")
    if cu_seqlens is not None:
        if stats is not None:
            stats.parts.clear()
        return _packed(lambda w, h, st, g: newton_slstm_fused(w, r, h, g, max_iters=max_iters, omega=omega,
                                                               eps=eps, picard_iters=picard_iters, stats=st,
                                                               want_residual=want_residual),
                       wx, h0, cu_seqlens, block_table, (4, r.shape[-1]), stats, states)
    h0 = gather_h0(h0, block_table, wx.shape[0], (4, r.shape[-1]))
    dev = _check_cuda(wx, r, h0, states)
    _check_iters(max_iters)
    if wx.dim() != 3 or wx.shape[-1] % 4:
        raise ValueError(f"wx must be (B, T, 4*d), got {tuple(wx.shape)}")
    B, T, d4 = wx.shape
    d = d4 // 4
    if tuple(r.shape) != (4, d):
        raise ValueError(f"r must be (4, {d}), got {tuple(r.shape)}")
    if h0 is not None and tuple(h0.shape) != (B, 4, d):
        raise ValueError(f"h0 must be ({B}, 4, {d}), got {tuple(h0.shape)}")
    if states is not None and tuple(states.shape) != (B, T, 4, d):
        raise ValueError(f"states must be ({B}, {T}, 4, {d}), got {tuple(states.shape)}")
    if T < 1:
        raise ValueError("time must be >= 1")
    if picard_iters < 0 or picard_iters + max_iters > 40:
        raise ValueError("picard_iters out of range")
    code = _dtype_code(wx)
    wx_c = wx.detach().contiguous()
    rc_, h0c, gc = _same(r, wx), _same(h0, wx), _same(states, wx)
    out = torch.empty(B, T, 4, d, dtype=wx.dtype, device=dev)
    st = stats or DeviceStats(dev, max_iters)
    lib = L.lib()
    with torch.cuda.device(dev):
        nbytes = lib.prb_newton_workspace_bytes(L.CELL_SLSTM_DIAG, code, B, T, d, 1, max_iters,
                                                int(picard_iters))
        ws = _workspace(nbytes, dev)
        rc = lib.prb_newton_slstm_fused(_ptr(wx_c), _ptr(rc_), _ptr(h0c), _ptr(gc), _ptr(out), B, T,
                                        d, code, int(max_iters), int(picard_iters), float(omega),
                                        float(eps), int(want_residual), _ptr(ws), ws.numel(),
                                        _ptr(st.buf), _stream(dev))
    _raise(rc, "newton_slstm_fused")
    return out


# ---------------------------------------------------------------------------- backward

def _bwd_common(states, wx, grad_states, h0):
    dev = _check_cuda(states, wx, grad_states, h0)
    code = _dtype_code(wx)
    st = states.detach().to(wx.dtype).contiguous()
    gs = grad_states.detach().to(wx.dtype).contiguous()
    return dev, code, st, wx.detach().contiguous(), gs, _same(h0, wx)


def _diag_reverse_vjp(what: str, cell_code: int, gates: int, states: Tensor, wx: Tensor, params: tuple,
                      grad_states: Tensor, h0: Tensor | None, want_bias: bool):
    """Shared body of the scalar-diagonal reverse scan + VJP operators: returns
    ``(g_wx, g_params (NP,d) fp32, g_h0 (B,d) fp32, g_bias (G*d,) fp32 or None)``."""
    dev, code, st, wxc, gs, h0c = _bwd_common(states, wx, grad_states, h0)
    B, T, dg = wx.shape
    if dg % gates:
        raise ValueError(f"wx must be (B, T, {gates}*d), got {tuple(wx.shape)}")
    d = dg // gates
    if tuple(states.shape) != (B, T, d) or tuple(grad_states.shape) != (B, T, d):
        raise ValueError("states / grad_states must be (B, T, d)")
    g_wx = torch.empty_like(wxc)
    g_par = torch.empty(len(params), d, dtype=torch.float32, device=dev)
    g_bias = torch.empty(gates * d, dtype=torch.float32, device=dev) if want_bias else None
    g_h0 = torch.empty(B, d, dtype=torch.float32, device=dev)
    sb = DeviceStats(dev, 0)
    pc = [_same(p, wx) for p in params] + [None] * (3 - len(params))  # keep alive across the call
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(lib.prb_bwd_workspace_bytes(cell_code, code, B, T, d, 1), dev)
        rc = lib.prb_bwd_diag_ex(cell_code, _ptr(st), _ptr(wxc), _ptr(pc[0]), _ptr(pc[1]), _ptr(pc[2]), _ptr(h0c),
                                 _ptr(gs), _ptr(g_wx), _ptr(g_par), _ptr(g_bias), _ptr(g_h0), B, T, d, code,
                                 _ptr(ws), ws.numel(), _ptr(sb.buf), _stream(dev))
    _raise(rc, what)
    _track_backward(sb)
    return g_wx, g_par, g_h0, g_bias


def gru_reverse_vjp(states: Tensor, wx: Tensor, a_z: Tensor, a_r: Tensor, a_n: Tensor,
                    grad_states: Tensor, h0: Tensor | None = None, *, want_bias: bool = False):
    """Eq. 2.6 reverse scan fused with the packed GRU VJP.

    Returns ``(g_wx, g_az, g_ar, g_an, g_h0)``; parameter grads are fp32 sums over batch and
    time with no clip mask (the caller applies it, reference ``solvers/vjp.py:141-144``).
    ``want_bias`` (all scalar-diagonal cells): one more result, ``g_bias (G*d,) fp32`` = the sum of
    ``g_wx`` over batch and time, accumulated by the same kernel."""
    g_wx, gp, g_h0, gb = _diag_reverse_vjp("gru_reverse_vjp", L.CELL_GRU_DIAG, 3, states, wx, (a_z, a_r, a_n),
                                           grad_states, h0, want_bias)
    return (g_wx, gp[0], gp[1], gp[2], g_h0) + ((gb,) if want_bias else ())


def nlru_reverse_vjp(states: Tensor, wx: Tensor, u: Tensor, grad_states: Tensor,
                     h0: Tensor | None = None, *, want_bias: bool = False):
    """Eq. 2.6 reverse scan fused with the packed NLRU VJP: ``(g_wx, g_u, g_h0)``."""
    g_wx, gp, g_h0, gb = _diag_reverse_vjp("nlru_reverse_vjp", L.CELL_NLRU, 2, states, wx, (u,), grad_states, h0,
                                           want_bias)
    return (g_wx, gp[0], g_h0) + ((gb,) if want_bias else ())


def cfc_reverse_vjp(states: Tensor, wx: Tensor, u: Tensor, grad_states: Tensor,
                    h0: Tensor | None = None, *, want_bias: bool = False):
    """Eq. 2.6 reverse scan fused with the packed CfC VJP (reference ``kernels/vjp_cfc.py:102-167``):
    ``(g_wx (B,T,4d) = grads of (f_pre, c_x, dt, b), g_u, g_h0)``."""
    g_wx, gp, g_h0, gb = _diag_reverse_vjp("cfc_reverse_vjp", L.CELL_CFC, 4, states, wx, (u,), grad_states, h0,
                                           want_bias)
    return (g_wx, gp[0], g_h0) + ((gb,) if want_bias else ())


def lstm_reverse_vjp(states: Tensor, wx: Tensor, a_f: Tensor, a_z: Tensor, a_o: Tensor, c_f: Tensor,
                     c_o: Tensor, grad_states: Tensor, h0: Tensor | None = None):
    """Eq. 2.6 reverse scan (2x2 blocks, J^T) fused with the packed LSTM VJP:
    ``(g_wx (B,T,3d), g_params (5,d) fp32 in the order a_f,a_z,a_o,c_f,c_o, g_h0 (B,2,d) fp32)``."""
    dev, code, st, wxc, gs, h0c = _bwd_common(states, wx, grad_states, h0)
    B, T, d3 = wx.shape
    d = d3 // 3
    if tuple(states.shape) != (B, T, 2, d) or tuple(grad_states.shape) != (B, T, 2, d):
        raise ValueError("states / grad_states must be (B, T, 2, d)")
    g_wx = torch.empty_like(wxc)
    g_par = torch.empty(5, d, dtype=torch.float32, device=dev)
    g_h0 = torch.empty(B, 2, d, dtype=torch.float32, device=dev)
    sb = DeviceStats(dev, 0)
    pars = [_same(p, wx) for p in (a_f, a_z, a_o, c_f, c_o)]
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(lib.prb_lstm_workspace_bytes(B, T, d, 0, 1), dev)
        rc = lib.prb_bwd_lstm(_ptr(st), _ptr(wxc), *[_ptr(p) for p in pars], _ptr(h0c), _ptr(gs), _ptr(g_wx),
                              _ptr(g_par), _ptr(g_h0), B, T, d, code, _ptr(ws), ws.numel(), _ptr(sb.buf),
                              _stream(dev))
    _raise(rc, "lstm_reverse_vjp")
    _track_backward(sb)
    return g_wx, g_par, g_h0


def titans_reverse_vjp(states: Tensor, wx: Tensor, u: Tensor, r: Tensor, grad_states: Tensor,
                       h0: Tensor | None = None, *, want_bias: bool = False):
    """Eq. 2.6 reverse scan fused with the Titans VJP: ``(g_wx (B,T,5d), g_u, g_r, g_h0)``."""
    g_wx, gp, g_h0, gb = _diag_reverse_vjp("titans_reverse_vjp", L.CELL_TITANS, 5, states, wx, (u, r), grad_states,
                                           h0, want_bias)
    return (g_wx, gp[0], gp[1], g_h0) + ((gb,) if want_bias else ())


def slstm_reverse_vjp(states: Tensor, wx: Tensor, r: Tensor, grad_states: Tensor,
                      h0: Tensor | None = None, eps: float = 1e-6, *, grad_slot: int | None = None,
                      want_bias: bool = False):
    """Eq. 2.6 reverse scan (4x4 blocks, J^T) fused with the packed sLSTM VJP:
    ``(g_wx (B,T,4d), g_r (4,d) fp32, g_h0 (B,4,d) fp32)``.

    ``grad_slot`` in 0..3: ``grad_states`` is ``(B,T,d)``, the cotangent of that state slot alone
    (what a layer that outputs the hidden slot receives) -- the zero-filled ``(B,T,4,d)`` array is
    never built.  ``want_bias``: a fourth result ``g_bias (4d,) fp32``, the sum of ``g_wx`` over
    batch and time (the gradient of the bias of ``W_x``) accumulated by the same kernel."""
    dev, code, st, wxc, gs, h0c = _bwd_common(states, wx, grad_states, h0)
    B, T, d4 = wx.shape
    d = d4 // 4
    want_g = (B, T, 4, d) if grad_slot is None else (B, T, d)
    if grad_slot is not None and not 0 <= int(grad_slot) <= 3:
        raise ValueError(f"grad_slot must be in 0..3, got {grad_slot}")
    if tuple(states.shape) != (B, T, 4, d) or tuple(grad_states.shape) != want_g:
        raise ValueError(f"states must be (B, T, 4, d) and grad_states {want_g}, got "
                         f"{tuple(states.shape)} / {tuple(grad_states.shape)}")
    g_wx = torch.empty_like(wxc)
    g_par = torch.empty(4, d, dtype=torch.float32, device=dev)
    g_bias = torch.empty(4 * d, dtype=torch.float32, device=dev) if want_bias else None
    g_h0 = torch.empty(B, 4, d, dtype=torch.float32, device=dev)
    sb = DeviceStats(dev, 0)
    rc_ = _same(r, wx)
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(lib.prb_bwd_workspace_bytes(L.CELL_SLSTM_DIAG, code, B, T, d, 1), dev)
        rc = lib.prb_bwd_slstm_ex(_ptr(st), _ptr(wxc), _ptr(rc_), _ptr(h0c), _ptr(gs),
                                  -1 if grad_slot is None else int(grad_slot), _ptr(g_wx), _ptr(g_par),
                                  _ptr(g_bias), _ptr(g_h0), B, T, d, code, float(eps), _ptr(ws), ws.numel(),
                                  _ptr(sb.buf), _stream(dev))
    _raise(rc, "slstm_reverse_vjp")
    _track_backward(sb)
    if want_bias:
        return g_wx, g_par, g_h0, g_bias
    return g_wx, g_par, g_h0


def residual_max(cell_code: int, wx: Tensor, params: Tensor, states: Tensor,
                 h0: Tensor | None = None, eps: float = 1e-6) -> float:
    """``max|f(H_{t-1}, x_t) - H_t|`` evaluated on the device (one host sync)."""
    dev = _check_cuda(wx, params, states, h0)
    code = _dtype_code(wx)
    B, T = wx.shape[:2]
    d = states.shape[-1]
    sb = DeviceStats(dev, 0)
    lib = L.lib()
    with torch.cuda.device(dev):
        ws = _workspace(1 << 20, dev)
        need = (params.numel() + (0 if h0 is None else h0.numel())) * 4 + 4096
        if need > ws.numel():
            ws = _workspace(need, dev)
        wxc, pc, h0c, stc = wx.detach().contiguous(), _same(params, wx), _same(h0, wx), _same(states, wx)
        rc = lib.prb_residual(int(cell_code), _ptr(wxc), _ptr(pc),
                              _ptr(h0c), _ptr(stc), B, T, d, code, float(eps),
                              _ptr(ws), ws.numel(), _ptr(sb.buf), _stream(dev))
    _raise(rc, "residual_max")
    return sb.read()[1]
