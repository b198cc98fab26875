"""Loader of the C-ABI library.  There is no fallback: if the library cannot be
loaded, every operator of this package raises."""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libpararnn_b200.so")

PRB_F32, PRB_BF16 = 0, 1
CELL_GRU_DIAG, CELL_NLRU, CELL_SLSTM_DIAG, CELL_GRU_HEAD, CELL_TITANS, CELL_LSTM, CELL_CFC = 0, 1, 2, 3, 4, 5, 6
MAX_ITERS = 16
STATS_BYTES = 80


class ExtensionMissingError(RuntimeError):
    """The CUDA extension is not built or cannot be loaded."""


_lib = None

_VOIDP = ctypes.c_void_p
_INT = ctypes.c_int
_SIZE = ctypes.c_size_t
_FLOAT = ctypes.c_float

_SIGNATURES = {
    "prb_version": (ctypes.c_char_p, []),
    "prb_error_string": (ctypes.c_char_p, [_INT]),
    "prb_debug_set": (_INT, [_INT, ctypes.c_longlong]),
    "prb_newton_workspace_bytes": (_SIZE, [_INT] * 8),
    "prb_bwd_workspace_bytes": (_SIZE, [_INT] * 6),
    "prb_newton_gru_fused": (_INT, [_VOIDP] * 6 + [_INT] * 5 + [_FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_newton_nlru_fused": (_INT, [_VOIDP] * 4 + [_INT] * 5 + [_FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_newton_cfc_fused": (_INT, [_VOIDP] * 4 + [_INT] * 5 + [_FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_cfc": (_INT, [_VOIDP] * 8 + [_INT] * 4 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_newton_titans_fused": (_INT, [_VOIDP] * 5 + [_INT] * 5 + [_FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_titans": (_INT, [_VOIDP] * 9 + [_INT] * 4 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_lstm_workspace_bytes": (_SIZE, [_INT] * 5),
    "prb_newton_lstm_fused": (_INT, [_VOIDP] * 8 + [_INT] * 5 + [_FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_lstm": (_INT, [_VOIDP] * 12 + [_INT] * 4 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_newton_slstm_fused": (_INT, [_VOIDP] * 5 + [_INT] * 6 + [_FLOAT, _FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_gru_head_workspace_bytes": (_SIZE, [_INT] * 5),
    "prb_newton_gru_head_fused": (_INT, [_VOIDP] * 6 + [_INT] * 6 + [_FLOAT, _INT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_gru_head": (_INT, [_VOIDP] * 11 + [_INT] * 5 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_gru": (_INT, [_VOIDP] * 10 + [_INT] * 4 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_nlru": (_INT, [_VOIDP] * 8 + [_INT] * 4 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_slstm": (_INT, [_VOIDP] * 8 + [_INT] * 4 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_diag_ex": (_INT, [_INT] + [_VOIDP] * 11 + [_INT] * 4 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_bwd_slstm_ex": (_INT, [_VOIDP] * 5 + [_INT] + [_VOIDP] * 4 + [_INT] * 4 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_residual": (_INT, [_INT] + [_VOIDP] * 4 + [_INT] * 4 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_pass_workspace_bytes": (_SIZE, [_INT] * 4),
    "prb_diag_guess": (_INT, [_INT] + [_VOIDP] * 4 + [_INT] * 4 + [_VOIDP]),
    "prb_diag_newton_pass": (_INT, [_INT] + [_VOIDP] * 8 + [_INT] * 5 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _INT, _VOIDP]),
    "prb_diag_bwd_pass": (_INT, [_INT] + [_VOIDP] * 10 + [_INT] * 5 + [_VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_slstm_picard_pass": (_INT, [_VOIDP] * 9 + [_INT] * 7 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_slstm_picard_sweep": (_INT, [_VOIDP] * 6 + [_INT] * 5 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_slstm_newton_sweep": (_INT, [_VOIDP] * 5 + [_INT] * 6 + [_FLOAT, _FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_slstm_newton_pass": (_INT, [_VOIDP] * 8 + [_INT] * 7 + [_FLOAT, _FLOAT, _VOIDP, _SIZE, _VOIDP, _INT, _VOIDP]),
    "prb_slstm_bwd_pass": (_INT, [_VOIDP] * 10 + [_INT] * 7 + [_FLOAT, _VOIDP, _SIZE, _VOIDP, _VOIDP]),
    "prb_plan_segments": (_INT, [_INT] * 5 + [_VOIDP, _VOIDP]),
    "prb_fold_segments": (_INT, [_INT, _VOIDP, _INT, _INT, _VOIDP, _INT, _INT, _VOIDP]),
    "prb_segment_carries": (_INT, [_INT, _VOIDP, _INT, _INT, _VOIDP, _VOIDP, _INT, _INT, _VOIDP]),
    "prb_shard_carries": (_INT, [_INT, _VOIDP, _INT, _INT, _INT, _INT, _VOIDP, _INT, _VOIDP, _VOIDP, _FLOAT, _VOIDP, _INT, _INT, _VOIDP]),
    "prb_fold_carries": (_INT, [_INT, _VOIDP, _INT, _INT, _INT, _VOIDP, _INT, _INT, _VOIDP]),
    "prb_decode_step": (_INT, [_INT, _VOIDP, _VOIDP, _VOIDP, _FLOAT, _VOIDP, _VOIDP, _INT, _INT, _INT, _FLOAT, _VOIDP]),
    "prb_static_scratch_bytes": (_SIZE, []),
    "prb_bwd_nlru_static": (_INT, [_VOIDP] * 8 + [_INT] * 4 + [_VOIDP, _VOIDP]),
    "prb_residual_pass": (_INT, [_INT] + [_VOIDP] * 4 + [_INT] * 5 + [_FLOAT, _VOIDP, _VOIDP]),
}


def exported_symbols() -> tuple[str, ...]:
    return tuple(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ExtensionMissingError(
                f"{LIB_PATH} not found: build it with `python -m pararnn_b200._build` "
                "(nvcc, sm_100a). This package has no CPU or PyTorch fallback."
            )
        try:
            handle = ctypes.CDLL(LIB_PATH)
        except OSError as exc:  # pragma: no cover
            raise ExtensionMissingError(f"cannot load {LIB_PATH}: {exc}") from exc
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


OPTIONS = {"kernel_family": 0, "picard_fused": 1, "newton_fused": 2, "spin_limit": 3}
KERNEL_FAMILY = {"auto": -1, "lookback": 0, "pipe": 2}
_DEFAULTS = {"kernel_family": -1, "picard_fused": 1, "newton_fused": 1, "spin_limit": 0}


def debug_set(option: str, value) -> None:
    """Test / profiling hook (``prb_debug_set``): force a kernel family or a wait limit."""
    if option == "kernel_family" and isinstance(value, str):
        value = KERNEL_FAMILY[value]
    rc = lib().prb_debug_set(OPTIONS[option], int(value))
    if rc != 0:
        raise ValueError(f"prb_debug_set({option}, {value}) failed: {error_string(rc)}")


def debug_reset() -> None:
    for name, value in _DEFAULTS.items():
        debug_set(name, value)


def error_string(code: int) -> str:
    return lib().prb_error_string(int(code)).decode()
