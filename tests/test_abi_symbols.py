"""The C-ABI library loads and exports every symbol the public header declares (no compute)."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pararnn_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(prb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared()
    for must in ("prb_newton_gru_fused", "prb_newton_nlru_fused", "prb_newton_slstm_fused",
                 "prb_bwd_gru", "prb_bwd_nlru", "prb_bwd_slstm", "prb_residual"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from pararnn_b200 import _build, _lib

    _build.build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert b"sm_100a" in ctypes.cast(handle.prb_version, ctypes.CFUNCTYPE(ctypes.c_char_p))()


def test_python_binding_covers_header():
    from pararnn_b200 import _lib

    assert set(_declared()) == set(_lib.exported_symbols())


def test_workspace_queries_are_pure():
    from pararnn_b200 import _lib

    lib = _lib.lib()
    a = lib.prb_newton_workspace_bytes(_lib.CELL_SLSTM_DIAG, _lib.PRB_BF16, 2, 1000, 64, 1, 2, 5)
    b = lib.prb_newton_workspace_bytes(_lib.CELL_SLSTM_DIAG, _lib.PRB_BF16, 2, 2000, 64, 1, 2, 5)
    assert 0 < a < b
    assert lib.prb_newton_workspace_bytes(_lib.CELL_GRU_DIAG, 0, 0, 10, 8, 1, 3, 0) == 0
    assert lib.prb_error_string(-2).decode().startswith("workspace")


def test_sweep_entry_points_validate_arguments_before_any_gpu_work():
    """Argument checks come first, so they can be exercised without a GPU."""
    from pararnn_b200 import _lib

    lib = _lib.lib()
    null = None
    # missing pointers
    assert lib.prb_slstm_picard_sweep(null, null, null, null, null, null, 6, 1, 8, 32, _lib.PRB_F32, 1e-6,
                                      null, 0, null, null) == -1
    assert lib.prb_slstm_newton_sweep(null, null, null, null, null, 2, 1, 1, 8, 32, _lib.PRB_F32, 1.0, 1e-6,
                                      null, 0, null, null) == -1
    # more passes than one sweep takes (pointers only need to be non-null to get that far)
    buf = ctypes.create_string_buffer(256)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.prb_slstm_picard_sweep(p, p, null, null, p, null, 7, 1, 8, 32, _lib.PRB_F32, 1e-6, null, 0,
                                      p, null) == -3
    assert lib.prb_slstm_newton_sweep(p, p, p, null, p, 5, 1, 1, 8, 32, _lib.PRB_F32, 1.0, 1e-6, null, 0, p,
                                      null) == -3
