"""Shared pytest configuration.

Markers: ``gpu`` = needs a CUDA device (parity tests proper, called through the
C ABI).  Everything else runs on CPU.
"""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "pararnn-torch_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture
def prb_options():
    """Setter for the library's test hook (``prb_debug_set``); every option is restored to its
    default after the test."""
    from pararnn_b200 import _lib

    yield _lib.debug_set
    _lib.debug_reset()
