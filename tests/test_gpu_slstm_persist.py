"""The same sLSTM parity tests, forced onto the persistent-chain TMA kernels.

By default small shapes take the look-back kernels (too few chains to fill a GPU); setting
PRB_KERNEL_PATH=persist makes every shape whose strides meet TMA's 16-byte rule run the
persistent kernels, so both kernel families face the golden vectors and the oracle."""

import pytest

from test_gpu_slstm import *  # noqa: F401,F403  (re-collect the tests in this module)
from test_gpu_slstm import pytestmark  # noqa: F401


@pytest.fixture(autouse=True)
def _force_persistent_kernels(monkeypatch):
    monkeypatch.setenv("PRB_KERNEL_PATH", "persist")
