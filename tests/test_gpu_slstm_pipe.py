"""The sLSTM parity tests once more, forced onto the warp-pipelined persistent kernels
(PRB_KERNEL_PATH=pipe); passes that have no pipelined variant fall back to the other families."""

import pytest

from test_gpu_slstm import *  # noqa: F401,F403
from test_gpu_slstm import pytestmark  # noqa: F401


@pytest.fixture(autouse=True)
def _force_pipelined_kernels(monkeypatch):
    monkeypatch.setenv("PRB_KERNEL_PATH", "pipe")
