"""Build the C-ABI shared library ``libpararnn_b200.so`` for sm_100a with nvcc.

The library is built in-tree next to this file so that it travels with the
source tree.  ``python -m pararnn_b200._build`` rebuilds it.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
LIB = os.path.join(HERE, "libpararnn_b200.so")
OBJ_DIR = os.path.join(CSRC, "build")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _newest_source_mtime() -> float:
    m = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(os.path.dirname(HERE)), "include")):
        for f in os.listdir(root):
            if f.endswith((".cu", ".cuh", ".h")):
                m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def is_fresh() -> bool:
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_source_mtime()


def _compile(src: str) -> str:
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    cmd = ["nvcc", *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``.cu`` under ``csrc/`` and link the shared library."""
    if not force and is_fresh():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    sources = [s for s in sorted(os.listdir(CSRC)) if s.endswith(".cu")]
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(_compile, sources))
    # the CUDA runtime is linked statically (nvcc default): the library has no
    # dependency on a libcudart.so being on the loader path
    cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build(force=True, verbose=True)
