"""Put an importable copy of the reference package under ``oracle/_ref/`` (git-ignored).

    python oracle/make_ref.py /path/to/reference      (or PARARNN_REFERENCE=/path/to/reference)

Test infrastructure only: with ``oracle/_ref/pararnn`` present, ``tests/test_gpu_dropin.py``
imports the unmodified reference next to this backend and drives the reference's own
``newton_apply`` through ``pararnn_b200.shim``; without it that test is skipped.  Nothing in the
product imports ``oracle/``.  The copy never enters the repository's history.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
# where the reference checkout is looked for when no path is given
DEFAULT_ROOT = os.environ.get("PARARNN_REFERENCE", os.path.join(os.sep, "root", "reference"))


def make_ref(reference_root: str) -> str | None:
    src = os.path.join(reference_root, "src", "pararnn")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(DEST, "pararnn")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(DEST, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return dst


if __name__ == "__main__":
    out = make_ref(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_ROOT)
    print(out or "reference package not found; nothing copied")
