"""Puts a copy of the reference project's `model/` tree (plain Python, 256 KB)
under oracle/_ref/, where the CPU arm of bench.py and the reference-side tests
import it from.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

    python oracle/make_ref.py /path/to/nnue-pytorch

oracle/_ref/ is listed in .gitignore: the copy never enters this repository's
history, it only sits beside the built library on machines that run the
benchmarks.  Nothing is edited on the way; `verify()` compares every file
with its source byte for byte.
"""

from __future__ import annotations

import filecmp
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
TREES = ("model",)


def make(ref_root: str) -> str:
    for tree in TREES:
        src = os.path.join(ref_root, tree)
        if not os.path.isdir(src):
            raise SystemExit(f"{src} is not a directory: pass the root of an nnue-pytorch checkout")
        dst = os.path.join(DEST, tree)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    verify(ref_root)
    return DEST


def verify(ref_root: str) -> None:
    """Raises if any copied file differs from the checkout it came from."""
    for tree in TREES:
        for dirpath, _, files in os.walk(os.path.join(DEST, tree)):
            for f in files:
                if f.endswith(".pyc"):
                    continue
                mine = os.path.join(dirpath, f)
                theirs = os.path.join(ref_root, os.path.relpath(mine, DEST))
                if not filecmp.cmp(mine, theirs, shallow=False):
                    raise SystemExit(f"{mine} differs from {theirs}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python oracle/make_ref.py /path/to/nnue-pytorch")
    print(make(sys.argv[1]))
