"""In-tree build of libnnue_b200.so with nvcc for sm_100a.

The library is plain CUDA C++ behind a C ABI (include/nnue_b200.h); it does
not link against torch.  `python -m nnue_pytorch_b200._build` rebuilds it,
`build(force=False)` rebuilds only when a source is newer than the library.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libnnue_b200.so"

SOURCES = [
    "core.cu",
    "ft_sparse.cu",
    "ft_sparse_static.cu",
    "ft_fused.cu",
    "ft_fused_q16.cu",
    "ft_segment.cu",
    "ft_table.cu",
    "ranger_lite.cu",
    "multi_tensor.cu",
    "ddp_fused.cu",
    "quant_eval.cu",
    "layer_stack.cu",
    "layer_stack_l1.cu",
    "layer_stack_l1_tc.cu",
    "layer_stack_tail.cu",
    "layer_stack_weights.cu",
    "batch_build.cu",
    "sf_loss.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "--expt-extended-lambda",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")
    return cand


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    lib_m = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > lib_m for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every kernel source and link the shared library in-tree."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        objs.append(str(obj))
        cmd = [nvcc, *flags, "-I", str(INCLUDE), "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed.append(f"--- {src} ---\n{out}")
        elif out.strip() and (verbose or ptxas_info):
            print(f"--- {src} ---\n{out}", flush=True)
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *objs, "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force=True, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
