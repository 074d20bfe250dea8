"""A stand-in for the small part of CuPy that the reference project's
feature-transformer kernels use, on top of NVRTC and the CUDA driver API
(the `cuda-python` bindings).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): it exists so that the
reference's own CUDA kernel sources, read from its files at run time, can be
compiled and launched with the reference's own launch geometry on a machine
without CuPy, as the GPU comparator of the benchmarks.

Covered: `cupy.RawKernel(source, name)`, `.compile()`, and the launch
`kernel(grid=(gx,), block=(bx,), args=(...))` where every argument is either a
Python int (a device pointer from `tensor.data_ptr()`) or a numpy scalar
(`np.int32`, `np.float32`, ...), which is how
model/modules/feature_transformer/fused_ft_functions.py:57-75 and
sparse_linear_functions.py:90-101 of the reference launch.  Launches go to
torch's current stream.  Nothing else of CuPy is imitated; `from_dlpack` and
array objects (which the reference's optimizer kernels use) raise.
"""

from __future__ import annotations

import ctypes
import sys
import types

import numpy as np
import torch


class CupyShimError(RuntimeError):
    pass


def _check(res, what: str):
    err = res[0]
    if int(err) != 0:
        raise CupyShimError(f"{what} failed: {err!r}")
    return res[1:] if len(res) > 2 else (res[1] if len(res) == 2 else None)


class RawKernel:
    def __init__(self, code: str, name: str, options: tuple = (), **_):
        self.code, self.name, self.options = code, name, tuple(options)
        self._fn = None
        self._module = None

    def compile(self) -> None:
        if self._fn is not None:
            return
        from cuda.bindings import driver, nvrtc

        torch.cuda.init()
        torch.zeros(1, device="cuda")  # makes the primary context current on this thread
        major, minor = torch.cuda.get_device_capability()
        prog = _check(nvrtc.nvrtcCreateProgram(self.code.encode(), (self.name + ".cu").encode(), 0, [], []),
                      "nvrtcCreateProgram")
        opts = [f"--gpu-architecture=sm_{major}{minor}".encode(), b"--std=c++17"] + [o.encode() for o in self.options]
        res = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
        if int(res[0]) != 0:
            size = _check(nvrtc.nvrtcGetProgramLogSize(prog), "nvrtcGetProgramLogSize")
            log = b" " * int(size)
            nvrtc.nvrtcGetProgramLog(prog, log)
            raise CupyShimError(f"NVRTC could not compile {self.name}: {log.decode(errors='replace')[:2000]}")
        size = _check(nvrtc.nvrtcGetCUBINSize(prog), "nvrtcGetCUBINSize")
        cubin = b" " * int(size)
        _check(nvrtc.nvrtcGetCUBIN(prog, cubin), "nvrtcGetCUBIN")
        nvrtc.nvrtcDestroyProgram(prog)
        self._module = _check(driver.cuModuleLoadData(np.char.array(cubin).ctypes.data), "cuModuleLoadData")
        self._fn = _check(driver.cuModuleGetFunction(self._module, self.name.encode()), "cuModuleGetFunction")

    def __call__(self, grid, block, args, shared_mem: int = 0, stream=None) -> None:
        from cuda.bindings import driver

        self.compile()
        values, types_ = [], []
        for a in args:
            if isinstance(a, np.generic):
                ct = np.ctypeslib.as_ctypes_type(a.dtype)
                values.append(a.item())
                types_.append(ct)
            elif isinstance(a, int):
                values.append(a)
                types_.append(ctypes.c_void_p)
            else:
                raise CupyShimError(f"unsupported kernel argument {type(a).__name__}")
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        s = torch.cuda.current_stream().cuda_stream if stream is None else int(stream)
        _check(driver.cuLaunchKernel(self._fn, g[0], g[1], g[2], b[0], b[1], b[2], int(shared_mem), s,
                                     (tuple(values), tuple(types_)), 0), f"cuLaunchKernel({self.name})")


def _unsupported(*_, **__):
    raise CupyShimError("this stand-in covers RawKernel launches with pointer / scalar arguments only")


def install() -> types.ModuleType:
    """Registers the stand-in as `cupy` unless a real CuPy can be imported."""
    try:
        import cupy  # noqa: F401

        return sys.modules["cupy"]
    except Exception:  # noqa: BLE001 - absent or broken: use the stand-in
        pass
    m = types.ModuleType("cupy")
    m.RawKernel = RawKernel
    m.from_dlpack = _unsupported
    m.__nnue_shim__ = True
    sys.modules["cupy"] = m
    return m
