"""CPU-side checks of the C-ABI library: it loads, exports every function
include/nnue_b200.h declares, and validates arguments on the host before any
CUDA call.  No kernel runs here."""

import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from nnue_pytorch_b200 import _build, _lib

    _build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "nnue_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nnue_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_function_is_exported_and_bound(lib):
    from nnue_pytorch_b200 import _lib

    names = _declared_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/nnue_b200.h but not exported"
    assert sorted(_lib.PROTOTYPES) == names


def test_abi_version(lib):
    assert lib.nnue_b200_abi_version() == 1


def test_host_side_argument_validation(lib):
    from nnue_pytorch_b200 import _lib

    # negative sizes and bad enums are rejected before any CUDA call
    assert lib.nnue_ft_sparse_fwd(None, None, None, None, -1, 4, 4, 4, None) == -1
    assert b"negative size" in lib.nnue_b200_last_error()
    assert lib.nnue_ft_fused_fwd(None, None, None, None, None, None, None, 1.0, 0.0, 0.0, 1.0, None, None, None, None,
                                 4, 4, 4, 7, 8, None) == -1  # odd l1
    assert b"even" in lib.nnue_b200_last_error()
    assert lib.nnue_ft_fused_bwd(None, None, None, None, None, 1.0, 1.0, None, None, None, None, None, None,
                                 4, 4, 4, 8, 8, None, 0, 9, None) == -1  # unknown mode
    assert lib.nnue_b200_tune(b"no_such_knob", 1) == -1
    assert lib.nnue_rangerlite_update(None, None, None, None, None, None, None, None, 1, 1, None, None) == -1
    # newer entry points: the same convention
    def sliced(n, *bounds, by_columns=0):
        sp = _lib.BwdSlices()
        sp.n_slices = n
        sp.by_columns = by_columns
        for i, b in enumerate(bounds):
            sp.row_bounds[i] = b
        return lib.nnue_ft_fused_bwd_sliced(None, None, None, None, None, 1.0, 1.0, None, None, None, None, None, None,
                                            4, 4, 10, 8, 8, None, 0, 2, C.byref(sp), None)

    assert sliced(2, 0, 10, 5) == -1 and b"row bounds" in lib.nnue_b200_last_error()   # bounds decrease / wrong end
    assert sliced(1, 1, 10) == -1 and b"row bounds" in lib.nnue_b200_last_error()      # does not start at row 0
    assert sliced(1, 0, 9) == -1 and b"row bounds" in lib.nnue_b200_last_error()       # does not end at N
    assert sliced(17, 0) == -1 and b"slices" in lib.nnue_b200_last_error()             # too many
    assert sliced(2, 0, 4, 10) == -1 and b"null output" in lib.nnue_b200_last_error()  # valid slices: next check
    assert sliced(1, 0, 10, by_columns=1) == -1 and b"column bounds" in lib.nnue_b200_last_error()   # must end at L1 + P
    assert sliced(2, 0, 8, 16, by_columns=1) == -1 and b"multiples of 128" in lib.nnue_b200_last_error()
    assert sliced(1, 0, 16, by_columns=1) == -1 and b"null output" in lib.nnue_b200_last_error()
    assert lib.nnue_ft_fused_bwd_column_tile(3072, 8) == 256 and lib.nnue_ft_fused_bwd_column_tile(7, 8) == 0
    assert lib.nnue_l2_read_probe(None, 0, 1, 1, 0, None, None) == -1
    assert lib.nnue_b200_profile(1) == 0 and lib.nnue_b200_profile(0) == 0
    assert lib.nnue_batch_build_halfka(None, 4, 7, 64, None, None, None, None, None, None, None, None, None) == -1  # layout
    assert lib.nnue_batch_build_halfka(None, 4, 1, 32, None, None, None, None, None, None, None, None, None) == -1  # K < 64
    assert lib.nnue_batch_build_halfka(None, 0, 0, 32, None, None, None, None, None, None, None, None, None) == 0
    assert lib.nnue_sf_loss(None, None, None, None, None, None, None, None, None, None, None, None, 4, None) == -1
    assert lib.nnue_grad_sumsq_multi(None, None, 3, None, None) == -1 and lib.nnue_grad_sumsq_multi(None, None, 0, None, None) == 0
    assert lib.nnue_rangerlite_update_multi(None, 2, None, None) == -1 and lib.nnue_rangerlite_update_multi(None, 0, None, None) == 0
    assert lib.nnue_ls_effective_weights(*([None] * 15), 0, 8, None) == -1       # L1 = 0
    assert lib.nnue_ls_plan(None, 4, 99, None, 0, None) == -4                    # too many buckets
    # empty batches are a no-op that needs no device
    assert lib.nnue_ft_sparse_fwd(None, None, None, None, 0, 4, 4, 4, None) == 0
    assert lib.nnue_ft_fused_fwd(None, None, None, None, None, None, None, 1.0, 0.0, 0.0, 1.0, None, None, None, None,
                                 0, 4, 4, 8, 8, None) == 0


def test_workspace_sizes_are_monotone(lib):
    f = lib.nnue_ft_fused_bwd_workspace_bytes
    a = f(1024, 64, 23232, 1024, 8, 2)
    b = f(16384, 64, 23232, 3072, 8, 2)
    assert 0 < a < b
    # G [2B, W] dominates: 2*16384*3080*4 bytes
    assert b >= 2 * 16384 * 3080 * 4
    assert f(16384, 64, 23232, 3072, 8, 1) == 256
    assert f(-1, 64, 23232, 3072, 8, 2) == 0


def test_product_refuses_cpu_tensors():
    import torch

    from nnue_pytorch_b200 import SparseLinearFunction, double_feature_transform

    idx = torch.zeros(2, 4, dtype=torch.int32)
    w = torch.zeros(8, 16)
    b = torch.zeros(16)
    with pytest.raises(RuntimeError):
        SparseLinearFunction.apply(idx, w, b)
    with pytest.raises(RuntimeError):
        SparseLinearFunction.apply(idx, w, b, "torch")
    with pytest.raises(ValueError):
        SparseLinearFunction.apply(idx, w, b, "nonsense")
    us = torch.zeros(2, 1)
    with pytest.raises(RuntimeError):
        double_feature_transform(us, us, idx, idx, torch.zeros(2, dtype=torch.int64), w, b, 1.0, 8)
    with pytest.raises(ValueError):
        double_feature_transform(us, us, idx, idx, torch.zeros(2, dtype=torch.int64), w, b, 1.0, 8, "nonsense")


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "nnue_pytorch_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
                assert "_work/" not in src, f


def test_packed_position_record_matches_the_header_struct():
    import ctypes as C

    from nnue_pytorch_b200 import batch_build

    class Packed(C.Structure):  # field by field as declared in include/nnue_b200.h
        _fields_ = [("piece", C.c_uint16 * 32), ("score", C.c_int16), ("outcome2", C.c_uint8),
                    ("stm_white", C.c_uint8), ("count", C.c_uint8), ("pad", C.c_uint8 * 3)]

    assert C.sizeof(Packed) == batch_build.PACKED_DTYPE.itemsize == 72
    for name in ("piece", "score", "outcome2", "stm_white", "count", "pad"):
        assert getattr(Packed, name).offset == batch_build.PACKED_DTYPE.fields[name][1]
    header = open(os.path.join(ROOT, "include", "nnue_b200.h")).read()
    body = header[header.index("typedef struct nnue_packed_position {"):header.index("} nnue_packed_position;")]
    assert [ln.split()[1].split("[")[0].rstrip(";") for ln in body.splitlines()[1:] if ln.strip()] == [
        "piece", "score", "outcome2", "stm_white", "count", "pad"]


def test_column_slices_of_the_benchmark_sit_on_tile_borders():
    """`bench.column_slices` asks the library for the backward's column tile (a host-side query) and cuts the
    table's row into slices on tile borders, the last one taking the PSQT columns."""
    import importlib.util
    import os

    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(os.path.dirname(__file__), os.pardir, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.column_slices(3072, 8, 4) == [0, 768, 1536, 2304, 3080]
    assert bench.column_slices(3072, 8, 1) == [0, 3080]
    assert bench.column_slices(3072, 8, 13) == [256 * i for i in range(13)] + [3080]
    assert bench.column_slices(128, 8, 4) == [0, 136]  # one tile only: nothing to cut


def test_kept_integer_table_cache_keys_on_storage_and_version():
    """The cache of the integer table is fresh only for the very storage and torch version counter it was made
    from, with the same sizes and scales; a write through `.data` moves neither (which is why callers that make one
    invalidate the cache themselves)."""
    import torch

    from nnue_pytorch_b200._launch import QuantTableCache

    w = torch.nn.Parameter(torch.zeros(6, 24))
    q16, psqt, stats = torch.zeros(7, 16, dtype=torch.int16), torch.zeros(6, 8), torch.zeros(2, dtype=torch.int32)
    cache = QuantTableCache()
    assert not cache.fresh(w, 16, 256.0, 9600.0) and cache.emit_struct(w) is None
    cache.store(w, 16, 256.0, 9600.0, q16, psqt, stats)
    assert cache.fresh(w, 16, 256.0, 9600.0)
    assert not cache.fresh(w, 16, 128.0, 9600.0) and not cache.fresh(w, 8, 256.0, 9600.0)  # other scale, other split
    e = cache.emit_struct(w)
    assert e is not None and (e.L1, e.P, e.q16_pitch) == (16, 8, 16) and e.q16 == q16.data_ptr()
    with torch.no_grad():
        w.add_(1.0)                      # an in-place change through torch moves the version counter
    assert not cache.fresh(w, 16, 256.0, 9600.0) and cache.emit_struct(w) is None
    cache.mark(w)                        # "the buffers hold the table of w as it is now"
    assert cache.fresh(w, 16, 256.0, 9600.0)
    w.data.mul_(2.0)                     # a write behind the counter's back is NOT seen ...
    assert cache.fresh(w, 16, 256.0, 9600.0)
    cache.invalidate()                   # ... so whoever makes one says so
    assert not cache.fresh(w, 16, 256.0, 9600.0)
    w.data = torch.ones(6, 24)           # new storage: never fresh
    cache.store(torch.nn.Parameter(torch.zeros(6, 24)), 16, 256.0, 9600.0, q16, psqt, stats)
    assert not cache.fresh(w, 16, 256.0, 9600.0)
