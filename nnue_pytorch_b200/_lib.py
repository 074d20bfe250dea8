"""ctypes binding of libnnue_b200.so (declared in include/nnue_b200.h).

Loading never falls back to anything: a missing or unloadable library raises,
and so does every call made without a CUDA device.  The library is built
in-tree by `nnue_pytorch_b200._build`.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libnnue_b200.so"

NNUE_OK = 0
BWD_AUTO, BWD_ATOMIC, BWD_SEGMENT = 0, 1, 2
_BWD_MODES = {"auto": BWD_AUTO, "atomic": BWD_ATOMIC, "segment": BWD_SEGMENT}


class RangerHParams(C.Structure):
    """Mirror of `nnue_ranger_hparams`."""

    _fields_ = [
        ("beta2", C.c_float),
        ("one_minus_beta2", C.c_float),
        ("mom", C.c_float),
        ("one_minus_mom", C.c_float),
        ("one_plus_f", C.c_float),
        ("f", C.c_float),
        ("noise_norm_inv", C.c_float),
        ("step_size", C.c_float),
        ("bc2_sqrt", C.c_float),
        ("eps", C.c_float),
        ("wd_keep", C.c_float),
        ("alpha", C.c_float),
        ("one_minus_alpha", C.c_float),
        ("use_pnm", C.c_int32),
        ("step_is_odd", C.c_int32),
        ("do_merge", C.c_int32),
        ("phase", C.c_int32),
    ]


class RangerTensor(C.Structure):
    """Mirror of `nnue_ranger_tensor`."""

    _fields_ = [("p", C.c_void_p), ("grad", C.c_void_p), ("grad_ma", C.c_void_p), ("neg_grad_ma", C.c_void_p),
                ("variance_ma", C.c_void_p), ("slow", C.c_void_p), ("n", C.c_int64), ("hp", RangerHParams)]


MULTI_MAX = 16  # NNUE_MULTI_MAX


class QuantParams(C.Structure):
    """Mirror of `nnue_quant_params`."""

    _fields_ = [
        ("ft_max", C.c_int32),
        ("ft_shift", C.c_int32),
        ("hidden_max", C.c_int32),
        ("sqr_shift_l1", C.c_int32),
        ("sqr_eps_l1", C.c_int32),
        ("lin_shift_l1", C.c_int32),
        ("sqr_shift_l2", C.c_int32),
        ("sqr_eps_l2", C.c_int32),
        ("lin_shift_l2", C.c_int32),
        ("skip_mul", C.c_int32),
        ("out_mul", C.c_int32),
        ("out_div", C.c_int32),
    ]


MAX_SLICES = 16  # NNUE_BWD_MAX_SLICES


class BwdSlices(C.Structure):
    """Mirror of `nnue_bwd_slices`."""

    _fields_ = [("n_slices", C.c_int32), ("row_bounds", C.c_int64 * (MAX_SLICES + 1)), ("events", C.c_void_p * MAX_SLICES),
                ("by_columns", C.c_int32)]


class FtBlock(C.Structure):
    """Mirror of `nnue_ft_block`."""

    _fields_ = [("weight", C.c_void_p), ("virtual_weight", C.c_void_p), ("rows", C.c_int64), ("n_virtual", C.c_int64)]


class TableEmit(C.Structure):
    """Mirror of `nnue_table_emit`."""

    _fields_ = [("q16", C.c_void_p), ("q16_pitch", C.c_int64), ("psqt", C.c_void_p), ("d_stats", C.c_void_p),
                ("L1", C.c_int32), ("P", C.c_int32), ("scale_main", C.c_float), ("scale_psqt", C.c_float)]


class DdpEmit(C.Structure):
    """Mirror of `nnue_ddp_emit`."""

    _fields_ = [("h_q16_ptrs", C.POINTER(C.c_void_p)), ("h_psqt_ptrs", C.POINTER(C.c_void_p)),
                ("h_stats_ptrs", C.POINTER(C.c_void_p)), ("d_stats_local", C.c_void_p), ("q16_pitch", C.c_int64),
                ("L1", C.c_int32), ("P", C.c_int32), ("scale_main", C.c_float), ("scale_psqt", C.c_float),
                ("fp32_to_peers", C.c_int32)]


class LsWeightScales(C.Structure):
    """Mirror of `nnue_ls_weight_scales`."""

    _fields_ = [(n, C.c_float) for n in ("w1", "b1", "w2", "b2", "w3", "b3")] + [("quantize", C.c_int32)]


class LossParams(C.Structure):
    """Mirror of `nnue_loss_params`."""

    _fields_ = [(n, C.c_float) for n in (
        "in_offset", "out_offset", "in_scaling", "out_scaling", "pow_exp", "qp_asymmetry", "w1", "w2",
        "tb_remap_base", "tb_remap_scale", "tb_remap_decay", "lam", "net_scale")]


class LsParams(C.Structure):
    """Mirror of `nnue_ls_params`."""

    _fields_ = [
        ("act_scale", C.c_float),
        ("act_eps", C.c_float),
        ("sqr_corr", C.c_float),
        ("max_hidden", C.c_float),
        ("out_den", C.c_float),
        ("out_mul", C.c_float),
        ("quantize_out", C.c_int32),
    ]


_P = C.c_void_p
_I64 = C.c_int64
_I32 = C.c_int32
_SZ = C.c_size_t

# name -> (restype, argtypes); the complete export list of include/nnue_b200.h
PROTOTYPES = {
    "nnue_b200_abi_version": (C.c_int, []),
    "nnue_b200_last_error": (C.c_char_p, []),
    "nnue_b200_launch_count": (C.c_int64, []),
    "nnue_b200_tune": (C.c_int, [C.c_char_p, C.c_int]),
    "nnue_b200_device_status": (C.c_int, [_P, C.POINTER(_I64), C.POINTER(_I64)]),
    "nnue_b200_profile": (C.c_int, [_I32]),
    "nnue_b200_profile_read": (C.c_int, [_I32, C.POINTER(C.c_char_p), C.POINTER(C.c_double), C.POINTER(_I64)]),
    "nnue_l2_read_probe": (C.c_int, [_P, _I64, _I64, _I32, _I32, _P, _P]),
    "nnue_ft_sparse_fwd": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _I64, _I32, _P]),
    "nnue_ft_sparse_bwd_workspace_bytes": (_SZ, [_I64, _I32, _I64, _I32, _I32]),
    "nnue_ft_sparse_bwd": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _I64, _I32, _P, _SZ, _I32, _P]),
    "nnue_ft_sparse_bwd_static": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _I64, _I32, _P]),
    "nnue_ft_fused_fwd": (
        C.c_int,
        [_P, _P, _P, _P, _P, _P, _P, C.c_float, C.c_float, C.c_float, C.c_float, _P, _P, _P, _P,
         _I64, _I32, _I64, _I32, _I32, _P],
    ),
    "nnue_ft_fused_bwd_workspace_bytes": (_SZ, [_I64, _I32, _I64, _I32, _I32, _I32]),
    "nnue_ft_fused_bwd": (
        C.c_int,
        [_P, _P, _P, _P, _P, C.c_float, C.c_float, _P, _P, _P, _P, _P, _P, _I64, _I32, _I64, _I32, _I32,
         _P, _SZ, _I32, _P],
    ),
    "nnue_ft_fused_bwd_sliced": (
        C.c_int,
        [_P, _P, _P, _P, _P, C.c_float, C.c_float, _P, _P, _P, _P, _P, _P, _I64, _I32, _I64, _I32, _I32,
         _P, _SZ, _I32, C.POINTER(BwdSlices), _P],
    ),
    "nnue_ft_prepare_table": (C.c_int, [_P, _P, _P, _I64, _I64, _I32, _I32, C.c_float, C.c_float, _P]),
    "nnue_ft_quantize_table": (C.c_int, [_P, _P, _P, _I64, _P, _I64, _I64, _I32, _I32, C.c_float, C.c_float, _P, _P]),
    "nnue_ft_fused_fwd_q16": (
        C.c_int,
        [_P] * 6 + [_I64, _P, _P, C.c_float, _P, _I32, C.POINTER(FtBlock), _I32, C.c_float, C.c_float, C.c_float, C.c_float,
                    _P, _P, _P, _P, _I64, _I32, _I64, _I32, _I32, _P],
    ),
    "nnue_ft_virtual_grad": (C.c_int, [_P, _P, _I64, _I64, _I32, _P]),
    "nnue_rangerlite_update": (
        C.c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, C.POINTER(RangerHParams), _P],
    ),
    "nnue_rangerlite_update_emit": (
        C.c_int,
        [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I64, C.POINTER(RangerHParams), C.POINTER(TableEmit), _P],
    ),
    "nnue_ddp_reduce_shard": (C.c_int, [C.POINTER(_P), _I32, _I32, _I64, _I64, _P, _P]),
    "nnue_ddp_update_shard": (
        C.c_int,
        [C.POINTER(_P), _I32, _I32, _I64, _I64, _P, _P, _P, _P, _P, _P, C.POINTER(RangerHParams), _P],
    ),
    "nnue_ddp_update_shard_emit": (
        C.c_int,
        [C.POINTER(_P), _I32, _I32, _I64, _I64, _P, _P, _P, _P, _P, _P, C.POINTER(RangerHParams), C.POINTER(DdpEmit), _P],
    ),
    "nnue_ddp_reduce_block": (C.c_int, [C.POINTER(_P), _I32, _I32, _I64, _I64, _I64, _I64, _I64, _P, _P]),
    "nnue_ft_fused_bwd_column_tile": (_I32, [_I32, _I32]),
    "nnue_ddp_publish_stats": (C.c_int, [C.POINTER(DdpEmit), _I32, _I32, _P]),
    "nnue_grad_sumsq_multi": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_int64), _I32, _P, _P]),
    "nnue_rangerlite_update_multi": (C.c_int, [C.POINTER(RangerTensor), _I32, _P, _P]),
    "nnue_lookahead_merge": (C.c_int, [_P, _P, _I64, C.c_float, _P]),
    "nnue_grad_sumsq": (C.c_int, [_P, _I64, _P, _P]),
    "nnue_clip_coef": (C.c_int, [_P, C.c_float, C.c_float, _P, _P]),
    "nnue_ls_plan_bytes": (_SZ, [_I64, _I32]),
    "nnue_ls_plan": (C.c_int, [_P, _I64, _I32, _P, _SZ, _P]),
    "nnue_ls_l1_fwd": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _P]),
    "nnue_ls_l1_fwd_tc": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _P]),
    "nnue_ls_l1_bwd_tc_workspace_bytes": (_SZ, [_I32, _I32]),
    "nnue_ls_l1_bwd_tc": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I32, _P, _SZ, _P]),
    "nnue_ls_l1_bwd": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I32, _P]),
    "nnue_ls_tail_fwd": (C.c_int, [_P, _P, _P, _P, _P, _P, C.POINTER(LsParams), _P, _P, _I64, _I32, _P]),
    "nnue_ls_tail_bwd_workspace_bytes": (_SZ, [_I64, _I32]),
    "nnue_ls_tail_bwd": (
        C.c_int,
        [_P, _P, _P, _P, _P, _P, C.POINTER(LsParams), _P, _P, _P, _P, _P, _P, _SZ, _I64, _I32, _P],
    ),
    "nnue_quant_eval": (
        C.c_int,
        [_P] * 14 + [_I64, _I32, _I64, _I32, _I32, _I32, _I32, _I32, C.POINTER(QuantParams), _P],
    ),
    "nnue_ls_effective_weights": (C.c_int, [_P] * 8 + [C.POINTER(LsWeightScales)] + [_P] * 6 + [_I32, _I32, _P]),
    "nnue_ls_fold_grads": (C.c_int, [_P, _P, _P, _P, _I32, _I32, _P]),
    "nnue_sf_loss_workspace_bytes": (_SZ, []),
    "nnue_sf_loss": (C.c_int, [_P] * 6 + [C.POINTER(LossParams), _P, _P, _P, _P, _P, _I64, _P]),
    "nnue_quant_eval_workspace_bytes": (_SZ, [_I64, _I32]),
    "nnue_quant_eval_tiled": (
        C.c_int,
        [_P] * 14 + [_I64, _I32, _I64, _I32, _I32, _I32, _I32, _I32, C.POINTER(QuantParams), _P, _SZ, _P],
    ),
    "nnue_ft_prepare_bias_q16": (C.c_int, [_P, _P, _I32, _I32, C.c_float, _P, _I32, _P]),
    "nnue_quant_pack_table": (C.c_int, [_P, _P, _P, _I64, _I32, _P]),
    "nnue_quant_eval_packed": (
        C.c_int,
        [_P] * 5 + [_I32] + [_P] * 9 + [_I64, _I32, _I64, _I32, _I32, _I32, _I32, _I32, C.POINTER(QuantParams), _P, _SZ, _P],
    ),
    "nnue_batch_build_halfka": (C.c_int, [_P, _I64, _I32, _I32, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
}

_lib = None


class NnueB200Error(RuntimeError):
    pass


def load() -> C.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NnueB200Error(
            f"{LIB_PATH} is missing: build it with `python -m nnue_pytorch_b200._build` "
            "(there is no CPU or PyTorch fallback for these kernels)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the export is missing
        fn.restype = res
        fn.argtypes = args
    if lib.nnue_b200_abi_version() != 1:
        raise NnueB200Error("libnnue_b200.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != NNUE_OK:
        msg = load().nnue_b200_last_error().decode("utf-8", "replace")
        raise NnueB200Error(f"{what} failed with status {status}: {msg}")


def bwd_mode(name: str) -> int:
    try:
        return _BWD_MODES[name]
    except KeyError:
        raise ValueError(f"unknown backward mode {name!r}; expected one of {sorted(_BWD_MODES)}") from None


def tune(key: str, value: int) -> None:
    check(load().nnue_b200_tune(key.encode(), int(value)), f"nnue_b200_tune({key})")


def profile(enable: bool) -> None:
    """Start (and clear) or stop the library's per-kernel event record."""
    check(load().nnue_b200_profile(1 if enable else 0), "nnue_b200_profile")


def profile_summary() -> dict[str, dict]:
    """{kernel name: {"launches": n, "total_ms": t, "mean_ms": t / n}} of the record; synchronises the device."""
    lib, out, i = load(), {}, 0
    while True:
        name, ms, n = C.c_char_p(), C.c_double(0.0), _I64(0)
        if lib.nnue_b200_profile_read(i, C.byref(name), C.byref(ms), C.byref(n)) != NNUE_OK:
            break
        out[name.value.decode()] = {"launches": int(n.value), "total_ms": ms.value,
                                    "mean_ms": ms.value / max(int(n.value), 1)}
        i += 1
    return out


def device_status(stream_ptr: int) -> None:
    """Synchronise the stream and raise if a kernel skipped bad indices or a wait ran out."""
    bad, tmo = _I64(0), _I64(0)
    check(load().nnue_b200_device_status(stream_ptr, C.byref(bad), C.byref(tmo)), "device status")
