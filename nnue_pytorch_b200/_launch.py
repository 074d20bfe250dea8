"""Thin launch helpers between torch tensors and the C ABI.

torch is used here for device memory, the current stream and nothing else:
every function takes tensors, checks the contract the reference asserts
(model/modules/feature_transformer/sparse_linear_functions.py:58-76 and
fused_ft_functions.py:23-45 of the reference project), and hands raw device
pointers to libnnue_b200.so.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_BWD_MODE = "auto"


class KernelTimer:
    """Optional CUDA-event timing of the C-ABI calls, on the stream they launch
    on.  Nothing synchronises until `summary()` is read."""

    def __init__(self):
        self.spans: dict[str, list] = {}

    def span(self, name: str, device: torch.device):
        return _Span(self, name, device)

    def summary(self) -> dict[str, dict]:
        torch.cuda.synchronize()
        out = {}
        for name, pairs in self.spans.items():
            ms = [a.elapsed_time(b) for a, b in pairs]
            out[name] = {"calls": len(ms), "total_ms": sum(ms), "mean_ms": sum(ms) / max(len(ms), 1)}
        return out


class _Span:
    def __init__(self, timer, name, device):
        self.timer, self.name, self.device = timer, name, device

    def __enter__(self):
        self.a = torch.cuda.Event(enable_timing=True)
        self.b = torch.cuda.Event(enable_timing=True)
        self.a.record(torch.cuda.current_stream(self.device))

    def __exit__(self, *exc):
        self.b.record(torch.cuda.current_stream(self.device))
        self.timer.spans.setdefault(self.name, []).append((self.a, self.b))


class _NoSpan:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


def exchange_of(t: torch.Tensor | None):
    """The data-parallel table exchange (`ddp.ShardedTableExchange`) that owns tensor `t`,
    or None.  The exchange marks its table parameter; tables derived from the parameter
    (`PrepareTableFunction`) carry the mark on.  With an exchange, the fused backward writes
    the table gradient into the exchange's shared buffer instead of a fresh tensor and the
    autograd functions hand no gradient to the parameter."""
    return getattr(t, "_nnue_exchange", None) if t is not None else None


TIMER: KernelTimer | None = None
_NO_SPAN = _NoSpan()


def _span(name: str, device: torch.device):
    return TIMER.span(name, device) if TIMER is not None else _NO_SPAN


def set_backward_mode(mode: str) -> None:
    """Select the scatter strategy of the backward kernels: auto | atomic | segment."""
    global _BWD_MODE
    _lib.bwd_mode(mode)
    _BWD_MODE = mode


def get_backward_mode() -> str:
    return _BWD_MODE


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(
                "nnue_pytorch_b200 kernels run on CUDA tensors only (there is no CPU or PyTorch fallback)"
            )
        if t.device != dev:
            raise RuntimeError("all tensors must live on the same CUDA device")
    return dev


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


# --------------------------------------------------------------------------
def sparse_linear_forward(indices: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    assert indices.dim() == 2 and indices.dtype == torch.int32
    assert weight.dim() == 2 and weight.dtype == torch.float32
    assert bias.dim() == 1 and bias.dtype == torch.float32
    assert weight.shape[1] == bias.shape[0]
    dev = _require_cuda(indices, weight, bias)
    assert indices.is_contiguous() and weight.is_contiguous() and bias.is_contiguous()
    B, K = indices.shape
    N, W = weight.shape
    out = torch.empty(B, W, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev), _span("sparse_fwd", dev):
        st = _lib.load().nnue_ft_sparse_fwd(
            _ptr(indices), _ptr(weight), _ptr(bias), _ptr(out), B, K, N, W, _stream(dev)
        )
    _lib.check(st, "nnue_ft_sparse_fwd")
    return out


def sparse_linear_backward(
    indices: torch.Tensor, grad_out: torch.Tensor, num_inputs: int, mode: str | None = None
) -> tuple[torch.Tensor, torch.Tensor]:
    dev = _require_cuda(indices, grad_out)
    grad_out = grad_out.contiguous()
    assert grad_out.dtype == torch.float32
    B, K = indices.shape
    W = grad_out.shape[1]
    m = _lib.bwd_mode(mode or _BWD_MODE)
    lib = _lib.load()
    grad_w = torch.empty(num_inputs, W, dtype=torch.float32, device=dev)
    grad_b = torch.empty(W, dtype=torch.float32, device=dev)
    ws = _workspace(lib.nnue_ft_sparse_bwd_workspace_bytes(B, K, num_inputs, W, m), dev)
    with torch.cuda.device(dev), _span("sparse_bwd", dev):
        st = lib.nnue_ft_sparse_bwd(
            _ptr(indices), _ptr(grad_out), _ptr(grad_w), _ptr(grad_b), B, K, num_inputs, W,
            _ptr(ws), ws.numel(), m, _stream(dev),
        )
    _lib.check(st, "nnue_ft_sparse_bwd")
    return grad_w, grad_b


# --------------------------------------------------------------------------
def fused_forward(us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, l1_size,
                  act_quant_scale: float = 0.0, act_quant_eps: float = 0.0, out_scale: float = 1.0):
    assert l1_size % 2 == 0
    dev = _require_cuda(us, them, white_indices, black_indices, psqt_indices, weight, bias)
    assert us.dtype == torch.float32 and them.dtype == torch.float32
    assert white_indices.dtype == torch.int32 and black_indices.dtype == torch.int32
    assert psqt_indices.dtype == torch.int64
    assert weight.dtype == torch.float32 and bias.dtype == torch.float32
    assert white_indices.dim() == 2 and black_indices.dim() == 2 and psqt_indices.dim() == 1
    assert weight.dim() == 2 and bias.dim() == 1 and weight.shape[1] == bias.shape[0]
    assert white_indices.shape == black_indices.shape
    assert white_indices.shape[0] == psqt_indices.shape[0]
    assert us.numel() == white_indices.shape[0] and them.numel() == white_indices.shape[0]
    assert us.is_contiguous() and them.is_contiguous()
    assert white_indices.is_contiguous() and black_indices.is_contiguous() and psqt_indices.is_contiguous()
    assert weight.is_contiguous() and bias.is_contiguous()
    B, K = white_indices.shape
    N, W = weight.shape
    P = W - l1_size
    assert P >= 0
    l0 = torch.empty(B, l1_size, dtype=torch.float32, device=dev)
    wpsqt = torch.empty(B, 1, dtype=torch.float32, device=dev)
    bpsqt = torch.empty(B, 1, dtype=torch.float32, device=dev)
    saved = torch.empty(B, 4, l1_size // 2, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev), _span("fused_fwd", dev):
        st = _lib.load().nnue_ft_fused_fwd(
            _ptr(us), _ptr(them), _ptr(white_indices), _ptr(black_indices), _ptr(psqt_indices),
            _ptr(weight), _ptr(bias), float(max_ft_activation),
            float(act_quant_scale), float(act_quant_eps), float(out_scale),
            _ptr(l0), _ptr(wpsqt), _ptr(bpsqt), _ptr(saved), B, K, N, l1_size, P, _stream(dev),
        )
    _lib.check(st, "nnue_ft_fused_fwd")
    return l0, wpsqt, bpsqt, saved


def fused_backward(
    us, them, white_indices, black_indices, psqt_indices, max_ft_activation, l1_size, num_inputs, num_outputs,
    grad_l0, grad_wpsqt, grad_bpsqt, saved, mode: str | None = None, out_scale: float = 1.0,
    sink: torch.Tensor | None = None, slices=None,
):
    """`sink`: preallocated [num_inputs, num_outputs] destination of the table gradient (a fresh
    tensor otherwise).  `slices`: (bounds, torch events[, by_columns]) to deliver the gradient slice by slice
    (`nnue_ft_fused_bwd_sliced`: row bounds, or column bounds in floats with by_columns); they belong to this one call."""
    dev = _require_cuda(us, grad_l0, grad_wpsqt, grad_bpsqt, saved)
    grad_l0 = grad_l0.contiguous()
    grad_wpsqt = grad_wpsqt.contiguous()
    grad_bpsqt = grad_bpsqt.contiguous()
    B, K = white_indices.shape
    P = num_outputs - l1_size
    m = _lib.bwd_mode(mode or _BWD_MODE)
    lib = _lib.load()
    if sink is not None:
        assert tuple(sink.shape) == (num_inputs, num_outputs) and sink.device == dev and sink.is_contiguous()
        assert sink.dtype == torch.float32
        grad_w = sink
    else:
        grad_w = torch.empty(num_inputs, num_outputs, dtype=torch.float32, device=dev)
    grad_b = torch.empty(num_outputs, dtype=torch.float32, device=dev)
    spec = None
    if slices is not None:
        bounds, events = slices[0], slices[1]
        assert len(bounds) - 1 == len(events) <= _lib.MAX_SLICES
        spec = _lib.BwdSlices()
        spec.n_slices = len(events)
        spec.by_columns = int(bool(slices[2])) if len(slices) > 2 else 0
        for i, b in enumerate(bounds):
            spec.row_bounds[i] = int(b)
        for i, e in enumerate(events):
            spec.events[i] = e.cuda_event
    ws = _workspace(lib.nnue_ft_fused_bwd_workspace_bytes(B, K, num_inputs, l1_size, P, m), dev)
    with torch.cuda.device(dev), _span("fused_bwd", dev):
        st = lib.nnue_ft_fused_bwd_sliced(
            _ptr(us), _ptr(them), _ptr(white_indices), _ptr(black_indices), _ptr(psqt_indices),
            float(max_ft_activation), float(out_scale), _ptr(grad_l0), _ptr(grad_wpsqt), _ptr(grad_bpsqt), _ptr(saved),
            _ptr(grad_w), _ptr(grad_b), B, K, num_inputs, l1_size, P, _ptr(ws), ws.numel(), m,
            C.byref(spec) if spec is not None else None, _stream(dev),
        )
    _lib.check(st, "nnue_ft_fused_bwd_sliced")
    return grad_w, grad_b


# --------------------------------------------------------------------------
def prepare_table(weight, virtual_weight, l1_size: int, scale_main: float, scale_psqt: float,
                  out: torch.Tensor | None = None, span: str = "prepare_table") -> torch.Tensor:
    """fq(weight + virtual_weight.repeat(N // n_virtual, 1)) in one pass (see nnue_ft_prepare_table).
    `out`: optional contiguous destination with at least weight.numel() elements."""
    dev = _require_cuda(weight) if virtual_weight is None else _require_cuda(weight, virtual_weight)
    assert weight.dtype == torch.float32 and weight.dim() == 2 and weight.is_contiguous()
    N, W = weight.shape
    nv = 0
    if virtual_weight is not None:
        assert virtual_weight.dtype == torch.float32 and virtual_weight.is_contiguous()
        assert virtual_weight.shape[1] == W and N % virtual_weight.shape[0] == 0
        nv = virtual_weight.shape[0]
    if out is None:
        out = torch.empty_like(weight)
    else:
        assert out.dtype == torch.float32 and out.is_contiguous() and out.numel() >= weight.numel() and out.device == dev
    with torch.cuda.device(dev), _span(span, dev):
        st = _lib.load().nnue_ft_prepare_table(
            _ptr(weight), _ptr(virtual_weight), _ptr(out), N, nv, l1_size, W - l1_size,
            float(scale_main), float(scale_psqt), _stream(dev),
        )
    _lib.check(st, "nnue_ft_prepare_table")
    return out


def prepare_bias_q16(bias: torch.Tensor, l1_size: int, scale_main: float, stats: torch.Tensor, overwrite: bool) -> torch.Tensor:
    """`nnue_ft_prepare_bias_q16`: the fake-quantized bias the int16 forward adds (PSQT part zero) and its range
    statistics into `stats` (int32 [2]; added, or written over with `overwrite`), one launch."""
    dev = _require_cuda(bias, stats)
    assert bias.dtype == torch.float32 and bias.is_contiguous() and stats.dtype == torch.int32 and stats.numel() == 2
    out = torch.empty_like(bias)
    with torch.cuda.device(dev), _span("prepare_bias", dev):
        st = _lib.load().nnue_ft_prepare_bias_q16(_ptr(bias), _ptr(out), int(l1_size), bias.numel() - int(l1_size),
                                                  float(scale_main), _ptr(stats), int(bool(overwrite)), _stream(dev))
    _lib.check(st, "nnue_ft_prepare_bias_q16")
    return out


def quantize_blocks(blocks, l1_size: int, scale_main: float, scale_psqt: float, overflow: torch.Tensor | None = None,
                    out=None):
    """The integer form of the table the forward reads when weights are fake-quantized
    (`nnue_ft_quantize_table`, one launch per parameter block).  `blocks` is a list of
    (weight [rows, W], virtual_weight [n_virtual, W] or None) in table order.  Returns
    (q16 int16 [N, L1], psqt float32 [N, P], stats int32 [2] = entries outside int16, max |k|); a given
    `overflow` (the stats of an earlier call) is updated instead of a fresh one; `out` = (q16 [N + 1, L1], psqt [N, P])
    to write into existing buffers."""
    dev = _require_cuda(*[t for b in blocks for t in b if t is not None])
    W = blocks[0][0].shape[1]
    P = W - l1_size
    n_total = sum(w.shape[0] for w, _ in blocks)
    pitch = l1_size  # rows back to back (a padded pitch was measured: no faster on B200)
    if out is not None:
        q16, psqt = out
        assert q16.dtype == torch.int16 and tuple(q16.shape) == (n_total + 1, pitch) and q16.is_contiguous()
        assert psqt.dtype == torch.float32 and tuple(psqt.shape) == (n_total, P) and psqt.is_contiguous()
    else:
        q16 = torch.empty(n_total + 1, pitch, dtype=torch.int16, device=dev)
        psqt = torch.empty(n_total, max(P, 1), dtype=torch.float32, device=dev)[:, :P]
    q16[n_total].zero_()  # the all-zero row that padding and out-of-range list entries read
    if overflow is None:
        overflow = torch.zeros(2, dtype=torch.int32, device=dev)
    lib = _lib.load()
    at = 0
    with torch.cuda.device(dev), _span("quantize_table", dev):
        for w, v in blocks:
            assert w.dtype == torch.float32 and w.dim() == 2 and w.is_contiguous() and w.shape[1] == W
            nv = 0
            if v is not None:
                assert v.dtype == torch.float32 and v.is_contiguous() and v.shape[1] == W and w.shape[0] % v.shape[0] == 0
                nv = v.shape[0]
            rows = w.shape[0]
            st = lib.nnue_ft_quantize_table(
                _ptr(w), _ptr(v), q16.data_ptr() + at * pitch * 2, pitch, psqt.data_ptr() + at * P * 4, rows, nv,
                l1_size, P, float(scale_main), float(scale_psqt), _ptr(overflow), _stream(dev))
            _lib.check(st, "nnue_ft_quantize_table")
            at += rows
    return q16, psqt, overflow


def fused_forward_q16(us, them, white_indices, black_indices, psqt_indices, q16, psqt, bias_fq, overflow, blocks,
                      scale_main: float, max_ft_activation, l1_size, act_quant_scale: float = 0.0,
                      act_quant_eps: float = 0.0, out_scale: float = 1.0, master: bool = True):
    """`nnue_ft_fused_fwd_q16`: the fused forward on the tensors `quantize_blocks` made (same outputs
    and saved tensor as `fused_forward`).  `overflow` holds one or more [overflow count, max |k|] pairs.
    `master=False`: the fp32 rows of the (single) block are not valid on this device; a forward that would need
    them is reported by `device_status` instead."""
    dev = _require_cuda(us, them, white_indices, black_indices, psqt_indices, q16, bias_fq, overflow)
    assert us.dtype == torch.float32 and them.dtype == torch.float32
    assert white_indices.dtype == torch.int32 and black_indices.dtype == torch.int32 and psqt_indices.dtype == torch.int64
    assert white_indices.shape == black_indices.shape and white_indices.shape[0] == psqt_indices.shape[0]
    assert us.is_contiguous() and them.is_contiguous() and white_indices.is_contiguous() and black_indices.is_contiguous()
    assert psqt_indices.is_contiguous() and q16.is_contiguous() and bias_fq.is_contiguous()
    assert q16.dtype == torch.int16 and q16.shape[1] >= l1_size and bias_fq.dtype == torch.float32
    B, K = white_indices.shape
    N = q16.shape[0] - 1  # the last row is the all-zero row
    P = bias_fq.shape[0] - l1_size
    arr = (_lib.FtBlock * len(blocks))()
    for d, (w, v) in zip(arr, blocks):
        d.weight, d.virtual_weight, d.rows, d.n_virtual = _ptr(w), _ptr(v), w.shape[0], 0 if v is None else v.shape[0]
    if not master:
        assert len(blocks) == 1 and blocks[0][1] is None
        arr[0].weight = None
    assert overflow.dtype == torch.int32 and overflow.numel() % 2 == 0 and overflow.is_contiguous()
    l0 = torch.empty(B, l1_size, dtype=torch.float32, device=dev)
    wpsqt = torch.empty(B, 1, dtype=torch.float32, device=dev)
    bpsqt = torch.empty(B, 1, dtype=torch.float32, device=dev)
    saved = torch.empty(B, 4, l1_size // 2, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev), _span("fused_fwd", dev):
        st = _lib.load().nnue_ft_fused_fwd_q16(
            _ptr(us), _ptr(them), _ptr(white_indices), _ptr(black_indices), _ptr(psqt_indices), _ptr(q16), q16.shape[1],
            psqt.data_ptr() if P > 0 else None, _ptr(bias_fq), float(scale_main), _ptr(overflow), overflow.numel() // 2, arr, len(blocks),
            float(max_ft_activation), float(act_quant_scale), float(act_quant_eps), float(out_scale),
            _ptr(l0), _ptr(wpsqt), _ptr(bpsqt), _ptr(saved), B, K, N, l1_size, P, _stream(dev))
    _lib.check(st, "nnue_ft_fused_fwd_q16")
    return l0, wpsqt, bpsqt, saved


def virtual_grad(grad: torch.Tensor, n_virtual: int) -> torch.Tensor:
    dev = _require_cuda(grad)
    grad = grad.contiguous()
    N, W = grad.shape
    out = torch.empty(n_virtual, W, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev), _span("virtual_grad", dev):
        st = _lib.load().nnue_ft_virtual_grad(_ptr(grad), _ptr(out), N, n_virtual, W, _stream(dev))
    _lib.check(st, "nnue_ft_virtual_grad")
    return out


def l2_read_probe(rows: int = 23232, total_rows: int = 16384 * 68, rows_per_warp: int = 68, pattern: int = 1,
                  iters: int = 20, device: torch.device | None = None) -> float:
    """GB/s of `nnue_l2_read_probe` over a rows x 1 KiB buffer (24 MB by default: the slice of the
    table one column tile of the forward touches), timed with CUDA events over `iters` launches
    after two warm-ups."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    buf = torch.ones(rows * 256, dtype=torch.float32, device=dev)
    warps = max(total_rows // rows_per_warp, 1)
    sink = torch.empty(warps * 128, dtype=torch.float32, device=dev)
    lib = _lib.load()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.device(dev):
        for i in range(iters + 2):
            if i == 2:
                a.record(torch.cuda.current_stream(dev))
            _lib.check(lib.nnue_l2_read_probe(_ptr(buf), rows, warps, rows_per_warp, pattern, _ptr(sink), _stream(dev)),
                       "nnue_l2_read_probe")
        b.record(torch.cuda.current_stream(dev))
        b.synchronize()
    ms = a.elapsed_time(b) / iters
    return warps * rows_per_warp * 1024 / (ms * 1e-3) / 1e9


def device_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel since the last call skipped an
    out-of-range index or gave up on a bounded wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _lib.device_status(_stream(dev))


def hparams_struct(**kw) -> _lib.RangerHParams:
    hp = _lib.RangerHParams()
    for k, v in kw.items():
        setattr(hp, k, v)
    return hp


class QuantTableCache:
    """The integer table of ONE parameter block without factor rows, kept between steps.

    The forward gathers `q16` / `psqt` (see `quantize_blocks`); writing them costs a pass over the
    whole table.  When the optimizer is this package's RangerLite, its update kernel writes the new
    table while it has the new weights in registers, and the forward finds the cache fresh.  Fresh
    means: made from this very storage (`data_ptr`) at this very `_version` with the same scales.
    Any in-place change through torch (clipping, `copy_`, loading a state dict) moves `_version`,
    a swap of `.data` moves the pointer, and either makes the next forward quantize from scratch.
    Code that writes the parameter through raw pointers must call `mark` (after re-emitting) or
    `invalidate`."""

    def __init__(self, owner=None):
        """`owner`: who keeps the buffers up to date when they are shared between devices (a
        `ddp.ShardedTableExchange`): a stale cache is then rebuilt by `owner.rebuild_integer_rows()`, into the
        same buffers, and `owner.fp32_rows_valid` tells whether the fp32 rows may be read on this device."""
        self.q16 = self.psqt = self.stats = None
        self.key = None
        self.owner = owner

    @staticmethod
    def _key(w, l1, scale_main, scale_psqt):
        return (w.data_ptr(), w._version, tuple(w.shape), int(l1), float(scale_main), float(scale_psqt))

    def fresh(self, w, l1, scale_main, scale_psqt) -> bool:
        return self.q16 is not None and self.key == self._key(w, l1, scale_main, scale_psqt)

    def store(self, w, l1, scale_main, scale_psqt, q16, psqt, stats) -> None:
        self.q16, self.psqt, self.stats = q16, psqt, stats
        self.key = self._key(w, l1, scale_main, scale_psqt)

    def invalidate(self) -> None:
        self.key = None

    def emit_struct(self, w):
        """`nnue_table_emit` for an optimizer update of `w`, or None when the cache does not describe
        the tensor as it is now."""
        if self.q16 is None or self.key is None or self.key[:3] != (w.data_ptr(), w._version, tuple(w.shape)):
            return None
        e = _lib.TableEmit()
        e.q16, e.q16_pitch, e.psqt, e.d_stats = self.q16.data_ptr(), self.q16.shape[1], self.psqt.data_ptr(), self.stats.data_ptr()
        e.L1, e.P, e.scale_main, e.scale_psqt = self.key[3], w.shape[1] - self.key[3], self.key[4], self.key[5]
        return e

    def mark(self, w) -> None:
        """The buffers now hold the table of `w` as it is (an emitting update has just run)."""
        self.key = (w.data_ptr(), w._version, tuple(w.shape)) + self.key[3:]


def ranger_update(p, grad, grad_ma, neg_grad_ma, variance_ma, slow, row_active, grad_scale, hp, emit=None) -> None:
    """`emit`: a `_lib.TableEmit` to have the kernel also write the integer table of the new weights."""
    dev = _require_cuda(p, grad, grad_ma, variance_ma)
    for t in (p, grad, grad_ma, neg_grad_ma, variance_ma, slow):
        if t is not None:
            assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == p.numel()
    if row_active is not None:
        assert row_active.dtype == torch.uint8 and p.dim() == 2 and row_active.numel() == p.shape[0]
        rows, width = p.shape
    elif emit is not None:
        assert p.dim() == 2  # the integer table is written row by row
        rows, width = p.shape
    else:
        rows, width = 1, p.numel()
    with torch.cuda.device(dev), _span("ranger_table" if row_active is not None or p.numel() > (1 << 22) else "ranger_small", dev):
        st = _lib.load().nnue_rangerlite_update_emit(
            _ptr(p), _ptr(grad), _ptr(grad_ma), _ptr(neg_grad_ma), _ptr(variance_ma), _ptr(slow),
            _ptr(row_active), _ptr(grad_scale), rows, width, C.byref(hp),
            C.byref(emit) if emit is not None else None, _stream(dev),
        )
    _lib.check(st, "nnue_rangerlite_update_emit")


def ranger_update_multi(items, grad_scale) -> None:
    """items: list of (p, grad, grad_ma, neg_grad_ma, variance_ma, slow, hp): all
    of them updated by one launch per sixteen tensors."""
    if not items:
        return
    dev = _require_cuda(items[0][0])
    arr = (_lib.RangerTensor * len(items))()
    for d, (p, grad, grad_ma, neg_grad_ma, variance_ma, slow, hp) in zip(arr, items):
        for t in (p, grad, grad_ma, neg_grad_ma, variance_ma, slow):
            if t is not None:
                assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() == p.numel() and t.device == dev
        d.p, d.grad, d.grad_ma, d.neg_grad_ma = _ptr(p), _ptr(grad), _ptr(grad_ma), _ptr(neg_grad_ma)
        d.variance_ma, d.slow, d.n, d.hp = _ptr(variance_ma), _ptr(slow), p.numel(), hp
    with torch.cuda.device(dev), _span("ranger_small", dev):
        st = _lib.load().nnue_rangerlite_update_multi(arr, len(items), _ptr(grad_scale), _stream(dev))
    _lib.check(st, "nnue_rangerlite_update_multi")


def grad_sumsq_multi(grads, out_sumsq) -> None:
    """out_sumsq += sum over the listed gradients of their sums of squares."""
    if not grads:
        return
    dev = _require_cuda(out_sumsq, *grads)
    for g in grads:
        assert g.dtype == torch.float32 and g.is_contiguous()
    ptrs = (C.c_void_p * len(grads))(*[g.data_ptr() for g in grads])
    sizes = (C.c_int64 * len(grads))(*[g.numel() for g in grads])
    with torch.cuda.device(dev):
        st = _lib.load().nnue_grad_sumsq_multi(ptrs, sizes, len(grads), _ptr(out_sumsq), _stream(dev))
    _lib.check(st, "nnue_grad_sumsq_multi")


def lookahead_merge(p, slow, alpha: float) -> None:
    dev = _require_cuda(p, slow)
    assert p.dtype == torch.float32 and slow.dtype == torch.float32
    assert p.is_contiguous() and slow.is_contiguous() and p.numel() == slow.numel()
    with torch.cuda.device(dev):
        st = _lib.load().nnue_lookahead_merge(_ptr(p), _ptr(slow), p.numel(), float(alpha), _stream(dev))
    _lib.check(st, "nnue_lookahead_merge")


def grad_sumsq(grad, out_sumsq) -> None:
    dev = _require_cuda(grad, out_sumsq)
    assert grad.dtype == torch.float32 and grad.is_contiguous()
    with torch.cuda.device(dev):
        st = _lib.load().nnue_grad_sumsq(_ptr(grad), grad.numel(), _ptr(out_sumsq), _stream(dev))
    _lib.check(st, "nnue_grad_sumsq")


def clip_coef(sumsq, max_norm: float, out_coef, prescale: float = 1.0) -> None:
    dev = _require_cuda(sumsq, out_coef)
    with torch.cuda.device(dev):
        st = _lib.load().nnue_clip_coef(_ptr(sumsq), float(max_norm), float(prescale), _ptr(out_coef), _stream(dev))
    _lib.check(st, "nnue_clip_coef")


def ddp_reduce_shard(grad_ptrs: list[int], rank: int, elem_begin: int, elem_end: int, sumsq: torch.Tensor) -> None:
    dev = _require_cuda(sumsq)
    arr = (C.c_void_p * len(grad_ptrs))(*grad_ptrs)
    with torch.cuda.device(dev), _span("ddp_reduce", dev):
        st = _lib.load().nnue_ddp_reduce_shard(arr, len(grad_ptrs), rank, elem_begin, elem_end, _ptr(sumsq), _stream(dev))
    _lib.check(st, "nnue_ddp_reduce_shard")


def ddp_reduce_block(grad_ptrs: list[int], rank: int, row_begin: int, row_end: int, col_begin: int, col_end: int,
                     width: int, sumsq: torch.Tensor) -> None:
    dev = _require_cuda(sumsq)
    arr = (C.c_void_p * len(grad_ptrs))(*grad_ptrs)
    with torch.cuda.device(dev), _span("ddp_reduce", dev):
        st = _lib.load().nnue_ddp_reduce_block(arr, len(grad_ptrs), rank, row_begin, row_end, col_begin, col_end, width,
                                               _ptr(sumsq), _stream(dev))
    _lib.check(st, "nnue_ddp_reduce_block")


def bwd_column_tile(l1_size: int, n_psqt: int) -> int:
    """Floats per column tile of the segment backward at this shape (what column slice bounds must be multiples of)."""
    return int(_lib.load().nnue_ft_fused_bwd_column_tile(int(l1_size), int(n_psqt)))


def ddp_emit_struct(q16_ptrs, psqt_ptrs, stats_ptrs, stats_local, pitch, l1, p, scale_main, scale_psqt, fp32_to_peers):
    """`nnue_ddp_emit` over every rank's integer-table buffers; the pointer arrays stay alive with the struct."""
    e = _lib.DdpEmit()
    e._keep = tuple((C.c_void_p * len(a))(*a) for a in (q16_ptrs, psqt_ptrs, stats_ptrs))
    e.h_q16_ptrs, e.h_psqt_ptrs, e.h_stats_ptrs = e._keep
    e.d_stats_local, e.q16_pitch, e.L1, e.P = stats_local.data_ptr(), pitch, l1, p
    e.scale_main, e.scale_psqt, e.fp32_to_peers = float(scale_main), float(scale_psqt), int(bool(fp32_to_peers))
    return e


def ddp_update_shard(table_ptrs: list[int], rank: int, elem_begin: int, elem_end: int, grad, grad_ma, neg_grad_ma,
                     variance_ma, slow, grad_scale, hp, emit=None) -> None:
    dev = _require_cuda(grad, grad_ma, variance_ma)
    arr = (C.c_void_p * len(table_ptrs))(*table_ptrs)
    with torch.cuda.device(dev), _span("ddp_update", dev):
        st = _lib.load().nnue_ddp_update_shard_emit(
            arr, len(table_ptrs), rank, elem_begin, elem_end, _ptr(grad), _ptr(grad_ma), _ptr(neg_grad_ma),
            _ptr(variance_ma), _ptr(slow), _ptr(grad_scale), C.byref(hp),
            C.byref(emit) if emit is not None else None, _stream(dev),
        )
    _lib.check(st, "nnue_ddp_update_shard_emit")


def ddp_publish_stats(emit, world: int, rank: int, device) -> None:
    with torch.cuda.device(device):
        st = _lib.load().nnue_ddp_publish_stats(C.byref(emit), world, rank, _stream(device))
    _lib.check(st, "nnue_ddp_publish_stats")
