"""Integer evaluation of a quantized net on the GPU.

The reference project defines its quantized evaluation through the float
forward with fake quantization on (model/quantize.py, layer_stacks.py,
model.py:107-133) and exports integer weights with
`QuantizationManager.quantize_*` (model/quantize.py:175-235: scale, round,
refuse values outside the target type).  `QuantizedNet` performs that export
into device tensors and runs the all-integer kernel `nnue_quant_eval`.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .quantize import QuantizationManager


def _to_int(x: torch.Tensor, scale: float, dtype: torch.dtype) -> torch.Tensor:
    """round(x*scale) in `dtype`; out-of-range values raise like the reference's `_safe_convert`."""
    r = x.detach().double().mul(scale).round()
    lim = torch.iinfo(dtype).max
    bad = int((r.abs() > lim).sum())
    if bad:
        raise RuntimeError(
            f"Found {bad} out of bounds values when converting to target dtype {dtype}. "
            f"Min: {r.min().item()}, max: {r.max().item()}."
        )
    return r.to(dtype).contiguous()


class QuantizedNet:
    def __init__(self, ft_weight, ft_bias, l1_weight, l1_bias, l2_weight, l2_bias, out_weight, out_bias,
                 l1_size: int, num_buckets: int, quantization: QuantizationManager | None = None):
        """All arguments are float tensors on one CUDA device: `ft_weight`
        [N, L1+P] is the merged table, `l1_*` the first layer with its shared
        factor already folded in ([buckets*L2, L1] / [buckets*L2])."""
        q = quantization or QuantizationManager()
        self.consts = q.integer_constants()
        s = q.weight_scales_dict
        if not ft_weight.is_cuda:
            raise RuntimeError("QuantizedNet needs CUDA tensors (there is no CPU path)")
        self.device = ft_weight.device
        self.L1, self.buckets = int(l1_size), int(num_buckets)
        self.N = ft_weight.shape[0]
        self.P = ft_weight.shape[1] - self.L1
        self.L2 = l1_weight.shape[0] // self.buckets
        self.L3 = l2_weight.shape[0] // self.buckets
        self.ft_w = _to_int(ft_weight[:, : self.L1], s["ft_weight"], torch.int16)
        self.ft_psqt = _to_int(ft_weight[:, self.L1 :], s["ft_psqt_weight"], torch.int32)
        self.ft_b = _to_int(ft_bias[: self.L1], s["ft_bias"], torch.int32)
        self.l1_w = _to_int(l1_weight, s["ls_l1_weight"], torch.int8)
        self.l1_b = _to_int(l1_bias, s["ls_l1_bias"], torch.int32)
        self.l2_w = _to_int(l2_weight, s["ls_l2_weight"], torch.int8)
        self.l2_b = _to_int(l2_bias, s["ls_l2_bias"], torch.int32)
        self.out_w = _to_int(out_weight, s["ls_output_weight"], torch.int8)
        self.out_b = _to_int(out_bias.reshape(-1), s["ls_output_bias"], torch.int32)
        self._qp = _lib.QuantParams(**self.consts)
        self._pack()

    PACKED_MAX_ABS = 4095  # the packed gather's limit on |ft_w| (nnue_quant_eval_packed)

    def _pack(self) -> None:
        """The packed copy of the table the fast gather reads (`nnue_quant_pack_table`) and max |ft_w|, read once."""
        self.ft_w_packed, self.ft_max_abs = None, None
        if self.L1 % 32 != 0 or self.N == 0:
            return
        packed = torch.empty(self.N + 1, self.L1, dtype=torch.int16, device=self.device)
        max_abs = torch.zeros(1, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            st = _lib.load().nnue_quant_pack_table(self.ft_w.data_ptr(), packed.data_ptr(), max_abs.data_ptr(), self.N,
                                                   self.L1, torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(st, "nnue_quant_pack_table")
        self.ft_max_abs = int(max_abs.item())
        if self.ft_max_abs <= self.PACKED_MAX_ABS:
            self.ft_w_packed = packed

    @classmethod
    def from_model(cls, model) -> "QuantizedNet":
        """From an `NNUEModel` of this package (or the reference's: same attribute names)."""
        ls = model.layer_stacks
        table, bias = model.input.merged_weight_and_bias(False)
        count = ls.count
        l1_w = ls.l1.linear.weight + ls.l1.factorized_linear.weight.repeat(count, 1)
        l1_b = ls.l1.linear.bias + ls.l1.factorized_linear.bias.repeat(count)
        return cls(table, bias, l1_w, l1_b, ls.l2.linear.weight, ls.l2.linear.bias, ls.output.linear.weight,
                   ls.output.linear.bias, model.L1, count, model.quantization)

    @classmethod
    def from_integers(cls, nf, quantization: QuantizationManager | None = None,
                      device: torch.device | str = "cuda") -> "QuantizedNet":
        """From the integer tensors of a `.nnue` file (`serialize.NNUEFile`): nothing is rescaled
        or rounded again, the kernel evaluates the stored numbers."""
        import numpy as np

        q = quantization or QuantizationManager()
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("QuantizedNet needs a CUDA device (there is no CPU path)")
        self = cls.__new__(cls)
        self.consts = q.integer_constants()
        self.device = dev
        self.L1, self.buckets, self.P = int(nf.L1), int(nf.buckets), int(nf.P)
        self.L2, self.L3 = int(nf.L2), int(nf.L3)
        self.N = int(nf.ft_weight.shape[0])

        def put(a, dtype):
            return torch.from_numpy(np.ascontiguousarray(a)).to(device=dev, dtype=dtype).contiguous()

        self.ft_w = put(nf.ft_weight, torch.int16)
        self.ft_psqt = put(nf.ft_psqt, torch.int32)
        self.ft_b = put(nf.ft_bias.astype(np.int32), torch.int32)
        self.l1_w = put(np.concatenate([b[0][0] for b in nf.fc]), torch.int8)
        self.l1_b = put(np.concatenate([b[0][1] for b in nf.fc]), torch.int32)
        self.l2_w = put(np.concatenate([b[1][0] for b in nf.fc]), torch.int8)
        self.l2_b = put(np.concatenate([b[1][1] for b in nf.fc]), torch.int32)
        self.out_w = put(np.concatenate([b[2][0] for b in nf.fc]), torch.int8)
        self.out_b = put(np.concatenate([b[2][1] for b in nf.fc]), torch.int32)
        self._qp = _lib.QuantParams(**self.consts)
        self._pack()
        return self

    @torch.no_grad()
    def evaluate(self, white_indices, black_indices, stm_white, piece_count, tiled: bool = True,
                 packed: bool = True) -> torch.Tensor:
        """int32 [B]: the evaluation in units of 1/(2 * nnue2score * weight_scale_out)
        (= 1/19200 by default) of the float model output.  `tiled=False` runs the
        one-kernel form (no scratch memory, slower), `packed=False` the tiled form on the plain
        int16 table (what nets with |ft_w| > 4095 or lists beyond 511 rows get anyway); the
        results are the same bits."""
        dev = self.device
        assert white_indices.dtype == torch.int32 and black_indices.dtype == torch.int32
        assert white_indices.is_cuda and white_indices.is_contiguous() and black_indices.is_contiguous()
        assert white_indices.shape == black_indices.shape
        B, K = white_indices.shape
        stm = stm_white.reshape(-1).to(device=dev, dtype=torch.uint8).contiguous()
        bucket = ((piece_count.reshape(-1) - 1) // 4).to(device=dev, dtype=torch.int32).contiguous()
        out = torch.empty(B, dtype=torch.int32, device=dev)
        lib = _lib.load()
        if tiled and B > 0:
            ws = torch.empty(lib.nnue_quant_eval_workspace_bytes(B, self.L1), dtype=torch.uint8, device=dev)
            if packed and self.ft_w_packed is not None and K <= 511:
                with torch.cuda.device(dev):
                    st = lib.nnue_quant_eval_packed(
                        white_indices.data_ptr(), black_indices.data_ptr(), stm.data_ptr(), bucket.data_ptr(),
                        self.ft_w_packed.data_ptr(), self.ft_max_abs, self.ft_psqt.data_ptr(), self.ft_b.data_ptr(),
                        self.l1_w.data_ptr(), self.l1_b.data_ptr(), self.l2_w.data_ptr(), self.l2_b.data_ptr(),
                        self.out_w.data_ptr(), self.out_b.data_ptr(), out.data_ptr(),
                        B, K, self.N, self.L1, self.L2, self.L3, self.P, self.buckets,
                        C.byref(self._qp), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(dev).cuda_stream,
                    )
                _lib.check(st, "nnue_quant_eval_packed")
                return out
            with torch.cuda.device(dev):
                st = lib.nnue_quant_eval_tiled(
                    white_indices.data_ptr(), black_indices.data_ptr(), stm.data_ptr(), bucket.data_ptr(),
                    self.ft_w.data_ptr(), self.ft_psqt.data_ptr(), self.ft_b.data_ptr(),
                    self.l1_w.data_ptr(), self.l1_b.data_ptr(), self.l2_w.data_ptr(), self.l2_b.data_ptr(),
                    self.out_w.data_ptr(), self.out_b.data_ptr(), out.data_ptr(),
                    B, K, self.N, self.L1, self.L2, self.L3, self.P, self.buckets,
                    C.byref(self._qp), ws.data_ptr(), ws.numel(), torch.cuda.current_stream(dev).cuda_stream,
                )
            _lib.check(st, "nnue_quant_eval_tiled")
            return out
        with torch.cuda.device(dev):
            st = _lib.load().nnue_quant_eval(
                white_indices.data_ptr(), black_indices.data_ptr(), stm.data_ptr(), bucket.data_ptr(),
                self.ft_w.data_ptr(), self.ft_psqt.data_ptr(), self.ft_b.data_ptr(),
                self.l1_w.data_ptr(), self.l1_b.data_ptr(), self.l2_w.data_ptr(), self.l2_b.data_ptr(),
                self.out_w.data_ptr(), self.out_b.data_ptr(), out.data_ptr(),
                B, K, self.N, self.L1, self.L2, self.L3, self.P, self.buckets,
                C.byref(self._qp), torch.cuda.current_stream(dev).cuda_stream,
            )
        _lib.check(st, "nnue_quant_eval")
        return out
