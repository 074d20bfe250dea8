"""`FusedDoubleFtFunction`: both perspectives of the feature transformer in
one autograd op.

Mirrors model/modules/feature_transformer/fused_ft_functions.py:17-122 of the
reference project (argument order, output triple, gradients only for weight
and bias).  Differences that follow the parity target, the torch composition
of double_ft_functions.py:62-80: the tensor saved for backward holds the
pre-clamp activations, so the clamp passes gradient on the closed interval
[0, max] exactly like `torch.clamp`, and the gradient tensors are produced by
a segment reduction that writes every row once (no `torch.zeros` pass).
"""

from __future__ import annotations

import torch
from torch import autograd

from . import _launch

_HAS_CUPY_KERNELS = True
BACKWARD_TILE_SIZE = 1  # kept for importers of the reference module; unused here


class FusedDoubleFtFunction(autograd.Function):
    """The reference's nine arguments, plus three optional ones that fuse the
    dense passes the reference runs right after the op on `l0`
    (composed_feature_transformer.py:143-149): `act_quant_scale` > 0 applies
    floor(l0 * scale + act_quant_eps) / scale with a straight-through gradient,
    `out_scale` multiplies the result (and the incoming gradient)."""

    @staticmethod
    def forward(ctx, us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, l1_size,
                act_quant_scale=0.0, act_quant_eps=0.0, out_scale=1.0):
        ctx.max_ft_activation = float(max_ft_activation)
        ctx.l1_size = int(l1_size)
        ctx.out_scale = float(out_scale)
        l0, wpsqt, bpsqt, saved = _launch.fused_forward(
            us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, int(l1_size),
            act_quant_scale, act_quant_eps, out_scale,
        )
        ctx.save_for_backward(us, them, white_indices, black_indices, psqt_indices, saved)
        ctx.weight_shape = tuple(weight.shape)
        # a table made by PrepareTableFunction still needs its gradient routed to the factor rows
        ctx.table_is_derived = weight.grad_fn is not None
        ctx.exchange = _launch.exchange_of(weight)  # data-parallel owner of the table, if any
        return l0, wpsqt, bpsqt

    @staticmethod
    def backward(ctx, grad_l0, grad_wpsqt, grad_bpsqt):
        us, them, white_indices, black_indices, psqt_indices, saved = ctx.saved_tensors
        num_inputs, num_outputs = ctx.weight_shape
        ex = ctx.exchange
        grad_weight, grad_bias = _launch.fused_backward(
            us, them, white_indices, black_indices, psqt_indices, ctx.max_ft_activation, ctx.l1_size,
            num_inputs, num_outputs, grad_l0, grad_wpsqt, grad_bpsqt, saved, out_scale=ctx.out_scale,
            sink=None if ex is None else ex.grad_view, slices=None if ex is None else ex.slice_spec(),
        )
        if ex is not None and not ctx.table_is_derived:
            grad_weight = None  # the exchange reads its shared buffer itself
        return None, None, None, None, None, grad_weight, grad_bias, None, None, None, None, None


class PrepareTableFunction(autograd.Function):
    """table = fq(weight + virtual_weight.repeat(buckets, 1)) in one kernel.
    Backward: straight-through to `weight` (the same tensor, no copy), the
    bucket sum to `virtual_weight` (halfka_v2_hm.py:68-69 and the fake
    quantization of composed_feature_transformer.py:61-76 of the reference)."""

    @staticmethod
    def forward(ctx, weight, virtual_weight, l1_size, scale_main, scale_psqt):
        ctx.n_virtual = 0 if virtual_weight is None else virtual_weight.shape[0]
        ctx.exchange = _launch.exchange_of(weight)
        return _launch.prepare_table(weight, virtual_weight, int(l1_size), scale_main, scale_psqt)

    @staticmethod
    def backward(ctx, grad):
        gv = None
        if ctx.n_virtual and ctx.needs_input_grad[1]:
            gv = _launch.virtual_grad(grad, ctx.n_virtual)
        ex = ctx.exchange
        if ex is not None and grad.data_ptr() == ex.grad_view.data_ptr():
            if gv is not None:
                ex.note_local_reader()  # the reduce overwrites the buffer: it must wait for the kernel above
            grad = None  # the exchange reads its shared buffer itself
        return grad, gv, None, None, None


class PrepareBiasFunction(autograd.Function):
    """bias_full = [fq(bias[:l1]), zeros(psqt)]: the bias the operator adds
    (composed_feature_transformer.py:61-76 of the reference fake-quantizes the
    bias and drops its PSQT part, which never trains).  One fill and one kernel;
    the backward is a view of the incoming gradient."""

    @staticmethod
    def forward(ctx, bias, l1_size, scale):
        l1 = int(l1_size)
        out = torch.zeros_like(bias)
        _launch.prepare_table(bias.detach()[:l1].reshape(1, l1), None, l1, scale, 1.0, out=out, span="prepare_bias")
        ctx.pad = bias.numel() - l1
        ctx.l1 = l1
        return out

    @staticmethod
    def backward(ctx, grad):
        return torch.nn.functional.pad(grad[: ctx.l1], (0, ctx.pad)), None, None


class QuantizedFusedDoubleFtFunction(autograd.Function):
    """The whole feature transformer of one step when weights are fake-quantized at a power-of-two
    scale: table preparation (factor fold + fake quantization, written as int16), bias fake
    quantization and the fused operator, as ONE autograd node over the raw parameters.

    Same values, bit for bit, as `PrepareTableFunction` + `PrepareBiasFunction` +
    `FusedDoubleFtFunction` (every partial sum of the fp32 form is exact, see
    csrc/ft_fused_q16.cu); half the bytes through the L2.  Backward: the operator's gradient goes
    straight through both fake quantizations to every block's `weight`, summed over the repeats to
    its `virtual_weight`, and to the L1 part of the bias.

    apply(us, them, white_indices, black_indices, psqt_indices, bias, max_ft_activation, l1_size,
          act_quant_scale, act_quant_eps, out_scale, scale_main, scale_psqt, cache, w0, v0, w1, v1, ...)
    with (w_i, v_i) the parameter blocks in table order, v_i None for a block without factor rows.
    `cache`: a `_launch.QuantTableCache` (or None) for a single block without factor rows: the integer
    table is then kept between steps and only rebuilt when the parameter changed behind its back."""

    @staticmethod
    def forward(ctx, us, them, white_indices, black_indices, psqt_indices, bias, max_ft_activation, l1_size,
                act_quant_scale, act_quant_eps, out_scale, scale_main, scale_psqt, cache, *params):
        l1 = int(l1_size)
        blocks = [(params[i].detach(), None if params[i + 1] is None else params[i + 1].detach())
                  for i in range(0, len(params), 2)]
        if cache is not None and (len(blocks) != 1 or blocks[0][1] is not None):
            cache = None
        master = True
        if cache is not None and cache.owner is not None:
            # buffers shared between data-parallel ranks, rewritten by the exchange's update kernel
            if not cache.fresh(params[0], l1, scale_main, scale_psqt):
                cache.owner.rebuild_integer_rows()  # collective: every rank sees the same staleness
                if not cache.fresh(params[0], l1, scale_main, scale_psqt):
                    raise RuntimeError("the exchange ships integer rows at another L1 size or scale than the forward uses")
            q16, psqt, overflow = cache.q16, cache.psqt, cache.stats
            master = cache.owner.fp32_rows_valid
        elif cache is not None and cache.fresh(params[0], l1, scale_main, scale_psqt):
            q16, psqt, overflow = cache.q16, cache.psqt, cache.stats
        else:
            q16, psqt, overflow = _launch.quantize_blocks(blocks, l1, scale_main, scale_psqt)
            if cache is not None:
                cache.store(params[0], l1, scale_main, scale_psqt, q16, psqt, overflow)
                params[0]._nnue_q16_cache = cache  # where this package's optimizer looks for it
        # per-rank parts of the table first and the bias in a pair of its own (written over every step), or one
        # pair that the bias's figures are added to (the optimizer kernel resets it when it rewrites the table)
        parts = overflow.numel() > 2
        bias_fq = _launch.prepare_bias_q16(bias.detach(), l1, scale_main, overflow[-2:] if parts else overflow, parts)
        l0, wpsqt, bpsqt, saved = _launch.fused_forward_q16(
            us, them, white_indices, black_indices, psqt_indices, q16, psqt, bias_fq, overflow, blocks, scale_main,
            max_ft_activation, l1, act_quant_scale, act_quant_eps, out_scale, master=master)
        ctx.save_for_backward(us, them, white_indices, black_indices, psqt_indices, saved)
        ctx.max_ft_activation, ctx.l1_size, ctx.out_scale = float(max_ft_activation), l1, float(out_scale)
        ctx.rows = [w.shape[0] for w, _ in blocks]
        ctx.n_virtual = [0 if v is None else v.shape[0] for _, v in blocks]
        ctx.num_outputs = bias.shape[0]
        # a single block owned by a data-parallel exchange: its gradient lands in the exchange's buffer
        ctx.exchange = _launch.exchange_of(params[0]) if len(blocks) == 1 else None
        return l0, wpsqt, bpsqt

    @staticmethod
    def backward(ctx, grad_l0, grad_wpsqt, grad_bpsqt):
        us, them, white_indices, black_indices, psqt_indices, saved = ctx.saved_tensors
        ex = ctx.exchange
        n_total = sum(ctx.rows)
        grad_table, grad_bias = _launch.fused_backward(
            us, them, white_indices, black_indices, psqt_indices, ctx.max_ft_activation, ctx.l1_size,
            n_total, ctx.num_outputs, grad_l0, grad_wpsqt, grad_bpsqt, saved, out_scale=ctx.out_scale,
            sink=None if ex is None else ex.grad_view, slices=None if ex is None else ex.slice_spec(),
        )
        grads, at = [], 0
        for i, (rows, nv) in enumerate(zip(ctx.rows, ctx.n_virtual)):
            gw = grad_table if len(ctx.rows) == 1 else grad_table[at : at + rows]
            at += rows
            gv = None
            if nv and ctx.needs_input_grad[14 + 2 * i + 1]:
                gv = _launch.virtual_grad(gw, nv)
                if ex is not None:
                    ex.note_local_reader()  # the reduce overwrites the buffer: it must wait for the kernel above
            grads += [None if ex is not None else gw, gv]
        pad = ctx.num_outputs - ctx.l1_size
        grad_bias = torch.nn.functional.pad(grad_bias[: ctx.l1_size], (0, pad))  # the PSQT part of the bias never trains
        return (None, None, None, None, None, grad_bias, None, None, None, None, None, None, None, None, *grads)
