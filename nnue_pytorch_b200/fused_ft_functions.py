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
