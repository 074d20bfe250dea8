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

from torch import autograd

from . import _launch

_HAS_CUPY_KERNELS = True
BACKWARD_TILE_SIZE = 1  # kept for importers of the reference module; unused here


class FusedDoubleFtFunction(autograd.Function):
    @staticmethod
    def forward(ctx, us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, l1_size):
        ctx.max_ft_activation = float(max_ft_activation)
        ctx.l1_size = int(l1_size)
        l0, wpsqt, bpsqt, saved = _launch.fused_forward(
            us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, int(l1_size)
        )
        ctx.save_for_backward(us, them, white_indices, black_indices, psqt_indices, saved)
        ctx.weight_shape = tuple(weight.shape)
        return l0, wpsqt, bpsqt

    @staticmethod
    def backward(ctx, grad_l0, grad_wpsqt, grad_bpsqt):
        us, them, white_indices, black_indices, psqt_indices, saved = ctx.saved_tensors
        num_inputs, num_outputs = ctx.weight_shape
        grad_weight, grad_bias = _launch.fused_backward(
            us, them, white_indices, black_indices, psqt_indices, ctx.max_ft_activation, ctx.l1_size,
            num_inputs, num_outputs, grad_l0, grad_wpsqt, grad_bpsqt, saved,
        )
        return None, None, None, None, None, grad_weight, grad_bias, None, None
