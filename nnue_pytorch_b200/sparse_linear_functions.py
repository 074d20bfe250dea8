"""`SparseLinearFunction`: the reference's single-perspective sparse linear op.

Mirrors model/modules/feature_transformer/sparse_linear_functions.py:142-165
of the reference project: same entry point (`SparseLinearFunction.apply`),
same argument order, same contract on the tensors.  Every CUDA backend name
routes to the sm_100a kernels of libnnue_b200.so; there is no multi-backend
dispatch and no CPU path, so `backend="torch"` (the reference's
`F.embedding_bag` fallback) and CPU tensors raise.
"""

from __future__ import annotations

import torch
from torch import autograd

from . import _launch

# The reference exposes this flag for "are the custom kernels importable";
# tests and `double_ft_functions` read it.  Here the kernels are the product.
_HAS_CUPY_KERNELS = True


class _CudaSparseLinearFunction(autograd.Function):
    """output[b] = bias + sum_k weight[indices[b, k]]; the first -1 ends a row."""

    @staticmethod
    def forward(ctx, feature_indices, weight, bias):
        out = _launch.sparse_linear_forward(feature_indices, weight, bias)
        ctx.save_for_backward(feature_indices)
        ctx.num_inputs = weight.shape[0]
        return out

    @staticmethod
    def backward(ctx, grad_output):
        assert not ctx.needs_input_grad[0]
        (feature_indices,) = ctx.saved_tensors
        grad_w, grad_b = _launch.sparse_linear_backward(feature_indices, grad_output, ctx.num_inputs)
        return None, grad_w, grad_b


class SparseLinearFunction:
    # The kernels are reached through ctypes with raw device pointers, which a tracing compiler cannot
    # follow: like the reference's kernel factories (sparse_linear_kernel.py:50,172), the operator is
    # excluded from torch.compile and runs eagerly inside a compiled model.
    @staticmethod
    @torch.compiler.disable
    def apply(feature_indices, weight, bias, backend: str = "auto"):
        if backend in ("auto", "sparse"):
            if not (feature_indices.is_cuda and weight.is_cuda and bias.is_cuda):
                raise RuntimeError(
                    "Sparse CUDA kernel requested but tensors are not on CUDA "
                    "(nnue_pytorch_b200 has no CPU fallback)."
                )
            return _CudaSparseLinearFunction.apply(feature_indices, weight, bias)
        if backend == "torch":
            raise RuntimeError(
                "backend='torch' is the reference's PyTorch fallback; nnue_pytorch_b200 "
                "ships the sm_100a kernels only."
            )
        raise ValueError(f"Invalid SparseLinear backend requested: {backend}")
