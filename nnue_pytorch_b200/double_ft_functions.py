"""`double_feature_transform`: the operator boundary the model calls.

Mirrors model/modules/feature_transformer/double_ft_functions.py:7-82 of the
reference project.  `backend` is kept for signature compatibility:
"auto" and "fused" run the fused kernels, "sparse" composes two sparse-linear
kernel calls with the same torch glue the reference uses, "torch" raises
because this package has no PyTorch fallback, anything else is a ValueError.
"""

from __future__ import annotations

import torch

from .fused_ft_functions import _HAS_CUPY_KERNELS, FusedDoubleFtFunction  # noqa: F401
from .sparse_linear_functions import SparseLinearFunction


@torch.compiler.disable  # ctypes launches: runs eagerly inside a compiled model, as the reference's kernels do
def double_feature_transform(
    us: torch.Tensor,
    them: torch.Tensor,
    white_indices: torch.Tensor,
    black_indices: torch.Tensor,
    psqt_indices: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    max_ft_activation: float,
    l1_size: int,
    backend: str = "auto",
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    all_cuda = all(
        t.is_cuda for t in (us, them, white_indices, black_indices, psqt_indices, weight, bias)
    )
    if backend in ("auto", "fused"):
        if not all_cuda:
            raise RuntimeError(
                "Fused double FT backend requested, but not all tensors/parameters are on CUDA "
                "(nnue_pytorch_b200 has no CPU fallback)."
            )
        return FusedDoubleFtFunction.apply(
            us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, l1_size
        )
    if backend == "sparse":
        if not all_cuda:
            raise RuntimeError("Sparse backend requested, but not all tensors/parameters are on CUDA.")
        assert l1_size % 2 == 0
        wp = SparseLinearFunction.apply(white_indices, weight, bias, backend="sparse")
        bp = SparseLinearFunction.apply(black_indices, weight, bias, backend="sparse")
        w, wpsqt = torch.split(wp, l1_size, dim=1)
        b, bpsqt = torch.split(bp, l1_size, dim=1)
        sel = psqt_indices.unsqueeze(dim=1)
        wpsqt = wpsqt.gather(1, sel)
        bpsqt = bpsqt.gather(1, sel)
        x = (us * torch.cat([w, b], dim=1)) + (them * torch.cat([b, w], dim=1))
        x = torch.clamp(x, 0.0, max_ft_activation)
        c = torch.split(x, l1_size // 2, dim=1)
        return torch.cat([c[0] * c[1], c[2] * c[3]], dim=1), wpsqt, bpsqt
    if backend == "torch":
        raise RuntimeError(
            "backend='torch' is the reference's PyTorch fallback; nnue_pytorch_b200 ships the "
            "sm_100a kernels only."
        )
    raise ValueError(f"Invalid double FT implementation mode: {backend}")
