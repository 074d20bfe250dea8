"""Restatement of the reference's CPU path of the feature transformer.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

`sparse_linear` follows `_torch_sparse_linear`,
model/modules/feature_transformer/sparse_linear_functions.py:16-50 of the
reference project (an `embedding_bag` sum where negative entries are padding,
plus the bias).  `double_feature_transform` follows the torch composition in
double_ft_functions.py:62-80.  Both are differentiable torch code, so
gradients come from autograd exactly as they do in the reference; run them on
float64 inputs for the high-precision variant.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def sparse_linear(indices: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """out[b] = sum over non-negative indices[b, k] of weight[indices[b, k]], plus bias."""
    batch, max_active = indices.shape
    keep = (indices >= 0).to(weight.dtype).reshape(-1)
    flat = indices.clamp(min=0).long().reshape(-1)
    starts = torch.arange(0, batch * max_active, max_active, device=indices.device)
    summed = F.embedding_bag(flat, weight, starts, mode="sum", per_sample_weights=keep)
    return summed + bias


def double_feature_transform(us, them, white_indices, black_indices, psqt_indices, weight, bias, max_ft_activation, l1_size):
    """(l0 [B, l1], wpsqt [B, 1], bpsqt [B, 1]) of both perspectives."""
    assert l1_size % 2 == 0
    white = sparse_linear(white_indices, weight, bias)
    black = sparse_linear(black_indices, weight, bias)
    w, wpsqt = torch.split(white, l1_size, dim=1)
    b, bpsqt = torch.split(black, l1_size, dim=1)
    pick = psqt_indices.unsqueeze(1)
    wpsqt = wpsqt.gather(1, pick)
    bpsqt = bpsqt.gather(1, pick)
    x = us * torch.cat([w, b], dim=1) + them * torch.cat([b, w], dim=1)
    x = torch.clamp(x, 0.0, max_ft_activation)
    q = torch.split(x, l1_size // 2, dim=1)
    return torch.cat([q[0] * q[1], q[2] * q[3]], dim=1), wpsqt, bpsqt


def double_feature_transform_with_grads(us, them, white_indices, black_indices, psqt_indices, weight, bias,
                                        max_ft_activation, l1_size, grad_l0=None, grad_wpsqt=None, grad_bpsqt=None):
    """Forward plus d(loss)/d(weight, bias) for loss = <grad_l0, l0> + <grad_wpsqt, wpsqt> + <grad_bpsqt, bpsqt>
    (all-ones cotangents when none are given).  Returns a dict of detached tensors."""
    weight = weight.detach().clone().requires_grad_(True)
    bias = bias.detach().clone().requires_grad_(True)
    l0, wp, bp = double_feature_transform(us, them, white_indices, black_indices, psqt_indices, weight, bias,
                                          max_ft_activation, l1_size)
    gl0 = torch.ones_like(l0) if grad_l0 is None else grad_l0.to(l0.dtype)
    gwp = torch.ones_like(wp) if grad_wpsqt is None else grad_wpsqt.to(wp.dtype)
    gbp = torch.ones_like(bp) if grad_bpsqt is None else grad_bpsqt.to(bp.dtype)
    loss = (l0 * gl0).sum() + (wp * gwp).sum() + (bp * gbp).sum()
    loss.backward()
    return {
        "l0": l0.detach(), "wpsqt": wp.detach(), "bpsqt": bp.detach(),
        "grad_weight": weight.grad.detach(), "grad_bias": bias.grad.detach(),
    }


def sparse_linear_with_grads(indices, weight, bias, grad_out=None):
    weight = weight.detach().clone().requires_grad_(True)
    bias = bias.detach().clone().requires_grad_(True)
    out = sparse_linear(indices, weight, bias)
    g = torch.ones_like(out) if grad_out is None else grad_out.to(out.dtype)
    (out * g).sum().backward()
    return {"out": out.detach(), "grad_weight": weight.grad.detach(), "grad_bias": bias.grad.detach()}
