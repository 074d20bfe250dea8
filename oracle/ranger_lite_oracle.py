"""Restatement of the reference's RangerLite optimizer step (Python path).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Follows model/optimizers/ranger_lite.py:592-768 of the reference project for
the configuration the trainer uses by default (no legacy scoping, no norm
loss): Adam second moment, positive-negative momentum on alternating buffers,
optional stable weight decay normalised by the global debiased variance, and
a lookahead merge every `mergetime` steps.  Works on plain tensors.
"""

from __future__ import annotations

import math

import torch


class RangerLiteState:
    def __init__(self, params: list[torch.Tensor], pnm: bool = True, lookahead: bool = True):
        self.step = 0
        self.lookahead_step = 0
        self.param_size = 0
        self.grad_ma = [torch.zeros_like(p) for p in params]
        self.variance_ma = [torch.zeros_like(p) for p in params]
        self.neg_grad_ma = [torch.zeros_like(p) for p in params] if pnm else None
        self.slow = [p.clone() for p in params] if lookahead else None


@torch.no_grad()
def ranger_lite_step(params, grads, state: RangerLiteState, lr, weight_decay=0.0, betas=(0.9, 0.999), eps=1e-7,
                     pnm=True, pnm_momentum=1.0, lookahead=True, mergetime=5, alpha=0.5):
    """One optimizer step over parallel lists `params` / `grads` (updated in place).
    `lr` and `weight_decay` may be scalars or per-tensor lists."""
    n = len(params)
    lrs = lr if isinstance(lr, (list, tuple)) else [lr] * n
    wds = weight_decay if isinstance(weight_decay, (list, tuple)) else [weight_decay] * n
    beta1, beta2 = betas
    state.step += 1
    step = state.step
    bc2 = 1 - beta2**step

    var_sum = torch.zeros(1, dtype=params[0].dtype)
    for i in range(n):
        v = state.variance_ma[i]
        v.mul_(beta2).addcmul_(grads[i], grads[i], value=1 - beta2)
        var_sum += (v / bc2).sum()
    if not state.param_size:
        state.param_size = sum(p.numel() for p in params)
    var_norm = torch.sqrt(var_sum / state.param_size).clamp_min(eps)

    for i in range(n):
        p, g = params[i], grads[i]
        if wds[i]:
            p.mul_(1 - wds[i] * lrs[i] / var_norm)
        denom = (state.variance_ma[i].sqrt() / math.sqrt(bc2)).add_(eps)
        if pnm:
            if step % 2 == 1:
                pos, neg = state.grad_ma[i], state.neg_grad_ma[i]
            else:
                pos, neg = state.neg_grad_ma[i], state.grad_ma[i]
            pos.mul_(beta1**2).add_(g, alpha=1 - beta1**2)
            effective = ((step + 1) // 2) * 2
            bc1 = 1 - beta1**effective
            norm = math.sqrt((1 + pnm_momentum) ** 2 + pnm_momentum**2)
            upd = pos.mul(1 + pnm_momentum).add(neg, alpha=-pnm_momentum).mul(1 / norm)
        else:
            bc1 = 1 - beta1**step
            state.grad_ma[i].mul_(beta1).add_(g, alpha=1 - beta1)
            upd = state.grad_ma[i]
        p.addcdiv_(upd, denom, value=-(lrs[i] / bc1))

    if lookahead:
        state.lookahead_step += 1
        if state.lookahead_step >= mergetime:
            state.lookahead_step = 0
            for i in range(n):
                params[i].mul_(alpha).add_(state.slow[i], alpha=1.0 - alpha)
                state.slow[i].copy_(params[i])
