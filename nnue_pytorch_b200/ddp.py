"""Gradient exchange between data-parallel ranks (one process per GPU).

The reference wraps its model in `DistributedDataParallel`
(trainer/engine.py:149-162 of the reference project): every gradient is
averaged over the ranks during backward and every rank then runs the same
optimizer step.  `make_grad_hook` gives `TrainStep` the same result: the small
dense-layer gradients travel as one flat bucket, the feature-transformer
table gradient (23232 x 3080 fp32, 286 MB) as its own all-reduce.  NCCL over
NVLink/NVSwitch does the wire work; with one rank nothing is exchanged.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_BIG = 1 << 22  # elements; tensors at least this large are reduced on their own


def make_grad_hook(model: torch.nn.Module, world: int, average: bool = True):
    """`average=False` leaves rank SUMS in `.grad`; the caller then folds the
    division by `world` into the scalar its optimizer multiplies gradients by
    (`TrainStep` does), which saves a read-modify-write pass over the table."""
    if world <= 1:
        return None
    inv = 1.0 / world if average else 1.0

    def hook(m: torch.nn.Module) -> None:
        grads = [p.grad for p in m.parameters() if p.grad is not None]
        small = [g for g in grads if g.numel() < _BIG]
        for g in grads:
            if g.numel() >= _BIG:
                dist.all_reduce(g)
                if inv != 1.0:
                    g.mul_(inv)
        if small:
            flat = torch.cat([g.reshape(-1) for g in small])
            dist.all_reduce(flat)
            if inv != 1.0:
                flat.mul_(inv)
            at = 0
            for g in small:
                n = g.numel()
                g.copy_(flat[at : at + n].view_as(g))
                at += n

    return hook
