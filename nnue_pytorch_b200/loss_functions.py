"""The training loss as one kernel launch.

`sf_loss_fused` computes `calculate_sf_loss` of the reference (model/nnue.py:39-69,
with `remap_tablebase_score`, model/nnue.py:18-36) on
`(y + (wpsqt - bpsqt) * (us - 0.5)) * net_scale`, and the gradient with respect
to y, wpsqt and bpsqt in the same launch.  `SfLossFunction` wraps it for
autograd; `TrainStep` uses the raw form and seeds the backward pass with the
three gradients directly.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._launch import _ptr, _stream

_WORKSPACES: dict[int, torch.Tensor] = {}


def _workspace(dev: torch.device) -> torch.Tensor:
    """One zeroed workspace per device; every launch leaves it zeroed.  Launches
    on one device are ordered by the stream they share."""
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    ws = _WORKSPACES.get(key)
    if ws is None:
        n = _lib.load().nnue_sf_loss_workspace_bytes()
        ws = torch.zeros((n + 7) // 8, dtype=torch.int64, device=dev)
        _WORKSPACES[key] = ws
    return ws


def loss_params_struct(lp, lam: float, net_scale: float) -> _lib.LossParams:
    s = _lib.LossParams()
    for name in ("in_offset", "out_offset", "in_scaling", "out_scaling", "pow_exp", "qp_asymmetry", "w1", "w2",
                 "tb_remap_base", "tb_remap_scale", "tb_remap_decay"):
        setattr(s, name, float(getattr(lp, name)))
    s.lam, s.net_scale = float(lam), float(net_scale)
    return s


def sf_loss_fused(y, wpsqt, bpsqt, us, score, outcome, lp, lam: float, net_scale: float, want_grads: bool = True):
    """Returns (loss [] , d_y, d_wpsqt, d_bpsqt); the gradients are None when
    not wanted, and the PSQT ones when wpsqt is None.  All inputs float32 CUDA
    tensors of B elements.  `lam` is one number for the whole batch: the reference's
    `LambdaController` (model/lambda_utils.py:59-81) hands out a per-batch or per-sample TENSOR
    when lambda jitter is configured; such a lambda goes through the elementwise form
    (`model.sf_loss`), which broadcasts it."""
    if torch.is_tensor(lam):
        raise TypeError("sf_loss_fused takes a scalar lambda; use model.sf_loss for a per-sample lambda tensor")
    if not y.is_cuda:
        raise _lib.NnueB200Error("sf_loss_fused runs on the GPU only; pass CUDA tensors")
    dev, B = y.device, y.numel()
    ins = [y, wpsqt, bpsqt, us, score, outcome]
    for i, t in enumerate(ins):
        if t is not None:
            if t.dtype != torch.float32 or t.numel() != B or t.device != dev:
                raise ValueError("sf_loss_fused: every input must be float32 with one value per position")
            ins[i] = t.detach().contiguous()
    y_, wp_, bp_, us_, sc_, oc_ = ins
    loss = torch.empty((), dtype=torch.float32, device=dev)
    d_y = torch.empty_like(y_) if want_grads else None
    d_wp = torch.empty_like(wp_) if want_grads and wp_ is not None else None
    d_bp = torch.empty_like(bp_) if want_grads and bp_ is not None else None
    params = loss_params_struct(lp, lam, net_scale)
    with torch.cuda.device(dev):
        _lib.check(
            _lib.load().nnue_sf_loss(_ptr(y_), _ptr(wp_), _ptr(bp_), _ptr(us_), _ptr(sc_), _ptr(oc_), C.byref(params),
                                     _ptr(loss), _ptr(d_y), _ptr(d_wp), _ptr(d_bp), _ptr(_workspace(dev)), B,
                                     _stream(dev)),
            "nnue_sf_loss",
        )
    return loss, d_y, d_wp, d_bp


class SfLossFunction(torch.autograd.Function):
    """loss = SfLossFunction.apply(y, wpsqt, bpsqt, us, score, outcome, loss_params, lam, net_scale)"""

    @staticmethod
    def forward(ctx, y, wpsqt, bpsqt, us, score, outcome, lp, lam, net_scale):
        loss, d_y, d_wp, d_bp = sf_loss_fused(y, wpsqt, bpsqt, us, score, outcome, lp, lam, net_scale)
        ctx.save_for_backward(d_y, d_wp, d_bp)
        ctx.shapes = (y.shape, None if wpsqt is None else wpsqt.shape, None if bpsqt is None else bpsqt.shape)
        return loss

    @staticmethod
    def backward(ctx, g):
        d_y, d_wp, d_bp = ctx.saved_tensors
        sy, sw, sb = ctx.shapes
        return ((d_y * g).view(sy), None if d_wp is None else (d_wp * g).view(sw),
                None if d_bp is None else (d_bp * g).view(sb), None, None, None, None, None, None)
