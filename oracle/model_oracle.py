"""Restatement of the reference's network graph and loss around the feature
transformer, on plain tensors.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Follows, in the reference project:
  model/model.py:100-133                    bucket choice, PSQT term
  model/modules/feature_transformer/composed_feature_transformer.py:61-76,114-151
  model/modules/layer_stacks.py:33-84       three bucketed layers, squared/linear activations
  model/modules/stacked_linear.py:38-66,88-102
  model/quantize.py:36-56,133-147           fake quantization
  model/nnue.py:22-70,350-364               loss

`params` is a dict of tensors:
  ft_weight [N, L1+P] (already merged), ft_bias [L1+P],
  l1_w [C*L2, L1], l1_b [C*L2], l1f_w [L2, L1], l1f_b [L2]   (l1f = shared factor of the first layer)
  l2_w [C*L3, 2*L2], l2_b [C*L3], out_w [C, 2*L2+2*L3], out_b [C]
with C layer-stack buckets.  Everything is differentiable torch code; pass
float64 tensors for the exact variant.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .ft_oracle import double_feature_transform

EPS = 1e-5


@dataclass
class Quant:
    nnue2score: float = 600.0
    ws_l1: float = 128.0
    ws_l2: float = 64.0
    ws_lout: float = 128.0
    ws_out: float = 16.0
    ft_one: float = 256.0
    ft_max: float = 255.0
    hidden_one: float = 128.0
    hidden_max: float = 127.0
    l0_div: float = 512.0
    sqr_div: float = 128.0


def _ste(hard, soft):
    return hard.detach() + (soft - soft.detach())


def fq_weight(x, scale):
    return _ste(x.mul(scale).round().div(scale), x)


def fq_act(x, scale):
    return _ste(x.mul(scale).add(EPS).floor().div(scale), x)


def fq_output(x, q: Quant):
    mult = int(q.nnue2score * q.ws_out)
    den = int(q.hidden_one * q.ws_lout * 2.0)
    as_int = torch.round(x * den).to(torch.int64)
    out = torch.div(as_int * mult, den, rounding_mode="trunc")
    return _ste(out.to(x.dtype) / float(mult), x)


def merge_virtual(weight, virtual_weight, repeats):
    return weight + virtual_weight.repeat(repeats, 1)


def _select(stacked, bucket, width, count):
    rows = stacked.reshape(-1, width)
    base = torch.arange(0, bucket.shape[0] * count, count, device=stacked.device)
    return rows[bucket.flatten() + base]


def layer_stacks(params, l0, bucket, q: Quant = Quant(), fq_acts=True, fq_weights=True, trace: dict | None = None):
    """The three bucketed layers behind the feature transformer (model/modules/layer_stacks.py:33-84):
    `l0` [B, L1] -> [B, 1].  `trace`, when given, receives the values that go into each `floor` of the
    activation fake quantization ("pre_floor": [B, 2*L2 + 2*L3], in units of one quantization step),
    so that a caller can tell which positions sit on a step boundary."""
    L2 = params["l1f_w"].shape[0]
    count = params["out_w"].shape[0]
    L3 = params["l2_w"].shape[0] // count
    max_hidden = q.hidden_max / q.hidden_one
    sqr_corr = q.hidden_one / q.sqr_div
    pre = []

    w1 = params["l1_w"] + params["l1f_w"].repeat(count, 1)
    b1 = params["l1_b"] + params["l1f_b"].repeat(count)
    if fq_weights:
        w1, b1 = fq_weight(w1, q.ws_l1), fq_weight(b1, q.ws_l1 * q.hidden_one)
    o1 = _select(F.linear(l0, w1, b1), bucket, L2, count)
    skip = o1[:, -2].view(-1, 1) - o1[:, -1].view(-1, 1)
    sq = torch.pow(o1, 2.0)
    lin = o1
    if fq_acts:
        pre += [sq.detach() * q.hidden_one, lin.detach() * q.hidden_one]
        sq = fq_act(sq, q.hidden_one)
    sq = sq * sqr_corr
    if fq_acts:
        lin = fq_act(lin, q.hidden_one)
    x1 = torch.clamp(torch.cat([sq, lin], dim=1), 0, max_hidden)

    w2, b2 = params["l2_w"], params["l2_b"]
    if fq_weights:
        w2, b2 = fq_weight(w2, q.ws_l2), fq_weight(b2, q.ws_l2 * q.hidden_one)
    o2 = _select(F.linear(x1, w2, b2), bucket, L3, count)
    sq = torch.pow(o2, 2.0)
    lin = o2
    if fq_acts:
        pre += [sq.detach() * q.hidden_one, lin.detach() * q.hidden_one]
        sq = fq_act(sq, q.hidden_one)
    sq = sq * sqr_corr
    if fq_acts:
        lin = fq_act(lin, q.hidden_one)
    x2 = torch.clamp(torch.cat([sq, lin], dim=1), 0, max_hidden)

    w3, b3 = params["out_w"], params["out_b"]
    if fq_weights:
        w3, b3 = fq_weight(w3, q.ws_lout), fq_weight(b3, q.ws_lout * q.hidden_one)
    o3 = _select(F.linear(torch.cat([x1, x2], dim=1), w3, b3), bucket, 1, count)
    y = o3 + skip
    if trace is not None:
        trace["pre_floor"] = torch.cat(pre, dim=1) if pre else None
        trace["pre_output"] = y.detach()
    if fq_acts:
        y = fq_output(y, q)
    return y


def forward(params, us, them, white, black, piece_count, q: Quant = Quant(), fq_acts=True, fq_weights=True):
    L1 = params["l1_w"].shape[1]
    bucket = (piece_count - 1) // 4

    table, fb = params["ft_weight"], params["ft_bias"][:L1]
    if fq_weights:
        table = torch.cat([fq_weight(table[:, :L1], q.ft_one), fq_weight(table[:, L1:], q.nnue2score * q.ws_out)], dim=1)
        fb = fq_weight(fb, q.ft_one)
    bias = torch.cat([fb, torch.zeros_like(params["ft_bias"][L1:], dtype=fb.dtype)])
    l0, wpsqt, bpsqt = double_feature_transform(us, them, white, black, bucket, table, bias, q.ft_max / q.ft_one, L1)
    if fq_acts:
        l0 = fq_act(l0, q.hidden_one)
    l0 = l0 * (q.ft_one**2 / q.l0_div / q.hidden_one)
    y = layer_stacks(params, l0, bucket, q, fq_acts, fq_weights)
    return y + (wpsqt - bpsqt) * (us - 0.5)


@dataclass
class Loss:
    in_offset: float = 270.0
    out_offset: float = 270.0
    in_scaling: float = 340.0
    out_scaling: float = 380.0
    pow_exp: float = 2.5
    qp_asymmetry: float = 0.0
    w1: float = 0.0
    w2: float = 0.5
    tb_base: float = 4000.0
    tb_scale: float = 4000.0
    tb_decay: float = 0.85


def sf_loss(scorenet, score, outcome, lam=1.0, lp: Loss = Loss()):
    """`scorenet` already multiplied by nnue2score (centipawn-like units)."""
    mate, max_ply = 32000, 245
    a = score.abs()
    remapped = lp.tb_base + (lp.tb_decay ** (mate - a).clamp(min=0)) * lp.tb_scale
    score = torch.where(a >= mate - max_ply, torch.where(score < 0, -remapped, remapped), score)

    def wdl(v, off, sc):
        return 0.5 * (1.0 + ((v - off) / sc).sigmoid() - ((-v - off) / sc).sigmoid())

    qf = wdl(scorenet, lp.in_offset, lp.in_scaling)
    pf = wdl(score, lp.out_offset, lp.out_scaling)
    pt = pf * lam + outcome * (1.0 - lam)
    loss = torch.pow(torch.abs(pt - qf), lp.pow_exp)
    if lp.qp_asymmetry != 0.0:
        loss = loss * ((qf > pt) * lp.qp_asymmetry + 1)
    wts = 1 + (2.0**lp.w1 - 1) * torch.pow((pf - 0.5) ** 2 * pf * (1 - pf), lp.w2)
    return (loss * wts).sum() / wts.sum()


def training_loss(params, batch, q: Quant = Quant(), lam=1.0, lp: Loss = Loss()):
    us, them, white, black, outcome, score, piece_count = batch
    y = forward(params, us, them, white, black, piece_count, q, True, True)
    return sf_loss(y * q.nnue2score, score, outcome, lam, lp)
