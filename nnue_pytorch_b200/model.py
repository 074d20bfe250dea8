"""Host-side network around the feature transformer, for running whole
training steps without the reference checkout.

The feature transformer is this package's `ComposedFeatureTransformer` (CUDA
kernels); everything after it is ordinary torch (cuBLAS GEMMs and elementwise
ops), restating the graph of the reference project:
  model/model.py:9-133                      `NNUEModel`
  model/modules/layer_stacks.py:12-84       `LayerStacks`
  model/modules/stacked_linear.py:9-127     bucketed linear layers
  model/nnue.py:22-70,117-182               loss and the ten optimizer groups
Parameter names match the reference so state dicts are interchangeable.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from .composed_feature_transformer import ComposedFeatureTransformer
from .features import get_feature_cls
from .quantize import QuantizationConfig, QuantizationManager
from .ranger_lite import RangerLite


class StackedLinear(nn.Module):
    """`count` independent linear layers stored as one wide layer; a position
    uses the slice of its bucket."""

    def __init__(self, in_features: int, out_features: int, count: int, quantization=None, layer_key=None):
        super().__init__()
        self.in_features, self.out_features, self.count = in_features, out_features, count
        self.linear = nn.Linear(in_features, out_features * count)
        self.quantization, self.layer_key = quantization, layer_key
        with torch.no_grad():  # every bucket starts from the same weights
            self.linear.weight.copy_(self.linear.weight[:out_features].repeat(count, 1))
            self.linear.bias.copy_(self.linear.bias[:out_features].repeat(count))

    def _weights(self):
        return self.linear.weight, self.linear.bias

    def forward(self, x, ls_indices, fake_quantize_weights: bool = False):
        w, b = self._weights()
        if fake_quantize_weights:
            w = self.quantization.fake_quantize_weights(w, f"{self.layer_key}_weight")
            b = self.quantization.fake_quantize_weights(b, f"{self.layer_key}_bias")
        wide = F.linear(x, w, b).reshape(-1, self.out_features)
        base = torch.arange(0, ls_indices.shape[0] * self.count, self.count, device=wide.device)
        return wide[ls_indices.flatten() + base]


class FactorizedStackedLinear(StackedLinear):
    """Adds one layer shared by all buckets (folded in weight space)."""

    def __init__(self, in_features, out_features, count, quantization, layer_key):
        super().__init__(in_features, out_features, count, quantization, layer_key)
        self.factorized_linear = nn.Linear(in_features, out_features)
        self.zero_virtual_weights()

    def _weights(self):
        return (
            self.linear.weight + self.factorized_linear.weight.repeat(self.count, 1),
            self.linear.bias + self.factorized_linear.bias.repeat(self.count),
        )

    @torch.no_grad()
    def zero_virtual_weights(self):
        self.factorized_linear.weight.zero_()
        self.factorized_linear.bias.zero_()


class LayerStacks(nn.Module):
    def __init__(self, count: int, L1: int, L2: int, L3: int, quantization: QuantizationManager):
        super().__init__()
        self.count, self.L1, self.L2, self.L3 = count, L1, L2, L3
        self.quantization = quantization
        self.l1 = FactorizedStackedLinear(L1, L2, count, quantization, "ls_l1")
        self.l2 = StackedLinear(L2 * 2, L3, count, quantization, "ls_l2")
        self.output = StackedLinear(L2 * 2 + L3 * 2, 1, count, quantization, "ls_output")
        with torch.no_grad():
            self.output.linear.bias.zero_()

    def _activate(self, x, fake_quantize_acts):
        q = self.quantization
        sq = torch.pow(x, 2.0)
        if fake_quantize_acts:
            sq = q.fake_quantize_ls_act(sq)
        sq = sq * q.sqr_crelu_correction_factor
        if fake_quantize_acts:
            x = q.fake_quantize_ls_act(x)
        return q.clip_ls_act(torch.cat([sq, x], dim=1))

    fused = True  # use the bucket-aware kernels when the shapes allow it
    tensor_core_l1 = True  # first layer on the tensor cores when its inputs are exact in TF32 (quantized model)

    @torch.compiler.disable  # ctypes launches: runs eagerly inside a compiled model
    def plan_ahead(self, ls_indices):
        """Starts the bucket plan of this batch on a second stream (CUDA only); pass the result to
        `forward(..., plan_ahead=...)`.  None when the fused kernels do not apply."""
        from . import layer_stack_functions as lsf

        if self.fused and ls_indices.is_cuda and self.L2 == 32 and self.L3 == 32 and self.L1 % 32 == 0 and self.count <= 16:
            return lsf.PlanAhead(ls_indices, self.count)
        return None

    @torch.compiler.disable  # ctypes launches: runs eagerly inside a compiled model
    def _fused_forward(self, x, ls_indices, fake_quantize_acts, fake_quantize_weights, plan_ahead):
        from . import layer_stack_functions as lsf

        l1, l2, out = self.l1, self.l2, self.output
        w1, b1, w2, b2, w3, b3 = lsf.LayerStackWeightsFunction.apply(
            l1.linear.weight, l1.linear.bias, l1.factorized_linear.weight, l1.factorized_linear.bias,
            l2.linear.weight, l2.linear.bias, out.linear.weight, out.linear.bias, self.quantization,
            fake_quantize_weights)
        # quantized model: activations on the 1/128 grid and fake-quantized weights are exact in TF32
        exact = bool(self.tensor_core_l1 and fake_quantize_acts and fake_quantize_weights)
        return lsf.FusedLayerStackFunction.apply(x, ls_indices, w1, b1, w2, b2, w3, b3, self.quantization,
                                                 fake_quantize_acts, plan_ahead, exact)

    def forward(self, x, ls_indices, fake_quantize_acts=True, fake_quantize_weights=True, plan_ahead=None):
        from . import layer_stack_functions as lsf

        if self.fused and lsf.supported(x, self.L1, self.L2, self.L3, self.count):
            return self._fused_forward(x, ls_indices, fake_quantize_acts, fake_quantize_weights, plan_ahead)
        o1 = self.l1(x, ls_indices, fake_quantize_weights)
        skip = o1[:, -2].view(-1, 1) - o1[:, -1].view(-1, 1)
        x1 = self._activate(o1, fake_quantize_acts)
        x2 = self._activate(self.l2(x1, ls_indices, fake_quantize_weights), fake_quantize_acts)
        y = self.output(torch.cat([x1, x2], dim=1), ls_indices, fake_quantize_weights)
        if fake_quantize_acts:
            skip = self.quantization.fake_quantize_skip_act(skip)
        y = y + skip
        if fake_quantize_acts:
            y = self.quantization.fake_quantize_output(y)
        return y


@dataclass
class ModelConfig:
    L1: int = 1024
    L2: int = 32
    L3: int = 32
    quantize_config: QuantizationConfig = field(default_factory=QuantizationConfig)


class NNUEModel(nn.Module):
    def __init__(self, feature_name: str, config: ModelConfig, num_psqt_buckets: int = 8, num_ls_buckets: int = 8):
        super().__init__()
        self.L1, self.L2, self.L3 = config.L1, config.L2, config.L3
        self.quantization = QuantizationManager(config.quantize_config)
        self.num_psqt_buckets, self.num_ls_buckets = num_psqt_buckets, num_ls_buckets
        self.input = ComposedFeatureTransformer(get_feature_cls(feature_name), self.L1, num_psqt_buckets, self.quantization)
        self.layer_stacks = LayerStacks(num_ls_buckets, self.L1, self.L2, self.L3, self.quantization)
        self.input.init_weights()

    def forward_parts(self, us, them, white_indices, black_indices, piece_count, fake_quantize_acts=True,
                      fake_quantize_weights=True):
        """(layer-stack output, white PSQT, black PSQT), each [B, 1]: the three
        terms `forward` combines."""
        bucket = (piece_count - 1) // 4
        ahead = self.layer_stacks.plan_ahead(bucket)  # built beside the feature transformer
        l0, wpsqt, bpsqt = self.input(us, them, white_indices, black_indices, bucket, fake_quantize_acts, fake_quantize_weights)
        return self.layer_stacks(l0, bucket, fake_quantize_acts, fake_quantize_weights, ahead), wpsqt, bpsqt

    def forward(self, us, them, white_indices, black_indices, piece_count, fake_quantize_acts=True, fake_quantize_weights=True):
        y, wpsqt, bpsqt = self.forward_parts(us, them, white_indices, black_indices, piece_count, fake_quantize_acts,
                                             fake_quantize_weights)
        # PSQT: averaged over the perspectives, sign by side to move
        return y + (wpsqt - bpsqt) * (us - 0.5)


@dataclass
class LossParams:
    in_offset: float = 270.0
    out_offset: float = 270.0
    in_scaling: float = 340.0
    out_scaling: float = 380.0
    pow_exp: float = 2.5
    qp_asymmetry: float = 0.0
    w1: float = 0.0
    w2: float = 0.5
    tb_remap_base: float = 4000.0
    tb_remap_scale: float = 4000.0
    tb_remap_decay: float = 0.85


def sf_loss(scorenet, score, outcome, lp: LossParams, lam: float):
    """Win-rate-space power loss between the net and the (tablebase-remapped)
    search score blended with the game outcome."""
    a = score.abs()
    remap = lp.tb_remap_base + (lp.tb_remap_decay ** (32000 - a).clamp(min=0)) * lp.tb_remap_scale
    score = torch.where(a >= 32000 - 245, torch.where(score < 0, -remap, remap), score)
    q = (scorenet - lp.in_offset) / lp.in_scaling
    qm = (-scorenet - lp.in_offset) / lp.in_scaling
    qf = 0.5 * (1.0 + q.sigmoid() - qm.sigmoid())
    s = (score - lp.out_offset) / lp.out_scaling
    sm = (-score - lp.out_offset) / lp.out_scaling
    pf = 0.5 * (1.0 + s.sigmoid() - sm.sigmoid())
    pt = pf * lam + outcome * (1.0 - lam)
    loss = torch.pow(torch.abs(pt - qf), lp.pow_exp)
    if lp.qp_asymmetry != 0.0:
        loss = loss * ((qf > pt) * lp.qp_asymmetry + 1)
    weights = 1 + (2.0**lp.w1 - 1) * torch.pow((pf - 0.5) ** 2 * pf * (1 - pf), lp.w2)
    return (loss * weights).sum() / weights.sum()


def optimizer_groups(model: NNUEModel, lr: float, ft_wd=0.0, dense_wd=0.0, factorized_wd=0.0) -> list[dict]:
    """The ten parameter groups of the reference trainer, in its order."""
    ft_w = [p for n, p in model.input.named_parameters() if "bias" not in n]
    ft_b = [p for n, p in model.input.named_parameters() if "bias" in n]
    ls = model.layer_stacks
    spec = [
        (ft_w, ft_wd), (ft_b, 0.0),
        ([ls.l1.factorized_linear.weight], factorized_wd), ([ls.l1.factorized_linear.bias], 0.0),
        ([ls.l1.linear.weight], dense_wd), ([ls.l1.linear.bias], 0.0),
        ([ls.l2.linear.weight], dense_wd), ([ls.l2.linear.bias], 0.0),
        ([ls.output.linear.weight], dense_wd), ([ls.output.linear.bias], 0.0),
    ]
    return [{"params": ps, "lr": lr, "weight_decay": wd} for ps, wd in spec]


class TrainStep:
    """One optimizer step as the reference trainer performs it
    (trainer/engine.py:295-322): forward, loss, backward, clip the global
    gradient norm to `clip`, RangerLite update.  The clip is folded into the
    update kernels: one sum-of-squares pass per gradient, a device scalar, and
    the update multiplies by it.  `grad_hook(model)` (optional) runs between
    backward and the norm, which is where data-parallel ranks exchange
    gradients."""

    def __init__(self, model: NNUEModel, lr: float = 8.75e-4, clip: float = 2.0, lam: float = 1.0,
                 loss_params: LossParams | None = None, grad_hook=None, grad_prescale: float = 1.0,
                 table_exchange=None, fused_loss: bool = True, integer_rows: bool | str = True):
        """`grad_prescale`: factor that turns what `grad_hook` leaves in `.grad` into the true
        gradient (1/world when the hook sums over ranks without averaging).
        `table_exchange`: a `ddp.ShardedTableExchange` that owns the feature-transformer table
        (gradient reduce-scatter, sharded update, all-gather); the table then leaves the
        optimizer's parameter groups.
        `integer_rows`: True lets the exchange send the ranks the int16 / PSQT rows their forward reads instead of
        the fp32 rows (`ShardedTableExchange.ship_integer_rows`; the fp32 parameter is then current on every rank
        only after `table_exchange.sync_table()`), "with_fp32" sends both, False only the fp32 rows.  Applies when
        the table is the model's single feature block without factor rows and its scale is a power of two."""
        self.model = model
        # this loop's only writers of the table are the optimizer kernels, which rewrite the integer table too
        model.input.keep_integer_table = True
        self.clip, self.lam = clip, lam
        # False, or a tensor-valued `lam` (per-sample lambda jitter): the loss as elementwise torch ops (`sf_loss`)
        self.fused_loss = fused_loss
        self.loss_params = loss_params or LossParams()
        self.grad_hook = grad_hook
        self.table_exchange = table_exchange
        groups = optimizer_groups(model, lr)
        if table_exchange is not None:
            groups[0]["params"] = [p for p in groups[0]["params"] if p is not table_exchange.param]
            groups = [g for g in groups if g["params"]]
            table_exchange.install()
            inp = model.input
            if (integer_rows and len(inp.features) == 1 and inp.features[0].weight is table_exchange.param
                    and getattr(inp.features[0], "virtual_weight", None) is None and inp.integer_table_possible()):
                s = inp.quantization.weight_scales_dict
                table_exchange.ship_integer_rows(inp.l1_size, s["ft_weight"], s["ft_psqt_weight"],
                                                 fp32_to_peers=(integer_rows == "with_fp32"))
        self._table_group = {"lr": lr, "betas": (0.9, 0.999), "eps": 1e-7, "pnm_momentum": 1.0}
        self.optimizer = RangerLite(
            groups, lr=1.0, weight_decay=0.0, use_legacy_scoping_bug=False,
            normloss_active=False, pnm_activate=True, pnm_momentum=1.0, lookahead_blending_alpha=0.5,
            lookahead_mergetime=5,
        )
        dev = next(model.parameters()).device
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.grad_prescale = float(grad_prescale)
        self._coef = torch.full((1,), self.grad_prescale, dtype=torch.float32, device=dev)
        self._clipping = bool(clip and clip > 0)
        self.optimizer.grad_scale = self._coef if (self._clipping or self.grad_prescale != 1.0) else None

    def loss(self, batch):
        us, them, white, black, outcome, score, piece_count = batch
        y = self.model(us, them, white, black, piece_count, True, True)
        return sf_loss(y * self.model.quantization.nnue2score, score, outcome, self.loss_params, self.lam)

    def _loss_and_backward(self, batch):
        """Forward, loss and backward with the loss head (PSQT term, scaling,
        loss, its gradient) as one kernel: the backward pass starts from the
        gradients of the three model outputs."""
        from .loss_functions import sf_loss_fused

        us, them, white, black, outcome, score, piece_count = batch
        y, wpsqt, bpsqt = self.model.forward_parts(us, them, white, black, piece_count, True, True)
        loss, d_y, d_wp, d_bp = sf_loss_fused(y, wpsqt, bpsqt, us, score, outcome, self.loss_params, self.lam,
                                              self.model.quantization.nnue2score)
        self.optimizer.zero_grad(set_to_none=True)
        torch.autograd.backward([y, wpsqt, bpsqt], [d_y.view_as(y), d_wp.view_as(wpsqt), d_bp.view_as(bpsqt)])
        return loss

    def __call__(self, batch):
        from . import _launch

        if self.fused_loss and batch[0].is_cuda and not torch.is_tensor(self.lam):
            loss = self._loss_and_backward(batch)
        else:
            loss = self.loss(batch)
            self.optimizer.zero_grad(set_to_none=True)
            loss.backward()
        ex = self.table_exchange
        if ex is not None:
            ex.param.grad = None  # its gradient lives in the exchange's buffer
        if ex is not None and ex.sliced:
            # slice by slice on the exchange's own stream, beside the rest of the backward; issued before
            # the dense-gradient collective so that the per-slice collectives are not queued behind it
            ft_sumsq = ex.reduce()
        if self.grad_hook is not None:
            self.grad_hook(self.model)  # a collective: every rank's backward is complete after it
        if ex is not None and not ex.sliced:
            ft_sumsq = ex.reduce()
        if self._clipping:
            self._sumsq.zero_()
            grads = [p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                     for p in self.model.parameters() if p.grad is not None]
            _launch.grad_sumsq_multi(grads, self._sumsq)
            if ex is not None:
                self._sumsq.add_(ft_sumsq)
            _launch.clip_coef(self._sumsq, self.clip, self._coef, self.grad_prescale)
        opt = self.optimizer
        merge = opt.lookahead_active and opt.lookahead_step + 1 >= opt.lookahead_mergetime
        opt.step()
        if ex is not None:
            ex.step += 1
            ex.update(opt._hparams(self._table_group, ex.step, merge, phase=0), opt.grad_scale)
        return loss.detach()
