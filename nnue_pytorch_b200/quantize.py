"""Quantization scheme of the net: fake quantization for training and the
integer constants of the quantized evaluation.

Behaviour follows model/quantize.py of the reference project
(`QuantizationConfig` :58-73, `QuantizationManager` :76-249): weights are
rounded to the grid `1/scale` (half to even), activations are floored onto
`1/hidden_one` after adding 1e-5, the output is truncated toward zero in
units of `1/(nnue2score*weight_scale_out)`; all three use a straight-through
gradient.  When this package is overlaid on the reference tree the reference's
own `model.quantize` objects are used instead; this module serves standalone
use (benchmarks, the integer evaluation) and derives the integer constants.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

FAKE_QUANTIZE_EPS = 1e-5


@dataclass
class QuantizationConfig:
    nnue2score: float = 600.0
    weight_scale_l1: float = 128.0
    weight_scale_l2: float = 64.0
    weight_scale_l_out: float = 128
    weight_scale_out: float = 16.0
    weight_quantized_max_hidden: float = 127.0
    ft_quantized_one: float = 256.0
    ft_quantized_max: float = 255.0
    hidden_quantized_one: float = 128.0
    hidden_quantized_max: float = 127.0
    inference_l0_division_factor: float = 512.0
    inference_sqr_crelu_division_factor: float = 128.0


def _ste(hard: torch.Tensor, soft: torch.Tensor) -> torch.Tensor:
    """Value of `hard`, gradient of `soft`."""
    return hard.detach() + (soft - soft.detach())


def fake_quantize_acts(value: torch.Tensor, act_scale: float) -> torch.Tensor:
    return _ste(value.mul(act_scale).add(FAKE_QUANTIZE_EPS).floor().div(act_scale), value)


def fake_quantize_weights(value: torch.Tensor, weight_scale: float) -> torch.Tensor:
    return _ste(value.mul(weight_scale).round().div(weight_scale), value)


class QuantizationManager:
    def __init__(self, config: QuantizationConfig | None = None):
        c = config or QuantizationConfig()
        self.config = c
        self.nnue2score = c.nnue2score
        self.weight_scale_hidden = [c.weight_scale_l1, c.weight_scale_l2, c.weight_scale_l_out]
        self.weight_scale_out = c.weight_scale_out
        self.weight_quantized_max_hidden = c.weight_quantized_max_hidden
        self.hidden_quantized_one = c.hidden_quantized_one
        self.ft_quantized_one = c.ft_quantized_one
        self.max_hidden_weight = [c.weight_quantized_max_hidden / s for s in self.weight_scale_hidden]
        self.min_threat_weight = -127 / c.ft_quantized_one
        self.max_threat_weight = 127 / c.ft_quantized_one
        self.l0_correction_factor = (
            c.ft_quantized_one**2 / c.inference_l0_division_factor / c.hidden_quantized_one
        )
        self.sqr_crelu_correction_factor = c.hidden_quantized_one / c.inference_sqr_crelu_division_factor
        self.max_ft_activation = c.ft_quantized_max / c.ft_quantized_one
        self.max_hidden_activation = c.hidden_quantized_max / c.hidden_quantized_one
        h = c.hidden_quantized_one
        self.weight_scales_dict = {
            "ft_weight": c.ft_quantized_one,
            "ft_bias": c.ft_quantized_one,
            "ft_psqt_weight": c.nnue2score * c.weight_scale_out,
            "ls_l1_weight": c.weight_scale_l1,
            "ls_l1_bias": c.weight_scale_l1 * h,
            "ls_l2_weight": c.weight_scale_l2,
            "ls_l2_bias": c.weight_scale_l2 * h,
            "ls_output_weight": c.weight_scale_l_out,
            "ls_output_bias": c.weight_scale_l_out * h,
        }

    # -- training-time fake quantization ---------------------------------
    def clip_ft_act(self, x):
        return torch.clamp(x, 0.0, self.max_ft_activation)

    def clip_ls_act(self, x):
        return torch.clamp(x, 0, self.max_hidden_activation)

    def fake_quantize_ft_act(self, x):
        return fake_quantize_acts(x, self.config.hidden_quantized_one)

    def fake_quantize_ls_act(self, x):
        return fake_quantize_acts(x, self.config.hidden_quantized_one)

    def fake_quantize_skip_act(self, x):
        return x

    def fake_quantize_weights(self, tensor: torch.Tensor, key: str) -> torch.Tensor:
        return fake_quantize_weights(tensor, self.weight_scales_dict[key])

    def fake_quantize_output(self, x: torch.Tensor) -> torch.Tensor:
        mult = int(self.config.nnue2score * self.config.weight_scale_out)
        den = int(self.config.hidden_quantized_one * self.config.weight_scale_l_out * 2.0)
        as_int = torch.round(x * den).to(torch.int64)
        out_int = torch.div(as_int * mult, den, rounding_mode="trunc")
        return _ste(out_int.to(x.dtype) / float(mult), x)

    # -- integer evaluation constants --------------------------------------
    def integer_constants(self) -> dict[str, int]:
        """Shifts, epsilons and divisors of the integer evaluation.

        Exists only for schemes whose float fake-quantized forward is exactly
        an integer computation: both correction factors equal to 1 and every
        scale a power of two.  Raises ValueError otherwise.
        """
        c = self.config

        def log2_exact(x: float, what: str) -> int:
            e = round(math.log2(x))
            if x <= 0 or 2.0**e != x:
                raise ValueError(f"{what} = {x} is not a power of two; no exact integer evaluation")
            return e

        if self.l0_correction_factor != 1.0 or self.sqr_crelu_correction_factor != 1.0:
            raise ValueError("integer evaluation needs both correction factors equal to 1.0")
        h = c.hidden_quantized_one
        s1, s2, s3 = c.weight_scale_l1 * h, c.weight_scale_l2 * h, c.weight_scale_l_out * h
        if s3 % s1 != 0:
            raise ValueError("output-layer scale must be a multiple of the first-layer scale")
        return {
            "ft_max": int(c.ft_quantized_max),
            "ft_shift": log2_exact(c.ft_quantized_one**2 / h, "ft_one^2/hidden_one"),
            "hidden_max": int(c.hidden_quantized_max),
            "sqr_shift_l1": log2_exact(s1 * s1 / h, "l1 square scale"),
            "sqr_eps_l1": int(math.floor(FAKE_QUANTIZE_EPS * s1 * s1 / h)),
            "lin_shift_l1": log2_exact(s1 / h, "weight_scale_l1"),
            "sqr_shift_l2": log2_exact(s2 * s2 / h, "l2 square scale"),
            "sqr_eps_l2": int(math.floor(FAKE_QUANTIZE_EPS * s2 * s2 / h)),
            "lin_shift_l2": log2_exact(s2 / h, "weight_scale_l2"),
            "skip_mul": int(s3 // s1),
            "out_mul": int(c.nnue2score * c.weight_scale_out),
            "out_div": int(h * c.weight_scale_l_out * 2.0),
        }
