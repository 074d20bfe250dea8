"""`ComposedFeatureTransformer`: the module that owns the shared bias, merges
the per-feature weight tables and calls the fused double-FT operator.

Mirrors model/modules/feature_transformer/composed_feature_transformer.py:11-151
of the reference project (constructor, attributes, helper methods and
`forward` signature), so the reference's `NNUEModel` can build it unchanged.
"""

from __future__ import annotations

import math
from collections.abc import Callable

import torch
from torch import nn

from .double_ft_functions import double_feature_transform
from .fused_ft_functions import (
    FusedDoubleFtFunction,
    PrepareBiasFunction,
    PrepareTableFunction,
    QuantizedFusedDoubleFtFunction,
)

_FAKE_QUANTIZE_EPS = 1e-5  # model/quantize.py:10 of the reference


def _fusable_feature(f) -> bool:
    """Features that declare (`FUSED_TABLE = True`) that their merged table is `weight` or
    `weight + virtual_weight.repeat(k, 1)`, which the table kernel computes in one pass."""
    return bool(getattr(f, "FUSED_TABLE", False))


class ComposedFeatureTransformer(nn.Module):
    def __init__(self, feature_classes: list[Callable[[int], nn.Module]], l1_size: int, num_psqt_buckets: int, quantization):
        super().__init__()
        if l1_size % 2 != 0:
            raise ValueError(f"l1_size must be even, got {l1_size}.")
        self.l1_size = l1_size
        self.num_psqt_buckets = num_psqt_buckets
        self.num_outputs = l1_size + num_psqt_buckets

        features = [make(self.num_outputs) for make in feature_classes]
        self.features = nn.ModuleList(features)
        self.bias = nn.Parameter(torch.empty(self.num_outputs, dtype=torch.float32))

        self.NUM_INPUTS = sum(f.NUM_INPUTS for f in features)
        self.MAX_ACTIVE_FEATURES = sum(f.MAX_ACTIVE_FEATURES for f in features)
        self.NUM_REAL_FEATURES = sum(f.NUM_REAL_FEATURES for f in features)
        self.FEATURE_NAME = "+".join(f.FEATURE_NAME for f in features)
        self.INPUT_FEATURE_NAME = "+".join(f.INPUT_FEATURE_NAME for f in features)
        self.HASH = self._combined_hash()
        self.quantization = quantization

        bound = math.sqrt(1 / self.NUM_INPUTS)
        with torch.no_grad():
            self.bias.uniform_(-bound, bound)

    def _combined_hash(self) -> int:
        h = 0
        for f in self.features:
            h = ((h << 1) | (h >> 31)) & 0xFFFFFFFF  # rotate left by one, 32 bits
            h ^= f.HASH
        return h

    def merged_weight_and_bias(self, fake_quantize_weights: bool = False):
        """Table [NUM_INPUTS, l1+psqt] and bias the operator sees this step.
        The PSQT part of the bias is replaced by zeros (it never trains)."""
        b = self.bias[: self.l1_size]
        q = self.quantization
        if self.bias.is_cuda and all(_fusable_feature(f) for f in self.features):
            # one kernel per feature block: fold the factor rows and quantize in a single pass
            sm = q.weight_scales_dict["ft_weight"] if fake_quantize_weights else 0.0
            sp = q.weight_scales_dict["ft_psqt_weight"] if fake_quantize_weights else 0.0
            tables = []
            for f in self.features:
                virt = getattr(f, "virtual_weight", None)
                if virt is None and not fake_quantize_weights:
                    tables.append(f.weight)
                else:
                    t = PrepareTableFunction.apply(f.weight, virt, self.l1_size, sm, sp)
                    ex = getattr(f.weight, "_nnue_exchange", None)
                    if ex is not None:
                        t._nnue_exchange = ex  # the derived table's gradient lands in the exchange's buffer
                    tables.append(t)
            merged = tables[0] if len(tables) == 1 else torch.cat(tables, dim=0)
            sb = q.weight_scales_dict["ft_bias"] if fake_quantize_weights else 0.0
            return merged, PrepareBiasFunction.apply(self.bias, self.l1_size, sb)
        tables = [f.merged_weight() for f in self.features]
        merged = tables[0] if len(tables) == 1 else torch.cat(tables, dim=0)
        if fake_quantize_weights:
            merged = torch.cat(
                [
                    q.fake_quantize_weights(merged[:, : self.l1_size], "ft_weight"),
                    q.fake_quantize_weights(merged[:, self.l1_size :], "ft_psqt_weight"),
                ],
                dim=1,
            )
            b = q.fake_quantize_weights(b, "ft_bias")
        bias = torch.cat([b, torch.zeros_like(self.bias[self.l1_size :], dtype=b.dtype)], dim=0)
        return merged, bias

    integer_table = True  # gather an int16 table when weights are fake-quantized (same bits, half the bytes)

    # True: keep the integer table between forwards and let this package's optimizer rewrite it inside its
    # update kernel (saves a pass over the table per step).  The table is rebuilt when the parameter's storage or
    # torch version counter changes; a write through `.data` moves neither, so whoever makes one must call
    # `invalidate_integer_table()` (this module's own methods do).  Off by default; `TrainStep` switches it on.
    keep_integer_table = False

    def invalidate_integer_table(self) -> None:
        for cache in (getattr(self, "_q16_cache", None), getattr(self.features[0].weight, "_nnue_q16_cache", None)):
            if cache is not None:
                cache.invalidate()

    def _table_cache(self):
        """One feature block without factor rows: its integer table can be kept between steps."""
        if len(self.features) != 1 or getattr(self.features[0], "virtual_weight", None) is not None:
            return None
        shared = getattr(self.features[0].weight, "_nnue_q16_cache", None)
        if shared is not None and shared.owner is not None:
            return shared  # a data-parallel exchange ships the integer rows between the ranks
        if not self.keep_integer_table:
            return None
        cache = getattr(self, "_q16_cache", None)
        if cache is None:
            from ._launch import QuantTableCache

            cache = self._q16_cache = QuantTableCache()
        return cache

    def _integer_table_applies(self, indices: torch.Tensor, fake_quantize_weights: bool) -> bool:
        """The int16 form of the table is exact when every fake-quantized entry is an integer over a
        power-of-two scale shared by weights and bias, and a list holds at most 511 rows."""
        if not (fake_quantize_weights and indices.is_cuda and indices.shape[1] <= 511):
            return False
        return self.integer_table_possible()

    def integer_table_possible(self) -> bool:
        """What `_integer_table_applies` asks of the module itself, whatever the batch."""
        if not (self.integer_table and self.bias.is_cuda):
            return False
        if not all(_fusable_feature(f) for f in self.features) or len(self.features) > 8:
            return False
        s = self.quantization.weight_scales_dict
        scale = float(s["ft_weight"])
        pow2 = scale > 0 and math.frexp(scale)[0] == 0.5
        return pow2 and float(s["ft_bias"]) == scale and self.l1_size % 16 == 0 and self.num_psqt_buckets % 4 == 0

    @torch.no_grad()
    def coalesce(self) -> None:
        for f in self.features:
            f.coalesce()
        self.invalidate_integer_table()

    @torch.no_grad()
    def zero_virtual_weights(self) -> None:
        for f in self.features:
            f.zero_virtual_weights()
        self.invalidate_integer_table()

    @torch.no_grad()
    def init_weights(self) -> None:
        for f in self.features:
            f.init_weights(self.num_psqt_buckets, self.quantization.nnue2score)
        self.bias[self.l1_size :] = 0.0
        self.invalidate_integer_table()

    @torch.no_grad()
    def get_export_weights(self) -> torch.Tensor:
        return torch.cat([f.get_export_weights() for f in self.features], dim=0)

    @torch.no_grad()
    def load_export_weights(self, export_weight: torch.Tensor) -> None:
        at = 0
        for f in self.features:
            f.load_export_weights(export_weight[at : at + f.NUM_REAL_FEATURES])
            at += f.NUM_REAL_FEATURES
        self.invalidate_integer_table()

    def clip_weights(self, quantization) -> None:
        for f in self.features:
            f.clip_weights(quantization)
        self.invalidate_integer_table()

    @torch.compiler.disable  # ctypes launches: runs eagerly inside a compiled model
    def forward(
        self,
        us: torch.Tensor,
        them: torch.Tensor,
        white_indices: torch.Tensor,
        black_indices: torch.Tensor,
        psqt_indices: torch.Tensor,
        fake_quantize_acts: bool,
        fake_quantize_weights: bool,
        backend: str = "auto",
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if backend in ("auto", "fused") and self._integer_table_applies(white_indices, fake_quantize_weights):
            q = self.quantization
            params = []
            for f in self.features:
                params += [f.weight, getattr(f, "virtual_weight", None)]
            return QuantizedFusedDoubleFtFunction.apply(
                us, them, white_indices, black_indices, psqt_indices, self.bias, q.max_ft_activation, self.l1_size,
                q.config.hidden_quantized_one if fake_quantize_acts else 0.0, _FAKE_QUANTIZE_EPS,
                q.l0_correction_factor, q.weight_scales_dict["ft_weight"], q.weight_scales_dict["ft_psqt_weight"],
                self._table_cache(), *params)
        merged, bias = self.merged_weight_and_bias(fake_quantize_weights)
        if backend in ("auto", "fused") and merged.is_cuda:
            # activation fake quantization and the correction factor ride in the kernel epilogue
            q = self.quantization
            return FusedDoubleFtFunction.apply(
                us, them, white_indices, black_indices, psqt_indices, merged, bias, q.max_ft_activation,
                self.l1_size, q.config.hidden_quantized_one if fake_quantize_acts else 0.0, _FAKE_QUANTIZE_EPS,
                q.l0_correction_factor,
            )
        l0, wpsqt, bpsqt = double_feature_transform(
            us, them, white_indices, black_indices, psqt_indices, merged, bias,
            self.quantization.max_ft_activation, self.l1_size, backend,
        )
        if fake_quantize_acts:
            l0 = self.quantization.fake_quantize_ft_act(l0)
        # inference divides by a power of two; the factor keeps both grids aligned
        l0 = l0 * self.quantization.l0_correction_factor
        return l0, wpsqt, bpsqt
