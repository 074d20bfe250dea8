"""Feature blocks that own the feature-transformer weight table.

`HalfKav2Hm` mirrors the reference's class of the same name
(model/modules/features/halfka_v2_hm.py:39-170 of the reference project):
a real table of 24576 rows (32 king buckets x 12 piece planes x 64 squares)
plus 768 factor ("virtual") rows that are folded in weight space,
`merged_weight = weight + virtual_weight.repeat(32, 1)`.

`HalfKav2HmFlat` is the layout the headline benchmark is quoted on: one table
of 23232 rows (22528 real + 704 factor rows) where factor features are extra
*indices* of a position, so no merge pass exists.

`FullThreats` and `PP3Wide` mirror the two other blocks of the reference's
default feature set `Full_Threats+PP_3Wide+HalfKAv2_hm^`
(model/modules/features/full_threats.py:7-57, pp_3wide.py:7-55,
features/__init__.py:13-19): plain tables without factor rows, PSQT columns
zero, weights kept inside the int8 export range by `clip_weights`.
`full_features.py` builds their index lists.

Any object with the same attributes works with `ComposedFeatureTransformer`,
including the reference's own feature classes.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .positions import KING_BUCKETS, NUM_INPUTS_BASELINE, NUM_REAL_BASELINE

# material values used for the initial PSQT columns, by piece type 1..5
_PIECE_VALUES = {1: 126, 2: 781, 3: 825, 4: 1276, 5: 2538}


class InputFeature(nn.Module):
    HASH: int
    FEATURE_NAME: str
    INPUT_FEATURE_NAME: str
    NUM_INPUTS: int
    MAX_ACTIVE_FEATURES: int
    NUM_REAL_FEATURES: int
    EXPORT_WEIGHT_DTYPE: torch.dtype = torch.int16

    def clip_weights(self, quantization) -> None:
        pass

    def reset_parameters(self) -> None:
        sigma = math.sqrt(1 / self.NUM_INPUTS)
        with torch.no_grad():
            self.weight.uniform_(-sigma, sigma)


def _inverse_king_buckets() -> list[int]:
    inv = [0] * 32
    for sq in range(64):
        if KING_BUCKETS[sq] >= 0:
            inv[int(KING_BUCKETS[sq])] = sq
    return inv


class HalfKav2Hm(InputFeature):
    FUSED_TABLE = True  # merged table = weight + virtual_weight.repeat(buckets, 1)
    HASH = 0x7F234CB8
    FEATURE_NAME = "HalfKAv2_hm^"
    INPUT_FEATURE_NAME = "HalfKAv2_hm"
    MAX_ACTIVE_FEATURES = 32
    NUM_PLANES = 768
    NUM_BUCKETS = 32
    NUM_INPUTS = 768 * 32
    NUM_INPUTS_VIRTUAL = 768
    NUM_REAL_FEATURES = 704 * 32

    def __init__(self, num_outputs: int):
        super().__init__()
        self.num_outputs = num_outputs
        self.weight = nn.Parameter(torch.empty(self.NUM_INPUTS, num_outputs, dtype=torch.float32))
        self.virtual_weight = nn.Parameter(torch.zeros(self.NUM_INPUTS_VIRTUAL, num_outputs, dtype=torch.float32))
        self.reset_parameters()

    def merged_weight(self) -> torch.Tensor:
        return self.weight + self.virtual_weight.repeat(self.NUM_BUCKETS, 1)

    @torch.no_grad()
    def coalesce(self) -> None:
        self.weight.add_(self.virtual_weight.repeat(self.NUM_BUCKETS, 1))
        self.zero_virtual_weights()

    @torch.no_grad()
    def zero_virtual_weights(self) -> None:
        self.virtual_weight.zero_()

    @staticmethod
    def initial_psqt_values() -> torch.Tensor:
        """Material value of the piece a row stands for, from white's point of
        view: +v for an own piece, -v for an opposing one, 0 for kings.  Same
        for every king bucket and square."""
        plane = torch.zeros(12)
        for pt, v in _PIECE_VALUES.items():
            plane[(pt - 1) * 2] = v
            plane[(pt - 1) * 2 + 1] = -v
        return plane.repeat_interleave(64).repeat(32)

    @torch.no_grad()
    def init_weights(self, num_psqt_buckets: int, nnue2score: float) -> None:
        self.zero_virtual_weights()
        l1 = self.num_outputs - num_psqt_buckets
        vals = self.initial_psqt_values().to(self.weight) / nnue2score
        self.weight[:, l1:] = vals[:, None]

    @torch.no_grad()
    def get_export_weights(self) -> torch.Tensor:
        """Merged table in the 11-plane export layout (22528 rows): planes 0-9
        copied, the two king planes share plane 10 (opposing king everywhere,
        own king on the bucket's king square)."""
        merged = self.merged_weight().view(32, 12, 64, -1)
        out = merged.new_zeros(32, 11, 64, merged.shape[-1])
        out[:, :10] = merged[:, :10]
        out[:, 10] = merged[:, 11]
        for b, ksq in enumerate(_inverse_king_buckets()):
            out[b, 10, ksq] = merged[b, 10, ksq]
        return out.reshape(self.NUM_REAL_FEATURES, -1)

    @torch.no_grad()
    def load_export_weights(self, export_weight: torch.Tensor) -> None:
        src = export_weight.view(32, 11, 64, -1)
        full = export_weight.new_zeros(32, 12, 64, src.shape[-1])
        full[:, :10] = src[:, :10]
        full[:, 11] = src[:, 10]
        for b, ksq in enumerate(_inverse_king_buckets()):
            full[b, 10, ksq] = src[b, 10, ksq]
            full[b, 11, ksq] = 0
        self.weight.data.copy_(full.reshape(self.NUM_INPUTS, -1))
        self.zero_virtual_weights()


class HalfKav2HmFlat(InputFeature):
    """22528 real + 704 factor rows in one table; factor rows are addressed by
    the position's own index list (see positions.baseline_indices)."""

    FUSED_TABLE = True  # merged table = weight
    HASH = 0x7F234CB8
    FEATURE_NAME = "HalfKAv2_hm^"
    INPUT_FEATURE_NAME = "HalfKAv2_hm^"
    MAX_ACTIVE_FEATURES = 64
    NUM_INPUTS = NUM_INPUTS_BASELINE
    NUM_REAL_FEATURES = NUM_REAL_BASELINE

    def __init__(self, num_outputs: int):
        super().__init__()
        self.num_outputs = num_outputs
        self.weight = nn.Parameter(torch.empty(self.NUM_INPUTS, num_outputs, dtype=torch.float32))
        self.reset_parameters()

    def merged_weight(self) -> torch.Tensor:
        return self.weight

    @torch.no_grad()
    def coalesce(self) -> None:
        real = self.weight[: self.NUM_REAL_FEATURES].view(32, 704, -1)
        real.add_(self.weight[self.NUM_REAL_FEATURES :].unsqueeze(0))
        self.zero_virtual_weights()

    @torch.no_grad()
    def zero_virtual_weights(self) -> None:
        self.weight[self.NUM_REAL_FEATURES :].zero_()

    @torch.no_grad()
    def init_weights(self, num_psqt_buckets: int, nnue2score: float) -> None:
        self.zero_virtual_weights()
        l1 = self.num_outputs - num_psqt_buckets
        plane = torch.zeros(11)
        for pt, v in _PIECE_VALUES.items():
            plane[(pt - 1) * 2] = v
            plane[(pt - 1) * 2 + 1] = -v
        vals = plane.repeat_interleave(64).repeat(32).to(self.weight) / nnue2score
        self.weight[: self.NUM_REAL_FEATURES, l1:] = vals[:, None]

    @torch.no_grad()
    def get_export_weights(self) -> torch.Tensor:
        real = self.weight[: self.NUM_REAL_FEATURES].view(32, 704, -1)
        return (real + self.weight[self.NUM_REAL_FEATURES :].unsqueeze(0)).reshape(self.NUM_REAL_FEATURES, -1)

    @torch.no_grad()
    def load_export_weights(self, export_weight: torch.Tensor) -> None:
        self.weight[: self.NUM_REAL_FEATURES].copy_(export_weight)
        self.zero_virtual_weights()


class _PlainTable(InputFeature):
    """A feature block that is one trainable table: no factor rows, no piece values."""

    FUSED_TABLE = True  # merged table = weight
    MAX_ACTIVE_FEATURES = 128
    EXPORT_WEIGHT_DTYPE = torch.int8

    def __init__(self, num_outputs: int):
        super().__init__()
        self.num_outputs = num_outputs
        self.weight = nn.Parameter(torch.empty(self.NUM_INPUTS, num_outputs, dtype=torch.float32))
        self.reset_parameters()

    def merged_weight(self) -> torch.Tensor:
        return self.weight

    @torch.no_grad()
    def coalesce(self) -> None:
        pass

    @torch.no_grad()
    def zero_virtual_weights(self) -> None:
        pass

    @torch.no_grad()
    def init_weights(self, num_psqt_buckets: int, nnue2score: float) -> None:
        self.weight[:, self.num_outputs - num_psqt_buckets :] = 0.0

    @torch.no_grad()
    def get_export_weights(self) -> torch.Tensor:
        return self.weight.data.clone()

    @torch.no_grad()
    def load_export_weights(self, export_weight: torch.Tensor) -> None:
        self.weight.data.copy_(export_weight)

    def clip_weights(self, quantization) -> None:
        """Keeps every weight inside what the int8 export can hold (+-127 / ft_quantized_one)."""
        self.weight.data.clamp_(quantization.min_threat_weight, quantization.max_threat_weight)


class FullThreats(_PlainTable):
    """One row per (attacking piece, from, attacked piece, to) relation: 59808 rows."""

    HASH = 0x2E6B9D04
    FEATURE_NAME = "Full_Threats"
    INPUT_FEATURE_NAME = "Full_Threats"
    NUM_INPUTS = 59808
    NUM_REAL_FEATURES = 59808


class PP3Wide(_PlainTable):
    """One row per pair of pawns on the same or adjacent files: 96 * 95 / 2 = 4560 rows."""

    HASH = 0x86F2B1DD
    FEATURE_NAME = "PP_3Wide"
    INPUT_FEATURE_NAME = "PP_3Wide"
    NUM_INPUTS = 4560
    NUM_REAL_FEATURES = 4560


DEFAULT_FEATURES = "Full_Threats+PP_3Wide+HalfKAv2_hm^"
_FEATURES = {"HalfKAv2_hm^": HalfKav2Hm, "HalfKAv2_hm^flat": HalfKav2HmFlat, "Full_Threats": FullThreats,
             "PP_3Wide": PP3Wide}


def get_feature_cls(name: str):
    return [_FEATURES[p] for p in name.split("+")]
