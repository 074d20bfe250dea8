"""Stand-ins for optional packages the reference project imports at module
scope, so that its `model` package imports where they are not installed.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

  chess         only piece constants and a `Piece(type, color)` record are used
                (initial PSQT values, model/modules/features/halfka_v2_hm.py:173-194)
  torchmetrics  running means of the loss (model/nnue.py:108-114)
  numba         `njit` as a plain decorator (model/utils/serialize.py)
A package that is installed is left alone.
"""

from __future__ import annotations

import importlib.util
import sys
import types

import torch


def _missing(name: str) -> bool:
    if name in sys.modules:
        return False
    try:
        return importlib.util.find_spec(name) is None
    except (ImportError, ValueError):
        return True


def install() -> None:
    if _missing("chess"):
        chess = types.ModuleType("chess")
        chess.PAWN, chess.KNIGHT, chess.BISHOP, chess.ROOK, chess.QUEEN, chess.KING = 1, 2, 3, 4, 5, 6
        chess.WHITE, chess.BLACK = True, False

        class Piece:
            def __init__(self, piece_type, color):
                self.piece_type, self.color = piece_type, color

        chess.Piece = Piece
        sys.modules["chess"] = chess

    if _missing("torchmetrics"):
        tm = types.ModuleType("torchmetrics")

        class MeanMetric(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.total, self.n = 0.0, 0

            def update(self, v):
                self.total += float(v.detach()) if torch.is_tensor(v) else float(v)
                self.n += 1

            def compute(self):
                return torch.tensor(self.total / max(self.n, 1))

            def reset(self):
                self.total, self.n = 0.0, 0

        class MetricCollection(torch.nn.ModuleDict):
            pass

        tm.MeanMetric, tm.MetricCollection = MeanMetric, MetricCollection
        sys.modules["torchmetrics"] = tm

    if _missing("numba"):
        nb = types.ModuleType("numba")
        nb.njit = lambda f=None, **kw: (f if f is not None else (lambda g: g))
        sys.modules["numba"] = nb
