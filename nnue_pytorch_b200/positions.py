"""Seeded synthetic chess positions and their HalfKAv2_hm feature lists.

Stand-in for the binpack training data of the reference (its loader,
data_loader/cpp/training_data_loader.cpp:29-73, emits the same index lists
from real games).  Positions are not legal chess, only shaped like it:

  piece count k ~ U{2..32}; two kings on distinct uniform squares; k-2 other
  pieces of uniform type {P,N,B,R,Q} and colour on distinct free squares.

Two index layouts are produced from the same positions:

  "native"   the training layout of the reference's `HalfKav2Hm` feature
             (model/modules/features/halfka_v2_hm.py:27-50): 12 piece planes,
             N = 24576 rows, at most 32 active indices;
  "baseline" 11 planes (both kings share plane 10) with the 704 factor
             ("virtual") features as extra indices: N = 22528 + 704 = 23232
             rows, at most 64 active indices, reals first, then virtuals.

Lists are int32, padded with -1 on the right.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

# king bucket of the oriented king square (king always on files e-h after the
# horizontal mirror); square 0 = a1, 63 = h8.  Files a-d never occur.
KING_BUCKETS = np.full(64, -1, dtype=np.int64)
for _rank in range(8):
    for _f in range(4, 8):
        KING_BUCKETS[_rank * 8 + _f] = (7 - _rank) * 4 + (7 - _f)

NUM_PLANES_NATIVE = 12 * 64       # 768
NUM_INPUTS_NATIVE = 768 * 32      # 24576
MAX_ACTIVE_NATIVE = 32
NUM_PLANES_BASELINE = 11 * 64     # 704
NUM_REAL_BASELINE = 704 * 32      # 22528
NUM_INPUTS_BASELINE = NUM_REAL_BASELINE + NUM_PLANES_BASELINE  # 23232
MAX_ACTIVE_BASELINE = 64


@dataclass
class PositionBatch:
    """Raw positions: slot 0 is the white king, slot 1 the black king."""

    squares: np.ndarray      # [B, 32] int64, distinct per row
    piece_type: np.ndarray   # [B, 32] int64, 1..6 (6 = king)
    is_white: np.ndarray     # [B, 32] bool
    piece_count: np.ndarray  # [B] int64, slots >= piece_count are empty
    stm_white: np.ndarray    # [B] bool


def generate_positions(batch: int, seed: int, fixed_count: int | None = None) -> PositionBatch:
    rng = np.random.default_rng(seed)
    if fixed_count is None:
        k = rng.integers(2, 33, size=batch)
    else:
        if not 2 <= fixed_count <= 32:
            raise ValueError("fixed_count must be in 2..32")
        k = np.full(batch, fixed_count, dtype=np.int64)
    squares = np.argsort(rng.random((batch, 64)), axis=1)[:, :32].astype(np.int64)
    piece_type = rng.integers(1, 6, size=(batch, 32))
    is_white = rng.integers(0, 2, size=(batch, 32)).astype(bool)
    piece_type[:, 0] = 6
    piece_type[:, 1] = 6
    is_white[:, 0] = True
    is_white[:, 1] = False
    stm_white = rng.integers(0, 2, size=batch).astype(bool)
    return PositionBatch(squares, piece_type, is_white, k.astype(np.int64), stm_white)


def _perspective(pos: PositionBatch, white_pov: bool):
    ksq = pos.squares[:, 0] if white_pov else pos.squares[:, 1]
    flip = np.where(ksq % 8 < 4, 7, 0) ^ (0 if white_pov else 56)
    osq = pos.squares ^ flip[:, None]
    bucket = KING_BUCKETS[ksq ^ flip]
    assert (bucket >= 0).all()
    theirs = pos.is_white != white_pov
    active = np.arange(32)[None, :] < pos.piece_count[:, None]
    return osq, bucket, theirs, active


def native_indices(pos: PositionBatch, white_pov: bool) -> np.ndarray:
    """[B, 32] int32 lists in the reference's 12-plane training layout."""
    osq, bucket, theirs, active = _perspective(pos, white_pov)
    plane = (pos.piece_type - 1) * 2 + theirs
    idx = osq + plane * 64 + bucket[:, None] * NUM_PLANES_NATIVE
    return np.where(active, idx, -1).astype(np.int32)


def baseline_indices(pos: PositionBatch, white_pov: bool) -> np.ndarray:
    """[B, 64] int32 lists: k real rows, then the k matching factor rows."""
    osq, bucket, theirs, active = _perspective(pos, white_pov)
    plane = np.where(pos.piece_type == 6, 10, (pos.piece_type - 1) * 2 + theirs)
    within = plane * 64 + osq
    real = within + bucket[:, None] * NUM_PLANES_BASELINE
    virt = within + NUM_REAL_BASELINE
    k = pos.piece_count[:, None]
    j = np.arange(MAX_ACTIVE_BASELINE)[None, :]
    src = np.where(j < k, j, j - k)
    src = np.clip(src, 0, 31)
    both = np.where(j < k, np.take_along_axis(real, src, 1), np.take_along_axis(virt, src, 1))
    return np.where(j < 2 * k, both, -1).astype(np.int32)


@dataclass
class TrainingBatch:
    """One synthetic training batch in the order the reference trainer uses
    (data_loader/_native.py `SparseBatch.get_tensors`): us, them, white,
    black, outcome, score, piece_count."""

    us: np.ndarray           # [B, 1] float32, 1.0 = white to move
    them: np.ndarray         # [B, 1] float32
    white: np.ndarray        # [B, K] int32
    black: np.ndarray        # [B, K] int32
    outcome: np.ndarray      # [B, 1] float32 in {0, 0.5, 1}
    score: np.ndarray        # [B, 1] float32 centipawns
    piece_count: np.ndarray  # [B] int64

    def as_tuple(self):
        return (self.us, self.them, self.white, self.black, self.outcome, self.score, self.piece_count)


def generate_targets(batch: int, seed: int) -> tuple[np.ndarray, np.ndarray]:
    """score [B, 1] ~ N(0, 400) cp clipped to +-3000 and outcome [B, 1] uniform
    in {0, 0.5, 1}."""
    rng = np.random.default_rng([seed, 0x7A7])
    score = np.clip(rng.normal(0.0, 400.0, size=(batch, 1)), -3000, 3000).astype(np.float32)
    outcome = (rng.integers(0, 3, size=(batch, 1)) * 0.5).astype(np.float32)
    return score, outcome


def generate_batch(batch: int, seed: int, layout: str = "baseline", fixed_count: int | None = None) -> TrainingBatch:
    pos = generate_positions(batch, seed, fixed_count)
    fn = {"baseline": baseline_indices, "native": native_indices}[layout]
    score, outcome = generate_targets(batch, seed)
    us = pos.stm_white.astype(np.float32)[:, None]
    return TrainingBatch(us, 1.0 - us, fn(pos, True), fn(pos, False), outcome, score, pos.piece_count.copy())
