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

`skew="zipf"` draws king squares and (type, colour, square) of the other
pieces from Zipf-like distributions instead of uniform ones.  Real games put
about a third of all active features on a few dozen table rows (castled
kings, pawns on their home squares: on one batch of 16384 real positions the
reference's loader, data_loader/cpp/training_data_loader.cpp:487-544, fills a
single row more than 12000 times); the skewed generator reproduces that
concentration, which is what decides between atomics and a segment reduction
in the backward pass.
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


def _zipf_weights(n: int, exponent: float, perm_seed: int) -> np.ndarray:
    """Probabilities proportional to 1 / rank^exponent over a fixed (seeded) ranking of n items."""
    ranks = np.random.default_rng(perm_seed).permutation(n) + 1
    w = 1.0 / ranks.astype(np.float64) ** exponent
    return w / w.sum()


def _skewed_slots(rng, batch: int):
    """Distinct squares per row with both kings and the other pieces drawn from skewed distributions:
    squares come out as the order of `weight / Exp(1)` keys (a weighted permutation), the kings from a steeper
    ranking of their own, and (type, colour) of a piece from a ranking tied to its square."""
    king_w = _zipf_weights(64, 2.0, 101)
    sq_w = _zipf_weights(64, 1.1, 202)
    keys = sq_w[None, :] / rng.exponential(1.0, size=(batch, 64))
    order = np.argsort(-keys, axis=1).astype(np.int64)          # likely squares first
    wk = rng.choice(64, size=batch, p=king_w)
    bk = rng.choice(64, size=batch, p=king_w[::-1])
    bk = np.where(bk == wk, (bk + 8) % 64, bk)
    squares = np.empty((batch, 32), dtype=np.int64)
    squares[:, 0], squares[:, 1] = wk, bk
    # the other slots: the row's likely squares in order, skipping the two king squares
    free = (order != wk[:, None]) & (order != bk[:, None])
    rank_among_free = np.cumsum(free, axis=1) - 1
    take = free & (rank_among_free < 30)
    squares[:, 2:] = order[take].reshape(batch, 30)
    # piece on a square: one dominant (type, colour) per square, the rest uniform
    combo_of_sq = np.random.default_rng(303).integers(0, 10, size=64)
    dominant = rng.random((batch, 32)) < 0.8
    combo = np.where(dominant, combo_of_sq[squares], rng.integers(0, 10, size=(batch, 32)))
    return squares, combo // 2 + 1, (combo % 2).astype(bool)


def generate_positions(batch: int, seed: int, fixed_count: int | None = None, skew: str = "uniform") -> PositionBatch:
    rng = np.random.default_rng(seed)
    if fixed_count is None:
        k = rng.integers(2, 33, size=batch)
    else:
        if not 2 <= fixed_count <= 32:
            raise ValueError("fixed_count must be in 2..32")
        k = np.full(batch, fixed_count, dtype=np.int64)
    if skew == "zipf":
        squares, piece_type, is_white = _skewed_slots(rng, batch)
    elif skew == "uniform":
        squares = np.argsort(rng.random((batch, 64)), axis=1)[:, :32].astype(np.int64)
        piece_type = rng.integers(1, 6, size=(batch, 32))
        is_white = rng.integers(0, 2, size=(batch, 32)).astype(bool)
    else:
        raise ValueError(f"unknown skew {skew!r}; expected 'uniform' or 'zipf'")
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


def generate_batch(batch: int, seed: int, layout: str = "baseline", fixed_count: int | None = None,
                   skew: str = "uniform") -> TrainingBatch:
    pos = generate_positions(batch, seed, fixed_count, skew)
    fn = {"baseline": baseline_indices, "native": native_indices}[layout]
    score, outcome = generate_targets(batch, seed)
    us = pos.stm_white.astype(np.float32)[:, None]
    return TrainingBatch(us, 1.0 - us, fn(pos, True), fn(pos, False), outcome, score, pos.piece_count.copy())
