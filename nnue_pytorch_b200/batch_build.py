"""Packed positions and their expansion into a training batch on the GPU.

The reference's loader expands every position into its active-index lists on
CPU threads and copies the lists to the GPU (data_loader/cpp/
training_data_loader.cpp:29-73, data_loader/_native.py:48-96 of the reference
project: 2 x K x 4 bytes of indices per position).  Here a loader ships a
72-byte record per position and `build_batch` expands it with one kernel
launch into the tuple `SparseBatch.get_tensors` returns, in the order
`TrainStep` takes it: us, them, white, black, outcome, score, piece_count.
"""

from __future__ import annotations

import numpy as np
import torch

from . import _lib
from ._launch import _ptr, _stream
from .positions import PositionBatch

# little-endian image of `nnue_packed_position` (include/nnue_b200.h)
PACKED_DTYPE = np.dtype(
    [("piece", "<u2", (32,)), ("score", "<i2"), ("outcome2", "u1"), ("stm_white", "u1"), ("count", "u1"),
     ("pad", "u1", (3,))]
)
assert PACKED_DTYPE.itemsize == 72

LAYOUTS = {"native": (0, 32), "baseline": (1, 64)}


def pack_positions(pos: PositionBatch, score: np.ndarray, outcome: np.ndarray) -> np.ndarray:
    """[B] records.  Scores are stored as whole centipawns (the training data
    hold int16 scores, so nothing is lost on real data); outcomes as 0/1/2."""
    B = pos.squares.shape[0]
    rec = np.zeros(B, dtype=PACKED_DTYPE)
    piece = pos.squares.astype(np.uint16) | (pos.piece_type.astype(np.uint16) << 6) | (pos.is_white.astype(np.uint16) << 9)
    slot = np.arange(32)[None, :]
    rec["piece"] = np.where(slot < pos.piece_count[:, None], piece, 0)
    rec["score"] = np.clip(np.rint(np.asarray(score).reshape(B)), -32768, 32767).astype(np.int16)
    rec["outcome2"] = np.rint(np.asarray(outcome).reshape(B) * 2.0).astype(np.uint8)
    rec["stm_white"] = pos.stm_white.astype(np.uint8)
    rec["count"] = pos.piece_count.astype(np.uint8)
    return rec


def as_bytes(rec: np.ndarray) -> torch.Tensor:
    """uint8 [B, 72] CPU tensor sharing the records' memory."""
    return torch.from_numpy(np.ascontiguousarray(rec).view(np.uint8).reshape(-1, PACKED_DTYPE.itemsize))


def build_batch(packed: torch.Tensor, layout: str = "baseline", max_active: int | None = None):
    """packed: uint8 [B, 72] CUDA tensor.  Returns (us [B,1], them [B,1],
    white [B,K] int32, black [B,K] int32, outcome [B,1], score [B,1],
    piece_count [B] int64), all on the same device."""
    if not packed.is_cuda:
        raise _lib.NnueB200Error("build_batch runs on the GPU only; pass a CUDA tensor")
    if packed.dtype != torch.uint8 or packed.dim() != 2 or packed.shape[1] != PACKED_DTYPE.itemsize:
        raise ValueError("packed must be uint8 [B, 72]")
    code, k_min = LAYOUTS[layout]
    K = k_min if max_active is None else int(max_active)
    packed = packed.contiguous()
    dev, B = packed.device, packed.shape[0]
    white = torch.empty(B, K, dtype=torch.int32, device=dev)
    black = torch.empty(B, K, dtype=torch.int32, device=dev)
    f = torch.empty(4, B, 1, dtype=torch.float32, device=dev)
    piece_count = torch.empty(B, dtype=torch.int64, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        _lib.check(
            lib.nnue_batch_build_halfka(_ptr(packed), B, code, K, _ptr(white), _ptr(black), _ptr(f[0]), _ptr(f[1]),
                                        _ptr(f[2]), _ptr(f[3]), _ptr(piece_count), None, _stream(dev)),
            "nnue_batch_build_halfka",
        )
    return f[0], f[1], white, black, f[2], f[3], piece_count
