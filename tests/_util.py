"""Shared helpers of the test suite (no product code)."""

from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name: str) -> dict:
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def t(a, dtype=None):
    x = torch.from_numpy(np.ascontiguousarray(a))
    return x if dtype is None else x.to(dtype)


def max_rel_err(ours: torch.Tensor, ref: torch.Tensor) -> float:
    """max |ours - ref| relative to the max-norm of ref (elementwise relative
    error is meaningless where contributions cancel)."""
    denom = max(float(ref.abs().max()), 1e-30)
    return float((ours.double() - ref.double()).abs().max()) / denom


def small_model_params(seed: int = 11) -> dict:
    """The grid-aligned weights tests/golden/make_golden.py installs into the
    reference model (same generator, same draw order), native HalfKAv2_hm^
    layout with L1 = 64, as float64 numpy arrays in the oracle's layout."""
    gen = np.random.default_rng(seed)
    w = gen.integers(-40, 41, (24576, 72)) / 256.0
    w[:, 64:] = gen.integers(-3000, 3001, (24576, 8)) / 9600.0
    v = gen.integers(-20, 21, (768, 72)) / 256.0
    v[:, 64:] = gen.integers(-900, 901, (768, 8)) / 9600.0
    bias = np.zeros(72)
    bias[:64] = gen.integers(-60, 61, 64) / 256.0
    p = {"ft_real": w, "ft_virtual": v, "ft_bias": bias}
    p["l1_w"] = gen.integers(-90, 91, (256, 64)) / 128.0
    p["l1f_w"] = gen.integers(-30, 31, (32, 64)) / 128.0
    p["l1_b"] = gen.integers(-9000, 9001, 256) / 16384.0
    p["l1f_b"] = gen.integers(-3000, 3001, 32) / 16384.0
    p["l2_w"] = gen.integers(-100, 101, (256, 64)) / 64.0
    p["l2_b"] = gen.integers(-6000, 6001, 256) / 8192.0
    p["out_w"] = gen.integers(-120, 121, (8, 128)) / 128.0
    p["out_b"] = gen.integers(-9000, 9001, 8) / 16384.0
    p["ft_weight"] = w + np.tile(v, (32, 1))
    return p
