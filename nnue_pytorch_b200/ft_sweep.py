"""Forward / backward sweep of the fused double feature-transformer kernels.

    python -m nnue_pytorch_b200.ft_sweep                       # the full sweep
    python -m nnue_pytorch_b200.ft_sweep --l1 3072 --batch 16384 --active 0 \
        --tune bwd_u=1 --tune seg_chunk=256                   # one point, with tuning knobs

Shapes: HalfKAv2_hm^ as 22528 real + 704 factor rows (N = 23232, K = 64),
L1 in {1024, 2048, 3072}, batch in {4096, 16384, 65536}, `active` real
features per perspective fixed at 2, 8, 16 or 32 (0 = piece count ~ U[2,32]),
fp32 weights ~ N(0, 0.01).  Each point prints one JSON line with the mean
kernel time over 50 launches after 10 warm-ups (CUDA events on the launching
stream): "cold" with the L2 flushed between launches (the headline figures;
--no-flush skips it) and "steady" back to back and the algorithmic GB/s: every (position,
active row) counts one full row, as in an embedding bag; bytes served by the
L2 are therefore counted too and the figure can exceed the DRAM bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import _launch, _lib, positions

N_ROWS = positions.NUM_INPUTS_BASELINE
K = positions.MAX_ACTIVE_BASELINE


def _peak():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)  # 512 MB read-modify-write evicts the 126 MB L2
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        total += a.elapsed_time(b)
    return total / iters


FULL_ROWS, FULL_K, FULL_MEAN = 88944, 288, 52  # the reference's default feature set (threats + pawn patterns + HalfKA)


def _full_feature_lists(batch: int, seed: int):
    """Stand-in lists with the default feature set's shape: 88944 rows, up to
    288 active per perspective, about 52 on average, rows uniform at random."""
    import numpy as np

    rng = np.random.default_rng(seed)
    n_act = np.clip(np.rint(rng.normal(FULL_MEAN, 14, size=(2, batch))), 4, FULL_K).astype(np.int64)
    lists = []
    for side in range(2):
        idx = rng.integers(0, FULL_ROWS, size=(batch, FULL_K), dtype=np.int32)
        idx[np.arange(FULL_K)[None, :] >= n_act[side][:, None]] = -1
        lists.append(idx)
    us = rng.integers(0, 2, size=(batch, 1)).astype(np.float32)
    pc = rng.integers(2, 33, size=batch)
    return us, 1.0 - us, lists[0], lists[1], pc, float(n_act.mean())


def run_point(l1: int, batch: int, active: int, mode: str, iters: int, warmup: int, flush: bool, dev,
              features: str = "halfka"):
    P = 8
    W = l1 + P
    n_rows, k_max = (N_ROWS, K) if features == "halfka" else (FULL_ROWS, FULL_K)
    if features == "halfka":
        b = positions.generate_batch(batch, 0, layout="baseline", fixed_count=active if active else None)
        rows_per_persp = 2.0 * (active if active else float(b.piece_count.mean()))
        arrays, piece_count = (b.us, b.them, b.white, b.black), b.piece_count
    else:
        u, t_, wl, bl, piece_count, rows_per_persp = _full_feature_lists(batch, 0)
        arrays = (u, t_, wl, bl)
    us, them, wi, bi = (torch.from_numpy(x).to(dev) for x in arrays)
    ps = torch.from_numpy((piece_count - 1) // 4).to(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    w = torch.randn(n_rows, W, generator=g, device=dev) * 0.01
    bias = torch.randn(W, generator=g, device=dev) * 0.01
    gl0 = torch.randn(batch, l1, generator=g, device=dev)
    gp = torch.randn(batch, 1, generator=g, device=dev)
    fl = torch.zeros(128 * 1024 * 1024, device=dev) if flush else None
    max_act = 255.0 / 256.0

    saved = [None]

    def fwd():
        saved[0] = _launch.fused_forward(us, them, wi, bi, ps, w, bias, max_act, l1)[3]

    def bwd():
        _launch.fused_backward(us, them, wi, bi, ps, max_act, l1, n_rows, W, gl0, gp, gp, saved[0], mode)

    t_f = _time(fwd, iters, warmup, fl)
    t_b = _time(bwd, iters, warmup, fl)
    warm = None
    if flush:  # the steady-state figures as well: same launches back to back, nothing evicted in between
        warm = (_time(fwd, iters, warmup, None), _time(bwd, iters, warmup, None))
    _launch.device_status(dev)
    common = batch * (2 * rows_per_persp * W * 4 + 2 * k_max * 4 + 24 + 3 * l1 * 4 + 8)
    peak, kind = _peak()
    out = {
        "l1": l1, "batch": batch, "active_real_per_perspective": active or "U[2,32]", "rows_per_perspective": rows_per_persp,
        "fwd_ms": t_f, "fwd_algorithmic_GBps": common / t_f / 1e6, "fwd_frac_of_hbm": common / t_f / 1e6 / peak,
        "bwd_ms": t_b, "bwd_algorithmic_GBps": (common + n_rows * W * 4) / t_b / 1e6,
        "bwd_frac_of_hbm": (common + n_rows * W * 4) / t_b / 1e6 / peak,
        "rows": n_rows, "max_active": k_max,
        "fwd_ms_steady": warm[0] if warm else None, "bwd_ms_steady": warm[1] if warm else None,
        "bwd_mode": mode, "hbm_peak_GBps": peak, "peak_source": kind, "l2_flushed": bool(flush),
    }
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--l1", type=int, nargs="*", default=[1024, 2048, 3072])
    ap.add_argument("--batch", type=int, nargs="*", default=[4096, 16384, 65536])
    ap.add_argument("--active", type=int, nargs="*", default=[2, 8, 16, 32])
    ap.add_argument("--mode", default="auto", choices=["auto", "atomic", "segment"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--features", default="halfka", choices=["halfka", "full"],
                    help="full = the shape of the reference's default feature set (88944 rows, K = 288, ~52 active); "
                         "--active is ignored")
    ap.add_argument("--tune", action="append", default=[], help="key=value, passed to nnue_b200_tune")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("ft_sweep needs a CUDA device")
    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.load()
    tuned = {}
    for kv in a.tune:
        k, v = kv.split("=")
        _lib.tune(k, int(v))
        tuned[k] = int(v)
    for l1 in a.l1:
        for batch in a.batch:
            for act in a.active:
                r = run_point(l1, batch, act, a.mode, a.iters, a.warmup, not a.no_flush, dev, a.features)
                if tuned:
                    r["tune"] = tuned
                print(json.dumps(r), flush=True)
                torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
