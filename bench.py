#!/usr/bin/env python
"""Benchmark of the sparse feature-transformer training step on B200.

    python bench.py --gpus N --steps K --warmup W            (this repository's arm)
    python bench.py --impl reference --steps K --warmup W     (CPU arm, host cores)

Workload (the headline configuration): HalfKAv2_hm^ as one table of
22528 real + 704 factor rows, feature transformer 23232 -> 3072 for both
perspectives, pairwise clipped product, eight layer-stack buckets, fp32, batch
16384 per GPU, RangerLite, gradient-norm clip at 2.0, sigmoid-scaled loss with
lambda 1.0, synthetic positions (piece count ~ U[2,32]).  A step is one
forward + backward + optimizer update over one batch.

One JSON line is printed by rank 0.  `value` is positions/s with the batches
already resident in HBM; `e2e` repeats the measurement with the batch copied
from pinned host memory on a side stream (one batch ahead) and the loss of
every step copied back to the host, which reads it one step later.  With
`--feed packed` (default) the host copy is the 72-byte packed position records
and the index lists are written on the GPU inside the timed region; with
`--feed lists` it is the expanded lists, as the reference's loader ships them.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "training positions/sec at L1=3072"
UNIT = "positions/s"
N_ROWS = 23232
K_ACTIVE = 64
MEAN_ACTIVE = 34.0  # expected rows per perspective: 2 * E[k], k ~ U{2..32}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--l1", type=int, default=3072)
    ap.add_argument("--batch", type=int, default=16384, help="positions per GPU per step")
    ap.add_argument("--pool", type=int, default=4, help="distinct synthetic batches cycled through")
    ap.add_argument("--bwd-mode", default="auto", choices=["auto", "atomic", "segment"])
    ap.add_argument("--cpu-sample-batch", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tune", action="append", default=[], help="key=value, passed to nnue_b200_tune")
    ap.add_argument("--slices", default="auto", choices=["auto", "on", "off"],
                    help="fused exchange with the backward delivered in two row slices and the reduce of the first "
                         "one overlapped with the second.  auto = on from 8 GPUs (measured there: 3.42 ms against "
                         "3.55 ms per step; at 2 GPUs the two orders tie)")
    ap.add_argument("--feed", default="packed", choices=["packed", "lists"],
                    help="what the end-to-end run copies from pinned host memory every step: 72-byte packed "
                         "positions expanded on the GPU, or the expanded index lists")
    ap.add_argument("--ddp", default="fused", choices=["fused", "allreduce"],
                    help="table exchange at N > 1: peer-memory reduce-scatter/update/all-gather kernels, or NCCL all-reduce")
    return ap.parse_args()


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines, self.skip = index, None, [], 0

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            # nvidia-smi needs a moment to start: wait for its first line, then count only what follows,
            # so that every sample kept was taken while the timed region ran
            t0 = time.time()
            while not self.lines and time.time() - t0 < 3.0:
                time.sleep(0.005)
            self.skip = len(self.lines)
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()  # exact child we started
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines[self.skip:]:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
def algorithmic_bytes_fwd(batch: int, l1: int, rows_per_persp: float) -> float:
    """Embedding-bag accounting: every (position, active row) counts a full row."""
    W = l1 + 8
    return batch * (2 * rows_per_persp * W * 4 + 2 * K_ACTIVE * 4 + 24 + 3 * l1 * 4 + 8)


def algorithmic_bytes_bwd(batch: int, l1: int, rows_per_persp: float) -> float:
    return algorithmic_bytes_fwd(batch, l1, rows_per_persp) + N_ROWS * (l1 + 8) * 4


def make_pool(args, rank: int, n: int, batch: int):
    from nnue_pytorch_b200 import positions

    return [positions.generate_batch(batch, 1000 * rank + i, layout="baseline") for i in range(n)]


def make_packed_pool(args, rank: int, n: int, batch: int):
    """The same positions as `make_pool`, as pinned [B, 72] byte records."""
    from nnue_pytorch_b200 import batch_build, positions

    out = []
    for i in range(n):
        seed = 1000 * rank + i
        score, outcome = positions.generate_targets(batch, seed)
        rec = batch_build.pack_positions(positions.generate_positions(batch, seed), score, outcome)
        out.append((batch_build.as_bytes(rec).pin_memory(),))
    return out


def to_pinned(b):
    out = []
    for a in b.as_tuple():
        x = torch.from_numpy(np.ascontiguousarray(a))
        out.append(x.pin_memory() if torch.cuda.is_available() else x)
    return tuple(out)


# ---------------------------------------------------------------------------
def run_b200(args):
    import torch.distributed as dist

    from nnue_pytorch_b200 import _launch, _lib
    from nnue_pytorch_b200.ddp import make_grad_hook
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel, TrainStep

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the kernels")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", init_method="env://", device_id=dev)
    lib = _lib.load()
    _launch.set_backward_mode(args.bwd_mode)
    tuned = {}
    for kv in args.tune:
        k, v = kv.split("=")
        _lib.tune(k, int(v))
        tuned[k] = int(v)

    torch.manual_seed(1)
    model = NNUEModel("HalfKAv2_hm^flat", ModelConfig(L1=args.l1, L2=32, L3=32))
    with torch.no_grad():  # config: weights ~ N(0, 0.01) (standard deviation), PSQT columns keep their material init
        model.input.features[0].weight[:, : args.l1].normal_(0.0, 0.01)
    model.to(dev)
    hook = exchange = None
    if world > 1:
        table = model.input.features[0].weight
        if args.ddp == "fused":
            from nnue_pytorch_b200.ddp import ShardedTableExchange

            # --slices: the 704 factor rows (half of all entries) form the last slice, so the reduce of the
            # 22528 real rows can run while the factor rows' gradient is still being computed
            sliced = args.slices == "on" or (args.slices == "auto" and world >= 8)
            slices = [0, table.shape[0] - 704, table.shape[0]] if sliced else None
            exchange = ShardedTableExchange(table, slices=slices, reduce_ctas=tuned.get("ddp_reduce_ctas", 32))
        hook = make_grad_hook(model, world, average=False, skip=[table] if exchange is not None else [])
    step = TrainStep(model, lr=8.75e-4, clip=2.0, lam=1.0, grad_hook=hook, grad_prescale=1.0 / world,
                     table_exchange=exchange)

    pool_host = [to_pinned(b) for b in make_pool(args, rank, args.pool, args.batch)]
    pool_dev = [tuple(x.to(dev) for x in b) for b in pool_host]
    if args.feed == "packed":
        from nnue_pytorch_b200.batch_build import build_batch

        feed_host = make_packed_pool(args, rank, args.pool, args.batch)
    else:
        feed_host = pool_host
    h2d_bytes = sum(x.numel() * x.element_size() for x in feed_host[0])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host_ms = [0.0]
    # pinned landing slots for the loss and the copy stream exist before any timed region
    slots = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]
    done = [torch.cuda.Event(), torch.cuda.Event()]
    copy_stream = torch.cuda.Stream(dev)

    def timed(n_steps, resident: bool):
        """Returns (ms per step over this rank, last loss)."""
        from nnue_pytorch_b200.prefetch import DevicePrefetcher

        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        loss_host = 0.0
        e0.record()
        if resident:
            t_host = time.perf_counter()
            for i in range(n_steps):
                loss = step(pool_dev[i % len(pool_dev)])
            host_ms[0] = (time.perf_counter() - t_host) * 1e3 / n_steps  # host time to enqueue one step
        else:
            # every batch starts in pinned host memory inside the timed region: its copy runs on a side
            # stream while the previous step computes, and the loss is read back by the host every step
            host_iter = (feed_host[i % len(feed_host)] for i in range(n_steps))
            for i, batch in enumerate(DevicePrefetcher(host_iter, dev, copy_stream=copy_stream)):
                if args.feed == "packed":
                    batch = build_batch(batch[0], "baseline")  # index lists and targets written on the GPU
                loss = step(batch)
                slots[i % 2].copy_(loss.reshape(1), non_blocking=True)  # device -> host, every step
                done[i % 2].record()
                if i > 0:  # the host reads step i-1's loss while step i runs
                    done[(i - 1) % 2].synchronize()
                    loss_host = float(slots[(i - 1) % 2])
            done[(n_steps - 1) % 2].synchronize()
            loss_host = float(slots[(n_steps - 1) % 2])
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / n_steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms, (loss_host if not resident else float(loss))

    timed(max(args.warmup, 3), True)  # warm-up (also builds allocator pools, lazy attributes)

    launches0 = lib.nnue_b200_launch_count()
    _launch.TIMER = _launch.KernelTimer()
    with ClockSampler(local) as clocks:
        ms_resident, loss_val = timed(args.steps, True)
    spans = _launch.TIMER.summary()
    _launch.TIMER = None
    launches = (lib.nnue_b200_launch_count() - launches0) // max(args.steps, 1)
    timed(max(args.warmup, 3), False)  # warm-up of the end-to-end path (copy-stream allocations, pinned slots)
    ms_e2e, loss_e2e = timed(args.steps, False)
    _launch.device_status(dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak_gbs()
    fwd_ms = spans.get("fused_fwd", {}).get("mean_ms")
    bwd_ms = spans.get("fused_bwd", {}).get("mean_ms")
    opt_ms = spans.get("ranger_table", {}).get("mean_ms")
    fwd_bytes = algorithmic_bytes_fwd(args.batch, args.l1, MEAN_ACTIVE)
    bwd_bytes = algorithmic_bytes_bwd(args.batch, args.l1, MEAN_ACTIVE)
    fwd_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9 if fwd_ms else None
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9 if bwd_ms else None
    opt_gbs = 32.0 * N_ROWS * (args.l1 + 8) / (opt_ms * 1e-3) / 1e9 if opt_ms else None
    # dram__bytes_read.sum + dram__bytes_write.sum per launch of k_fused_fwd.  At the headline shape: measured by
    # ncu on this very workload (0.388 GB read + 0.562 GB written; profiles/ft_kernels_L3072_B4096_ncu_full.md has
    # the command).  Other batch sizes at L1 = 3072: scaled from it, the table read (<= 286 MB) does not grow with
    # the batch, the outputs do.
    traffic = None
    if args.l1 == 3072:
        table = N_ROWS * (args.l1 + 8) * 4
        traffic = 0.950316288e9 if args.batch == 16384 else table + (0.950316288e9 - table) * args.batch / 16384
    line = {
        "metric": METRIC,
        "value": world * args.batch / (ms_resident * 1e-3),
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": ms_resident,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": f"full training step: FT {N_ROWS}->{args.l1} x2 perspectives, 8 layer-stack buckets (L2=32, L3=32), "
                        f"RangerLite, clip 2.0, batch {args.batch}/GPU, HalfKAv2_hm^ real+factor indices (K=64)",
            "global_batch": world * args.batch,
            "l1": args.l1,
            "parallelism": f"dp{world}",
            "table_exchange": (args.ddp if world > 1 else "none"),
            "exchange_slices": (len(exchange.bounds) - 1) if exchange is not None else None,
            "backward": args.bwd_mode,
            "l2_policy": "working set per step (table 286 MB + gradient + moments + activations > 2 GB) exceeds the 126 MB L2; "
                         f"{args.pool} distinct batches cycled",
        },
        "e2e": {"value": world * args.batch / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "feed": args.feed},
        "gpu_launches": int(launches) * args.steps,
        "gpu_launches_per_step": int(launches),
        "host_enqueue_ms_per_step": round(host_ms[0], 3),
        "loss": loss_val,
        "clocks": clocks.summary(),
        "roofline": {
            "kernel": "k_fused_fwd (fused double-FT forward gather)",
            "bound": "hbm",
            "achieved": fwd_gbs,
            "peak": peak,
            "peak_source": f"{peak_kind} copy bandwidth",
            "unit": "GB/s",
            "frac": (fwd_gbs / peak) if fwd_gbs else None,
            "traffic": traffic,
            "algorithmic_bytes_per_launch": fwd_bytes,
            "ms_per_launch": fwd_ms,
        },
        "kernels": {
            "fused_fwd": {"ms": fwd_ms, "algorithmic_GBps": fwd_gbs, "frac": (fwd_gbs / peak) if fwd_gbs else None},
            "fused_bwd": {"ms": bwd_ms, "algorithmic_GBps": bwd_gbs, "frac": (bwd_gbs / peak) if bwd_gbs else None,
                          "note": "prologue + CSR build + segment gather-sum + bias column sum"},
            "ranger_table": {"ms": opt_ms, "GBps_at_32B_per_element": opt_gbs,
                             "frac": (opt_gbs / peak) if opt_gbs else None},
        },
        "spans_ms": {k: round(v["mean_ms"], 4) for k, v in sorted(spans.items())},
    }
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_reference_steps(args, steps=2, warmup=1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
def cpu_reference_steps(args, steps: int, warmup: int):
    """The CPU restatement of the reference's own path (oracle/: embedding-bag
    feature transformer, torch layer stacks, loss, autograd, RangerLite Python
    path) timed on this host's cores on a bounded sample of the workload."""
    from oracle import model_oracle, ranger_lite_oracle
    from nnue_pytorch_b200 import positions

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B = min(args.cpu_sample_batch, args.batch)
    g = torch.Generator().manual_seed(1)
    L1 = args.l1
    p = {
        "ft_weight": torch.randn(N_ROWS, L1 + 8, generator=g) * 0.01,
        "ft_bias": torch.randn(L1 + 8, generator=g) * 0.01,
        "l1_w": torch.randn(256, L1, generator=g) * 0.02, "l1_b": torch.zeros(256),
        "l1f_w": torch.zeros(32, L1), "l1f_b": torch.zeros(32),
        "l2_w": torch.randn(256, 64, generator=g) * 0.1, "l2_b": torch.zeros(256),
        "out_w": torch.randn(8, 128, generator=g) * 0.1, "out_b": torch.zeros(8),
    }
    order = list(p)
    state = ranger_lite_oracle.RangerLiteState([p[k] for k in order])
    times = []
    for i in range(warmup + steps):
        b = positions.generate_batch(B, 5000 + i, layout="baseline")
        batch = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in b.as_tuple())
        t0 = time.perf_counter()
        params = {k: v.requires_grad_(True) for k, v in p.items()}
        loss = model_oracle.training_loss(params, batch)
        grads = torch.autograd.grad(loss, [params[k] for k in order])
        total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(x) for x in grads]))
        coef = torch.clamp(2.0 / (total + 1e-6), max=1.0)
        for v in p.values():
            v.requires_grad_(False)
        ranger_lite_oracle.ranger_lite_step([p[k] for k in order], [x * coef for x in grads], state, lr=8.75e-4)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = statistics.median(times)
    return {
        "value": B / sec, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{warmup} warm-up + {steps} timed optimizer steps at batch {B} (the bench batch is {args.batch}), "
                  f"same model (L1={L1}), torch {torch.__version__} CPU ops, {cores} threads",
        "ms_per_step": sec * 1e3,
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 2))
    base = cpu_reference_steps(args, steps=steps, warmup=warm)
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": base["value"],
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": steps,
        "warmup": warm,
        "ms_per_step": base["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"full training step on host cores: FT {N_ROWS}->{args.l1} x2 perspectives, 8 layer-stack "
                               f"buckets, RangerLite, clip 2.0; bounded sample of batch {min(args.cpu_sample_batch, args.batch)}",
                   "l1": args.l1, "parallelism": "cpu"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_b200(a)
