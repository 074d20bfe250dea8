#!/usr/bin/env python
"""Benchmark of the sparse feature-transformer training step on B200.

    python bench.py --gpus N --steps K --warmup W            (this repository's arm)
    python bench.py --impl reference --steps K --warmup W     (CPU arm, host cores)
    python bench.py --workload sweep [--l1 ... --batch ... --active ...]   forward / backward kernel sweep
    python bench.py --workload step-native                    the same step in the reference's own table layout

Workload of the default run (the headline configuration): HalfKAv2_hm^ as one
table of 22528 real + 704 factor rows, feature transformer 23232 -> 3072 for
both perspectives, pairwise clipped product, eight layer-stack buckets, fp32,
batch 16384 per GPU, RangerLite, gradient-norm clip at 2.0, sigmoid-scaled
loss with lambda 1.0, synthetic positions (piece count ~ U[2,32]).  A step is
one forward + backward + optimizer update over one batch.

One JSON line is printed by rank 0.
  value       positions/s over exactly K steps with the batches resident in HBM, CUDA events, max over
              ranks, no per-call timers running; the host stays at most LOOKAHEAD steps ahead of the GPU.
  e2e         the same with every batch copied from pinned host memory on a side stream (one batch
              ahead) and the loss of every step copied back to the host, which reads it one step later.
              `--feed packed` (default): the host copy is the 72-byte packed position records and the
              index lists are written on the GPU inside the timed region; `--feed lists`: the expanded
              lists, as the reference's loader ships them.
  spans_ms / kernels / roofline   a separate pass with the per-call and per-kernel event timers on.
              `roofline` describes the kernel with the largest share of the step.  The gather kernels
              run out of the L2 (the table slice a column tile touches stays resident), so the bound
              is the L2 -> SM path: `peak` is measured in the same run by `nnue_l2_read_probe`.  The
              figure against the HBM copy peak (`hbm_algorithmic_frac`, embedding-bag accounting) and
              the DRAM utilisation from the recorded ncu traffic (`dram_frac`) stand beside it.
  sustained   a few seconds of back-to-back steps with the clock sampler running: the step time and
              SM clock the GPU settles at under its power limit.
  quant_eval  integer evaluation throughput of the same architecture (calls of one batch).
  exchange_check (N > 1)  untimed, after the timed loops: the fused table exchange against a plain
              all-reduce + full update from the same initial state (and against the same with the table
              gradient summed in rank order, which it must equal bit for bit), and whether all ranks hold
              the same table.
N > 1: `--slices auto|rows|cols|off` (overlap of the gradient reduce with the backward), `--rows-on-the-wire
int16|both|fp32` (what the sharded update stores into the other ranks), `--ddp fused|allreduce`.
"""

from __future__ import annotations

import argparse
import gc
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

LOOKAHEAD = 4  # steps the host may be ahead of the GPU in the resident-batch loop
METRIC = "training positions/sec at L1=3072"
UNIT = "positions/s"
N_ROWS = 23232
K_ACTIVE = 64
MEAN_ACTIVE = 34.0  # expected rows per perspective: 2 * E[k], k ~ U{2..32}

# dram__bytes_read.sum + dram__bytes_write.sum per launch at the headline shape (L1 = 3072, batch 16384), from
# ncu captures summarised under profiles/.  Recorded, not re-measured by a run of this file: the entry names
# the summary it comes from, and a kernel that changed since then has no entry.
RECORDED_DRAM_TRAFFIC = {
    "k_segment_chunks": (1.087e9, "profiles/train_step_L3072_B16384_dram_traffic.md"),
    "k_bwd_prologue": (0.955e9, "profiles/train_step_L3072_B16384_dram_traffic.md"),
    "k_ranger_rows": (2.350e9, "profiles/train_step_L3072_B16384_dram_traffic.md"),
    "k_fused_fwd_q16": (0.740e9, "profiles/train_step_L3072_B16384_dram_traffic.md"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="step", choices=["step", "sweep", "step-native"])
    ap.add_argument("--l1", type=int, nargs="*", default=None, help="L1 (step: one value, default 3072; sweep: a list)")
    ap.add_argument("--batch", type=int, nargs="*", default=None,
                    help="positions per GPU per step (step: one value, default 16384; sweep: a list)")
    ap.add_argument("--active", type=int, nargs="*", default=[2, 8, 16, 32],
                    help="sweep: real features per perspective (0 = piece count ~ U[2,32])")
    ap.add_argument("--features", default="halfka", choices=["halfka", "full"],
                    help="sweep: full = the table shape of the reference's default feature set (88944 rows, K = 288)")
    ap.add_argument("--skew", default="uniform", choices=["uniform", "zipf"],
                    help="sweep: zipf = king squares and piece placement drawn from a skewed distribution, so that "
                         "a few dozen rows collect a third of all entries, as real positions do")
    ap.add_argument("--no-flush", action="store_true", help="sweep: do not evict the L2 between launches")
    ap.add_argument("--pool", type=int, default=4, help="distinct synthetic batches cycled through")
    ap.add_argument("--bwd-mode", default="auto", choices=["auto", "atomic", "segment"])
    ap.add_argument("--cpu-sample-batch", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sustain-seconds", type=float, default=3.0, help="0 = skip the sustained block")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the timed loops: no spans pass, sustained block, L2 probe, quant_eval, exchange check")
    ap.add_argument("--tune", action="append", default=[], help="key=value, passed to nnue_b200_tune")
    ap.add_argument("--slices", default="auto", choices=["auto", "on", "rows", "cols", "off"],
                    help="fused exchange with the backward delivered in slices and the reduce of a slice overlapped "
                         "with the computation of the next: rows = two row slices (factor rows last), cols = "
                         "--col-slices column slices, on = rows, auto = rows from 4 GPUs (measured: 2 GPUs 2.69 ms "
                         "unsliced against 2.77 in column slices; 4 GPUs 2.76 unsliced, 2.72 rows, 2.78 columns; "
                         "8 GPUs 2.90 unsliced, 2.72 rows, 2.93 columns)")
    ap.add_argument("--col-slices", type=int, default=4, help="number of column slices of --slices cols")
    ap.add_argument("--clock-period-ms", type=int, default=50,
                    help="sampling period of nvidia-smi during the timed steps (every query takes a driver lock that "
                         "kernel launches wait for; measured per step at 20 ms 2.507 ms, at 100 ms 2.504)")
    ap.add_argument("--feed", default="packed", choices=["packed", "lists"],
                    help="what the end-to-end run copies from pinned host memory every step: 72-byte packed "
                         "positions expanded on the GPU, or the expanded index lists")
    ap.add_argument("--ddp", default="fused", choices=["fused", "allreduce"],
                    help="table exchange at N > 1: peer-memory reduce-scatter/update/all-gather kernels, or NCCL all-reduce")
    ap.add_argument("--rows-on-the-wire", default="int16", choices=["int16", "both", "fp32"],
                    help="what the fused exchange's update stores into the other ranks: the int16 / PSQT rows their "
                         "forward gathers (fp32 rows stay with their owner until sync_table), both, or the fp32 rows only")
    a = ap.parse_args()
    if a.workload != "sweep":
        a.l1 = (a.l1 or [3072])[0]
        a.batch = (a.batch or [16384])[0]
    return a


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs.

    nvidia-smi's start (it initialises the management library for every GPU of the machine) disturbs the process it
    watches for a moment, so the sampler is started BEFORE the warm-up steps; `window()` then marks the timed
    region, and only samples that arrived inside it are summarised."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 50):
        self.index, self.proc, self.lines, self.skip = index, None, [], 0
        self.period_ms = int(period_ms)
        self.t0, self.t1 = None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
            self.lines.append((time.time(), line.strip()))

    def window(self):
        """Context manager around the timed region: samples outside it are dropped from the summary."""
        sampler = self

        class _Window:
            def __enter__(self):
                sampler.t0 = time.time()

            def __exit__(self, *exc):
                sampler.t1 = time.time()

        return _Window()

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()  # exact child we started
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        kept = [ln for stamp, ln in self.lines[self.skip:]
                if not ((self.t0 is not None and stamp < self.t0) or (self.t1 is not None and stamp > self.t1))]
        if not kept:  # a timed region shorter than the sampling period: the samples of the warm-up steps before it
            kept = [ln for _, ln in self.lines[self.skip:]]
        for ln in kept:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power) if power else None}


# ---------------------------------------------------------------------------
def algorithmic_bytes_fwd(batch: int, l1: int, rows_per_persp: float, k_max: int = K_ACTIVE, table_bytes: int = 4) -> float:
    """Embedding-bag accounting: every (position, active row) counts a full row (`table_bytes` per L1 column:
    4 for the fp32 table, 2 for the int16 one; the one PSQT column a position reads stays fp32)."""
    row = l1 * table_bytes + (8 * 4 if table_bytes == 4 else 4)
    return batch * (2 * rows_per_persp * row + 2 * k_max * 4 + 24 + 3 * l1 * 4 + 8)


def algorithmic_bytes_bwd(batch: int, l1: int, rows_per_persp: float, n_rows: int = N_ROWS, k_max: int = K_ACTIVE) -> float:
    return algorithmic_bytes_fwd(batch, l1, rows_per_persp, k_max) + n_rows * (l1 + 8) * 4


def algorithmic_bytes_segment(batch: int, l1: int, rows_per_persp: float, n_rows: int = N_ROWS) -> float:
    """The segment gather-sum alone: one scratch-gradient row and one entry id per (position, perspective,
    active row), one write of the dense gradient."""
    W = l1 + 8
    return batch * 2 * rows_per_persp * (W * 4 + 4) + n_rows * W * 4


def make_pool(rank: int, n: int, batch: int):
    from nnue_pytorch_b200 import positions

    return [positions.generate_batch(batch, 1000 * rank + i, layout="baseline") for i in range(n)]


def make_packed_pool(rank: int, n: int, batch: int):
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


def build_model(l1: int, dev, feature: str = "HalfKAv2_hm^flat"):
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel

    torch.manual_seed(1)
    model = NNUEModel(feature, ModelConfig(L1=l1, L2=32, L3=32))
    with torch.no_grad():  # config: weights ~ N(0, 0.01) (standard deviation), PSQT columns keep their material init
        model.input.features[0].weight[:, :l1].normal_(0.0, 0.01)
    return model.to(dev)


def column_slices(l1: int, n_psqt: int, n: int) -> list[int]:
    """`n` column slices of the table's row (floats), on the backward's tile borders, tiles split evenly."""
    from nnue_pytorch_b200 import _launch

    w, tile = l1 + n_psqt, _launch.bwd_column_tile(l1, n_psqt)
    tiles = (w + tile - 1) // tile
    n = max(1, min(n, tiles))
    cuts = sorted({(tiles * i) // n for i in range(1, n)})
    return [0] + [c * tile for c in cuts if 0 < c * tile < w] + [w]


def build_step(model, world: int, ddp: str, slices, reduce_ctas: int, wire: str = "int16"):
    """(TrainStep, exchange or None) for `world` ranks."""
    from nnue_pytorch_b200.ddp import ShardedTableExchange, make_grad_hook
    from nnue_pytorch_b200.model import TrainStep

    hook = exchange = None
    if world > 1:
        table = model.input.features[0].weight
        if ddp == "fused":
            rows, cols = (slices or {}).get("rows"), (slices or {}).get("cols")
            exchange = ShardedTableExchange(table, slices=rows, col_slices=cols, reduce_ctas=reduce_ctas)
        hook = make_grad_hook(model, world, average=False, skip=[table] if exchange is not None else [])
    step = TrainStep(model, lr=8.75e-4, clip=2.0, lam=1.0, grad_hook=hook, grad_prescale=1.0 / world,
                     table_exchange=exchange, integer_rows={"int16": True, "both": "with_fp32", "fp32": False}[wire])
    return step, exchange


# ---------------------------------------------------------------------------
def exchange_check(args, dev, rank: int, world: int, bench_table: torch.Tensor, slices, reduce_ctas: int) -> dict:
    """Untimed correctness evidence for N > 1, at the benchmark's size: two optimizer steps of the fused
    exchange (peer-load reduce, sharded update, peer-store gather) against NCCL all-reduce + the full update on
    every rank, both from the same seeded state and on the same per-rank batches; and whether every rank holds
    the same table, both after those steps and in the table the timed loops left behind."""
    import torch.distributed as dist

    def agree(t: torch.Tensor) -> bool:
        other = t.detach().clone()
        dist.broadcast(other, src=0)
        flag = torch.tensor([0.0 if torch.equal(other, t.detach()) else 1.0], device=dev)
        dist.all_reduce(flag)
        return float(flag) == 0.0

    def rel(a, b):
        return float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)

    out = {"bench_table_ranks_agree": agree(bench_table)}
    batches = [tuple(torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in b.as_tuple())
               for b in make_pool(rank + 100, 2, args.batch)]
    ref = build_model(args.l1, dev)
    step_ref, _ = build_step(ref, world, "allreduce", None, reduce_ctas)
    losses_ref = [float(step_ref(b)) for b in batches]
    fused = build_model(args.l1, dev)
    step_fused, ex = build_step(fused, world, "fused", slices, reduce_ctas, args.rows_on_the_wire)
    losses = [float(step_fused(b)) for b in batches]
    ex.uninstall()

    # the same reference with the table gradient summed in RANK ORDER, ((g0 + g1) + g2) + ..., which is the order
    # of the peer-load reduce: fp32 sums of more than two terms depend on the order, NCCL's is its own
    from nnue_pytorch_b200.ddp import make_grad_hook
    from nnue_pytorch_b200.model import TrainStep

    ordered = build_model(args.l1, dev)
    o_table = ordered.input.features[0].weight
    dense_hook = make_grad_hook(ordered, world, average=False, skip=[o_table])

    def ordered_hook(model):
        dense_hook(model)
        parts = [torch.empty_like(o_table.grad) for _ in range(world)]
        dist.all_gather(parts, o_table.grad.contiguous())
        total = parts[0]
        for part in parts[1:]:
            total += part
        o_table.grad = total

    step_ordered = TrainStep(ordered, lr=8.75e-4, clip=2.0, lam=1.0, grad_hook=ordered_hook, grad_prescale=1.0 / world)
    for b in batches:
        step_ordered(b)
    t_ordered = o_table.detach()
    t_ref, t_fused = ref.input.features[0].weight.detach(), fused.input.features[0].weight.detach()
    small = max(rel(p.detach(), q.detach()) for (n, p), (_, q) in zip(fused.named_parameters(), ref.named_parameters())
                if "features" not in n)
    out.update({
        "ranks_agree": agree(t_fused),
        "table_rel_err": rel(t_fused, t_ref),
        "table_step_rel_err": None,
        "small_params_rel_err": small,
        "loss_rel_err": max(abs(a - b) / abs(b) for a, b in zip(losses, losses_ref)),
        "steps": len(batches),
        "reference": "NCCL all-reduce of the table gradient + full RangerLite update on every rank",
        "table_rel_err_vs_rank_ordered_sum": rel(fused.input.features[0].weight.detach(), t_ordered),
        "table_bitwise_equal_to_rank_ordered_sum": bool(torch.equal(fused.input.features[0].weight.detach(), t_ordered)),
    })
    init = build_model(args.l1, dev).input.features[0].weight.detach()
    d_ref, d_fused = t_ref - init, t_fused - init
    out["table_step_rel_err"] = float((d_fused - d_ref).abs().max()) / max(float(d_ref.abs().max()), 1e-30)
    return out


def quant_eval_block(model, args, dev) -> dict:
    """Integer evaluation of the benchmark's architecture: positions/s in calls of one batch (index lists
    resident on the device), CUDA events, after warm-up."""
    from nnue_pytorch_b200 import _launch, _lib
    from nnue_pytorch_b200.quantized_eval import QuantizedNet

    net = QuantizedNet.from_model(model)
    pool = make_pool(7, 4, args.batch)
    dev_pool = [(torch.from_numpy(b.white).to(dev), torch.from_numpy(b.black).to(dev),
                 torch.from_numpy(b.us[:, 0] > 0.5).to(dev), torch.from_numpy(b.piece_count).to(dev)) for b in pool]
    for i in range(4):
        net.evaluate(*dev_pool[i % 4])
    iters = 40
    _lib.profile(True)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        out = net.evaluate(*dev_pool[i % 4])
    b.record()
    b.synchronize()
    _lib.profile(False)
    prof = _lib.profile_summary()
    _launch.device_status(dev)
    ms = a.elapsed_time(b) / iters
    return {"value": args.batch / (ms * 1e-3), "unit": "positions/s", "ms_per_call": ms, "batch": args.batch,
            "dtype": "int16 table, int32 accumulation, int8 layers", "checksum": int(out.sum()),
            "kernels_ms": {k: round(v["mean_ms"], 4) for k, v in prof.items()}}


# ---------------------------------------------------------------------------
def run_step(args):
    import torch.distributed as dist

    from nnue_pytorch_b200 import _launch, _lib

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

    native = args.workload == "step-native"
    layout = "native" if native else "baseline"
    model = build_model(args.l1, dev, "HalfKAv2_hm^" if native else "HalfKAv2_hm^flat")
    n_rows = model.input.features[0].weight.shape[0]
    # --slices: the 704 factor rows (half of all entries) form the last slice, so the reduce of the
    # 22528 real rows can run while the factor rows' gradient is still being computed
    slices = None
    if world > 1 and args.ddp == "fused":
        kind = args.slices
        if kind == "auto":
            kind = "rows" if world >= 4 else "off"
        if kind == "on":
            kind = "rows"
        if kind == "rows" and not native:
            slices = {"rows": [0, n_rows - 704, n_rows]}
        elif kind == "cols":
            slices = {"cols": column_slices(args.l1, 8, args.col_slices)}
    # grid cap of the reduce that runs beside the sliced backward: few CTAs fill the links of 7 peers, 3 peers need more
    reduce_ctas = tuned.get("ddp_reduce_ctas", 32 if world >= 8 else 96)
    step, exchange = build_step(model, world, args.ddp, slices, reduce_ctas, args.rows_on_the_wire)

    from nnue_pytorch_b200 import positions

    pool_host = [to_pinned(positions.generate_batch(args.batch, 1000 * rank + i, layout=layout)) for i in range(args.pool)]
    pool_dev = [tuple(x.to(dev) for x in b) for b in pool_host]
    if args.feed == "packed":
        from nnue_pytorch_b200.batch_build import build_batch

        feed_host = make_packed_pool(rank, args.pool, args.batch)
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
        """Returns (ms per step, max over ranks; last loss)."""
        from nnue_pytorch_b200.prefetch import DevicePrefetcher

        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        loss_host = 0.0
        # a full collection of the interpreter's garbage (tens of milliseconds with this heap) inside the loop would
        # stall the host while the GPU's queue is still shallow: collect now, keep the collector off while timing
        gc.collect()
        gc.disable()
        e0.record()
        if resident:
            # the host enqueues a step in less time than the GPU runs it; it is kept at most LOOKAHEAD steps ahead
            # (as a training loop that looks at its loss now and then is), which keeps the allocator's pools and the
            # launch queue as they are after the warm-up instead of letting them grow for the length of the loop
            marks = [torch.cuda.Event() for _ in range(LOOKAHEAD)]
            t_host = time.perf_counter()
            for i in range(n_steps):
                if i >= LOOKAHEAD:
                    marks[i % LOOKAHEAD].synchronize()  # step i - LOOKAHEAD has finished
                loss = step(pool_dev[i % len(pool_dev)])
                marks[i % LOOKAHEAD].record()
            host_ms[0] = (time.perf_counter() - t_host) * 1e3 / n_steps  # host time per step, waits included
        else:
            # every batch starts in pinned host memory inside the timed region: its copy runs on a side
            # stream while the previous step computes, and the loss is read back by the host every step
            host_iter = (feed_host[i % len(feed_host)] for i in range(n_steps))
            for i, batch in enumerate(DevicePrefetcher(host_iter, dev, copy_stream=copy_stream)):
                if args.feed == "packed":
                    batch = build_batch(batch[0], layout)  # index lists and targets written on the GPU
                loss = step(batch)
                slots[i % 2].copy_(loss.reshape(1), non_blocking=True)  # device -> host, every step
                done[i % 2].record()
                if i > 0:  # the host reads step i-1's loss while step i runs
                    done[(i - 1) % 2].synchronize()
                    loss_host = float(slots[(i - 1) % 2])
            done[(n_steps - 1) % 2].synchronize()
            loss_host = float(slots[(n_steps - 1) % 2])
        e1.record()
        gc.enable()
        barrier()
        ms = e0.elapsed_time(e1) / n_steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms, (loss_host if not resident else float(loss))

    warm = max(args.warmup, 3)
    with ClockSampler(local, args.clock_period_ms) as clocks:  # started before the warm-up: its start-up is not part of the timed steps
        timed(warm, True)  # warm-up (also builds allocator pools, lazy attributes)
        launches0 = lib.nnue_b200_launch_count()
        with clocks.window():
            ms_resident, loss_val = timed(args.steps, True)
        launches = (lib.nnue_b200_launch_count() - launches0) // max(args.steps, 1)
    timed(warm, False)  # warm-up of the end-to-end path (copy-stream allocations, pinned slots)
    ms_e2e, loss_e2e = timed(args.steps, False)
    _launch.device_status(dev)

    extras = not args.no_extras
    spans, kprof = {}, {}
    if extras:
        # separate pass with the timers on: per C-ABI call (torch events around the call) and per kernel (the
        # library's own events around its main launches)
        _launch.TIMER = _launch.KernelTimer()
        _lib.profile(True)
        timed(min(args.steps, 20), True)
        _lib.profile(False)
        spans = _launch.TIMER.summary()
        _launch.TIMER = None
        kprof = _lib.profile_summary()

    sustained = None
    if extras and args.sustain_seconds > 0:
        n_sus = max(int(args.sustain_seconds * 1e3 / ms_resident), args.steps)
        with ClockSampler(local) as sus_clocks:
            ms_sus, _ = timed(n_sus, True)
        sustained = {"steps": n_sus, "ms_per_step": ms_sus, "value": world * args.batch / (ms_sus * 1e-3), "unit": UNIT,
                     "seconds": n_sus * ms_sus * 1e-3, "clocks": sus_clocks.summary()}

    check = None
    if exchange is not None:
        exchange.sync_table()  # the fp32 rows the other ranks own (they stay there when only integer rows travel)
    if extras and world > 1 and exchange is not None:
        check = exchange_check(args, dev, rank, world, model.input.features[0].weight, slices, reduce_ctas)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak_gbs()
    l2 = None
    if extras:
        seq = _launch.l2_read_probe(pattern=0, device=dev)
        rnd = _launch.l2_read_probe(pattern=1, device=dev)
        l2 = {"random_rows_gbs": rnd, "sequential_rows_gbs": seq,
              "how": "nnue_l2_read_probe: 1.14 GB read per launch from a 24 MB buffer (23232 rows x 1 KiB), 8 x 16-byte "
                     "loads in flight per lane, 20 launches after 2 warm-ups, CUDA events"}
    l2_peak = max(l2["random_rows_gbs"], l2["sequential_rows_gbs"]) if l2 else None

    rows_pp = MEAN_ACTIVE if not native else MEAN_ACTIVE / 2
    k_max = 32 if native else K_ACTIVE
    alg = {
        "k_fused_fwd": algorithmic_bytes_fwd(args.batch, args.l1, rows_pp, k_max),
        "k_fused_fwd_q16": algorithmic_bytes_fwd(args.batch, args.l1, rows_pp, k_max, table_bytes=2),
        "k_segment_chunks": algorithmic_bytes_segment(args.batch, args.l1, rows_pp, n_rows),
        "k_bwd_prologue": args.batch * (5 * args.l1 * 4 + 2 * (args.l1 + 8) * 4 + 24),
        "k_ranger_rows": 32.0 * n_rows * (args.l1 + 8),
    }
    bound_of = {"k_fused_fwd": "l2", "k_fused_fwd_q16": "l2", "k_segment_chunks": "l2", "k_bwd_prologue": "hbm", "k_ranger_rows": "hbm"}
    kernels = {}
    for name, rec in kprof.items():
        ms = rec["total_ms"] / max(min(args.steps, 20), 1)  # per step (a step may launch a kernel more than once)
        entry = {"ms_per_step": round(ms, 4), "launches_per_step": rec["launches"] / max(min(args.steps, 20), 1)}
        if name in alg and ms > 0:
            gbs = alg[name] / (ms * 1e-3) / 1e9
            entry.update({"algorithmic_bytes": alg[name], "algorithmic_GBps": gbs, "bound": bound_of[name],
                          "hbm_algorithmic_frac": gbs / peak})
            if l2_peak and bound_of[name] == "l2":
                entry["l2_frac"] = gbs / l2_peak
            if name in RECORDED_DRAM_TRAFFIC and args.l1 == 3072 and args.batch == 16384 and not native and not tuned:
                traffic, src = RECORDED_DRAM_TRAFFIC[name]
                entry.update({"dram_traffic": traffic, "dram_frac": traffic / (ms * 1e-3) / 1e9 / peak,
                              "traffic_source": src + " (recorded, not re-measured by this run)"})
        kernels[name] = entry
    roofline = None
    timed_kernels = {k: v for k, v in kernels.items() if "algorithmic_GBps" in v}
    if timed_kernels:
        top = max(timed_kernels, key=lambda k: timed_kernels[k]["ms_per_step"])
        e = timed_kernels[top]
        use_l2 = e["bound"] == "l2" and l2_peak
        roofline = {
            "kernel": top,
            "share_of_step": e["ms_per_step"] / ms_resident,
            "bound": "l2" if use_l2 else "hbm",
            "achieved": e["algorithmic_GBps"],
            "peak": l2_peak if use_l2 else peak,
            "peak_source": ("L2 -> SM read rate measured in this run (nnue_l2_read_probe)" if use_l2
                            else f"{peak_kind} copy bandwidth"),
            "unit": "GB/s",
            "frac": e["algorithmic_GBps"] / (l2_peak if use_l2 else peak),
            "hbm_peak": peak,
            "hbm_peak_source": f"{peak_kind} copy bandwidth",
            "hbm_algorithmic_frac": e["hbm_algorithmic_frac"],
            "traffic": e.get("dram_traffic"),
            "traffic_source": e.get("traffic_source"),
            "dram_frac": e.get("dram_frac"),
            "algorithmic_bytes_per_launch": e["algorithmic_bytes"],
            "ms_per_launch": e["ms_per_step"] / max(e["launches_per_step"], 1),
            "l2_probe": l2,
        }
    fwd_ms = spans.get("fused_fwd", {}).get("mean_ms")
    bwd_ms = spans.get("fused_bwd", {}).get("mean_ms")
    calls = {}
    if fwd_ms:
        int16 = "k_fused_fwd_q16" in kprof  # the forward gathered the int16 table: half the bytes per row
        g = algorithmic_bytes_fwd(args.batch, args.l1, rows_pp, k_max, 2 if int16 else 4) / (fwd_ms * 1e-3) / 1e9
        calls["fused_fwd"] = {"ms": fwd_ms, "algorithmic_GBps": g, "hbm_algorithmic_frac": g / peak,
                              "table": "int16" if int16 else "fp32"}
    if bwd_ms:
        g = algorithmic_bytes_bwd(args.batch, args.l1, rows_pp, n_rows, k_max) / (bwd_ms * 1e-3) / 1e9
        calls["fused_bwd"] = {"ms": bwd_ms, "algorithmic_GBps": g, "hbm_algorithmic_frac": g / peak,
                              "note": "one C-ABI call: prologue + CSR build + segment gather-sum + bias column sum"}
    line = {
        "metric": METRIC,
        "value": world * args.batch / (ms_resident * 1e-3),
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": warm,
        "ms_per_step": ms_resident,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": f"full training step: FT {n_rows}->{args.l1} x2 perspectives, 8 layer-stack buckets (L2=32, L3=32), "
                        f"RangerLite, clip 2.0, batch {args.batch}/GPU, "
                        + ("HalfKAv2_hm^ native layout (factor rows folded in weight space, K=32)" if native
                           else "HalfKAv2_hm^ real+factor indices (K=64)"),
            "global_batch": world * args.batch,
            "l1": args.l1,
            "parallelism": f"dp{world}",
            "table_exchange": (args.ddp if world > 1 else "none"),
            "exchange_slices": (None if exchange is None else
                                {"columns": exchange.col_bounds} if exchange.col_bounds is not None else
                                {"rows": exchange.bounds}),
            "rows_on_the_wire": (args.rows_on_the_wire if exchange is not None and getattr(exchange, "_emit", None) is not None
                                 else ("fp32" if exchange is not None else None)),
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
        "roofline": roofline,
        "kernels": kernels,
        "calls": calls,
        "spans_ms": {k: round(v["mean_ms"], 4) for k, v in sorted(spans.items())},
        "sustained": sustained,
    }
    if tuned:
        line["config"]["tune"] = tuned
    if check is not None:
        line["exchange_check"] = check
    if extras and world == 1 and not native:
        line["quant_eval"] = quant_eval_block(model, args, dev)
    if not args.no_cpu_baseline and world == 1 and not native:
        line["cpu_baseline"] = cpu_reference_steps(args, steps=2, warmup=1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# kernel sweep: forward and backward of the fused double feature transformer, separately
FULL_ROWS, FULL_K, FULL_MEAN = 88944, 288, 52  # the reference's default feature set (threats + pawn patterns + HalfKA)


def _full_feature_lists(batch: int, seed: int):
    """Stand-in lists with the default feature set's shape: 88944 rows, up to
    288 active per perspective, about 52 on average, rows uniform at random."""
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


def _time_launches(fn, iters, warmup, flush):
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


def sweep_point(l1, batch, active, mode, iters, warmup, flush, dev, features, skew):
    from nnue_pytorch_b200 import _launch, positions

    P = 8
    W = l1 + P
    n_rows, k_max = (N_ROWS, K_ACTIVE) if features == "halfka" else (FULL_ROWS, FULL_K)
    stats = None
    if features == "halfka":
        b = positions.generate_batch(batch, 0, layout="baseline", fixed_count=active if active else None,
                                     **({"skew": "zipf"} if skew == "zipf" else {}))
        rows_per_persp = 2.0 * (active if active else float(b.piece_count.mean()))
        arrays, piece_count = (b.us, b.them, b.white, b.black), b.piece_count
        hits = np.bincount(np.concatenate([b.white[b.white >= 0], b.black[b.black >= 0]]), minlength=n_rows)
        top = np.sort(hits[: positions.NUM_REAL_BASELINE])[::-1]
        stats = {"max_hits_real_row": int(top[0]), "top64_share_real_rows": float(top[:64].sum() / max(top.sum(), 1))}
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

    # the forward of the quantized model: the same operator on the int16 image of the fake-quantized table
    q16, psqt_tab, q_stats = _launch.quantize_blocks([(w, None)], l1, 256.0, 9600.0)
    bias_fq = torch.zeros_like(bias)
    _launch.prepare_table(bias[:l1].reshape(1, l1), None, l1, 256.0, 1.0, out=bias_fq, span="prepare_bias")

    def fwd16():
        _launch.fused_forward_q16(us, them, wi, bi, ps, q16, psqt_tab, bias_fq, q_stats, [(w, None)], 256.0, max_act, l1)

    t_f = _time_launches(fwd, iters, warmup, fl)
    t_f16 = _time_launches(fwd16, iters, warmup, fl)
    t_b = _time_launches(bwd, iters, warmup, fl)
    warm = None
    if flush:  # the steady-state figures as well: same launches back to back, nothing evicted in between
        warm = (_time_launches(fwd, iters, warmup, None), _time_launches(bwd, iters, warmup, None))
    _launch.device_status(dev)
    common = algorithmic_bytes_fwd(batch, l1, rows_per_persp, k_max)
    peak, kind = measured_peak_gbs()
    return {
        "l1": l1, "batch": batch, "active_real_per_perspective": active or "U[2,32]", "rows_per_perspective": rows_per_persp,
        "skew": skew, "list_stats": stats,
        "fwd_ms": t_f, "fwd_algorithmic_GBps": common / t_f / 1e6, "fwd_frac_of_hbm": common / t_f / 1e6 / peak,
        "fwd_int16_ms": t_f16,
        "fwd_int16_algorithmic_GBps": algorithmic_bytes_fwd(batch, l1, rows_per_persp, k_max, 2) / t_f16 / 1e6,
        "fwd_int16_frac_of_hbm": algorithmic_bytes_fwd(batch, l1, rows_per_persp, k_max, 2) / t_f16 / 1e6 / peak,
        "bwd_ms": t_b, "bwd_algorithmic_GBps": (common + n_rows * W * 4) / t_b / 1e6,
        "bwd_frac_of_hbm": (common + n_rows * W * 4) / t_b / 1e6 / peak,
        "rows": n_rows, "max_active": k_max,
        "fwd_ms_steady": warm[0] if warm else None, "bwd_ms_steady": warm[1] if warm else None,
        "bwd_mode": mode, "hbm_peak_GBps": peak, "peak_source": kind, "l2_flushed": bool(flush),
    }


def run_sweep(args):
    """BASELINE config 3: L1 x batch x active features; one JSON line per point.  Mean kernel time over
    `--steps` launches after `--warmup` (CUDA events on the launching stream): "cold" with the L2 flushed
    between launches (the headline figures) and "steady" back to back."""
    from nnue_pytorch_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the kernels")
    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.load()
    tuned = {}
    for kv in args.tune:
        k, v = kv.split("=")
        _lib.tune(k, int(v))
        tuned[k] = int(v)
    for l1 in (args.l1 or [1024, 2048, 3072]):
        for batch in (args.batch or [4096, 16384, 65536]):
            for act in (args.active if args.features == "halfka" else [0]):
                r = sweep_point(l1, batch, act, args.bwd_mode, args.steps, max(args.warmup, 3), not args.no_flush, dev,
                                args.features, args.skew)
                if tuned:
                    r["tune"] = tuned
                print(json.dumps(r), flush=True)
                torch.cuda.empty_cache()


# ---------------------------------------------------------------------------
def cpu_reference_steps(args, steps: int, warmup: int):
    """The reference's own path of the step on this host's cores, on a bounded sample of the workload.
    With the reference's `model/` tree present under oracle/_ref (see oracle/make_ref.py) this is the
    reference's `NNUEModel` forward, loss, autograd, `clip_grad_norm_` and `RangerLite.step`, unmodified
    (kind "reference"); otherwise the oracle's restatement of the same path (kind "port")."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B = min(args.cpu_sample_batch, args.batch)
    from oracle import ref_runner

    runner = ref_runner.make_cpu_step(args.l1, N_ROWS)
    from nnue_pytorch_b200 import positions

    times = []
    for i in range(warmup + steps):
        b = positions.generate_batch(B, 5000 + i, layout=runner.layout)
        batch = tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in b.as_tuple())
        t0 = time.perf_counter()
        runner.step(batch)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = statistics.median(times)
    return {
        "value": B / sec, "unit": UNIT, "cores": cores, "kind": runner.kind,
        "sample": f"{warmup} warm-up + {steps} timed optimizer steps at batch {B} (the bench batch is {args.batch}), "
                  f"{runner.describe}, torch {torch.__version__} CPU ops, {cores} threads",
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
    if torch.cuda.is_available():
        line["reference_gpu"] = ref_gpu_kernels(args)
    print(json.dumps(line), flush=True)


def ref_gpu_kernels(args) -> dict:
    """The reference's own CUDA kernels (its fused double-FT forward and backward) on this GPU at the
    benchmark's shape, compiled at run time from the sources under oracle/_ref through the NVRTC stand-in for
    CuPy that oracle/cupy_shim.py provides; or the reason why they could not be run."""
    try:
        from oracle import ref_runner

        return ref_runner.time_reference_gpu_kernels(args.l1, args.batch, N_ROWS)
    except Exception as e:  # noqa: BLE001 - reported, never fatal for the CPU arm
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.workload == "sweep":
        run_sweep(a)
    else:
        run_step(a)
