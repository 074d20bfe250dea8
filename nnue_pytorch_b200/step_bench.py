"""Time of one whole training step for either HalfKAv2_hm^ table layout.

    python -m nnue_pytorch_b200.step_bench --layout native --l1 3072 --batch 16384

"baseline": 22528 real + 704 factor rows in one table, the factor rows named
by the index lists (up to 64 active rows per list); the headline benchmark's
workload.  "native": the reference project's own layout
(model/modules/features/halfka_v2_hm.py:39-70): 24576 real rows gathered
through lists of up to 32, the 768 factor rows folded into them in weight
space before the gather (here by the table-preparation kernel) and their
gradient obtained by summing the real rows' gradient over the king buckets.
Same network, same optimizer, synthetic positions from the same generator;
prints one JSON line (CUDA events, batches resident on the device).
"""

from __future__ import annotations

import argparse
import json

import torch

from . import _launch, _lib, positions
from .model import ModelConfig, NNUEModel, TrainStep


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layout", default="native", choices=["native", "baseline"])
    ap.add_argument("--l1", type=int, default=3072)
    ap.add_argument("--batch", type=int, default=16384)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("step_bench needs a CUDA device")
    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.load()
    torch.manual_seed(1)
    name = "HalfKAv2_hm^" if a.layout == "native" else "HalfKAv2_hm^flat"
    model = NNUEModel(name, ModelConfig(L1=a.l1, L2=32, L3=32))
    with torch.no_grad():
        model.input.features[0].weight[:, : a.l1].normal_(0.0, 0.01)
    model.to(dev)
    step = TrainStep(model, lr=8.75e-4, clip=2.0, lam=1.0)
    pool = []
    for i in range(4):
        b = positions.generate_batch(a.batch, i, layout=a.layout)
        pool.append(tuple(torch.from_numpy(x).to(dev) for x in b.as_tuple()))
    for i in range(max(a.warmup, 3)):
        step(pool[i % 4])
    _launch.TIMER = _launch.KernelTimer()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(a.steps):
        loss = step(pool[i % 4])
    e1.record()
    torch.cuda.synchronize()
    spans = _launch.TIMER.summary()
    _launch.TIMER = None
    _launch.device_status(dev)
    ms = e0.elapsed_time(e1) / a.steps
    print(json.dumps({
        "layout": a.layout, "rows": model.input.features[0].weight.shape[0], "max_active": pool[0][2].shape[1],
        "l1": a.l1, "batch": a.batch, "ms_per_step": ms, "positions_per_s": a.batch / (ms * 1e-3),
        "loss": float(loss), "spans_ms": {k: round(v["mean_ms"], 4) for k, v in sorted(spans.items())},
    }))


if __name__ == "__main__":
    main()
