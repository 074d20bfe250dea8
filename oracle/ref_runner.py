"""Runs the reference project's own code (the copy under oracle/_ref, see
oracle/make_ref.py) for the benchmarks' comparison legs.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): used by the CPU-baseline /
`--impl reference` legs of bench.py and by tests; never by the product.

  make_cpu_step(l1, n_rows)      one optimizer step on the host cores.  With oracle/_ref present:
                                 the reference's `NNUE` shell (model/nnue.py:72-182,296-364), its
                                 `train_step`, autograd, `clip_grad_norm_(2.0)` and the optimizer
                                 `configure_optimizers` builds (trainer/engine.py:295-322), unmodified,
                                 on its own table layout (24576 real rows, factor rows folded in weight
                                 space, lists of up to 32).  Without it: the oracle's restatement on the
                                 benchmark's flat table.
  time_reference_gpu_kernels()   the reference's CUDA kernels (fused double feature transformer,
                                 forward and backward), compiled from its sources through
                                 oracle/cupy_shim.py, timed at a benchmark shape.  Runs in a child
                                 process (`python -m oracle.ref_runner --gpu-kernels ...`).
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import time
from dataclasses import dataclass
from typing import Callable

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


def ref_available() -> bool:
    return os.path.isfile(os.path.join(REF_ROOT, "model", "nnue.py"))


def import_reference(with_cupy_shim: bool = False):
    """The reference's `model` package, imported from oracle/_ref."""
    if not ref_available():
        raise RuntimeError("oracle/_ref/model is absent: run `python oracle/make_ref.py /path/to/nnue-pytorch`")
    from . import ref_shims

    ref_shims.install()
    if with_cupy_shim:
        from . import cupy_shim

        cupy_shim.install()
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    import model  # noqa: PLC0415 - the reference package

    if not os.path.abspath(model.__file__).startswith(REF_ROOT):
        raise RuntimeError(f"`model` resolved to {model.__file__}, not to the copy under oracle/_ref")
    return model


@dataclass
class CpuStep:
    kind: str          # "reference" | "port"
    layout: str        # positions.generate_batch layout the step consumes
    describe: str
    step: Callable


def make_cpu_step(l1: int, n_rows: int) -> CpuStep:
    if ref_available():
        return _reference_cpu_step(l1)
    return _port_cpu_step(l1, n_rows)


def _reference_cpu_step(l1: int) -> CpuStep:
    import contextlib

    with contextlib.redirect_stdout(sys.stderr):  # the reference prints its optimizer choice; keep stdout for the caller
        model = import_reference()
        cfg = model.NNUELightningConfig(features="HalfKAv2_hm^", model_config=model.ModelConfig(L1=l1, L2=32, L3=32))
        torch.manual_seed(1)
        nnue = model.NNUE(cfg)
        with torch.no_grad():
            nnue.model.input.features[0].weight[:, :l1].normal_(0.0, 0.01)
        optimizers, _ = nnue.configure_optimizers()
    opt = optimizers[0]
    nnue.train()
    if hasattr(opt, "train"):
        opt.train()
    counter = [0]

    def step(batch):
        out = nnue.train_step(batch, 0, counter[0])
        opt.zero_grad(set_to_none=True)
        out["loss"].backward()
        torch.nn.utils.clip_grad_norm_(nnue.parameters(), 2.0)
        opt.step()
        counter[0] += 1
        return float(out["train_loss"])

    return CpuStep("reference", "native",
                   f"the reference's own NNUE.train_step + backward + clip_grad_norm_ + {type(opt).__name__}.step "
                   f"(oracle/_ref, HalfKAv2_hm^ in its native layout: 24576 rows + 768 factor rows folded in weight "
                   f"space, lists of up to 32, L1={l1})", step)


def _port_cpu_step(l1: int, n_rows: int) -> CpuStep:
    from . import model_oracle, ranger_lite_oracle

    g = torch.Generator().manual_seed(1)
    p = {
        "ft_weight": torch.randn(n_rows, l1 + 8, generator=g) * 0.01,
        "ft_bias": torch.randn(l1 + 8, generator=g) * 0.01,
        "l1_w": torch.randn(256, l1, generator=g) * 0.02, "l1_b": torch.zeros(256),
        "l1f_w": torch.zeros(32, l1), "l1f_b": torch.zeros(32),
        "l2_w": torch.randn(256, 64, generator=g) * 0.1, "l2_b": torch.zeros(256),
        "out_w": torch.randn(8, 128, generator=g) * 0.1, "out_b": torch.zeros(8),
    }
    order = list(p)
    state = ranger_lite_oracle.RangerLiteState([p[k] for k in order])

    def step(batch):
        params = {k: v.requires_grad_(True) for k, v in p.items()}
        loss = model_oracle.training_loss(params, batch)
        grads = torch.autograd.grad(loss, [params[k] for k in order])
        total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(x) for x in grads]))
        coef = torch.clamp(2.0 / (total + 1e-6), max=1.0)
        for v in p.values():
            v.requires_grad_(False)
        ranger_lite_oracle.ranger_lite_step([p[k] for k in order], [x * coef for x in grads], state, lr=8.75e-4)
        return float(loss)

    return CpuStep("port", "baseline",
                   f"the oracle's restatement of the reference's CPU path (embedding-bag feature transformer on the flat "
                   f"{n_rows}-row table, torch layer stacks, loss, autograd, RangerLite Python path; L1={l1})", step)


# ---------------------------------------------------------------------------
def time_reference_gpu_kernels(l1: int, batch: int, n_rows: int, iters: int = 10, timeout_s: int = 240) -> dict:
    """Child process: see `_gpu_kernels_main`.  Returns its JSON, or {"unavailable": reason}."""
    if not ref_available():
        return {"unavailable": "oracle/_ref is absent (python oracle/make_ref.py /path/to/nnue-pytorch)"}
    cmd = [sys.executable, "-m", "oracle.ref_runner", "--gpu-kernels", str(l1), str(batch), str(n_rows), str(iters)]
    try:
        r = subprocess.run(cmd, cwd=os.path.dirname(HERE), capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference kernels did not finish within {timeout_s} s"}
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or ["no output"]
    return {"unavailable": f"exit {r.returncode}: {tail[0][:300]}"}


def _gpu_kernels_main(l1: int, batch: int, n_rows: int, iters: int) -> dict:
    """Times the reference's `FusedDoubleFtFunction` (its CUDA kernels, its launch geometry: one block per
    position forward, one per four positions backward with scalar atomics) on the benchmark's lists and weights,
    and checks its outputs against this repository's kernels on the same inputs."""
    import numpy as np

    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    import_reference(with_cupy_shim=True)
    import importlib

    fused = importlib.import_module("model.modules.feature_transformer.fused_ft_functions")
    if not fused._HAS_CUPY_KERNELS:
        return {"unavailable": "the reference's kernel module did not import with the CuPy stand-in"}
    from nnue_pytorch_b200 import positions

    dev = torch.device("cuda:0")
    b = positions.generate_batch(batch, 0, layout="baseline")
    us, them, wi, bi = (torch.from_numpy(np.ascontiguousarray(x)).to(dev) for x in (b.us, b.them, b.white, b.black))
    ps = torch.from_numpy((b.piece_count - 1) // 4).to(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    w = (torch.randn(n_rows, l1 + 8, generator=g, device=dev) * 0.01).requires_grad_(True)
    bias = (torch.randn(l1 + 8, generator=g, device=dev) * 0.01).requires_grad_(True)
    gl0 = torch.randn(batch, l1, generator=g, device=dev)
    gp = torch.randn(batch, 1, generator=g, device=dev)
    max_act = 255.0 / 256.0

    def ev():
        return torch.cuda.Event(enable_timing=True)

    fwd_ms, bwd_ms = [], []
    out = None
    for i in range(iters + 2):
        w.grad = bias.grad = None
        a, m, z = ev(), ev(), ev()
        a.record()
        out = fused.FusedDoubleFtFunction.apply(us, them, wi, bi, ps, w, bias, max_act, l1)
        m.record()
        torch.autograd.backward(list(out), [gl0, gp, gp])
        z.record()
        z.synchronize()
        if i >= 2:
            fwd_ms.append(a.elapsed_time(m))
            bwd_ms.append(m.elapsed_time(z))
    ref_l0, ref_gw = out[0].detach(), w.grad.detach().clone()

    # this repository's kernels on the same tensors (closed-interval clamp gradient: differs from the reference
    # kernel only where a pre-activation is exactly 0 or the cap)
    from nnue_pytorch_b200 import double_feature_transform

    w2, b2 = w.detach().clone().requires_grad_(True), bias.detach().clone().requires_grad_(True)
    ours_f, ours_b = [], []
    for i in range(iters + 2):
        w2.grad = b2.grad = None
        a, m, z = ev(), ev(), ev()
        a.record()
        o = double_feature_transform(us, them, wi, bi, ps, w2, b2, max_act, l1)
        m.record()
        torch.autograd.backward(list(o), [gl0, gp, gp])
        z.record()
        z.synchronize()
        if i >= 2:
            ours_f.append(a.elapsed_time(m))
            ours_b.append(m.elapsed_time(z))
    rel = lambda x, y: float((x - y).abs().max()) / max(float(y.abs().max()), 1e-30)  # noqa: E731
    med = lambda v: sorted(v)[len(v) // 2]  # noqa: E731
    return {
        "fwd_ms": med(fwd_ms), "bwd_ms": med(bwd_ms),
        "this_repo_fwd_ms": med(ours_f), "this_repo_bwd_ms": med(ours_b),
        "l0_rel_diff": rel(o[0].detach(), ref_l0), "grad_weight_rel_diff": rel(w2.grad, ref_gw),
        "shape": {"batch": batch, "l1": l1, "rows": n_rows, "max_active": int(wi.shape[1])},
        "how": "the reference's FusedDoubleFtFunction (fused_ft_functions.py) with its kernel strings compiled by NVRTC "
               "through a RawKernel stand-in; CUDA events around the autograd forward and backward (the backward "
               f"includes its torch.zeros of the dense gradient), median of {iters} after 2 warm-ups",
    }


if __name__ == "__main__":
    if len(sys.argv) >= 6 and sys.argv[1] == "--gpu-kernels":
        t0 = time.time()
        try:
            res = _gpu_kernels_main(*(int(x) for x in sys.argv[2:6]))
        except Exception as e:  # noqa: BLE001 - the parent reports the reason
            res = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        res["seconds"] = round(time.time() - t0, 1)
        print(json.dumps(res))
    else:
        raise SystemExit("usage: python -m oracle.ref_runner --gpu-kernels L1 BATCH ROWS ITERS")
