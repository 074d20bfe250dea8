"""Check of the peer-memory table exchange (reduce-scatter + sharded RangerLite +
all-gather kernels, fp32 or integer rows on the wire) against the plain NCCL
all-reduce followed by the full optimizer step on every rank.  The one-rank case
runs the same kernels on a single device; the others need 2 and 4 CUDA devices
and report themselves as skipped on a smaller box."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from nnue_pytorch_b200 import _launch, positions
        from nnue_pytorch_b200.ddp import ShardedTableExchange, make_grad_hook
        from nnue_pytorch_b200.model import ModelConfig, NNUEModel, TrainStep

        def rel(a, b):
            return float((a - b).abs().max()) / max(float(b.abs().max()), 1e-30)

        def build(feature="HalfKAv2_hm^flat"):
            torch.manual_seed(0)
            m = NNUEModel(feature, ModelConfig(L1=128, L2=32, L3=32))
            with torch.no_grad():
                m.input.features[0].weight[:, :128].normal_(0, 0.05)
                m.layer_stacks.l1.linear.weight.normal_(0, 0.05)
            return m.to(dev)

        def make_batches(layout):
            out = []
            for i in range(6):
                b = positions.generate_batch(256, 50 + 10 * i + rank, layout=layout)
                out.append(tuple(torch.from_numpy(a).to(dev) for a in b.as_tuple()))
            return out

        # the reference's own table layout: factor rows are a separate parameter folded in weight space, so the
        # backward ALSO reads the table's gradient buffer (the bucket sum for the factor rows) while the sliced
        # exchange is already reducing it on its own stream
        native_batches = make_batches("native")
        nref = build("HalfKAv2_hm^")
        nstep = TrainStep(nref, clip=2.0, grad_hook=make_grad_hook(nref, world, average=False), grad_prescale=1.0 / world)
        nlosses = [float(nstep(b)) for b in native_batches]

        def run_native(slices):
            fused = build("HalfKAv2_hm^")
            f0 = fused.input.features[0]
            ex = ShardedTableExchange(f0.weight, slices=slices)
            step = TrainStep(fused, clip=2.0, grad_hook=make_grad_hook(fused, world, average=False, skip=[f0.weight]),
                             grad_prescale=1.0 / world, table_exchange=ex)
            losses = [float(step(b)) for b in native_batches]
            ex.uninstall()
            _launch.device_status(dev)
            return {
                "loss": max(abs(a - b) / abs(b) for a, b in zip(losses, nlosses)),
                "table": rel(f0.weight.detach(), nref.input.features[0].weight.detach()),
                "small": max(rel(p.detach(), q.detach()) for (n, p), (_, q) in
                             zip(fused.named_parameters(), nref.named_parameters()) if n != "input.features.0.weight"),
                "state": 0.0, "step": ex.step, "ranks_agree": True,
            }

        batches = make_batches("baseline")
        ref = build()
        step_ref = TrainStep(ref, clip=2.0, grad_hook=make_grad_hook(ref, world, average=False),
                             grad_prescale=1.0 / world)
        losses_ref = [float(step_ref(b)) for b in batches]
        ref_table = ref.input.features[0].weight.detach().clone()
        ref_state = {k: v.clone() for k, v in step_ref.optimizer.state[ref.input.features[0].weight].items()
                     if torch.is_tensor(v)}

        def run(slices, wire=True, cols=None):
            """`wire`: what the update stores into the other ranks (True: the int16 / PSQT rows of the table the
            forward gathers, "with_fp32": those and the fp32 rows, False: fp32 rows, quantized again by every rank)."""
            fused = build()
            table = fused.input.features[0].weight
            ex = ShardedTableExchange(table, slices=slices, col_slices=cols)
            step = TrainStep(fused, clip=2.0, grad_hook=make_grad_hook(fused, world, average=False, skip=[table]),
                             grad_prescale=1.0 / world, table_exchange=ex, integer_rows=wire)
            assert (ex._emit is not None) == bool(wire)
            losses = []
            for i, b in enumerate(batches):
                if i == 3 and wire:
                    # a write behind the exchange's back (every rank the same one, here one that changes no value):
                    # the integer rows are rebuilt from the owners' fp32 rows at the next forward
                    with torch.no_grad():
                        table.mul_(1.0)
                    fused.input.invalidate_integer_table()
                losses.append(float(step(b)))
            if wire is True and world > 1:
                assert not ex.fp32_rows_valid  # rows of other owners are stale here until the gather below
            ex.uninstall()
            assert ex.fp32_rows_valid
            _launch.device_status(dev)
            sd = ex.state_dict()
            # the checkpoint round trip: what state_dict gathered, load_state_dict scatters back to the same shares
            before = [t_.clone() for t_ in (ex.grad_ma, ex.variance_ma, ex.neg_grad_ma, ex.slow)]
            for t_ in (ex.grad_ma, ex.variance_ma, ex.neg_grad_ma, ex.slow):
                t_.fill_(float("nan"))
            ex.load_state_dict({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in sd.items()})
            assert all(torch.equal(a, b) for a, b in zip(before, (ex.grad_ma, ex.variance_ma, ex.neg_grad_ma, ex.slow)))
            rep = {
                "loss": max(abs(a - b) / abs(b) for a, b in zip(losses, losses_ref)),
                "table": rel(table.detach(), ref_table),
                "small": max(rel(p.detach(), q.detach()) for (n, p), (_, q) in
                             zip(fused.named_parameters(), ref.named_parameters()) if "features" not in n),
                "state": max(rel(sd[k], ref_state[k]) for k in ("grad_ma", "neg_grad_ma", "variance_ma", "lookahead_params")),
                "step": sd["step"],
            }
            # every rank must hold the same table after the all-gather
            mine = table.detach().clone()
            other = mine.clone()
            dist.broadcast(other, src=0)
            rep["ranks_agree"] = bool(torch.equal(mine, other))
            return rep

        n_rows = ref_table.shape[0]
        report = {
            "one_slice": run(None),
            "two_slices": run([0, n_rows - 704, n_rows]),           # factor rows last, reduce overlapped
            "four_slices": run([0, 9001, 9001, n_rows - 704, n_rows]),  # an empty slice and ragged shares
            "fp32_rows": run(None, wire=False),
            "both_rows": run([0, n_rows - 704, n_rows], wire="with_fp32"),
            "one_column_slice": run(None, cols=[0, 136]),
            "native_one_slice": run_native(None),
            "native_two_slices": run_native([0, 12288, 24576]),
        }
        # column slices sit on the gather-sum's tile borders: 128 floats with one float4 per lane, so the
        # 136-float rows of this small model split into two
        from nnue_pytorch_b200 import _lib

        _lib.tune("bwd_u", 1)
        try:
            assert _launch.bwd_column_tile(128, 8) == 128
            report["two_column_slices"] = run(None, cols=[0, 128, 136])
            report["column_slices_with_an_empty_one"] = run(None, cols=[0, 128, 128, 136], wire=False)
        finally:
            _lib.tune("bwd_u", 2)
        torch.save(report, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2, 4])
def test_sharded_table_exchange_matches_allreduce(tmp_path, world):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        report = torch.load(tmp_path / f"rank{r}.pt")
        for name, rep in report.items():
            assert rep["ranks_agree"], (name, rep)
            assert rep["step"] == 6
            assert rep["loss"] <= 1e-5, (name, rep)
            assert rep["table"] <= 1e-5 and rep["small"] <= 1e-5 and rep["state"] <= 1e-5, (name, rep)
