"""Data-parallel gradient exchange on CPU ranks (gloo, world size 2): the hook
`TrainStep` calls between backward and the optimizer must leave every rank
with the mean gradient, large tensors and the flat bucket of small ones alike."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, big, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nnue_pytorch_b200 import ddp

        ddp._BIG = big  # make one tensor take the "own all-reduce" route at test size
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(64, 48), torch.nn.Linear(48, 3))
        g = torch.Generator().manual_seed(100 + rank)
        for p in model.parameters():
            p.grad = torch.randn(p.shape, generator=g)
        model[1].bias.grad = None  # a parameter without gradient must be left alone
        hook = ddp.make_grad_hook(model, world)
        hook(model)
        torch.save([None if p.grad is None else p.grad.clone() for p in model.parameters()],
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_grad_hook_averages_over_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), 2000, str(tmp_path)), nprocs=world, join=True)
    got = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 48), torch.nn.Linear(48, 3))
    gens = [torch.Generator().manual_seed(100 + r) for r in range(world)]
    for i, p in enumerate(model.parameters()):
        per_rank = [torch.randn(p.shape, generator=g) for g in gens]
        if i == 3:
            assert got[0][i] is None and got[1][i] is None
            continue
        want = sum(per_rank) / world
        for r in range(world):
            assert torch.allclose(got[r][i], want, rtol=1e-6, atol=1e-7), (r, i)


def test_single_rank_needs_no_hook():
    from nnue_pytorch_b200 import ddp

    assert ddp.make_grad_hook(torch.nn.Linear(2, 2), 1) is None


def test_sliced_shares_tile_every_slice_exactly():
    """Every rank owns a part of every row slice; the parts are whole rows, disjoint,
    in rank order, and together cover the slice."""
    from nnue_pytorch_b200.ddp import shard_ranges

    width = 12
    for bounds in ([0, 23232], [0, 22528, 23232], [0, 7, 7, 10, 1001], [0, 3, 5]):
        for world in (1, 2, 3, 8):
            per_rank = [shard_ranges(bounds, width, world, r) for r in range(world)]
            for s, (b0, b1) in enumerate(zip(bounds[:-1], bounds[1:])):
                at = b0 * width
                for r in range(world):
                    e0, e1 = per_rank[r][s]
                    assert e0 == at and e1 >= e0 and e0 % width == 0 and e1 % width == 0
                    at = e1
                assert at == b1 * width


def _state_worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nnue_pytorch_b200.ddp import gather_sharded, scatter_full

        width = 12
        report = {}
        for bounds in ([0, 101], [0, 64, 101], [0, 7, 7, 10, 101], [0, 1]):
            full = torch.arange(bounds[-1] * width, dtype=torch.float32) * 0.5 + 3.0
            mine = scatter_full(full.view(bounds[-1], width), bounds, width, world, rank)
            back = gather_sharded(mine, bounds, width, dist.group.WORLD)
            report[str(bounds)] = (mine.numel(), bool(torch.equal(back, full)))
        torch.save(report, os.path.join(out_dir, f"state{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_sharded_optimizer_state_round_trip(tmp_path):
    """Checkpoint layout of the sharded table exchange: scattering a full-size state tensor into the
    per-rank shares (what `load_state_dict` does) and gathering it again (what `state_dict` does) is
    the identity, the shares partition the tensor, for one and several slices, ragged and empty ones."""
    for world in (2, 3):
        mp.spawn(_state_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
        reports = [torch.load(tmp_path / f"state{r}.pt") for r in range(world)]
        for key in reports[0]:
            rows = eval(key)[-1]  # noqa: S307 - the key is the bounds list this test wrote
            assert sum(rep[key][0] for rep in reports) == rows * 12, key
            assert all(rep[key][1] for rep in reports), key
