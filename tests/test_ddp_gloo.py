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
