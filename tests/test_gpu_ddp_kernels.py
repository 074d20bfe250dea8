"""The peer-memory exchange kernels on ONE GPU: the "ranks" are separate
buffers of the same device, handed to the kernels through the same pointer
table they get across GPUs.  Covers every world-size variant of the reduce
kernel and the shard update + store-to-every-rank against the plain update."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from nnue_pytorch_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")


@pytest.mark.parametrize("world", [1, 2, 3, 4, 5, 8, 16])
def test_reduce_shard_sums_in_rank_order(dev, world):
    from nnue_pytorch_b200 import _launch
    from nnue_pytorch_b200.ddp import shard_ranges

    rows, width = 1003, 136
    gen = torch.Generator().manual_seed(world)
    orig = [torch.randn(rows * width, generator=gen).to(dev) for _ in range(world)]
    want = orig[0].clone()
    for g in orig[1:]:
        want = want + g  # rank order, one rounding per add: what the kernel does
    for bounds in ([0, rows], [0, 400, 400, rows]):
        bufs = [g.clone() for g in orig]
        ptrs = [b.data_ptr() for b in bufs]
        total = 0.0
        for rank in range(world):
            sumsq = torch.zeros(1, device=dev)
            for e0, e1 in shard_ranges(bounds, width, world, rank):
                _launch.ddp_reduce_shard(ptrs, rank, e0, e1, sumsq)
                assert torch.equal(bufs[rank][e0:e1], want[e0:e1])
            total += float(sumsq)
            # elements outside the rank's share are untouched
            mask = torch.ones(rows * width, dtype=torch.bool, device=dev)
            for e0, e1 in shard_ranges(bounds, width, world, rank):
                mask[e0:e1] = False
            assert torch.equal(bufs[rank][mask], orig[rank][mask])
        ref = float((want.double() ** 2).sum())
        assert abs(total - ref) <= 1e-5 * ref


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("step_no,merge", [(1, 0), (2, 0), (5, 1)])
def test_update_shard_equals_plain_update_and_reaches_every_table(dev, world, step_no, merge):
    from nnue_pytorch_b200 import _launch
    from nnue_pytorch_b200.ddp import shard_ranges

    rows, width = 515, 72
    n = rows * width
    gen = torch.Generator().manual_seed(7)
    p0, g0 = torch.randn(n, generator=gen).to(dev) * 0.1, torch.randn(n, generator=gen).to(dev) * 0.01
    gm0, ngm0 = torch.randn(n, generator=gen).to(dev) * 0.02, torch.randn(n, generator=gen).to(dev) * 0.02
    vm0, slow0 = torch.rand(n, generator=gen).to(dev) * 1e-3, torch.randn(n, generator=gen).to(dev) * 0.1
    hp = _launch.hparams_struct(
        beta2=0.999, one_minus_beta2=0.001, mom=0.81, one_minus_mom=0.19, one_plus_f=2.0, f=1.0,
        noise_norm_inv=5.0 ** -0.5, step_size=8.75e-4, bc2_sqrt=(1 - 0.999 ** step_no) ** 0.5, eps=1e-7, wd_keep=1.0,
        alpha=0.5, one_minus_alpha=0.5, use_pnm=1, step_is_odd=step_no % 2, do_merge=merge, phase=0)
    scale = torch.full((1,), 0.5, device=dev)
    ref = [x.clone() for x in (p0, g0, gm0, ngm0, vm0, slow0)]
    _launch.ranger_update(ref[0], ref[1], ref[2], ref[3], ref[4], ref[5], None, scale, hp)

    tables = [p0.clone() for _ in range(world)]
    ptrs = [t_.data_ptr() for t_ in tables]
    bounds = [0, 200, rows]
    for rank in range(world):
        for e0, e1 in shard_ranges(bounds, width, world, rank):
            if e1 == e0:
                continue
            gm, ngm, vm, slow = gm0[e0:e1].clone(), ngm0[e0:e1].clone(), vm0[e0:e1].clone(), slow0[e0:e1].clone()
            _launch.ddp_update_shard(ptrs, rank, e0, e1, g0, gm, ngm, vm, slow, scale, hp)
            for got, want in ((gm, ref[2]), (ngm, ref[3]), (vm, ref[4]), (slow, ref[5])):
                assert torch.equal(got, want[e0:e1])
    for t_ in tables:  # every "rank" now holds the fully updated table
        assert torch.equal(t_, ref[0])
