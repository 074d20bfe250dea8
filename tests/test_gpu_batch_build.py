"""Device-side batch construction: the lists the GPU writes from packed
positions are exactly the lists the host formula produces (positions.py, which
the golden fixture `halfka_indices.npz` pins to the reference's index formula)."""

import numpy as np
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


@pytest.mark.parametrize("layout", ["baseline", "native"])
@pytest.mark.parametrize("B,seed,fixed", [(1, 5, None), (1000, 0, None), (4096, 3, 32), (257, 9, 2)])
def test_build_equals_host_lists(dev, layout, B, seed, fixed):
    from nnue_pytorch_b200 import _launch, batch_build, positions

    pos = positions.generate_positions(B, seed, fixed)
    score, outcome = positions.generate_targets(B, seed)
    want = positions.generate_batch(B, seed, layout=layout, fixed_count=fixed)
    packed = batch_build.as_bytes(batch_build.pack_positions(pos, score, outcome)).to(dev)
    us, them, white, black, oc, sc, pc = batch_build.build_batch(packed, layout)
    _launch.device_status(dev)
    assert np.array_equal(white.cpu().numpy(), want.white)
    assert np.array_equal(black.cpu().numpy(), want.black)
    assert np.array_equal(us.cpu().numpy(), want.us) and np.array_equal(them.cpu().numpy(), want.them)
    assert np.array_equal(oc.cpu().numpy(), want.outcome)
    assert np.array_equal(sc.cpu().numpy(), np.rint(want.score))  # records hold whole centipawns
    assert np.array_equal(pc.cpu().numpy(), want.piece_count)


def test_wider_lists_are_padded(dev):
    from nnue_pytorch_b200 import batch_build, positions

    pos = positions.generate_positions(64, 1)
    score, outcome = positions.generate_targets(64, 1)
    packed = batch_build.as_bytes(batch_build.pack_positions(pos, score, outcome)).to(dev)
    _, _, white, _, _, _, _ = batch_build.build_batch(packed, "baseline", max_active=96)
    want = positions.baseline_indices(pos, True)
    assert np.array_equal(white[:, :64].cpu().numpy(), want)
    assert bool((white[:, 64:] == -1).all())


def test_malformed_records_are_counted_and_left_empty(dev):
    from nnue_pytorch_b200 import _launch, _lib, batch_build, positions

    pos = positions.generate_positions(8, 2)
    score, outcome = positions.generate_targets(8, 2)
    rec = batch_build.pack_positions(pos, score, outcome)
    rec["count"][1] = 1                      # too few pieces
    rec["count"][2] = 40                     # too many
    rec["piece"][3, 0] &= ~np.uint16(7 << 6)   # white king loses its type
    rec["piece"][4, 1] |= np.uint16(1 << 9)    # second white king, no black king
    packed = batch_build.as_bytes(rec).to(dev)
    _launch.device_status(dev)
    _, _, white, black, _, _, _ = batch_build.build_batch(packed, "baseline")
    with pytest.raises(_lib.NnueB200Error):
        _launch.device_status(dev)
    good = positions.baseline_indices(pos, True)
    for i in range(8):
        if i in (1, 2, 3, 4):
            assert bool((white[i] == -1).all()) and bool((black[i] == -1).all())
        else:
            assert np.array_equal(white[i].cpu().numpy(), good[i])


def test_empty_batch_and_bad_arguments(dev):
    from nnue_pytorch_b200 import _lib, batch_build

    out = batch_build.build_batch(torch.empty(0, 72, dtype=torch.uint8, device=dev), "native")
    assert out[2].shape == (0, 32)
    with pytest.raises(_lib.NnueB200Error):
        batch_build.build_batch(torch.zeros(4, 72, dtype=torch.uint8, device=dev), "baseline", max_active=32)
    with pytest.raises(_lib.NnueB200Error):
        batch_build.build_batch(torch.zeros(4, 72, dtype=torch.uint8), "baseline")


def test_prefetcher_delivers_every_batch_in_order(dev):
    """Side-stream staging: every batch arrives once, in order, with the bytes
    of its pinned source, also when the consumer overwrites its inputs and the
    source list is shorter than the pipeline depth."""
    from nnue_pytorch_b200.prefetch import DevicePrefetcher

    gen = torch.Generator().manual_seed(0)
    for n in (0, 1, 2, 7):
        host = [(torch.randint(0, 255, (4096, 72), generator=gen, dtype=torch.uint8).pin_memory(),
                 torch.randn(513, generator=gen).pin_memory()) for _ in range(n)]
        seen = 0
        for i, (a, b) in enumerate(DevicePrefetcher(iter(host), dev)):
            assert a.is_cuda and b.is_cuda
            big = torch.empty(1 << 24, device=dev).normal_()  # keep the compute stream busy
            assert torch.equal(a.cpu(), host[i][0]) and torch.equal(b.cpu(), host[i][1])
            a.zero_()
            b.zero_()
            del big
            seen += 1
        assert seen == n
