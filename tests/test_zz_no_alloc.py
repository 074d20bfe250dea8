"""The allocation-free sparse-linear backward (`nnue_ft_sparse_bwd_static`).

Some programs that embed this library may not allocate device memory when
they need the gradient (their own pool owns the device, or allocation is banned
after start-up), so they cannot hand over the workspace `nnue_ft_sparse_bwd`
asks for.  The variant carries
its scratch as a fixed 32 MiB array in the library image.  Here it is called
straight through the C ABI, twice in a row on different inputs, and compared
with the workspace-taking entry point; shapes beyond the array are refused.
The file name sorts last so that a run stopping at the first failure has
already been through every other test.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, K, N, W, dev):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, N, (B, K), generator=g, dtype=torch.int32)
    n_act = torch.randint(0, K + 1, (B,), generator=g)
    idx[torch.arange(K)[None, :] >= n_act[:, None]] = -1
    go = torch.randn(B, W, generator=g)
    return idx.to(dev), go.to(dev)


def _reference(lib, idx, go, N):
    B, K = idx.shape
    W = go.shape[1]
    gw = torch.empty(N, W, device=go.device)
    gb = torch.empty(W, device=go.device)
    nbytes = lib.nnue_ft_sparse_bwd_workspace_bytes(B, K, N, W, 2)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=go.device)
    st = lib.nnue_ft_sparse_bwd(idx.data_ptr(), go.data_ptr(), gw.data_ptr(), gb.data_ptr(), B, K, N, W,
                                ws.data_ptr(), nbytes, 2, torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.nnue_b200_last_error()
    return gw, gb


def test_static_scratch_backward_matches_workspace_backward():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from nnue_pytorch_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    # the set-up call: the first use on a device looks up the array's address, and with the CUDA runtime's lazy
    # module loading that is also the moment the 32 MiB array itself takes its place in device memory
    idx, go = _case(0, 8, 4, 16, 8, dev)
    gw0, gb0 = torch.empty(16, 8, device=dev), torch.empty(8, device=dev)
    assert lib.nnue_ft_sparse_bwd_static(idx.data_ptr(), go.data_ptr(), gw0.data_ptr(), gb0.data_ptr(), 8, 4, 16, 8,
                                         stream) == 0, lib.nnue_b200_last_error()
    torch.cuda.synchronize()
    # two calls in a row, the second on other data and another shape: whatever the first
    # left in the shared array must not leak into the second
    for seed, (B, K, N, W) in ((1, (700, 32, 3000, 264)), (2, (333, 17, 1200, 132))):
        idx, go = _case(seed, B, K, N, W, dev)
        want_w, want_b = _reference(lib, idx, go, N)
        gw = torch.full((N, W), float("nan"), device=dev)
        gb = torch.full((W,), float("nan"), device=dev)
        torch.cuda.synchronize()
        # the CUDA driver's own count of free device memory (torch's allocator statistics would not see an
        # allocation made inside the library); the helper stream and the array are in place by now
        free_before, _ = torch.cuda.mem_get_info(dev)
        st = lib.nnue_ft_sparse_bwd_static(idx.data_ptr(), go.data_ptr(), gw.data_ptr(), gb.data_ptr(),
                                           B, K, N, W, stream)
        assert st == 0, lib.nnue_b200_last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(dev)
        assert free_after == free_before, "the call changed the amount of free device memory"
        # both entry points take the same deterministic segment route: the bits agree
        assert torch.equal(gw, want_w) and torch.equal(gb, want_b)


def test_static_scratch_refuses_shapes_beyond_its_array():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from nnue_pytorch_b200 import _lib

    lib = _lib.load()
    B, K, N, W = 16384, 64, 23232, 3080
    assert lib.nnue_ft_sparse_bwd_workspace_bytes(B, K, N, W, 2) > (32 << 20)
    st = lib.nnue_ft_sparse_bwd_static(None, None, None, None, B, K, N, W, None)
    assert st == -3
    msg = lib.nnue_b200_last_error().decode()
    assert "built-in array" in msg and "nnue_ft_sparse_bwd" in msg
    _ = C
