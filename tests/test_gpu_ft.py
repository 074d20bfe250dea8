"""GPU parity of the feature-transformer kernels against the CPU oracle and the
golden fixtures.  Everything goes through the C ABI (ctypes) by way of the
reference-shaped Python operators."""

import numpy as np
import pytest
import torch

from _util import load_golden, max_rel_err, t

pytestmark = pytest.mark.gpu

TOL = 1e-5  # relative to the tensor's max-norm, fp32 (the stated parity bar)


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from nnue_pytorch_b200 import _lib

    _lib.load()  # fail loudly if the library is missing
    return torch.device("cuda:0")


def _check(ours: torch.Tensor, ref32: torch.Tensor, ref64: torch.Tensor | None, what: str):
    ours = ours.detach().cpu()
    assert ours.shape == ref32.shape, what
    err = max_rel_err(ours, ref32)
    assert err <= TOL, f"{what}: max-norm relative error {err:.3e} > {TOL}"
    scale = max(float(ref32.abs().max()), 1e-30)
    assert torch.allclose(ours, ref32, rtol=1e-5, atol=1e-5 * scale), what
    if ref64 is not None:
        # kernel error vs float64 truth is no worse than the fp32 oracle's own
        e_ours = float((ours.double() - ref64).abs().max())
        e_ref = float((ref32.double() - ref64).abs().max())
        assert e_ours <= 2 * e_ref + 1e-7 * scale, f"{what}: {e_ours:.3e} vs oracle's own {e_ref:.3e}"


def _run_sparse(dev, idx, w, b, go, mode):
    from nnue_pytorch_b200 import SparseLinearFunction, _launch

    _launch.set_backward_mode(mode)
    try:
        wd = w.to(dev).requires_grad_(True)
        bd = b.to(dev).requires_grad_(True)
        out = SparseLinearFunction.apply(idx.to(dev), wd, bd)
        (out * go.to(dev)).sum().backward()
        _launch.device_status(dev)
        return out.detach(), wd.grad, bd.grad
    finally:
        _launch.set_backward_mode("auto")


@pytest.mark.parametrize("mode", ["segment", "atomic"])
def test_sparse_linear_golden(dev, mode):
    g = load_golden("sparse_linear")
    out, gw, gb = _run_sparse(dev, t(g["indices"]), t(g["weight"]), t(g["bias"]), t(g["grad_out"]), mode)
    _check(out, t(g["out"]), None, "out")
    _check(gw, t(g["grad_weight"]), None, "grad_weight")
    _check(gb, t(g["grad_bias"]), None, "grad_bias")


def test_sparse_linear_reference_test_shapes(dev):
    """The two cases of the reference's tests/test_feature_transformer.py: dense
    emulation with duplicate indices (tolerance 1e-4 there) and trailing padding."""
    from nnue_pytorch_b200 import SparseLinearFunction

    torch.manual_seed(0)
    w = torch.rand(10, 128)
    b = torch.rand(128)
    idx = (torch.rand(16, 32) * 10).to(torch.int32)
    counts = torch.zeros(16, 10)
    for i in range(16):
        for j in range(32):
            counts[i, idx[i, j]] += 1
    dense = torch.mm(counts, w) + b
    out = SparseLinearFunction.apply(idx.to(dev), w.to(dev), b.to(dev))
    assert float((out.cpu() - dense).abs().max()) < 1e-4
    torch.manual_seed(42)
    w = torch.rand(10, 64, device=dev)
    b = torch.rand(64, device=dev)
    act = (torch.rand(8, 5) * 10).to(torch.int32).to(dev)
    pad = torch.full((8, 3), -1, dtype=torch.int32, device=dev)
    a = SparseLinearFunction.apply(act, w, b)
    c = SparseLinearFunction.apply(torch.cat([act, pad], dim=1), w, b)
    assert torch.equal(a, c)


@pytest.mark.parametrize("B,N,K,W", [(1, 7, 1, 4), (37, 50, 9, 132), (300, 1000, 64, 1032), (64, 33, 40, 130), (5, 9, 3, 7)])
def test_sparse_linear_random_shapes(dev, B, N, K, W):
    from oracle import ft_oracle

    gen = torch.Generator().manual_seed(B * 1000 + W)
    idx = torch.randint(0, N, (B, K), generator=gen, dtype=torch.int32)
    n_act = torch.randint(0, K + 1, (B,), generator=gen)
    idx[torch.arange(K)[None, :] >= n_act[:, None]] = -1
    w = torch.randn(N, W, generator=gen) * 0.1
    b = torch.randn(W, generator=gen) * 0.1
    go = torch.randn(B, W, generator=gen)
    r32 = ft_oracle.sparse_linear_with_grads(idx, w, b, go)
    r64 = ft_oracle.sparse_linear_with_grads(idx, w.double(), b.double(), go.double())
    for mode in ("segment", "atomic"):
        out, gw, gb = _run_sparse(dev, idx, w, b, go, mode)
        _check(out, r32["out"], r64["out"], f"out[{mode}]")
        _check(gw, r32["grad_weight"], r64["grad_weight"], f"grad_weight[{mode}]")
        _check(gb, r32["grad_bias"], r64["grad_bias"], f"grad_bias[{mode}]")


def _run_fused(dev, c, mode, backend="fused"):
    from nnue_pytorch_b200 import _launch, double_feature_transform

    _launch.set_backward_mode(mode)
    try:
        wd = c["weight"].to(dev).requires_grad_(True)
        bd = c["bias"].to(dev).requires_grad_(True)
        l0, wp, bp = double_feature_transform(
            c["us"].to(dev), c["them"].to(dev), c["white"].to(dev), c["black"].to(dev), c["psqt"].to(dev),
            wd, bd, c["max_act"], c["l1"], backend)
        loss = (l0 * c["grad_l0"].to(dev)).sum() + (wp * c["grad_wpsqt"].to(dev)).sum() + (bp * c["grad_bpsqt"].to(dev)).sum()
        loss.backward()
        _launch.device_status(dev)
        return {"l0": l0.detach(), "wpsqt": wp.detach(), "bpsqt": bp.detach(), "grad_weight": wd.grad, "grad_bias": bd.grad}
    finally:
        _launch.set_backward_mode("auto")


def _golden_case(name):
    g = load_golden(name)
    c = {k: t(g[k]) for k in ("us", "them", "white", "black", "psqt", "weight", "bias", "grad_l0", "grad_wpsqt", "grad_bpsqt")}
    c["max_act"], c["l1"] = float(g["max_act"]), int(g["l1"])
    ref = {k: t(g[k]) for k in ("l0", "wpsqt", "bpsqt", "grad_weight", "grad_bias")}
    return c, ref


@pytest.mark.parametrize("name", ["fused_ft_randn", "fused_ft_stm"])
@pytest.mark.parametrize("mode", ["segment", "atomic"])
def test_fused_golden(dev, name, mode):
    c, ref = _golden_case(name)
    r = _run_fused(dev, c, mode)
    for k, v in ref.items():
        _check(r[k], v, None, f"{name}.{k}[{mode}]")


def _random_case(B, N, K, l1, P, seed, stm01=True, max_act=255.0 / 256.0, wscale=0.05, dup=True):
    gen = torch.Generator().manual_seed(seed)
    c = {}
    if stm01:
        c["us"] = torch.randint(0, 2, (B, 1), generator=gen).float()
        c["them"] = 1.0 - c["us"]
    else:
        c["us"] = torch.randn(B, 1, generator=gen)
        c["them"] = torch.randn(B, 1, generator=gen)
    for key in ("white", "black"):
        idx = torch.randint(0, N, (B, K), generator=gen, dtype=torch.int32)
        if not dup:
            idx = torch.stack([torch.randperm(N, generator=gen)[:K] for _ in range(B)]).to(torch.int32)
        n_act = torch.randint(0, K + 1, (B,), generator=gen)
        idx[torch.arange(K)[None, :] >= n_act[:, None]] = -1
        c[key] = idx
    c["psqt"] = torch.randint(0, max(P, 1), (B,), generator=gen, dtype=torch.int64)
    c["weight"] = torch.randn(N, l1 + P, generator=gen) * wscale
    c["bias"] = torch.randn(l1 + P, generator=gen) * wscale
    c["grad_l0"] = torch.randn(B, l1, generator=gen)
    c["grad_wpsqt"] = torch.randn(B, 1, generator=gen)
    c["grad_bpsqt"] = torch.randn(B, 1, generator=gen)
    c["max_act"], c["l1"] = max_act, l1
    return c


def _oracle(c, dtype):
    from oracle import ft_oracle

    f = lambda x: x.to(dtype)  # noqa: E731
    return ft_oracle.double_feature_transform_with_grads(
        f(c["us"]), f(c["them"]), c["white"], c["black"], c["psqt"], f(c["weight"]), f(c["bias"]),
        c["max_act"], c["l1"], f(c["grad_l0"]), f(c["grad_wpsqt"]), f(c["grad_bpsqt"]))


CASES = [
    # B, N, K, l1, P, stm01, max_act, wscale
    (4, 100, 32, 32, 8, False, 127.0, 1.0),       # reference test shape, l1 = 32
    (4, 100, 32, 2048, 8, False, 127.0, 1.0),     # reference test shape, l1 = 2048
    (13, 64, 5, 8, 4, True, 255.0 / 256.0, 0.3),  # one float4 per half, ragged batch
    (67, 500, 64, 512, 8, True, 255.0 / 256.0, 0.08),
    (40, 300, 33, 1024, 8, True, 255.0 / 256.0, 0.06),   # K not a multiple of 32
    (24, 200, 70, 3072, 8, True, 255.0 / 256.0, 0.04),   # K > 64, headline width
    (9, 50, 12, 6, 3, True, 255.0 / 256.0, 0.4),         # scalar kernels: l1 % 8 != 0, P % 4 != 0
    (48, 88944, 288, 256, 8, True, 255.0 / 256.0, 0.03),  # the default feature set's table: 88944 rows, K = 288
]


@pytest.mark.parametrize("case", CASES, ids=[f"B{c[0]}-N{c[1]}-K{c[2]}-L{c[3]}-P{c[4]}" for c in CASES])
def test_fused_random_shapes(dev, case):
    B, N, K, l1, P, stm01, max_act, wscale = case
    c = _random_case(B, N, K, l1, P, seed=l1 * 7 + B, stm01=stm01, max_act=max_act, wscale=wscale)
    r32, r64 = _oracle(c, torch.float32), _oracle(c, torch.float64)
    for mode in ("segment", "atomic"):
        r = _run_fused(dev, c, mode)
        for k in ("l0", "wpsqt", "bpsqt", "grad_weight", "grad_bias"):
            _check(r[k], r32[k], r64[k], f"{k}[{mode}]")


def test_fused_equals_sparse_composition(dev):
    """`backend="sparse"` (two sparse-linear kernels + torch glue) and the fused
    kernels agree, as the reference's tests/test_fused_double_ft.py checks."""
    c = _random_case(32, 400, 32, 256, 8, seed=5, stm01=False, max_act=127.0, wscale=0.5)
    a = _run_fused(dev, c, "segment", "fused")
    b = _run_fused(dev, c, "segment", "sparse")
    torch.testing.assert_close(a["l0"], b["l0"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(a["wpsqt"], b["wpsqt"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(a["grad_weight"], b["grad_weight"], atol=1e-4, rtol=1e-3)
    torch.testing.assert_close(a["grad_bias"], b["grad_bias"], atol=1e-4, rtol=1e-3)


def test_forward_is_bitwise_the_sequential_sum(dev):
    """bias first, then rows in list order: the accumulation order of the
    reference's CUDA kernels, reproduced bit for bit (0/1 side to move)."""
    c = _random_case(16, 300, 40, 64, 8, seed=77, dup=True)
    r = _run_fused(dev, c, "segment")
    W = c["weight"].numpy()
    bias = c["bias"].numpy()
    l1, h = 64, 32
    for p in range(16):
        acc = []
        for lst in (c["white"][p], c["black"][p]):
            a = bias.copy()
            for r_ in lst.tolist():
                if r_ < 0:
                    break
                a = (a + W[r_]).astype(np.float32)
            acc.append(a)
        first, second = (acc[0], acc[1]) if c["us"][p, 0] == 1 else (acc[1], acc[0])
        x = np.concatenate([first[:l1], second[:l1]])
        cl = np.clip(x, 0.0, np.float32(c["max_act"]))
        want = np.concatenate([cl[:h] * cl[h:l1], cl[l1:l1 + h] * cl[l1 + h:]]).astype(np.float32)
        assert np.array_equal(r["l0"][p].cpu().numpy(), want)
        pi = int(c["psqt"][p])
        assert float(r["wpsqt"][p, 0]) == float(acc[0][l1 + pi])
        assert float(r["bpsqt"][p, 0]) == float(acc[1][l1 + pi])


def test_config0_baseline_layout_parity(dev):
    """BASELINE configs[0]: HalfKAv2_hm^ as 22528 real + 704 factor rows,
    L1 = 1024, batch 1024, weights ~ N(0, 0.01), fp32."""
    from nnue_pytorch_b200 import positions

    b = positions.generate_batch(1024, 0, layout="baseline")
    gen = torch.Generator().manual_seed(1)
    L1, P = 1024, 8
    c = {
        "us": t(b.us), "them": t(b.them), "white": t(b.white), "black": t(b.black),
        "psqt": t((b.piece_count - 1) // 4),
        "weight": torch.randn(positions.NUM_INPUTS_BASELINE, L1 + P, generator=gen) * 0.01,
        "bias": torch.randn(L1 + P, generator=gen) * 0.01,
        "grad_l0": torch.randn(1024, L1, generator=gen), "grad_wpsqt": torch.randn(1024, 1, generator=gen),
        "grad_bpsqt": torch.randn(1024, 1, generator=gen), "max_act": 255.0 / 256.0, "l1": L1,
    }
    r32, r64 = _oracle(c, torch.float32), _oracle(c, torch.float64)
    for mode in ("segment", "atomic"):
        r = _run_fused(dev, c, mode)
        for k in ("l0", "wpsqt", "bpsqt", "grad_weight", "grad_bias"):
            _check(r[k], r32[k], r64[k], f"config0.{k}[{mode}]")


def test_segment_backward_is_reproducible(dev):
    """Two runs of the segment-reduce backward give identical bits, including
    rows that collect thousands of hits (factor rows)."""
    from nnue_pytorch_b200 import positions

    b = positions.generate_batch(4096, 3, layout="baseline")
    gen = torch.Generator().manual_seed(2)
    L1, P = 256, 8
    c = {
        "us": t(b.us), "them": t(b.them), "white": t(b.white), "black": t(b.black),
        "psqt": t((b.piece_count - 1) // 4),
        "weight": torch.randn(positions.NUM_INPUTS_BASELINE, L1 + P, generator=gen) * 0.02,
        "bias": torch.randn(L1 + P, generator=gen) * 0.02,
        "grad_l0": torch.randn(4096, L1, generator=gen), "grad_wpsqt": torch.randn(4096, 1, generator=gen),
        "grad_bpsqt": torch.randn(4096, 1, generator=gen), "max_act": 255.0 / 256.0, "l1": L1,
    }
    a = _run_fused(dev, c, "segment")
    for _ in range(2):
        b2 = _run_fused(dev, c, "segment")
        assert torch.equal(a["grad_weight"], b2["grad_weight"])
        assert torch.equal(a["grad_bias"], b2["grad_bias"])
    r32 = _oracle(c, torch.float32)
    _check(a["grad_weight"], r32["grad_weight"], None, "grad_weight")


def test_linearity_at_full_size(dev):
    """Size-independent property at the headline shape (L1 = 3072, batch
    16384, 23232 rows): the backward is linear in the incoming gradient, and
    the bias gradient equals the column sum identity sum_rows(gW[:, :L1]) ==
    sum over hits, checked through a scalar checksum."""
    from nnue_pytorch_b200 import _launch, double_feature_transform, positions

    B, L1, P = 16384, 3072, 8
    b = positions.generate_batch(B, 0, layout="baseline")
    gen = torch.Generator(device=dev).manual_seed(1)
    w = (torch.randn(positions.NUM_INPUTS_BASELINE, L1 + P, generator=gen, device=dev) * 0.01).requires_grad_(True)
    bias = (torch.randn(L1 + P, generator=gen, device=dev) * 0.01).requires_grad_(True)
    us, them, wi, bi = (t(x).to(dev) for x in (b.us, b.them, b.white, b.black))
    ps = t((b.piece_count - 1) // 4).to(dev)
    l0, wp, bp = double_feature_transform(us, them, wi, bi, ps, w, bias, 255.0 / 256.0, L1)
    g1 = torch.randn(B, L1, generator=gen, device=dev)
    g2 = torch.randn(B, L1, generator=gen, device=dev)
    z = torch.zeros(B, 1, device=dev)

    def grads(g):
        gw, gb = torch.autograd.grad([l0, wp, bp], [w, bias], [g, z, z], retain_graph=True)
        return gw, gb

    a, ab = grads(g1)
    b_, bb = grads(g2)
    s, sb = grads(g1 + g2)
    _launch.device_status(dev)
    scale = float(s.abs().max())
    assert float((a + b_ - s).abs().max()) <= 1e-5 * scale
    assert float((ab + bb - sb).abs().max()) <= 1e-5 * float(sb.abs().max())
    # every position contributes its gradient row once per active index: with n_w + n_b
    # active rows, sum over all table rows of gW[:, :L1] == sum_p (n_w(p) g_w(p) + n_b(p) g_b(p)).
    # Check the cheaper corollary on the PSQT block, which is exact to rounding:
    k = t(b.piece_count).to(dev).float()
    gp = torch.ones(B, 1, device=dev)
    gw_p, gb_p = torch.autograd.grad([l0, wp, bp], [w, bias], [torch.zeros_like(l0), gp, gp], retain_graph=False)
    assert abs(float(gw_p[:, L1:].sum()) - float((4 * k).sum())) <= 1e-3 * float((4 * k).sum())
    assert abs(float(gb_p[L1:].sum()) - 2 * B) <= 1e-3 * 2 * B


def test_bad_indices_are_skipped_not_dereferenced(dev):
    from nnue_pytorch_b200 import SparseLinearFunction, _launch, _lib

    w = torch.randn(10, 16, device=dev)
    b = torch.zeros(16, device=dev)
    idx = torch.tensor([[1, 2, 10_000_000, 3], [4, -1, 5, 6]], dtype=torch.int32, device=dev)
    _launch.device_status(dev)  # clear
    out = SparseLinearFunction.apply(idx, w, b)
    with pytest.raises(_lib.NnueB200Error):
        _launch.device_status(dev)
    _launch.device_status(dev)  # reading clears the word
    assert torch.allclose(out[0], w[1] + w[2] + w[3])
    assert torch.allclose(out[1], w[4])  # the first -1 ends the row


def test_prepare_table_matches_torch_composition(dev):
    """weight + virtual.repeat(32, 1), two fake quantizations and the concat of the
    reference module, against the one-pass kernel (bit for bit vs the CPU ops)."""
    from nnue_pytorch_b200.fused_ft_functions import PrepareTableFunction

    gen = torch.Generator().manual_seed(3)
    N, nv, L1, P = 768, 24, 40, 8
    w = torch.randn(N, L1 + P, generator=gen) * 0.3
    v = torch.randn(nv, L1 + P, generator=gen) * 0.1
    go = torch.randn(N, L1 + P, generator=gen)

    def ref(w, v, quant):
        m = w + v.repeat(N // nv, 1) if v is not None else w
        if not quant:
            return m
        fq = lambda x, s: x.mul(s).round().div(s)  # noqa: E731
        return torch.cat([fq(m[:, :L1], 256.0), fq(m[:, L1:], 9600.0)], dim=1)

    for virt, quant in ((v, True), (v, False), (None, True)):
        wd = w.to(dev).requires_grad_(True)
        vd = virt.to(dev).requires_grad_(True) if virt is not None else None
        out = PrepareTableFunction.apply(wd, vd, L1, 256.0 if quant else 0.0, 9600.0 if quant else 0.0)
        assert torch.equal(out.detach().cpu(), ref(w, virt, quant))
        out.backward(go.to(dev))
        assert torch.equal(wd.grad.cpu(), go)  # straight-through
        if virt is not None:
            want = go.view(N // nv, nv, -1).sum(0)
            assert max_rel_err(vd.grad.cpu(), want) <= 1e-6


def test_fused_epilogue_matches_separate_ops(dev):
    """Activation fake quantization and the correction factor inside the kernel
    equal the reference's separate tensor ops after the bare operator."""
    from nnue_pytorch_b200 import double_feature_transform
    from nnue_pytorch_b200.fused_ft_functions import FusedDoubleFtFunction

    c = _random_case(50, 300, 32, 128, 8, seed=9, wscale=0.1)
    for corr in (1.0, 0.75):
        outs = []
        for fused in (True, False):
            wd = c["weight"].to(dev).requires_grad_(True)
            bd = c["bias"].to(dev).requires_grad_(True)
            args = (c["us"].to(dev), c["them"].to(dev), c["white"].to(dev), c["black"].to(dev), c["psqt"].to(dev), wd, bd)
            if fused:
                l0, wp, bp = FusedDoubleFtFunction.apply(*args, c["max_act"], 128, 128.0, 1e-5, corr)
            else:
                l0, wp, bp = double_feature_transform(*args, c["max_act"], 128)
                hard = l0.mul(128.0).add(1e-5).floor().div(128.0)
                l0 = (hard.detach() + (l0 - l0.detach())) * corr
            ((l0 * c["grad_l0"].to(dev)).sum() + wp.sum()).backward()
            outs.append((l0.detach(), wd.grad, bd.grad))
        assert torch.equal(outs[0][0], outs[1][0])
        assert torch.equal(outs[0][1], outs[1][1])
        assert torch.equal(outs[0][2], outs[1][2])
        assert len(torch.unique(outs[0][0] * 128 / corr)) <= 129


@pytest.mark.parametrize("mode", ["segment", "atomic"])
@pytest.mark.parametrize("bounds", [[0, 23232], [0, 5000, 23232], [0, 7509, 15018, 22528, 23232], [0, 0, 1, 23231, 23232, 23232],
                                    ("cols", [0, 264]), ("cols", [0, 256, 264]), ("cols", [0, 0, 256, 256, 264, 264])])
def test_sliced_backward_is_bitwise_the_unsliced_one(dev, bounds, mode):
    """The gradient produced slice by slice (what the data-parallel exchange
    consumes while later slices are still computed) has the bits of the
    one-launch gradient, and every slice event is recorded by the call -- also
    on the atomic route, which finishes the whole gradient at once.  Slices are
    row ranges, or (marked "cols") column ranges on the gather-sum's tile borders."""
    by_columns = isinstance(bounds, tuple)
    if by_columns:
        bounds = bounds[1]
    from nnue_pytorch_b200 import _launch, positions

    b = positions.generate_batch(2048, 11, layout="baseline")
    c = {"us": t(b.us), "them": t(b.them), "white": t(b.white), "black": t(b.black),
         "psqt": t((b.piece_count - 1) // 4), "max_act": 255.0 / 256.0, "l1": 256}
    gen = torch.Generator().manual_seed(2)
    c["weight"] = torch.randn(positions.NUM_INPUTS_BASELINE, 264, generator=gen) * 0.05
    c["bias"] = torch.randn(264, generator=gen) * 0.05
    c["grad_l0"] = torch.randn(2048, 256, generator=gen)
    c["grad_wpsqt"] = torch.randn(2048, 1, generator=gen)
    c["grad_bpsqt"] = torch.randn(2048, 1, generator=gen)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in c.items()}
    _, _, _, saved = _launch.fused_forward(d["us"], d["them"], d["white"], d["black"], d["psqt"], d["weight"], d["bias"],
                                           c["max_act"], 256)

    def backward(slices, sink=None):
        return _launch.fused_backward(d["us"], d["them"], d["white"], d["black"], d["psqt"], c["max_act"], 256,
                                      positions.NUM_INPUTS_BASELINE, 264, d["grad_l0"], d["grad_wpsqt"], d["grad_bpsqt"],
                                      saved, mode=mode, slices=slices, sink=sink)

    ref_w, ref_b = backward(None)
    events = [torch.cuda.Event() for _ in range(len(bounds) - 1)]
    blocker = torch.cuda.Event()
    for e in events:
        e.record()  # a torch event has no CUDA handle until it is first recorded
    torch.cuda.synchronize()
    # keep the stream busy so that an event the call does NOT re-record would still read "done" from the
    # record above, while an event it does record stays pending until the work in front of it drains
    torch.cuda._sleep(200_000_000)
    sink = torch.full((positions.NUM_INPUTS_BASELINE, 264), float("nan"), device=dev)
    got_w, got_b = backward((bounds, events, by_columns), sink)
    assert not any(e.query() for e in events), "every slice event must be re-recorded behind the pending work"
    blocker.record()
    torch.cuda.synchronize()
    assert all(e.query() for e in events)
    assert got_w.data_ptr() == sink.data_ptr()
    if mode == "segment":
        assert torch.equal(got_w, ref_w) and torch.equal(got_b, ref_b)
    else:
        assert max_rel_err(got_w.cpu(), ref_w.cpu()) <= TOL and max_rel_err(got_b.cpu(), ref_b.cpu()) <= TOL


def test_column_slices_must_sit_on_tile_borders(dev):
    from nnue_pytorch_b200 import _launch, _lib

    assert _launch.bwd_column_tile(256, 8) == 256 and _launch.bwd_column_tile(3072, 8) == 256
    assert _launch.bwd_column_tile(255, 8) == 0  # the scalar route has no tiles
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=dev)  # noqa: E731
    ev = [torch.cuda.Event() for _ in range(2)]
    for e in ev:
        e.record()
    with pytest.raises(_lib.NnueB200Error, match="multiples of 256"):
        _launch.fused_backward(z(4, 1), z(4, 1), z(4, 8, dt=torch.int32), z(4, 8, dt=torch.int32), z(4, dt=torch.int64),
                               1.0, 256, 100, 264, z(4, 256), z(4, 1), z(4, 1), z(4, 4, 128), mode="segment",
                               slices=([0, 128, 264], ev, True))


def test_sliced_backward_records_events_for_an_empty_batch(dev):
    from nnue_pytorch_b200 import _launch

    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=dev)  # noqa: E731
    events = [torch.cuda.Event(), torch.cuda.Event()]
    for e in events:
        e.record()
    torch.cuda.synchronize()
    torch.cuda._sleep(100_000_000)
    gw, gb = _launch.fused_backward(z(0, 1), z(0, 1), z(0, 8, dt=torch.int32), z(0, 8, dt=torch.int32), z(0, dt=torch.int64),
                                    1.0, 16, 40, 24, z(0, 16), z(0, 1), z(0, 1), z(0, 4, 8), mode="segment",
                                    slices=([0, 10, 40], events))
    assert not any(e.query() for e in events)
    torch.cuda.synchronize()
    assert all(e.query() for e in events) and float(gw.abs().sum()) == 0.0 and float(gb.abs().sum()) == 0.0


def test_auto_mode_switches_to_atomics_on_nearly_empty_boards(dev):
    """mode=auto learns the density of the lists from its previous call (no
    synchronisation): dense boards stay on the segment route, boards with two
    pieces move to the atomic scatter within a few calls; the gradients
    agree with the segment route either way."""
    from nnue_pytorch_b200 import _lib, positions

    lib = _lib.load()

    def case(fixed):
        b = positions.generate_batch(3000, 5, layout="baseline", fixed_count=fixed)
        c = {"us": t(b.us), "them": t(b.them), "white": t(b.white), "black": t(b.black),
             "psqt": t((b.piece_count - 1) // 4), "max_act": 255.0 / 256.0, "l1": 256}
        gen = torch.Generator().manual_seed(2)
        c["weight"] = torch.randn(positions.NUM_INPUTS_BASELINE, 264, generator=gen) * 0.05
        c["bias"] = torch.randn(264, generator=gen) * 0.05
        c["grad_l0"] = torch.randn(3000, 256, generator=gen)
        c["grad_wpsqt"] = torch.randn(3000, 1, generator=gen)
        c["grad_bpsqt"] = torch.randn(3000, 1, generator=gen)
        return c

    def launches_of_auto(c):
        torch.cuda.synchronize()
        n0 = lib.nnue_b200_launch_count()
        r = _run_fused(dev, c, "auto")
        torch.cuda.synchronize()
        return lib.nnue_b200_launch_count() - n0, r

    sparse, dense = case(2), case(None)
    ref_sparse, ref_dense = _run_fused(dev, sparse, "segment"), _run_fused(dev, dense, "segment")
    launches_of_auto(dense)            # the probe of this call describes dense boards
    n_dense, r = launches_of_auto(dense)
    n_dense = max(n_dense, launches_of_auto(dense)[0])  # with or without the count kernel
    assert torch.equal(r["grad_weight"], ref_dense["grad_weight"])  # still the segment route, bit for bit
    for _ in range(4):                 # dense data are re-counted every fourth call: at most four calls late
        launches_of_auto(sparse)
    n_sparse, r = launches_of_auto(sparse)
    assert n_sparse < n_dense - 5, (n_sparse, n_dense)  # one scatter kernel instead of the CSR pipeline
    assert max_rel_err(r["grad_weight"].cpu(), ref_sparse["grad_weight"].cpu()) <= TOL
    assert max_rel_err(r["grad_bias"].cpu(), ref_sparse["grad_bias"].cpu()) <= TOL
    launches_of_auto(dense)
    n_again, r = launches_of_auto(dense)  # and back (sparse data are counted on every call)
    assert n_again >= n_dense - 1 and torch.equal(r["grad_weight"], ref_dense["grad_weight"])


def test_skewed_lists_with_rows_hit_thousands_of_times(dev):
    """Real positions concentrate a third of all entries on a few dozen rows; the skewed generator
    does the same (one real row collects more than 4096 entries in a batch of 8192).  Both scatter
    routes against the oracle, and the segment route bit for bit run to run: the long rows go
    through the per-row bitmap ordering of the CSR builder."""
    from nnue_pytorch_b200 import positions

    B, L1, P = 8192, 256, 8
    b = positions.generate_batch(B, 4, layout="baseline", skew="zipf")
    hits = np.bincount(np.concatenate([b.white[b.white >= 0], b.black[b.black >= 0]]),
                       minlength=positions.NUM_INPUTS_BASELINE)
    assert hits[: positions.NUM_REAL_BASELINE].max() > 4096
    gen = torch.Generator().manual_seed(2)
    c = {
        "us": t(b.us), "them": t(b.them), "white": t(b.white), "black": t(b.black),
        "psqt": t((b.piece_count - 1) // 4),
        "weight": torch.randn(positions.NUM_INPUTS_BASELINE, L1 + P, generator=gen) * 0.02,
        "bias": torch.randn(L1 + P, generator=gen) * 0.02,
        "grad_l0": torch.randn(B, L1, generator=gen), "grad_wpsqt": torch.randn(B, 1, generator=gen),
        "grad_bpsqt": torch.randn(B, 1, generator=gen), "max_act": 255.0 / 256.0, "l1": L1,
    }
    r32, r64 = _oracle(c, torch.float32), _oracle(c, torch.float64)
    a = _run_fused(dev, c, "segment")
    again = _run_fused(dev, c, "segment")
    assert torch.equal(a["grad_weight"], again["grad_weight"]) and torch.equal(a["grad_bias"], again["grad_bias"])
    for mode, r in (("segment", a), ("atomic", _run_fused(dev, c, "atomic"))):
        for k in ("l0", "wpsqt", "bpsqt", "grad_weight", "grad_bias"):
            # the float64 criterion compares summation quality with torch's pairwise sums; the atomic route adds
            # 12000 contributions to one address in arrival order, so it is held to the 1e-5 bar alone
            _check(r[k], r32[k], r64[k] if mode == "segment" or not k.startswith("grad") else None, f"zipf.{k}[{mode}]")


def test_row_named_twice_by_many_positions(dev):
    """The one documented exception to the ordered sums: a row that single positions name twice
    and that collects more than 4096 entries keeps its fill order (the per-row bitmap cannot
    hold duplicates and the shared-memory sort stops at 4096).  The sums are still right; only
    their order, hence the last bits, may differ between runs."""
    from nnue_pytorch_b200 import _launch

    B, N, K, L1, P = 3000, 500, 8, 64, 8
    c = _random_case(B, N, K, L1, P, seed=31, wscale=0.1)
    for key in ("white", "black"):
        c[key][:, 0] = 7
        c[key][:, 1] = 7        # every position names row 7 twice: 12000 entries, all duplicated
        c[key][:, 2:] = torch.where(c[key][:, 2:] == 7, torch.full_like(c[key][:, 2:], 8), c[key][:, 2:])
        c[key][::3, 4:] = -1
    r32, r64 = _oracle(c, torch.float32), _oracle(c, torch.float64)
    r = _run_fused(dev, c, "segment")
    for k in ("l0", "grad_weight", "grad_bias"):
        _check(r[k], r32[k], r64[k], f"dup.{k}")
    _launch.device_status(dev)


def _transformer_both_ways(dev, blocks, bias, c, l1, act=(128.0, 1e-5, 1.0)):
    """The feature transformer of one step through the int16 table (one autograd node over the raw
    parameters) and through the fp32 table (table preparation + bias preparation + operator);
    returns both result sets: outputs and the gradients of every parameter."""
    from nnue_pytorch_b200.fused_ft_functions import (FusedDoubleFtFunction, PrepareBiasFunction, PrepareTableFunction,
                                                      QuantizedFusedDoubleFtFunction)

    args = tuple(c[k].to(dev) for k in ("us", "them", "white", "black", "psqt"))
    res = []
    for integer in (True, False):
        ps = [(w.clone().to(dev).requires_grad_(True), None if v is None else v.clone().to(dev).requires_grad_(True))
              for w, v in blocks]
        bd = bias.clone().to(dev).requires_grad_(True)
        if integer:
            flat = [t_ for pair in ps for t_ in pair]
            l0, wp, bp = QuantizedFusedDoubleFtFunction.apply(*args, bd, c["max_act"], l1, *act, 256.0, 9600.0, None, *flat)
        else:
            tables = [PrepareTableFunction.apply(w, v, l1, 256.0, 9600.0) for w, v in ps]
            table = tables[0] if len(tables) == 1 else torch.cat(tables, dim=0)
            l0, wp, bp = FusedDoubleFtFunction.apply(*args, table, PrepareBiasFunction.apply(bd, l1, 256.0), c["max_act"],
                                                     l1, *act)
        torch.autograd.backward([l0, wp, bp], [c["grad_l0"].to(dev), c["grad_wpsqt"].to(dev), c["grad_bpsqt"].to(dev)])
        out = {"l0": l0.detach(), "wpsqt": wp.detach(), "bpsqt": bp.detach(), "bias.grad": bd.grad}
        for i, (w, v) in enumerate(ps):
            out[f"w{i}.grad"] = w.grad
            if v is not None:
                out[f"v{i}.grad"] = v.grad
        res.append(out)
    return res


Q16_CASES = [
    # B, blocks as (rows, factor rows or 0), K, l1
    (67, [(500, 0)], 64, 512),
    (40, [(768 * 4, 768)], 33, 1024),              # factor rows folded in weight space
    (24, [(200, 0)], 70, 3072),                    # headline width, K > 64
    (48, [(1200, 0), (96, 0), (768 * 2, 768)], 288, 256),  # three feature blocks, the default set's list length
    (9, [(64, 0)], 5, 16),                         # one 16-byte group per half
    (1, [(64, 32)], 1, 32),
]


@pytest.mark.parametrize("case", Q16_CASES, ids=[f"B{c[0]}-K{c[2]}-L{c[3]}-{len(c[1])}blk" for c in Q16_CASES])
def test_integer_table_forward_has_the_bits_of_the_fp32_forward(dev, case):
    """With fake-quantized weights the forward gathers an int16 table and sums in int32; nothing
    of the fp32 sum is ever rounded, so outputs (and, the backward being shared, gradients) are
    identical bit for bit; an oracle comparison of the same outputs rides along."""
    from oracle import ft_oracle

    B, blocks_spec, K, l1 = case
    P = 8
    n_total = sum(r for r, _ in blocks_spec)
    c = _random_case(B, n_total, K, l1, P, seed=l1 + B, wscale=0.05)
    gen = torch.Generator().manual_seed(5)
    blocks = [(torch.randn(r, l1 + P, generator=gen) * 0.2, torch.randn(nv, l1 + P, generator=gen) * 0.1 if nv else None)
              for r, nv in blocks_spec]
    bias = torch.randn(l1 + P, generator=gen) * 0.3
    a, b = _transformer_both_ways(dev, blocks, bias, c, l1)
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k
    # and against the oracle's restatement of the module (fold, two fake quantizations, operator, activation
    # fake quantization)
    fq = lambda x, s: x.mul(s).round().div(s)  # noqa: E731
    merged = torch.cat([w if v is None else w + v.repeat(w.shape[0] // v.shape[0], 1) for w, v in blocks])
    table = torch.cat([fq(merged[:, :l1], 256.0), fq(merged[:, l1:], 9600.0)], dim=1)
    bq = torch.cat([fq(bias[:l1], 256.0), torch.zeros(P)])
    l0, wp, bp = ft_oracle.double_feature_transform(c["us"], c["them"], c["white"], c["black"], c["psqt"], table, bq,
                                                    c["max_act"], l1)
    l0 = l0.mul(128.0).add(1e-5).floor().div(128.0)
    on_step = ((l0 - a["l0"].cpu()).abs() > 1e-6).float().mean()
    assert float(on_step) <= 2e-3  # floor() flips where an fp32 product lands within rounding of a step
    assert max_rel_err(a["wpsqt"].cpu(), wp) <= TOL and max_rel_err(a["bpsqt"].cpu(), bp) <= TOL


def test_integer_table_falls_back_when_a_weight_leaves_the_int16_range(dev):
    """An entry with |round(w * 256)| > 32767 (or such a bias) cannot live in the int16 table.  The
    emitting kernel tallies it on the device, and the forward then gathers the fp32 parameters with
    the fake quantization applied per element: same bits as the fp32 table, no host round trip."""
    B, K, l1, P = 50, 40, 256, 8
    c = _random_case(B, 600, K, l1, P, seed=3, wscale=0.05)
    gen = torch.Generator().manual_seed(6)
    for poke in ("weight", "factor", "bias", "split often", "beyond packed sums"):
        w = torch.randn(600, l1 + P, generator=gen) * 0.2
        v = torch.randn(100, l1 + P, generator=gen) * 0.1
        bias = torch.randn(l1 + P, generator=gen) * 0.3
        if poke == "weight":
            w[17, 5] = 200.0          # k = 51200
            w[300, 250] = -129.5
        elif poke == "factor":
            v[3, 100] = 150.0
        elif poke == "bias":
            bias[7] = -400.0
        elif poke == "split often":
            # |k| up to 3200: still the integer route, the pair sums are split every ten rows; rows that many
            # lists name carry the large values, with both signs in neighbouring columns
            w[:40, ::3] = 12.5
            w[:40, 1::3] = -12.25
            c["white"][:, 0] = torch.arange(B, dtype=torch.int32) % 40
            c["black"][:, :3] = torch.tensor([1, 2, 3], dtype=torch.int32)
        else:
            w[5, 9] = 20.0            # k = 5120: inside int16, beyond what the packed sums take
        a, b = _transformer_both_ways(dev, [(w, v)], bias, c, l1)
        for k in a:
            assert torch.equal(a[k], b[k]), (poke, k)
