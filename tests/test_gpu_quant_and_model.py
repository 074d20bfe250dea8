"""GPU checks of the integer evaluation (bit-exact) and of the whole training
step around the feature transformer."""

import numpy as np
import pytest
import torch

from _util import load_golden, max_rel_err, small_model_params, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return torch.device("cuda:0")


def _net_from_params(p, L1, dev, buckets=8):
    from nnue_pytorch_b200.quantized_eval import QuantizedNet

    f = lambda a: t(np.asarray(a), torch.float64).to(dev)  # noqa: E731
    l1_w = f(p["l1_w"] + np.tile(p["l1f_w"], (buckets, 1)))
    l1_b = f(p["l1_b"] + np.tile(p["l1f_b"], buckets))
    return QuantizedNet(f(p["ft_weight"]), f(p["ft_bias"]), l1_w, l1_b, f(p["l2_w"]), f(p["l2_b"]),
                        f(p["out_w"]), f(p["out_b"]), L1, buckets)


def test_integer_eval_matches_reference_float64(dev):
    """The reference's float64 fake-quantized forward, x19200 and rounded,
    on the golden positions (native HalfKAv2_hm^ layout)."""
    from nnue_pytorch_b200 import positions

    g = load_golden("model_small")
    net = _net_from_params(small_model_params(), 64, dev)
    b = positions.generate_batch(96, 21, layout="native")
    out = net.evaluate(t(b.white).to(dev), t(b.black).to(dev), t(b.us[:, 0] > 0.5), t(b.piece_count))
    assert np.array_equal(out.cpu().numpy().astype(np.int64), g["eval_int"][:, 0])


def _random_quant_params(L1, N, gen, buckets=8, L2=32, L3=32, ft_range=24):
    p = {}
    w = gen.integers(-ft_range, ft_range + 1, (N, L1 + 8)) / 256.0
    w[:, L1:] = gen.integers(-2000, 2001, (N, 8)) / 9600.0
    p["ft_weight"] = w
    bias = np.zeros(L1 + 8)
    bias[:L1] = gen.integers(-60, 61, L1) / 256.0
    p["ft_bias"] = bias
    p["l1_w"] = gen.integers(-100, 101, (buckets * L2, L1)) / 128.0
    p["l1f_w"] = gen.integers(-27, 28, (L2, L1)) / 128.0
    p["l1_b"] = gen.integers(-9000, 9001, buckets * L2) / 16384.0
    p["l1f_b"] = gen.integers(-3000, 3001, L2) / 16384.0
    p["l2_w"] = gen.integers(-127, 128, (buckets * L3, 2 * L2)) / 64.0
    p["l2_b"] = gen.integers(-6000, 6001, buckets * L3) / 8192.0
    p["out_w"] = gen.integers(-127, 128, (buckets, 2 * L2 + 2 * L3)) / 128.0
    p["out_b"] = gen.integers(-9000, 9001, buckets) / 16384.0
    return p


@pytest.mark.parametrize("L1,layout,B,ft_range", [(1024, "baseline", 4096, 24), (3072, "baseline", 2048, 24),
                                                  (256, "native", 3000, 24), (512, "baseline", 3001, 4095),
                                                  (512, "baseline", 1000, 4096), (256, "native", 2000, 30000)])
def test_integer_eval_matches_integer_oracle(dev, L1, layout, B, ft_range):
    """The three forms of the evaluation (packed gather, plain tiled gather, one kernel) against the integer
    oracle.  Table entries up to 4095 in magnitude take the packed gather (pair sums split every 8 rows at that
    size); one entry beyond it and the net is served by the plain int16 gather."""
    from oracle import quant_oracle
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.quantize import QuantizationManager

    gen = np.random.default_rng(L1 + ft_range)
    N = positions.NUM_INPUTS_BASELINE if layout == "baseline" else positions.NUM_INPUTS_NATIVE
    p = _random_quant_params(L1, N, gen, ft_range=ft_range)
    if ft_range > 24:
        p["ft_weight"][0, 0] = ft_range / 256.0  # the bound itself occurs
    b = positions.generate_batch(B, 17, layout=layout)
    consts = QuantizationManager().integer_constants()
    want = quant_oracle.integer_eval(quant_oracle.quantize_params(p, L1), b.white, b.black, b.us[:, 0] > 0.5,
                                     (b.piece_count - 1) // 4, consts)
    net = _net_from_params(p, L1, dev)
    args = (t(b.white).to(dev), t(b.black).to(dev), t(b.us[:, 0] > 0.5), t(b.piece_count))
    assert (net.ft_w_packed is not None) == (ft_range <= 4095) and net.ft_max_abs == ft_range
    got = net.evaluate(*args)                    # packed gather (when the table allows it) + layer kernel
    plain = net.evaluate(*args, packed=False)    # gather on the plain int16 table + layer kernel
    single = net.evaluate(*args, tiled=False)    # one kernel per position
    assert np.array_equal(got.cpu().numpy().astype(np.int64), want)
    assert torch.equal(got, single) and torch.equal(got, plain)
    assert len(np.unique(want)) > B // 4  # the outputs are not degenerate


def test_integer_eval_with_a_non_default_scheme(dev):
    """Every constant of the integer evaluation derives from `QuantizationConfig`
    (model/quantize.py:58-73 of the reference).  A power-of-two scheme other than the default one --
    feature transformer at 128, layers at 64 / 32 / 64, hidden activations at 64 -- against the float64
    fake-quantized forward of the same scheme (the definition) and the integer oracle.  A scheme whose
    scales are not powers of two (the 127 of a literal "int16 at scale 127") has no exact integer form
    and is refused."""
    from oracle import model_oracle, quant_oracle
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.quantize import QuantizationConfig, QuantizationManager
    from nnue_pytorch_b200.quantized_eval import QuantizedNet

    cfg = QuantizationConfig(weight_scale_l1=64.0, weight_scale_l2=32.0, weight_scale_l_out=64.0, ft_quantized_one=128.0,
                             ft_quantized_max=127.0, hidden_quantized_one=64.0, hidden_quantized_max=63.0,
                             inference_l0_division_factor=256.0, inference_sqr_crelu_division_factor=64.0)
    qm = QuantizationManager(cfg)
    consts = qm.integer_constants()
    assert (consts["ft_shift"], consts["sqr_shift_l1"], consts["lin_shift_l1"], consts["sqr_shift_l2"],
            consts["lin_shift_l2"], consts["out_div"], consts["ft_max"], consts["hidden_max"]) == (8, 18, 6, 16, 5, 8192, 127, 63)
    L1, B, N = 256, 3000, positions.NUM_INPUTS_BASELINE
    gen = np.random.default_rng(9)
    p = {"ft_weight": gen.integers(-20, 21, (N, L1 + 8)) / 128.0, "l1_w": gen.integers(-60, 61, (256, L1)) / 64.0,
         "l1f_w": gen.integers(-3, 4, (32, L1)) / 64.0, "l1_b": gen.integers(-4000, 4001, 256) / 4096.0,
         "l1f_b": gen.integers(-500, 501, 32) / 4096.0, "l2_w": gen.integers(-63, 64, (256, 64)) / 32.0,
         "l2_b": gen.integers(-2000, 2001, 256) / 2048.0, "out_w": gen.integers(-63, 64, (8, 128)) / 64.0,
         "out_b": gen.integers(-4000, 4001, 8) / 4096.0}
    p["ft_weight"][:, L1:] = gen.integers(-2000, 2001, (N, 8)) / 9600.0
    p["ft_bias"] = np.concatenate([gen.integers(-40, 41, L1) / 128.0, np.zeros(8)])
    b = positions.generate_batch(B, 23, layout="baseline")
    f = lambda a: t(np.asarray(a), torch.float64).to(dev)  # noqa: E731
    net = QuantizedNet(f(p["ft_weight"]), f(p["ft_bias"]), f(p["l1_w"] + np.tile(p["l1f_w"], (8, 1))),
                       f(p["l1_b"] + np.tile(p["l1f_b"], 8)), f(p["l2_w"]), f(p["l2_b"]), f(p["out_w"]), f(p["out_b"]),
                       L1, 8, qm)
    got = net.evaluate(t(b.white).to(dev), t(b.black).to(dev), t(b.us[:, 0] > 0.5), t(b.piece_count))
    scales = {"ft": 128.0, "psqt": 9600.0, "l1": 64.0, "l2": 32.0, "out": 64.0, "hidden": 64.0}
    want = quant_oracle.integer_eval(quant_oracle.quantize_params(p, L1, scales), b.white, b.black, b.us[:, 0] > 0.5,
                                     (b.piece_count - 1) // 4, consts)
    assert np.array_equal(got.cpu().numpy().astype(np.int64), want)
    # the definition: float64 forward with this scheme's fake quantization, in units of 1 / (2 * 600 * 16)
    quant = model_oracle.Quant(ws_l1=64.0, ws_l2=32.0, ws_lout=64.0, ft_one=128.0, ft_max=127.0, hidden_one=64.0,
                               hidden_max=63.0, l0_div=256.0, sqr_div=64.0)
    p64 = {k: t(np.asarray(v), torch.float64) for k, v in p.items()}
    y = model_oracle.forward(p64, t(b.us).double(), t(b.them).double(), t(b.white), t(b.black), t(b.piece_count), quant)
    assert np.array_equal(torch.round(y[:, 0] * 19200.0).to(torch.int64).numpy(), want)
    assert len(np.unique(want)) > B // 4
    with pytest.raises(ValueError):  # correction factors other than 1, scales that are no powers of two
        QuantizationManager(QuantizationConfig(ft_quantized_one=127.0, ft_quantized_max=127.0)).integer_constants()
    with pytest.raises(ValueError, match="power of two"):
        QuantizationManager(QuantizationConfig(weight_scale_l2=48.0)).integer_constants()


def test_tiled_integer_eval_in_several_passes(dev):
    """A workspace smaller than the batch needs: the batch is walked in passes; same bits."""
    import ctypes as C

    from nnue_pytorch_b200 import _lib, positions

    L1, B = 256, 1000
    p = _random_quant_params(L1, positions.NUM_INPUTS_BASELINE, np.random.default_rng(3))
    net = _net_from_params(p, L1, dev)
    b = positions.generate_batch(B, 5, layout="baseline")
    white, black = t(b.white).to(dev), t(b.black).to(dev)
    stm = t(b.us[:, 0] > 0.5).to(device=dev, dtype=torch.uint8)
    bucket = ((t(b.piece_count) - 1) // 4).to(device=dev, dtype=torch.int32)
    want = net.evaluate(white, black, t(b.us[:, 0] > 0.5), t(b.piece_count), tiled=False)
    lib = _lib.load()
    for positions_per_pass in (1, 37, 160, 5000):
        ws = torch.empty(256 + positions_per_pass * (L1 + 4) + 255, dtype=torch.uint8, device=dev)
        out = torch.full((B,), -7, dtype=torch.int32, device=dev)
        st = lib.nnue_quant_eval_tiled(
            white.data_ptr(), black.data_ptr(), stm.data_ptr(), bucket.data_ptr(), net.ft_w.data_ptr(),
            net.ft_psqt.data_ptr(), net.ft_b.data_ptr(), net.l1_w.data_ptr(), net.l1_b.data_ptr(), net.l2_w.data_ptr(),
            net.l2_b.data_ptr(), net.out_w.data_ptr(), net.out_b.data_ptr(), out.data_ptr(), B, white.shape[1], net.N,
            L1, net.L2, net.L3, net.P, net.buckets, C.byref(net._qp), ws.data_ptr(), ws.numel(),
            torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(st, "nnue_quant_eval_tiled")
        assert torch.equal(out, want), positions_per_pass
    tiny = torch.empty(64, dtype=torch.uint8, device=dev)
    st = lib.nnue_quant_eval_tiled(
        white.data_ptr(), black.data_ptr(), stm.data_ptr(), bucket.data_ptr(), net.ft_w.data_ptr(),
        net.ft_psqt.data_ptr(), net.ft_b.data_ptr(), net.l1_w.data_ptr(), net.l1_b.data_ptr(), net.l2_w.data_ptr(),
        net.l2_b.data_ptr(), net.out_w.data_ptr(), net.out_b.data_ptr(), out.data_ptr(), B, white.shape[1], net.N,
        L1, net.L2, net.L3, net.P, net.buckets, C.byref(net._qp), tiny.data_ptr(), tiny.numel(),
        torch.cuda.current_stream(dev).cuda_stream)
    assert st == -3  # workspace too small


def test_quantization_refuses_out_of_range_weights(dev):
    p = _random_quant_params(64, 100, np.random.default_rng(0))
    p["l2_w"][0, 0] = 3.0  # 3.0 * 64 = 192 > 127
    with pytest.raises(RuntimeError, match="out of bounds"):
        _net_from_params(p, 64, dev)


def test_model_forward_and_gradients_match_oracle(dev):
    """Whole network (feature transformer kernels + torch layer stacks + loss)
    against the oracle on the golden model: same loss, same gradients."""
    from oracle import model_oracle
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.model import LossParams, ModelConfig, NNUEModel, sf_loss

    g = load_golden("model_small")
    p = small_model_params()
    m = NNUEModel("HalfKAv2_hm^", ModelConfig(L1=64, L2=32, L3=32))
    with torch.no_grad():
        f = m.input.features[0]
        f.weight.copy_(t(p["ft_real"], torch.float32))
        f.virtual_weight.copy_(t(p["ft_virtual"], torch.float32))
        m.input.bias.copy_(t(p["ft_bias"], torch.float32))
        ls = m.layer_stacks
        for mod, wk, bk in ((ls.l1.linear, "l1_w", "l1_b"), (ls.l1.factorized_linear, "l1f_w", "l1f_b"),
                            (ls.l2.linear, "l2_w", "l2_b"), (ls.output.linear, "out_w", "out_b")):
            mod.weight.copy_(t(p[wk], torch.float32))
            mod.bias.copy_(t(p[bk], torch.float32))
    m.to(dev)
    b = positions.generate_batch(96, 21, layout="native")
    us, them, white, black, outcome, score, pc = (t(a).to(dev) for a in b.as_tuple())
    y = m(us, them, white, black, pc, True, True)
    assert max_rel_err(y.detach().cpu(), t(g["scorenet32"])) <= 1e-5
    loss = sf_loss(y * 600.0, score, outcome, LossParams(), 1.0)
    loss.backward()
    assert abs(float(loss) - float(g["loss"])) <= 1e-5 * float(g["loss"])
    # float64 run of the same graph: tells the kernels' error from the fp32 reference's own rounding
    p64 = {k: t(np.asarray(v), torch.float64).requires_grad_(True) for k, v in p.items()
           if k not in ("ft_real", "ft_virtual")}
    cpu_batch = tuple(t(a) for a in b.as_tuple())
    cpu_batch = tuple(x.double() if x.is_floating_point() else x for x in cpu_batch)
    model_oracle.training_loss(p64, cpu_batch).backward()
    g64 = {"g_ft_weight": p64["ft_weight"].grad, "g_ft_virtual": p64["ft_weight"].grad.view(32, 768, -1).sum(0),
           "g_ft_bias": p64["ft_bias"].grad, "g_l1_w": p64["l1_w"].grad, "g_out_w": p64["out_w"].grad}
    f = m.input.features[0]
    for ours, key in ((f.weight.grad, "g_ft_weight"), (f.virtual_weight.grad, "g_ft_virtual"),
                      (m.input.bias.grad, "g_ft_bias"), (m.layer_stacks.l1.linear.weight.grad, "g_l1_w"),
                      (m.layer_stacks.output.linear.weight.grad, "g_out_w")):
        ref32, ref64 = t(g[key]), g64[key]
        if key == "g_ft_bias":
            ref64 = ref64.clone()
            ref64[64:] = 0  # the reference drops the PSQT part of the bias from the graph
        err = max_rel_err(ours.cpu(), ref32)
        scale = float(ref32.abs().max())
        e_ours = float((ours.cpu().double() - ref64).abs().max())
        e_ref = float((ref32.double() - ref64).abs().max())
        print(f"{key}: vs fp32 reference {err:.2e}; vs float64: ours {e_ours / scale:.2e}, fp32 reference {e_ref / scale:.2e}")
        # the bar is 1e-5 against the fp32 reference; where two fp32 evaluations of a sum this long differ by
        # more, the float64 run decides: ours may be no further from it than twice the reference's own error
        assert err <= 1e-5 or e_ours <= 2 * e_ref + 1e-7 * scale, key


def test_training_steps_track_the_oracle(dev):
    """Twenty optimizer steps (four lookahead merges) of the whole model on the
    baseline layout: the loss of every step and the parameters after 1, 5 and
    20 steps follow the CPU oracle (forward + autograd + RangerLite
    restatement), each within 1e-5 of the tensor's max-norm."""
    from oracle import model_oracle, ranger_lite_oracle
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel, TrainStep

    torch.manual_seed(0)
    m = NNUEModel("HalfKAv2_hm^flat", ModelConfig(L1=128, L2=32, L3=32))
    with torch.no_grad():
        m.input.features[0].weight[:, :128].normal_(0, 0.05)
        m.layer_stacks.l1.linear.weight.normal_(0, 0.05)
    names = {"ft_weight": m.input.features[0].weight, "ft_bias": m.input.bias,
             "l1f_w": m.layer_stacks.l1.factorized_linear.weight, "l1f_b": m.layer_stacks.l1.factorized_linear.bias,
             "l1_w": m.layer_stacks.l1.linear.weight, "l1_b": m.layer_stacks.l1.linear.bias,
             "l2_w": m.layer_stacks.l2.linear.weight, "l2_b": m.layer_stacks.l2.linear.bias,
             "out_w": m.layer_stacks.output.linear.weight, "out_b": m.layer_stacks.output.linear.bias}
    order = list(names)  # the trainer's ten groups, in its order
    cpu = {k: v.detach().clone() for k, v in names.items()}
    state = ranger_lite_oracle.RangerLiteState([cpu[k] for k in order])
    m.to(dev)
    step = TrainStep(m, lr=8.75e-4, clip=2.0)
    worst = {}
    for i in range(20):
        b = positions.generate_batch(512, 100 + i, layout="baseline")
        batch = tuple(t(a) for a in b.as_tuple())
        params = {k: v.clone().requires_grad_(True) for k, v in cpu.items()}
        loss_ref = model_oracle.training_loss(params, batch)
        loss_ref.backward()
        grads = [params[k].grad for k in order]
        total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(g_) for g_ in grads]))
        coef = torch.clamp(2.0 / (total + 1e-6), max=1.0)
        ranger_lite_oracle.ranger_lite_step([cpu[k] for k in order], [g_ * coef for g_ in grads], state, lr=8.75e-4)
        loss = step(tuple(x.to(dev) for x in batch))
        assert abs(float(loss) - float(loss_ref)) <= 1e-5 * abs(float(loss_ref)), i
        if i in (0, 4, 19):  # after 1, 5 and 20 optimizer steps (four lookahead merges by then)
            worst[i + 1] = max(max_rel_err(names[k].detach().cpu(), cpu[k]) for k in order)
    print("max-norm relative parameter error after 1 / 5 / 20 steps:", worst)
    assert all(v <= 1e-5 for v in worst.values()), worst  # measured on B200: 8.8e-6, 6.3e-6, 5.2e-6


@pytest.mark.parametrize("B,L1,fq", [(300, 64, True), (2000, 256, True), (777, 96, False), (5, 32, True),
                                     (1, 32, False), (4097, 3072, False), (4097, 3072, True)])
def test_fused_layer_stack_matches_oracle(dev, B, L1, fq):
    """Bucket-aware layer-stack kernels against the CPU oracle of the layer stacks (fp32 and
    float64): output, input gradient and every parameter gradient.

    With fake quantization on, an activation is floor(v * 128 + 1e-5) / 128.  The first-layer sums are
    exact in fp32 (inputs and quantized weights are small multiples of 1/128; the test's parameters
    sit on a 2^-12 grid so that the factor merge is exact too), but the SQUARE of a sum is rounded.
    Where the float64 value of v * 128 + 1e-5 lies within fp32 rounding distance of an integer without
    v * 128 being that integer exactly, an fp32 evaluation may land on either side of the step; the
    same holds for the rounding of the output.  Such positions are identified FROM THE FLOAT64 RUN
    (not from the disagreement), take no part in the gradient comparison (their cotangent is zeroed
    for every implementation) and are the only ones allowed to differ in the output."""
    from oracle import model_oracle
    from nnue_pytorch_b200.model import LayerStacks
    from nnue_pytorch_b200.quantize import QuantizationManager

    torch.manual_seed(B)
    ls = LayerStacks(8, L1, 32, 32, QuantizationManager())
    with torch.no_grad():
        for p in ls.parameters():
            p.add_(torch.randn_like(p) * 0.05)
            p.copy_((p * 4096).round() / 4096)
    x0 = (torch.rand(B, L1) * 0.9).div(1 / 128).floor().div(128)  # quantized activations in [0, 0.9]
    bucket = torch.randint(0, 8, (B,))
    if B > 100:
        bucket[bucket == 5] = 4  # an empty bucket
    if B == 777:
        bucket[:] = 6            # everything in one bucket
    gy = torch.randn(B, 1)
    keys = {"l1_w": ls.l1.linear.weight, "l1_b": ls.l1.linear.bias, "l1f_w": ls.l1.factorized_linear.weight,
            "l1f_b": ls.l1.factorized_linear.bias, "l2_w": ls.l2.linear.weight, "l2_b": ls.l2.linear.bias,
            "out_w": ls.output.linear.weight, "out_b": ls.output.linear.bias}

    def oracle(dtype, cot, trace=None):
        params = {k: v.detach().to(dtype).requires_grad_(True) for k, v in keys.items()}
        x = x0.detach().clone().to(dtype).requires_grad_(True)
        y = model_oracle.layer_stacks(params, x, bucket, model_oracle.Quant(), fq, fq, trace)
        y.backward(cot.to(dtype))
        return y.detach(), x.grad, {k: v.grad for k, v in params.items()}

    trace = {}
    y64, _, _ = oracle(torch.float64, gy, trace)
    on_step = torch.zeros(B, dtype=torch.bool)
    if fq:
        # distance of every value that enters a floor() to the nearest integer, within eight fp32 ulp of the
        # value (exact integers excepted: fp32 holds them exactly), and of the scaled output to the nearest
        # half-integer (its round())
        v = trace["pre_floor"]
        dist = ((v + model_oracle.EPS) - (v + model_oracle.EPS).round()).abs()
        near = dist < 8 * 2.0**-23 * v.abs().clamp(min=1.0)
        on_step = (near & (v != v.round())).any(dim=1)
        z = trace["pre_output"][:, 0] * 32768.0
        on_step |= ((z - z.floor()) - 0.5).abs() < 1e-4
    cot = gy * (~on_step).float()[:, None]
    y32, dx32, g32 = oracle(torch.float32, cot)
    y64, dx64, g64 = oracle(torch.float64, cot)

    ls.to(dev)
    ls.fused = True
    ls.zero_grad(set_to_none=True)
    x = x0.detach().clone().to(dev).requires_grad_(True)
    y = ls(x, bucket.to(dev), fq, fq)
    y.backward(cot.to(dev))
    ya, xa = y.detach().cpu(), x.grad.cpu()
    ga = {k: v.grad.cpu() for k, v in keys.items()}

    def parity(ours, r32, r64, what):
        scale = max(float(r32.abs().max()), 1e-30)
        err = float((ours.double() - r32.double()).abs().max()) / scale
        e_ours = float((ours.double() - r64).abs().max())
        e_ref = float((r32.double() - r64).abs().max())
        assert err <= 1e-5 or e_ours <= 2 * e_ref + 1e-7 * scale, (what, err, e_ours / scale, e_ref / scale)

    ok = ~on_step
    differing = int(((ya - y32).abs() > 1e-5 * max(float(y32.abs().max()), 1e-30))[:, 0].sum())
    print(f"B={B} L1={L1} fq={fq}: {int(on_step.sum())} positions on a quantization step, {differing} outputs differ")
    # the explanation must stay an exception: a few percent of the positions at most (squares of sums near the
    # clipping bound of 127 steps have an fp32 ulp of 1e-5 of a step, so wide layers flag more), and no more
    # outputs may differ than positions were flagged
    assert float(on_step.float().mean()) <= 0.05 and differing <= int(on_step.sum())
    if ok.any():
        parity(ya[ok], y32[ok], y64[ok], "y")
        parity(xa[ok], dx32[ok], dx64[ok], "dx")
    for k in keys:
        parity(ga[k], g32[k], g64[k], k)


def test_training_is_reproducible(dev):
    """Two runs of eight optimizer steps from the same seed: every loss and every
    parameter agree bit for bit (the reference's atomics make its runs differ)."""
    from nnue_pytorch_b200 import batch_build, positions
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel, TrainStep

    def run():
        torch.manual_seed(0)
        m = NNUEModel("HalfKAv2_hm^flat", ModelConfig(L1=256, L2=32, L3=32))
        with torch.no_grad():
            m.input.features[0].weight[:, :256].normal_(0, 0.05)
        m.to(dev)
        step = TrainStep(m, clip=2.0)
        losses = []
        for i in range(8):
            pos = positions.generate_positions(2048, 40 + i)
            score, outcome = positions.generate_targets(2048, 40 + i)
            packed = batch_build.as_bytes(batch_build.pack_positions(pos, score, outcome)).to(dev)
            losses.append(step(batch_build.build_batch(packed, "baseline")).clone())
        return torch.stack(losses), [p.detach().clone() for p in m.parameters()]

    la, pa = run()
    lb, pb = run()
    assert torch.equal(la, lb)
    for a, b in zip(pa, pb):
        assert torch.equal(a, b)


def test_kept_integer_table_follows_every_change_of_the_weights(dev):
    """The forward keeps the int16 table between steps and the optimizer kernel rewrites it; a model that
    quantizes the table afresh in every forward must stay bit-identical through optimizer steps (a lookahead
    merge among them), through an in-place change made with torch between two steps (weight clipping), through
    the optimizer's train / eval pointer swap and through a step of a different optimizer path."""
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel, TrainStep

    def build(keep):
        torch.manual_seed(0)
        m = NNUEModel("HalfKAv2_hm^flat", ModelConfig(L1=256, L2=32, L3=32))
        with torch.no_grad():
            m.input.features[0].weight[:, :256].normal_(0, 0.05)
        m.input.keep_integer_table = keep
        return m.to(dev)

    a, b = build(True), build(False)
    sa, sb = TrainStep(a, clip=2.0), TrainStep(b, clip=2.0)
    assert a.input.keep_integer_table and b.input.keep_integer_table  # TrainStep switches it on
    b.input.keep_integer_table = False
    batches = [tuple(t(x).to(dev) for x in positions.generate_batch(1024, 60 + i, layout="baseline").as_tuple())
               for i in range(9)]

    def same():
        for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
            assert torch.equal(p, q), n

    for i, batch in enumerate(batches):
        la, lb = sa(batch), sb(batch)
        assert torch.equal(la, lb), i
        same()
        if i == 2:  # what a trainer's weight clipping does between steps: a write through .data, then the notice
            for m in (a, b):
                m.input.features[0].weight.data.clamp_(-0.08, 0.08)
                m.input.invalidate_integer_table()
        if i == 3:  # an in-place change torch itself tracks needs no notice
            for m in (a, b):
                with torch.no_grad():
                    m.input.features[0].weight.mul_(1.01)
        if i == 5:  # evaluation in between: the slow weights take the parameters' place and go back
            for s_, m in ((sa, a), (sb, b)):
                s_.optimizer.eval()
                with torch.no_grad():
                    ya = m(*batch[:4], batch[6], True, True)
                s_.optimizer.train()
                m._eval_out = ya
            assert torch.equal(a._eval_out, b._eval_out)
        if i == 7:  # a raw-pointer update that does not rewrite the table: the cache must notice
            for s_ in (sa, sb):
                s_.optimizer.touched_rows_only = False
    cache = a.input._q16_cache
    assert cache.q16 is not None and b.input._table_cache() is None


@pytest.mark.parametrize("B,L1", [(300, 64), (4097, 3072), (16384, 1024), (1, 32)])
def test_tensor_core_first_layer_has_the_bits_of_the_fma_kernel(dev, B, L1):
    """The quantized model's first layer-stack layer runs as tcgen05.mma (TF32 inputs, fp32 accumulation in
    tensor memory).  Activations on the 1/128 grid and fake-quantized weights are exact in TF32 and their
    partial sums exact in fp32, so the output equals the fp32 FMA kernel's bit for bit."""
    import ctypes as C  # noqa: F401

    from nnue_pytorch_b200 import _launch, _lib

    lib = _lib.load()
    gen = torch.Generator().manual_seed(B + L1)
    count = 8
    x = (torch.randint(0, 128, (B, L1), generator=gen).float() / 128.0).to(dev)
    x[x > 0.6] = 0.0  # sparse like the clipped products are
    W1 = (torch.randint(-127, 128, (count * 32, L1), generator=gen).float() / 128.0).to(dev)
    b1 = (torch.randint(-9000, 9001, (count * 32,), generator=gen).float() / 16384.0).to(dev)
    bucket = torch.randint(0, count, (B,), generator=gen).to(dev)
    if B > 100:
        bucket[bucket == 3] = 2  # an empty bucket
    plan = torch.empty(lib.nnue_ls_plan_bytes(B, count) // 4 + 4, dtype=torch.int32, device=dev)
    s = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(lib.nnue_ls_plan(bucket.data_ptr(), B, count, plan.data_ptr(), plan.numel() * 4, s), "nnue_ls_plan")
    outs = []
    for fn in (lib.nnue_ls_l1_fwd, lib.nnue_ls_l1_fwd_tc):
        o1 = torch.full((B, 32), float("nan"), device=dev)
        _lib.check(fn(x.data_ptr(), W1.data_ptr(), b1.data_ptr(), plan.data_ptr(), o1.data_ptr(), B, L1, count, s), "l1 fwd")
        outs.append(o1)
    _launch.device_status(dev)  # a bounded wait that ran out would show here
    want = torch.einsum("bk,bok->bo", x.double().cpu(), W1.double().cpu().view(count, 32, L1)[bucket.cpu()]) \
        + b1.double().cpu().view(count, 32)[bucket.cpu()]
    assert torch.equal(outs[0].cpu().double(), want)  # the FMA kernel is exact on these inputs
    assert torch.equal(outs[1], outs[0])


@pytest.mark.parametrize("B,L1", [(5, 128), (777, 512), (4097, 3072), (16384, 3072)])
def test_tensor_core_input_gradient_matches_the_fma_kernel(dev, B, L1):
    """The quantized model's first-layer INPUT gradient on tcgen05: d_o1 (an arbitrary fp32 gradient) goes in as
    three TF32-exact parts, W1 (k / 128) is exact, so every product is exact and only the fp32 accumulation
    rounds.  Against the float64 product, the tensor-core result must be as close as the fp32 FMA kernel's (within
    a factor of two) and within 1e-6 of the tensor's max-norm; the weight and bias gradients are the FMA kernel's."""
    from nnue_pytorch_b200 import _launch, _lib

    lib = _lib.load()
    gen = torch.Generator().manual_seed(3 * B + L1)
    count = 8
    x = (torch.randint(0, 128, (B, L1), generator=gen).float() / 128.0).to(dev)
    W1 = (torch.randint(-127, 128, (count * 32, L1), generator=gen).float() / 128.0).to(dev)
    d_o1 = (torch.randn(B, 32, generator=gen) * torch.rand(B, 1, generator=gen) * 1e-3).to(dev)  # a wide range of sizes
    bucket = torch.randint(0, count, (B,), generator=gen).to(dev)
    if B > 100:
        bucket[bucket == 3] = 2  # an empty bucket
    plan = torch.empty(lib.nnue_ls_plan_bytes(B, count) // 4 + 4, dtype=torch.int32, device=dev)
    s = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(lib.nnue_ls_plan(bucket.data_ptr(), B, count, plan.data_ptr(), plan.numel() * 4, s), "nnue_ls_plan")

    def run(tc):
        dx = torch.full((B, L1), float("nan"), device=dev)
        dW1 = torch.full_like(W1, float("nan"))
        db1 = torch.full((count * 32,), float("nan"), device=dev)
        if tc:
            ws = torch.empty(lib.nnue_ls_l1_bwd_tc_workspace_bytes(L1, count), dtype=torch.uint8, device=dev)
            st = lib.nnue_ls_l1_bwd_tc(x.data_ptr(), W1.data_ptr(), d_o1.data_ptr(), plan.data_ptr(), dx.data_ptr(),
                                       dW1.data_ptr(), db1.data_ptr(), B, L1, count, ws.data_ptr(), ws.numel(), s)
        else:
            st = lib.nnue_ls_l1_bwd(x.data_ptr(), W1.data_ptr(), d_o1.data_ptr(), plan.data_ptr(), dx.data_ptr(),
                                    dW1.data_ptr(), db1.data_ptr(), B, L1, count, s)
        _lib.check(st, "l1 bwd")
        return dx, dW1, db1

    fma = run(False)
    tc_dx_only = run(True)
    _lib.tune("ls_dw_tc", 1)  # off by default: the weight gradient's tensor-core form is correct but slower
    try:
        tc = run(True)
    finally:
        _lib.tune("ls_dw_tc", 0)
    _launch.device_status(dev)  # a bounded wait that ran out would show here
    assert torch.equal(tc_dx_only[1], fma[1]) and torch.equal(tc_dx_only[2], fma[2]) and torch.equal(tc_dx_only[0], tc[0])
    # the weight gradient: x is exact in TF32, d_o1 enters in three exact parts, sums of 512 positions in tensor memory
    onehot = torch.nn.functional.one_hot(bucket, count).double()
    want_w = torch.einsum("bc,bo,bk->cok", onehot, d_o1.double(), x.double()).reshape(count * 32, L1)
    want_b = torch.einsum("bc,bo->co", onehot, d_o1.double()).reshape(-1)
    for name, got_tc, got_fma, ref in (("dW1", tc[1], fma[1], want_w), ("db1", tc[2], fma[2], want_b)):
        sc = max(float(ref.abs().max()), 1e-30)
        e_t = float((got_tc.double() - ref).abs().max()) / sc
        e_f = float((got_fma.double() - ref).abs().max()) / sc
        print(f"B={B} L1={L1}: max-norm relative error of {name}: tensor cores {e_t:.3e}, FMA kernel {e_f:.3e}")
        assert not torch.isnan(got_tc).any()
        assert e_t <= 2e-6 and e_t <= 2 * e_f + 2e-7, name
    want = torch.einsum("bo,bok->bk", d_o1.double(), W1.double().view(count, 32, L1)[bucket])
    scale = float(want.abs().max())
    e_tc = float((tc[0].double() - want).abs().max()) / scale
    e_fma = float((fma[0].double() - want).abs().max()) / scale
    print(f"B={B} L1={L1}: max-norm relative error of dx: tensor cores {e_tc:.3e}, FMA kernel {e_fma:.3e}")
    assert not torch.isnan(tc[0]).any()
    assert e_tc <= 1e-6 and e_tc <= 2 * e_fma + 1e-7
