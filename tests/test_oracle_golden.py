"""Pins the CPU oracle against fixtures produced by the reference's own code
(tests/golden/make_golden.py).  CPU only."""

import numpy as np
import torch

from oracle import ft_oracle, model_oracle, quant_oracle, ranger_lite_oracle
from nnue_pytorch_b200 import positions
from nnue_pytorch_b200.quantize import QuantizationManager

from _util import load_golden, max_rel_err, small_model_params, t


def test_sparse_linear_matches_reference():
    g = load_golden("sparse_linear")
    r = ft_oracle.sparse_linear_with_grads(t(g["indices"]), t(g["weight"]), t(g["bias"]), t(g["grad_out"]))
    assert torch.equal(r["out"], t(g["out"]))
    assert torch.equal(r["grad_weight"], t(g["grad_weight"]))
    assert torch.equal(r["grad_bias"], t(g["grad_bias"]))


def test_fused_matches_reference():
    for name in ("fused_ft_randn", "fused_ft_stm"):
        g = load_golden(name)
        r = ft_oracle.double_feature_transform_with_grads(
            t(g["us"]), t(g["them"]), t(g["white"]), t(g["black"]), t(g["psqt"]), t(g["weight"]), t(g["bias"]),
            float(g["max_act"]), int(g["l1"]), t(g["grad_l0"]), t(g["grad_wpsqt"]), t(g["grad_bpsqt"]))
        for k in ("l0", "wpsqt", "bpsqt", "grad_weight", "grad_bias"):
            assert torch.equal(r[k], t(g[k])), (name, k)
        if name == "fused_ft_stm":  # the clamp must be active on both sides for this case to mean anything
            l0 = t(g["l0"])
            assert (l0 == 0).any() and (l0 >= (255.0 / 256.0) ** 2 - 1e-6).any()


def test_halfka_index_formula():
    g = load_golden("halfka_indices")
    pos = positions.generate_positions(64, 5)
    assert np.array_equal(positions.native_indices(pos, True), g["white"])
    assert np.array_equal(positions.native_indices(pos, False), g["black"])
    assert np.array_equal(positions.KING_BUCKETS, g["king_buckets"])


def test_baseline_layout_is_consistent_with_native():
    pos = positions.generate_positions(256, 9)
    for pov in (True, False):
        nat = positions.native_indices(pos, pov)
        base = positions.baseline_indices(pos, pov)
        k = pos.piece_count
        assert base.shape == (256, 64)
        for i in range(256):
            n = int(k[i])
            assert (base[i, 2 * n:] == -1).all() and (base[i, :2 * n] >= 0).all()
            real, virt = base[i, :n], base[i, n:2 * n]
            assert (real < positions.NUM_REAL_BASELINE).all()
            assert np.array_equal(virt, real % 704 + positions.NUM_REAL_BASELINE)
            # same bucket, square and (king-merged) plane as the native index
            assert np.array_equal(real // 704, nat[i, :n] // 768)
            assert np.array_equal(real % 64, nat[i, :n] % 64)
            plane12 = (nat[i, :n] % 768) // 64
            assert np.array_equal((real % 704) // 64, np.minimum(plane12, 10))


def test_ranger_lite_matches_reference():
    for name, wd in (("ranger_lite", 0.0), ("ranger_lite_wd", 0.01)):
        g = load_golden(name)
        params = [t(g[f"init{j}"]).clone() for j in range(3)]
        st = ranger_lite_oracle.RangerLiteState(params)
        for step in range(12):
            grads = [t(g[f"grad{step}_{j}"]) for j in range(3)]
            ranger_lite_oracle.ranger_lite_step(params, grads, st, lr=8.75e-4, weight_decay=[wd, 0.0, 0.0])
            for j in range(3):
                assert torch.equal(params[j], t(g[f"param{step}_{j}"])), (name, step, j)
        for j in range(3):
            assert torch.equal(st.grad_ma[j], t(g[f"grad_ma{j}"]))
            assert torch.equal(st.neg_grad_ma[j], t(g[f"neg_grad_ma{j}"]))
            assert torch.equal(st.variance_ma[j], t(g[f"variance_ma{j}"]))
            assert torch.equal(st.slow[j], t(g[f"slow{j}"]))


def test_sf_loss_matches_reference():
    g = load_golden("sf_loss")
    sn, sc, oc = t(g["scorenet"]), t(g["score"]), t(g["outcome"])
    assert float(model_oracle.sf_loss(sn, sc, oc, 1.0)) == float(g["loss_lambda_1"])
    assert float(model_oracle.sf_loss(sn, sc, oc, 0.6)) == float(g["loss_lambda_06"])


def _small_batch():
    b = positions.generate_batch(96, 21, layout="native")
    return tuple(t(a) for a in b.as_tuple())


def test_model_forward_loss_and_grads_match_reference():
    g = load_golden("model_small")
    p = small_model_params()
    real = t(p["ft_real"], torch.float32).requires_grad_(True)
    virt = t(p["ft_virtual"], torch.float32).requires_grad_(True)
    params = {k: t(v, torch.float32).requires_grad_(True) for k, v in p.items() if k not in ("ft_real", "ft_virtual", "ft_weight")}
    params["ft_weight"] = model_oracle.merge_virtual(real, virt, 32)
    batch = _small_batch()
    us, them, white, black, outcome, score, pc = batch
    with torch.no_grad():
        y = model_oracle.forward(params, us, them, white, black, pc)
    assert torch.equal(y, t(g["scorenet32"]))
    loss = model_oracle.training_loss(params, batch)
    loss.backward()
    assert float(loss) == float(g["loss"])
    assert max_rel_err(real.grad, t(g["g_ft_weight"])) < 1e-6
    assert max_rel_err(virt.grad, t(g["g_ft_virtual"])) < 1e-6
    assert max_rel_err(params["ft_bias"].grad, t(g["g_ft_bias"])) < 1e-6
    assert max_rel_err(params["l1_w"].grad, t(g["g_l1_w"])) < 1e-6
    assert max_rel_err(params["l1f_w"].grad, t(g["g_l1f_w"])) < 1e-6
    assert max_rel_err(params["out_w"].grad, t(g["g_out_w"])) < 1e-6


def test_integer_eval_matches_reference_float64_forward():
    g = load_golden("model_small")
    p = small_model_params()
    b = positions.generate_batch(96, 21, layout="native")
    consts = QuantizationManager().integer_constants()
    qp = quant_oracle.quantize_params(p, 64)
    bucket = (b.piece_count - 1) // 4
    got = quant_oracle.integer_eval(qp, b.white, b.black, b.us[:, 0] > 0.5, bucket, consts)
    assert np.array_equal(got, g["eval_int"][:, 0])
    # and the float64 restatement of the same forward agrees too
    params = {k: t(v, torch.float64) for k, v in p.items()}
    us, them, white, black, _, _, pc = (t(a) for a in b.as_tuple())
    y = model_oracle.forward(params, us.double(), them.double(), white, black, pc)
    assert np.array_equal(torch.round(y * 19200).to(torch.int64).numpy()[:, 0], g["eval_int"][:, 0])


def test_integer_eval_epsilon_window():
    """o1^2 just below a multiple of 2^21 rounds up, exactly as the 1e-5 the
    float path adds before its floor (model/quantize.py:41)."""
    for o1, eps, shift in ((1448, 20, 21), (2048, 20, 21), (724, 5, 19)):
        v = np.int64(o1)
        k = (v * v + eps) >> shift
        f = np.floor((float(v) / (1 << ((shift + 7) // 2))) ** 2 * 128 + 1e-5)
        assert int(k) == int(f)
    # every v below 3e6 whose square lands in the window behaves like the float path
    v = np.arange(0, 3_000_000, dtype=np.int64)
    sq = v * v
    window = (sq % (1 << 21)) >= (1 << 21) - 20
    vv = v[window]
    want = np.floor((vv.astype(np.float64) / 16384.0) ** 2 * 128 + 1e-5).astype(np.int64)
    assert np.array_equal((vv * vv + 20) >> 21, want)
    assert len(vv) > 0
