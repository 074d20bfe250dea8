"""The one-launch training loss against the reference's formula: the golden
fixture generated from the reference (tests/golden/sf_loss.npz), and the torch
restatement in float32 and float64 for the gradients."""

import numpy as np
import pytest
import torch

from _util import load_golden, max_rel_err, t

pytestmark = pytest.mark.gpu

TOL = 1e-5


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from nnue_pytorch_b200 import _lib

    _lib.load()
    return torch.device("cuda:0")


def test_loss_matches_reference_fixture(dev):
    from nnue_pytorch_b200.loss_functions import sf_loss_fused
    from nnue_pytorch_b200.model import LossParams

    g = load_golden("sf_loss")  # includes scores in the tablebase range
    sn, sc, oc = (t(g[k]).to(dev) for k in ("scorenet", "score", "outcome"))
    for lam, key in ((1.0, "loss_lambda_1"), (0.6, "loss_lambda_06")):
        loss, _, _, _ = sf_loss_fused(sn, None, None, None, sc, oc, LossParams(), lam, 1.0, want_grads=False)
        want = float(g[key])
        assert abs(float(loss) - want) <= TOL * abs(want), (lam, float(loss), want)


@pytest.mark.parametrize("B", [1, 37, 1024, 16384, 70001])
@pytest.mark.parametrize("variant", ["default", "asym", "lambda", "no_psqt"])
def test_loss_and_gradients_match_torch_formula(dev, B, variant):
    from nnue_pytorch_b200.loss_functions import SfLossFunction
    from nnue_pytorch_b200.model import LossParams, sf_loss

    gen = torch.Generator().manual_seed(B)
    y = torch.randn(B, 1, generator=gen) * 0.8
    wp, bp = torch.randn(B, 1, generator=gen) * 0.3, torch.randn(B, 1, generator=gen) * 0.3
    us = torch.randint(0, 2, (B, 1), generator=gen).float()
    score = (torch.randn(B, 1, generator=gen) * 400).clamp(-3000, 3000).round()
    score[:: 97] = 31990.0   # mate-range scores take the remap branch
    score[5:: 131] = -31800.0
    outcome = torch.randint(0, 3, (B, 1), generator=gen).float() * 0.5
    lp = LossParams()
    lam = 1.0
    if variant == "asym":
        lp = LossParams(qp_asymmetry=0.3, w1=1.5, w2=0.7, pow_exp=2.2)
    elif variant == "lambda":
        lam = 0.4

    def ref(dtype):
        yy, ww, bb = (x.to(dtype).clone().requires_grad_(True) for x in (y, wp, bp))
        net = yy if variant == "no_psqt" else yy + (ww - bb) * (us.to(dtype) - 0.5)
        loss = sf_loss(net * 600.0, score.to(dtype), outcome.to(dtype), lp, lam)
        loss.backward()
        return loss.detach(), yy.grad, (None if variant == "no_psqt" else ww.grad), (None if variant == "no_psqt" else bb.grad)

    l32, gy32, gw32, gb32 = ref(torch.float32)
    l64, gy64, gw64, gb64 = ref(torch.float64)
    yd, wd, bd = (x.to(dev).requires_grad_(True) for x in (y, wp, bp))
    if variant == "no_psqt":
        loss = SfLossFunction.apply(yd, None, None, None, score.to(dev), outcome.to(dev), lp, lam, 600.0)
    else:
        loss = SfLossFunction.apply(yd, wd, bd, us.to(dev), score.to(dev), outcome.to(dev), lp, lam, 600.0)
    loss.backward()
    assert abs(float(loss) - float(l64)) <= TOL * abs(float(l64))
    pairs = [(yd.grad, gy32, gy64)] + ([] if variant == "no_psqt" else [(wd.grad, gw32, gw64), (bd.grad, gb32, gb64)])
    for ours, r32, r64 in pairs:
        ours = ours.cpu()
        assert ours.shape == r32.shape
        err = max_rel_err(ours.double(), r64)
        assert err <= max(TOL, 2 * max_rel_err(r32.double(), r64)), err


def test_loss_is_reproducible_and_leaves_its_workspace_clean(dev):
    from nnue_pytorch_b200.loss_functions import _workspace, sf_loss_fused
    from nnue_pytorch_b200.model import LossParams

    gen = torch.Generator().manual_seed(3)
    B = 40000
    y, sc = torch.randn(B, generator=gen).to(dev), (torch.randn(B, generator=gen) * 500).to(dev)
    oc = (torch.randint(0, 3, (B,), generator=gen).float() * 0.5).to(dev)
    outs = [sf_loss_fused(y, None, None, None, sc, oc, LossParams(), 0.7, 600.0) for _ in range(4)]
    for o in outs[1:]:
        assert torch.equal(o[0], outs[0][0]) and torch.equal(o[1], outs[0][1])
    torch.cuda.synchronize()
    assert int(_workspace(dev)[0]) == 0  # the arrival counter is back at zero


def test_train_step_with_and_without_the_fused_loss_agree(dev):
    from nnue_pytorch_b200 import positions
    from nnue_pytorch_b200.model import ModelConfig, NNUEModel, TrainStep

    def run(fused):
        torch.manual_seed(0)
        m = NNUEModel("HalfKAv2_hm^flat", ModelConfig(L1=128, L2=32, L3=32))
        with torch.no_grad():
            m.input.features[0].weight[:, :128].normal_(0, 0.05)
        m.to(dev)
        step = TrainStep(m, clip=2.0, fused_loss=fused)
        losses = []
        for i in range(3):
            b = positions.generate_batch(512, 7 + i, layout="baseline")
            losses.append(float(step(tuple(t(a).to(dev) for a in b.as_tuple()))))
        return losses, m.input.features[0].weight.detach().cpu()

    la, wa = run(True)
    lb, wb = run(False)
    for a, b in zip(la, lb):
        assert abs(a - b) <= 2e-5 * abs(b)
    assert max_rel_err(wa, wb) <= 1e-4
