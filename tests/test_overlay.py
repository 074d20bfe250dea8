"""The drop-in: an unmodified copy of the reference's `model` package (oracle/_ref, see
oracle/make_ref.py) with `nnue_pytorch_b200.overlay` installed in front of it.

CPU: the reference imports, builds its `NNUE` shell and its ten optimizer groups on top of the
replacement modules, and its state dict keeps the reference's parameter names.
GPU: the reference's model, compiled with torch.compile as its train.py does, runs one training
step on these kernels and reproduces the loss and every gradient of the untouched reference run
on CPU through its own torch path.  Each run is a child process: the overlay changes what
`import model` means for a whole interpreter.
"""

import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHILD = os.path.join(ROOT, "tests", "_overlay_child.py")
HAVE_REF = os.path.isfile(os.path.join(ROOT, "oracle", "_ref", "model", "nnue.py"))
needs_ref = pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref is absent (python oracle/make_ref.py <checkout>)")


def _child(*args):
    r = subprocess.run([sys.executable, CHILD, *map(str, args)], cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]


@needs_ref
def test_reference_builds_on_the_overlay(tmp_path):
    out = tmp_path / "keys.pt"
    _child("keys", out)
    rep = torch.load(out)
    assert rep["ft_module"] == "nnue_pytorch_b200.composed_feature_transformer"
    assert rep["dft_module"] == "nnue_pytorch_b200.double_ft_functions"
    assert rep["optimizer_module"] == "nnue_pytorch_b200.ranger_lite"
    assert rep["has_cupy_flag"]
    assert rep["groups"] == [2, 1, 1, 1, 1, 1, 1, 1, 1, 1]  # table + factor rows, bias, then the eight dense tensors
    for key in ("input.bias", "input.features.0.weight", "input.features.0.virtual_weight",
                "layer_stacks.l1.linear.weight", "layer_stacks.output.linear.bias"):
        assert key in rep["model_keys"], key
        assert "model." + key in rep["state_keys"], key


def test_overlay_refuses_to_install_late():
    code = ("import sys, types; sys.modules['model'] = types.ModuleType('model');"
            "from nnue_pytorch_b200 import overlay\n"
            "try:\n    overlay.install()\nexcept RuntimeError as e:\n    print('refused'); raise SystemExit(0)\n"
            "raise SystemExit(1)")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "refused" in r.stdout, r.stderr[-2000:]


@needs_ref
@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["operators", "module"])
def test_compiled_reference_model_trains_on_the_overlay(tmp_path, variant):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    ref, out = tmp_path / "ref.pt", tmp_path / "out.pt"
    _child("reference", ref)
    _child("overlay", ref, out, variant)
    want, got = torch.load(ref), torch.load(out)
    assert got["launches"] > 0, "the step did not go through libnnue_b200"
    assert abs(got["loss"] - want["loss"]) <= 1e-5 * abs(want["loss"]), (got["loss"], want["loss"])
    assert set(got["grads"]) == set(want["grads"])
    for name, g_ref in want["grads"].items():
        scale = max(float(g_ref.abs().max()), 1e-30)
        err = float((got["grads"][name] - g_ref).abs().max()) / scale
        assert err <= 1e-5, (name, err)


@needs_ref
@pytest.mark.gpu
def test_default_feature_set_matches_the_reference_module(tmp_path):
    """`Full_Threats+PP_3Wide+HalfKAv2_hm^` (88944 rows, lists of up to 288): this package's model on the GPU
    (three feature blocks quantized into one int16 table, fused operator, fused layer stacks) against the
    reference's own model with the same parameters on CPU through its torch path: loss and the gradient of
    every parameter, the factor rows of the HalfKA block included."""
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from nnue_pytorch_b200.features import DEFAULT_FEATURES
    from nnue_pytorch_b200.model import LossParams, ModelConfig, NNUEModel, sf_loss

    ref = tmp_path / "ref.pt"
    _child("reference", ref, DEFAULT_FEATURES)
    want = torch.load(ref)
    dev = torch.device("cuda:0")
    m = NNUEModel(DEFAULT_FEATURES, ModelConfig(L1=256, L2=32, L3=32))
    assert m.input.NUM_INPUTS == 88944 and m.input.MAX_ACTIVE_FEATURES == 288
    m.load_state_dict(want["state"])
    m.to(dev)
    us, them, white, black, outcome, score, pc = (x.to(dev) for x in want["batch"])
    assert white.shape[1] == 288
    for integer_table in (True, False):
        m.input.integer_table = integer_table
        m.zero_grad(set_to_none=True)
        y = m(us, them, white, black, pc, True, True)
        loss = sf_loss(y * 600.0, score, outcome, LossParams(), 1.0)
        loss.backward()
        assert abs(float(loss) - want["loss"]) <= 1e-5 * abs(want["loss"]), (integer_table, float(loss), want["loss"])
        got = {n: p.grad.detach().cpu() for n, p in m.named_parameters() if p.grad is not None}
        assert set(got) == set(want["grads"])
        for name, g_ref in want["grads"].items():
            scale = max(float(g_ref.abs().max()), 1e-30)
            err = float((got[name] - g_ref).abs().max()) / scale
            assert err <= 1e-5, (integer_table, name, err)
