"""Child process of tests/test_overlay.py (a separate interpreter, because the
overlay changes what `import model` means for the whole process).

    python tests/_overlay_child.py reference OUT.pt [FEATURES]   the reference as it is, on CPU (its torch path)
    python tests/_overlay_child.py keys OUT.pt             overlay installed, CPU only: names and structure
    python tests/_overlay_child.py overlay IN.pt OUT.pt [module]   overlay installed, on cuda:0, model compiled
"""

import importlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

L1, B, SEED = 256, 192, 5


FEATURES = "HalfKAv2_hm^"


def _batch():
    """The tuple `SparseBatch.get_tensors` returns, for generated positions in the layout FEATURES needs."""
    from nnue_pytorch_b200 import full_features, positions

    b = positions.generate_batch(B, 77, layout="native")
    if FEATURES != "HalfKAv2_hm^":
        white, black = full_features.full_feature_lists(full_features.boards_of(positions.generate_positions(B, 77)))
        b.white, b.black = white, black
    return tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in b.as_tuple())


def _build(model_pkg):
    cfg = model_pkg.NNUELightningConfig(features=FEATURES, model_config=model_pkg.ModelConfig(L1=L1, L2=32, L3=32))
    torch.manual_seed(SEED)
    nnue = model_pkg.NNUE(cfg)
    with torch.no_grad():
        for f in nnue.model.input.features:
            f.weight[:, :L1].normal_(0.0, 0.05)
            if hasattr(f, "virtual_weight"):
                f.virtual_weight[:, :L1].normal_(0.0, 0.02)
    return nnue


def _grads(nnue):
    return {n: p.grad.detach().cpu().clone() for n, p in nnue.model.named_parameters() if p.grad is not None}


def main():
    global FEATURES
    mode = sys.argv[1]
    if mode == "reference" and len(sys.argv) > 3:
        FEATURES = sys.argv[3]
    from oracle import ref_runner, ref_shims

    ref_shims.install()
    sys.path.insert(0, ref_runner.REF_ROOT)
    if mode == "reference":
        import model

        nnue = _build(model)
        nnue.train()
        out = nnue.train_step(_batch(), 0, 0)
        out["loss"].backward()
        torch.save({"state": nnue.model.state_dict(), "loss": float(out["loss"]), "grads": _grads(nnue),
                    "batch": _batch()}, sys.argv[2])
        return
    from nnue_pytorch_b200 import overlay

    if mode == "keys":
        overlay.install(module=True)
        import model

        nnue = _build(model)
        opts, _ = nnue.configure_optimizers()
        torch.save({
            "ft_module": type(nnue.model.input).__module__,
            "dft_module": model.modules.feature_transformer.double_feature_transform.__module__,
            "optimizer_module": type(opts[0]).__module__,
            "groups": [len(g["params"]) for g in opts[0].param_groups],
            "state_keys": sorted(nnue.state_dict().keys()),
            "model_keys": sorted(nnue.model.state_dict().keys()),
            # the flag the reference's dispatcher and tests read, by the dotted name they import it from
            "has_cupy_flag": bool(importlib.import_module(
                "model.modules.feature_transformer.fused_ft_functions")._HAS_CUPY_KERNELS),
        }, sys.argv[2])
        return
    assert mode == "overlay"
    overlay.install(module=len(sys.argv) > 4 and sys.argv[4] == "module")
    import model

    ref = torch.load(sys.argv[2])
    nnue = _build(model)
    nnue.model.load_state_dict(ref["state"])
    dev = torch.device("cuda:0")
    nnue.to(dev)
    nnue.train()
    nnue.model = torch.compile(nnue.model, backend="eager")  # what the reference's train.py does before training
    batch = tuple(x.to(dev) for x in _batch())
    out = nnue.train_step(batch, 0, 0)
    out["loss"].backward()
    opts, _ = nnue.configure_optimizers()
    torch.nn.utils.clip_grad_norm_(nnue.parameters(), 2.0)
    opts[0].step()  # the replacement optimizer runs on the compiled model's parameters
    torch.cuda.synchronize()
    from nnue_pytorch_b200 import _lib

    torch.save({"loss": float(out["loss"]), "grads": {k.replace("_orig_mod.", ""): v for k, v in _grads(nnue).items()},
                "ft_module": type(nnue.model.input).__module__ if hasattr(nnue.model, "input") else "",
                "launches": int(_lib.load().nnue_b200_launch_count())}, sys.argv[3])


if __name__ == "__main__":
    main()
