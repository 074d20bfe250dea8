"""Registers this package under the reference project's module names, so that
an unmodified nnue-pytorch checkout trains on these kernels.

The reference resolves its feature-transformer operators and its optimizer
through package-relative imports (model/modules/__init__.py:2-4,
model/modules/feature_transformer/__init__.py:1-11,
model/optimizers/rangerlite_wrapper.py:5), and Python consults `sys.modules`
before the file system.  A launcher calls `install()` first and then imports
or runs the reference as usual:

    import runpy, sys
    sys.path.insert(0, "/path/to/nnue-pytorch")
    from nnue_pytorch_b200 import overlay
    overlay.install()
    runpy.run_path("/path/to/nnue-pytorch/train.py", run_name="__main__")

What is replaced: the three operator modules (`sparse_linear_functions`,
`fused_ft_functions`, `double_ft_functions`; the CuPy kernel modules behind
them are then never imported) and `model.optimizers.ranger_lite`.  With
`module=True` the reference's `ComposedFeatureTransformer` is replaced as well,
which moves the factor fold, the weight fake quantization and the activation
fake quantization from dense torch passes into the kernels; the reference's
feature blocks whose merged table is `weight + virtual_weight.repeat(k, 1)`
(`HalfKav2Hm`) are marked for that path.  Everything else of the reference
(model graph, layer stacks, loss, trainer, loader, CLI) runs as it is.
"""

from __future__ import annotations

import importlib
import sys

FT_PACKAGE = "model.modules.feature_transformer"
OPERATOR_MODULES = ("sparse_linear_functions", "fused_ft_functions", "double_ft_functions")
OPTIMIZER_MODULE = "model.optimizers.ranger_lite"
_installed: dict[str, object] = {}


def install(module: bool = False, optimizer: bool = True) -> None:
    """Must run before the reference's `model` package is imported."""
    already = [m for m in (f"{FT_PACKAGE}.{n}" for n in OPERATOR_MODULES) if m in sys.modules and m not in _installed]
    if already or ("model" in sys.modules and not _installed):
        raise RuntimeError("overlay.install() must run before the reference's `model` package is imported "
                           f"(already imported: {already or ['model']})")
    for name in OPERATOR_MODULES:
        _register(f"{FT_PACKAGE}.{name}", importlib.import_module(f"nnue_pytorch_b200.{name}"))
    if optimizer:
        _register(OPTIMIZER_MODULE, importlib.import_module("nnue_pytorch_b200.ranger_lite"))
    if module:
        _register(f"{FT_PACKAGE}.composed_feature_transformer",
                  importlib.import_module("nnue_pytorch_b200.composed_feature_transformer"))
        # the reference's feature blocks: importing them runs the reference's package initialisers, which now
        # pick the modules registered above
        hk = importlib.import_module("model.modules.features.halfka_v2_hm")
        hk.HalfKav2Hm.FUSED_TABLE = True  # merged_weight() is weight + virtual_weight.repeat(32, 1): halfka_v2_hm.py:68-69


def _register(name: str, mod) -> None:
    sys.modules[name] = mod
    _installed[name] = mod


def uninstall() -> None:
    """Removes the registrations (modules that already imported the replacements keep them)."""
    for name, mod in list(_installed.items()):
        if sys.modules.get(name) is mod:
            del sys.modules[name]
    _installed.clear()


def installed() -> bool:
    return bool(_installed)
