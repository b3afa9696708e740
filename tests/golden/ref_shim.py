"""Import the K-Fold reference's torch modules without its heavy dependencies.

The reference's package ``__init__`` files pull in rdkit, gemmi, omegaconf and
atlaslm, none of which the hot path needs.  This shim registers empty namespace
modules for those packages (with ``__path__`` pointing at the real directories)
so that the individual primitive/layer files can be imported unmodified.

Only the fixture generator (``make_golden.py``) and the optional
reference-vs-oracle tests use this file; nothing shipped depends on it.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

# default: a checkout named "reference" beside this repository; KFOLD_REFERENCE_ROOT overrides it
_DEFAULT_ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")


def reference_root() -> str | None:
    root = os.environ.get("KFOLD_REFERENCE_ROOT", _DEFAULT_ROOT)
    return root if os.path.isdir(os.path.join(root, "src", "kfold")) else None


def _namespace(name: str, path: str) -> None:
    if name in sys.modules:
        return
    mod = types.ModuleType(name)
    mod.__path__ = [path]
    sys.modules[name] = mod
    parent, _, child = name.rpartition(".")
    if parent and parent in sys.modules:
        setattr(sys.modules[parent], child, mod)


def load_reference():
    """Return a namespace of the reference classes on the hot path."""
    root = reference_root()
    if root is None:
        raise RuntimeError("K-Fold reference tree not found")
    src = os.path.join(root, "src")
    if src not in sys.path:
        sys.path.insert(0, src)
    import kfold  # noqa: F401  (top-level package has a light __init__)

    base = os.path.join(src, "kfold")
    for name, rel in [
        ("kfold.model", "model"),
        ("kfold.model.layers", "model/layers"),
        ("kfold.model.layers.folding", "model/layers/folding"),
        ("kfold.model.modules", "model/modules"),
        ("kfold.data", "data"),
        ("kfold.data.types", "data/types"),
        ("kfold.utils", "utils"),
    ]:
        _namespace(name, os.path.join(base, rel))

    if "omegaconf" not in sys.modules:
        oc = types.ModuleType("omegaconf")
        oc.OmegaConf = type("OmegaConf", (), {})
        oc.DictConfig = type("DictConfig", (), {})
        sys.modules["omegaconf"] = oc
    if "kfold.data.types.model_input" not in sys.modules:
        mi = types.ModuleType("kfold.data.types.model_input")
        mi.FoldingInput = type("FoldingInput", (), {})
        sys.modules["kfold.data.types.model_input"] = mi

    ns = types.SimpleNamespace()
    prim = importlib.import_module("kfold.model.primitives")
    for k in (
        "LayerNorm", "Linear", "LinearNoBias", "AdaLN", "SwiGLU",
        "TriangleMultiplicationOutgoing", "TriangleMultiplicationIncoming",
        "TriangleAttentionStartingNode", "TriangleAttentionEndingNode",
    ):
        setattr(ns, k, getattr(prim, k))
    ns.attention = importlib.import_module("kfold.model.primitives.attention")
    ns.Transition = importlib.import_module(
        "kfold.model.layers.folding.transition").Transition
    apb = importlib.import_module("kfold.model.layers.folding.attention_pair_bias")
    ns.SelfAttentionPairBias = apb.SelfAttentionPairBias
    ns.CrossAttentionPairBias = apb.CrossAttentionPairBias
    return ns
