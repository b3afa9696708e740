"""Import the K-Fold reference's torch modules without its heavy dependencies.

The reference's package ``__init__`` files pull in rdkit, gemmi, omegaconf and
atlaslm, none of which the hot path needs.  This shim registers empty namespace
modules for those packages (with ``__path__`` pointing at the real directories)
so that the individual primitive/layer files can be imported unmodified.

The reference is looked for, in this order, at ``$KFOLD_REFERENCE_ROOT``, in
``baseline/_ref`` of this repository (where ``pip install --no-deps --target
baseline/_ref <kfold checkout>`` puts the package; that directory is not under
version control) and in a checkout named ``reference`` beside the repository.

Only the fixture generator (``make_golden.py``), the reference-vs-oracle tests and
the CPU reference arm of ``bench.py`` use this file; nothing shipped depends on it.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _package_parent(root: str) -> str | None:
    """The directory that holds the ``kfold`` package under `root`: ``root/src`` (a checkout) or ``root`` (an install)."""
    for parent in (os.path.join(root, "src"), root):
        if os.path.isfile(os.path.join(parent, "kfold", "model", "primitives", "__init__.py")):
            return parent
    return None


def reference_root() -> str | None:
    """Directory to put on sys.path so that ``import kfold`` finds the reference, or None."""
    cands = [os.environ.get("KFOLD_REFERENCE_ROOT"), os.path.join(_REPO, "baseline", "_ref"),
             os.path.join(os.path.dirname(_REPO), "reference")]
    for root in cands:
        if root and os.path.isdir(root):
            parent = _package_parent(root)
            if parent is not None:
                return parent
    return None


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
    src = reference_root()
    if src is None:
        raise RuntimeError("K-Fold reference tree not found")
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


class _AnyMeta(type):
    def __getattr__(cls, name):
        return cls


class _Any(metaclass=_AnyMeta):
    """Stands for any class of a module that cannot be imported here; attribute access on it yields itself."""


class _StubModule(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _Any


def load_reference_model():
    """Import the reference's ``kfold.model.model`` (LMToPair, the Parcae dynamics of KFold) after ``load_reference()``.
    The modules it pulls in for the parts of K-Fold outside the hot path (input embedder, sequence / structure encoders,
    heads) need rdkit and friends; they are replaced by stub modules whose every attribute is a placeholder class, which
    is all the import needs (class-level annotations such as ``input_embedder.InputEmbedder.Config``)."""
    load_reference()
    mods = sys.modules["kfold.model.modules"]
    for n in ("input_embedder", "prot_seq_encoder", "prot_struct_encoder", "rna_seq_encoder", "patch_geometry", "distogram_head",
              "confidence_head", "apo_module"):
        full = "kfold.model.modules." + n
        if full not in sys.modules:
            stub = _StubModule(full)
            sys.modules[full] = stub
            setattr(mods, n, stub)
    return importlib.import_module("kfold.model.model")


def _sub(weights: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in weights.items() if k.startswith(p)}


def build_reference_block(ns, w: dict, c_z: int = 128, c_s: int = 384, tri_heads: int = 4, single_heads: int = 16):
    """The composite Pairformer block of the benchmark, assembled from REFERENCE modules only (torch backend): the pair
    track in the order of ``PairformerBlock.forward`` (model/modules/apo_module.py:145-172) with ``Transition(c_z, 4)``,
    then the single track of ``ConfidencePairSingleBlock.forward`` (model/modules/confidence_head.py:152-175).
    Returns ``fn(z, s, pair_mask, mask) -> (z, s)``; the inputs are updated in place, as the reference does in eval."""
    import torch

    def load(mod, sd):
        mod.load_state_dict(sd, strict=True)
        return mod.eval()

    tmo = load(ns.TriangleMultiplicationOutgoing(c_z), _sub(w, "tri_mul_out"))
    tmi = load(ns.TriangleMultiplicationIncoming(c_z), _sub(w, "tri_mul_in"))
    tas = load(ns.TriangleAttentionStartingNode(c_z, tri_heads), _sub(w, "tri_att_start"))
    tae = load(ns.TriangleAttentionEndingNode(c_z, tri_heads), _sub(w, "tri_att_end"))
    trz = load(ns.Transition(c_z, 4), _sub(w, "transition_z"))
    lnz = load(ns.LayerNorm(c_z), _sub(w, "layernorm_z"))
    lin = load(ns.LinearNoBias(c_z, single_heads), _sub(w, "linear_pair_bias"))
    att = load(ns.SelfAttentionPairBias(c_s, single_heads, None, "confidence", kernel_backend="torch"), _sub(w, "attention"))
    trs = load(ns.Transition(c_s, 4), _sub(w, "transition"))

    @torch.no_grad()
    def block(z, s, pair_mask, mask):
        z.add_(tmo(z, pair_mask))
        z.add_(tmi(z, pair_mask))
        z.add_(tas(z, pair_mask))
        z.add_(tae(z, pair_mask))
        z.add_(trz(z))
        pair_bias = lin(lnz(z)).movedim(-1, -3)
        s.add_(att(s, None, pair_bias, mask))
        s.add_(trs(s))
        return z, s

    return block
