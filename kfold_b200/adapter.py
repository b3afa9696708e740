"""Hooks that put the B200 kernels behind K-Fold's own ``kernel_backend`` dispatch.

K-Fold's primitives choose an implementation by comparing ``self.kernel_backend`` with a string
inside ``forward`` (model/primitives/triangle_multiplication.py:194-210,
model/primitives/triangle_attention.py:404-408, model/primitives/attention.py:62-73).  This module adds
the value ``"b200"`` to that dispatch without editing K-Fold:

  * ``b200_triangular_mult`` / ``b200_triangular_attn`` / ``b200_attention_pair_bias`` are the backend
    entry points, written against the *reference* modules (they read the reference's parameter names) and
    following the conventions of the reference's Triton entry points
    (model/primitives/triangle_multiplication.py:94-145);
  * ``install()`` patches an imported ``kfold`` package so that modules whose ``kernel_backend`` is
    ``"b200"`` route to them, and ``select_kernel_backend`` accepts the new name;
  * ``convert(model)`` switches the modules of an already constructed model over (the pair-bias
    attention modules are constructed with a hard-coded ``"sdpa"``, so a post-construction pass is needed).
"""
from __future__ import annotations

import functools
import importlib

import torch

from . import functional as F
from . import packing

BACKEND = "b200"


def _check(x: torch.Tensor, what: str) -> None:
    if torch.is_grad_enabled():
        raise RuntimeError(f"The B200 {what} backend is inference-only.")
    if not x.is_cuda:
        raise RuntimeError(f"The B200 {what} backend requires CUDA.")


def _compute_dtype(x: torch.Tensor) -> torch.dtype:
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type)
    return x.dtype


def _is_precise(dt: torch.dtype, what: str) -> bool:
    """bfloat16 compute -> the tensor-core path; float32 compute -> the fp32-accurate path."""
    if dt == torch.bfloat16:
        return False
    if dt == torch.float32:
        return True
    raise NotImplementedError(f"The B200 {what} backend computes in bfloat16 or float32; got compute dtype {dt}")


def _cached_pack(module: torch.nn.Module, x: torch.Tensor, dtype: torch.dtype, slot: str, pack_fn):
    """Pack once per module; re-pack when a parameter's storage or version changes
    (the cache key of model/primitives/triangle_multiplication.py:73-91)."""
    key = (x.device.type, x.device.index, dtype) + tuple(
        v for p in module.parameters() for v in (p.data_ptr(), None if torch.is_inference(p) else p._version))
    cache = getattr(module, "_b200_cache", None)
    if cache is None:
        cache = {}
        module._b200_cache = cache
    hit = cache.get(slot)
    if hit is None or hit[0] != key:
        hit = (key, pack_fn(module.state_dict(), x.device))
        cache[slot] = hit
    return hit[1]


@torch.compiler.disable
def b200_triangular_mult(module: torch.nn.Module, x: torch.Tensor, mask: torch.Tensor, direction: str) -> torch.Tensor:
    """Stands where ``triton_triangluar_mult(module, x, mask, direction)`` stands."""
    _check(x, "triangle multiplication")
    cd = _compute_dtype(x)
    precise = _is_precise(cd, "triangle multiplication")
    pk = _cached_pack(module, x, cd, "trimul", lambda sd, dev: packing.pack_trimul(sd, dev, precise=precise))
    with torch.autocast(x.device.type, enabled=False):
        out = F.triangle_multiplication(x.float() if precise else x, mask.bool(), pk, direction, eps=module.layernorm_in.eps)
    return out.to(x.dtype)


@torch.compiler.disable
def b200_triangular_attn(module: torch.nn.Module, x: torch.Tensor, mask: torch.Tensor | None, starting: bool) -> torch.Tensor:
    """Stands where ``triton_triangular_attn(module, x, mask)`` stands, but takes the UNtransposed tensors:
    the ending node is handled inside the kernels."""
    _check(x, "triangle attention")
    cd = _compute_dtype(x)
    precise = _is_precise(cd, "triangle attention")
    heads = module.no_heads
    pk = _cached_pack(module, x, cd, "triatt", lambda sd, dev: packing.pack_triatt(sd, heads, dev, precise=precise))
    lead = x.shape[:-3]
    x4 = x.reshape(-1, *x.shape[-3:])
    if precise:
        x4 = x4.float()
    m4 = None if mask is None else mask.reshape(-1, *mask.shape[-2:]).bool()
    with torch.autocast(x.device.type, enabled=False):
        out = F.triangle_attention(x4, m4, pk, starting, eps=module.layer_norm.eps)
    return out.reshape(*lead, *x.shape[-3:]).to(x.dtype)


def apb_supported(module: torch.nn.Module) -> bool:
    """Shapes the pair-bias attention kernel takes: head dim a multiple of 8 in [16, 64], default mask offset."""
    d = getattr(module, "head_dim", 0)
    return d % 8 == 0 and 16 <= d <= 64 and getattr(module, "inf", 1e9) == 1e9


@torch.compiler.disable
def b200_attention_pair_bias(module, x_q, x_k, pair_bias, mask, *, call_site: str) -> torch.Tensor:
    """Stands where ``triton_attention_pair_bias(module, x_q, x_k, pair_bias, mask, call_site=...)`` stands: the
    token-level self-attention call sites "diffusion_global" and "confidence" (x_q is x_k), and the windowed cross
    attention of the atom transformers, "diffusion_local" (x_q (..., W, 32, c), x_k (..., W, 128, c))."""
    _check(x_q, "pair-bias attention")
    cd = _compute_dtype(x_q)
    precise = _is_precise(cd, "pair-bias attention")
    heads = module.num_heads
    keys = ("linear_q.weight", "linear_q.bias", "linear_k.weight", "linear_v.weight", "linear_g.weight",
            "linear_g.bias", "linear_out.weight", "linear_out.bias")
    if x_q is not x_k:
        def pack_cross(sd, dev):
            return packing.pack_apb_cross({k: sd[k] for k in keys if k in sd}, heads, dev, precise=precise)

        pkc = _cached_pack(module, x_q, cd, "apb_cross", pack_cross)
        with torch.autocast(x_q.device.type, enabled=False):
            return F.attention_pair_bias_cross_bcast(x_q.float() if precise else x_q, x_k.float() if precise else x_k, pair_bias,
                                                     mask, pkc, out_dtype=x_q.dtype)

    def pack(sd, dev):
        return packing.pack_apb({k: sd[k] for k in keys if k in sd}, heads, dev, precise=precise)

    pk = _cached_pack(module, x_q, cd, "apb", pack)
    with torch.autocast(x_q.device.type, enabled=False):
        out = F.attention_pair_bias(x_q.float() if precise else x_q, pair_bias, mask, pk, out_dtype=x_q.dtype)
    return out


# ------------------------------------------------------------------------------------------------
# patching an imported kfold package
# ------------------------------------------------------------------------------------------------
_installed = False


def install() -> None:
    """Teach an importable ``kfold`` package the ``"b200"`` backend.  Idempotent.  Does not edit any file."""
    global _installed
    if _installed:
        return
    runtime = importlib.import_module("kfold.utils.runtime")
    tm = importlib.import_module("kfold.model.primitives.triangle_multiplication")
    ta = importlib.import_module("kfold.model.primitives.triangle_attention")
    att = importlib.import_module("kfold.model.primitives.attention")

    orig_select = runtime.select_kernel_backend

    @functools.wraps(orig_select)
    def select_kernel_backend(backend: str = "auto") -> str:
        if backend == BACKEND:
            if not torch.cuda.is_available():
                raise ValueError("The 'b200' backend needs a CUDA device.")
            return BACKEND
        return orig_select(backend)

    runtime.select_kernel_backend = select_kernel_backend

    def wrap_trimul(cls, direction):
        orig = cls.forward

        @functools.wraps(orig)
        def forward(self, x, mask):
            if self.kernel_backend == BACKEND:
                return b200_triangular_mult(self, x, mask, direction=direction)
            return orig(self, x, mask)

        cls.forward = forward

    wrap_trimul(tm.TriangleMultiplicationOutgoing, "outgoing")
    wrap_trimul(tm.TriangleMultiplicationIncoming, "incoming")

    orig_ta = ta.TriangleAttention.forward

    @functools.wraps(orig_ta)
    def ta_forward(self, x, mask=None):
        if self.kernel_backend == BACKEND:
            return b200_triangular_attn(self, x, mask, starting=self.starting)
        return orig_ta(self, x, mask)

    ta.TriangleAttention.forward = ta_forward

    orig_apb = att.attention_pair_bias

    @functools.wraps(orig_apb)
    def attention_pair_bias(module, x_q, x_k, pair_bias, mask, *, kernel_backend, call_site):
        if kernel_backend == BACKEND:
            return b200_attention_pair_bias(module, x_q, x_k, pair_bias, mask, call_site=call_site)
        return orig_apb(module, x_q, x_k, pair_bias, mask, kernel_backend=kernel_backend, call_site=call_site)

    att.attention_pair_bias = attention_pair_bias
    # the layer module imported the function by name
    try:
        layer = importlib.import_module("kfold.model.layers.folding.attention_pair_bias")
        layer.attention_pair_bias = attention_pair_bias
    except Exception:  # the layer package may be unimportable without K-Fold's optional dependencies
        pass
    _installed = True


def convert(model: torch.nn.Module, diffusion: bool = False) -> int:
    """Switch every supported module of a constructed model to the ``"b200"`` backend; returns how many.

    The sampler's token transformer runs in float32 in K-Fold (model/model.py:409-429).  Under float32 compute the
    backend takes its fp32-accurate path (split-operand GEMMs around a CUDA-core attention kernel), which is
    correct but slow; its attention modules (call site "diffusion_global") are therefore left alone unless
    ``diffusion`` is set.
    """
    n = 0
    for m in model.modules():
        name = type(m).__name__
        if name in ("TriangleMultiplicationOutgoing", "TriangleMultiplicationIncoming"):
            c = m.layernorm_in.normalized_shape
            if c % 64 == 0 and 64 <= c <= 512:
                m.kernel_backend = BACKEND
                n += 1
        elif name in ("TriangleAttentionStartingNode", "TriangleAttentionEndingNode", "TriangleAttention"):
            d = m.c_hidden
            if d % 8 == 0 and 16 <= d <= 64 and m.inf == 1e9:
                m.kernel_backend = BACKEND
                n += 1
        elif name == "SelfAttentionPairBias" and apb_supported(m):
            if getattr(m, "call_site", "") == "diffusion_global" and not diffusion:
                continue
            m.kernel_backend = BACKEND
            n += 1
        elif name == "CrossAttentionPairBias" and apb_supported(m) and diffusion:
            # the atom transformers of the sampler and of the input embedder ("diffusion_local"); float32 there too
            m.kernel_backend = BACKEND
            n += 1
    return n
