"""Host-side mirror of the reference modules on the hot path.

Same class names, constructor arguments, parameter names (so a reference
``state_dict`` loads with ``strict=True``) and ``forward`` signatures as the K-Fold
modules they stand in for, with the CUDA kernels behind them:

  TriangleMultiplicationOutgoing / Incoming   model/primitives/triangle_multiplication.py:148-313
  TriangleAttentionStartingNode / EndingNode  model/primitives/triangle_attention.py:338-465
  Transition                                  model/layers/folding/transition.py:20-68
  SelfAttentionPairBias (channel_s=None)      model/layers/folding/attention_pair_bias.py:70-158
  TriangularBlock                             model/modules/tri_stack.py:86-151
  PairformerBlock (pair + single track)       model/modules/apo_module.py:107-172 +
                                              model/modules/confidence_head.py:125-175

Conventions copied from the reference's Triton backend
(model/primitives/triangle_multiplication.py:94-145): inference only (``RuntimeError``
when autograd is recording or the input is not on a CUDA device), compute dtype =
autocast dtype if autocast is on else the input dtype, result returned in the input
dtype, weights packed once per module and re-packed when a parameter's storage or
version changes.
"""
from __future__ import annotations

import torch
from torch import nn

from . import functional as F
from . import packing

__all__ = [
    "LayerNorm", "LinearNoBias", "Linear",
    "TriangleMultiplicationOutgoing", "TriangleMultiplicationIncoming",
    "TriangleAttentionStartingNode", "TriangleAttentionEndingNode",
    "Transition", "AdaLN", "SelfAttentionPairBias", "ConditionedTransitionBlock", "CachedGlobalTransformerBlock",
    "CachedGlobalTransformerStack", "TriangularBlock", "PairformerBlock",
]


# --------------------------------------------------------------------------------------------
# parameter holders (names match the reference so that state dicts are interchangeable)
# --------------------------------------------------------------------------------------------
class LayerNorm(nn.Module):
    """LayerNorm with fp32 statistics (model/primitives/normalization.py:24-91)."""

    def __init__(self, normalized_shape: int, create_scale: bool = True, create_offset: bool = True, eps: float = 1e-5):
        super().__init__()
        self.normalized_shape = normalized_shape
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(normalized_shape)) if create_scale else None
        self.bias = nn.Parameter(torch.zeros(normalized_shape)) if create_offset else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        _check_inference(x)
        return F.layer_norm(x, self.weight, self.bias, self.eps)


class Linear(nn.Module):
    """Parameter holder for a projection; N(0, 1/fan_in) init (model/primitives/linear.py:25-107)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(out_features, in_features) * in_features ** -0.5)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)


class LinearNoBias(Linear):
    def __init__(self, in_features: int, out_features: int):
        super().__init__(in_features, out_features, bias=False)


class _SwiGLU(nn.Module):
    def __init__(self, channel_in: int, channel_out: int):
        super().__init__()
        self.linear = LinearNoBias(channel_in, channel_out * 2)


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def _check_inference(x: torch.Tensor) -> None:
    if torch.is_grad_enabled():
        raise RuntimeError("The kfold_b200 kernel backend is inference-only (run under torch.no_grad()).")
    if not x.is_cuda:
        raise RuntimeError("The kfold_b200 kernel backend requires CUDA tensors.")


def compute_dtype(x: torch.Tensor) -> torch.dtype:
    """Autocast dtype when autocast is on, else the input dtype
    (model/primitives/triangle_multiplication.py:67-70)."""
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type)
    return x.dtype


def _is_precise(dt: torch.dtype, what: str) -> bool:
    """bfloat16 compute -> the tensor-core path; float32 compute -> the fp32-accurate path (split operands)."""
    if dt == torch.bfloat16:
        return False
    if dt == torch.float32:
        return True
    raise NotImplementedError(f"{what}: compute dtype {dt} is not available (bfloat16 and float32 are)")


def _tensor_key(t: torch.Tensor) -> tuple:
    """Identity of an activation tensor for a cache: storage address, shape, dtype and in-place version.  Tensors created
    under ``torch.inference_mode()`` (how the reference runs, model/model.py:294 and :361) carry no version counter; for
    them the key has no version, and a caller that overwrites such a tensor in place must call ``reset_caches()``."""
    return (t.data_ptr(), tuple(t.shape), t.dtype, None if torch.is_inference(t) else t._version)


class _PackedMixin:
    """Packs the module's weights once and re-packs when any parameter changes
    (same cache key as model/primitives/triangle_multiplication.py:73-91)."""

    _pack_cache = None
    _pack_key = None

    def _packed(self, device: torch.device, dtype: torch.dtype, pack_fn):
        key = (device.type, device.index, dtype) + tuple(
            v for p in self.parameters() for v in (p.data_ptr(), None if torch.is_inference(p) else p._version))
        if self._pack_cache is None or self._pack_key != key:
            sd = {k: v for k, v in self.state_dict().items()}
            self._pack_cache = pack_fn(sd, device)
            self._pack_key = key
        return self._pack_cache


# --------------------------------------------------------------------------------------------
# primitives
# --------------------------------------------------------------------------------------------
class _TriangleMultiplication(nn.Module, _PackedMixin):
    direction = "outgoing"

    def __init__(self, dim: int = 128, kernel_backend: str = "b200") -> None:
        super().__init__()
        self.kernel_backend = kernel_backend
        self.layernorm_in = LayerNorm(dim)
        self.linear_p_in = LinearNoBias(dim, 2 * dim)
        self.linear_g_in = LinearNoBias(dim, 2 * dim)
        self.layernorm_out = LayerNorm(dim)
        self.linear_p_out = LinearNoBias(dim, dim)
        self.linear_g_out = LinearNoBias(dim, dim)

    @torch.compiler.disable
    def forward(self, x: torch.Tensor, mask: torch.Tensor, residual: bool = False) -> torch.Tensor:
        """x (B,N,N,D), mask (B,N,N) -> update (B,N,N,D); with ``residual`` returns x + update."""
        _check_inference(x)
        cd = compute_dtype(x)
        precise = _is_precise(cd, type(self).__name__)
        pk = self._packed(x.device, cd, lambda sd, dev: packing.pack_trimul(sd, dev, precise=precise))
        with torch.autocast(x.device.type, enabled=False):
            out = F.triangle_multiplication(x.float() if precise else x, mask, pk, self.direction,
                                            eps=self.layernorm_in.eps, residual=residual)
        return out.to(x.dtype)


class TriangleMultiplicationOutgoing(_TriangleMultiplication):
    direction = "outgoing"


class TriangleMultiplicationIncoming(_TriangleMultiplication):
    direction = "incoming"


class _MHAParams(nn.Module):
    def __init__(self, c_in: int, c_hidden: int, no_heads: int):
        super().__init__()
        self.linear_q = LinearNoBias(c_in, c_hidden * no_heads)
        self.linear_k = LinearNoBias(c_in, c_hidden * no_heads)
        self.linear_v = LinearNoBias(c_in, c_hidden * no_heads)
        self.linear_o = LinearNoBias(c_hidden * no_heads, c_in)
        self.linear_g = LinearNoBias(c_in, c_hidden * no_heads)


class _TriangleAttention(nn.Module, _PackedMixin):
    starting = True

    def __init__(self, c_in: int, no_heads: int, inf: float = 1e9, kernel_backend: str = "b200") -> None:
        super().__init__()
        assert c_in % no_heads == 0, f"c_in ({c_in}) must be divisible by no_heads ({no_heads})"
        if inf != 1e9:
            raise ValueError("the kernel's key-mask offset is fixed at 1e9 (the reference default)")
        self.c_in, self.no_heads, self.c_hidden, self.inf = c_in, no_heads, c_in // no_heads, inf
        self.kernel_backend = kernel_backend
        self.layer_norm = LayerNorm(c_in)
        self.linear = LinearNoBias(c_in, no_heads)
        self.mha = _MHAParams(c_in, self.c_hidden, no_heads)

    @torch.compiler.disable
    def forward(self, x: torch.Tensor, mask: torch.Tensor | None = None, residual: bool = False) -> torch.Tensor:
        """x (*,I,J,C), mask (*,I,J) or None -> update (*,I,J,C)."""
        _check_inference(x)
        cd = compute_dtype(x)
        precise = _is_precise(cd, type(self).__name__)
        pk = self._packed(x.device, cd, lambda sd, dev: packing.pack_triatt(sd, self.no_heads, dev, precise=precise))
        lead = x.shape[:-3]
        x4 = x.reshape(-1, *x.shape[-3:])
        if precise:
            x4 = x4.float()
        m4 = None if mask is None else mask.reshape(-1, *mask.shape[-2:])
        with torch.autocast(x.device.type, enabled=False):
            out = F.triangle_attention(x4, m4, pk, self.starting, eps=self.layer_norm.eps, residual=residual)
        return out.reshape(*lead, *x.shape[-3:]).to(x.dtype)


class TriangleAttentionStartingNode(_TriangleAttention):
    starting = True


class TriangleAttentionEndingNode(_TriangleAttention):
    starting = False


class Transition(nn.Module, _PackedMixin):
    def __init__(self, channel: int, expansion_factor: int) -> None:
        super().__init__()
        self.model_dim = channel * expansion_factor
        self.layernorm = LayerNorm(channel)
        self.swiglu = _SwiGLU(channel, self.model_dim)
        self.linear_out = LinearNoBias(self.model_dim, channel)

    @torch.compiler.disable
    def forward(self, x: torch.Tensor, residual: bool = False) -> torch.Tensor:
        _check_inference(x)
        cd = compute_dtype(x)
        precise = _is_precise(cd, "Transition")
        pk = self._packed(x.device, cd, lambda sd, dev: packing.pack_transition(sd, dev, precise=precise))
        with torch.autocast(x.device.type, enabled=False):
            out = F.transition(x.float() if precise else x, pk, eps=self.layernorm.eps, residual=residual)
        return out.to(x.dtype)


class AdaLN(nn.Module, _PackedMixin):
    """Adaptive LayerNorm (model/primitives/normalization.py:94-125)."""

    def __init__(self, channel_a: int, channel_s: int):
        super().__init__()
        self.channel_a, self.channel_s = channel_a, channel_s
        self.layernorm_s = LayerNorm(channel_s, create_scale=True, create_offset=False)
        self.linear_g = Linear(channel_s, channel_a)
        self.linear_bias = LinearNoBias(channel_s, channel_a)

    def gate_shift(self, s: torch.Tensor, precise: bool = False) -> torch.Tensor:
        """[sigmoid logits | shift] of the conditioning, (..., L, 2 c_a): one small LayerNorm + GEMM per token.
        bf16, or float32 from the split-operand GEMM when ``precise``."""
        if precise:
            pk = self._packed(s.device, torch.float32, lambda sd, dev: packing.pack_adaln(sd, dev, precise=True))
            sn = F.layer_norm(s.float(), pk["ln_s_w"], None, self.layernorm_s.eps, out_dtype=torch.float32)
            return F.linear_fp32(sn, pk["w_gs"], pk["b_gs"])
        pk = self._packed(s.device, torch.bfloat16, packing.pack_adaln)
        sn = F.layer_norm(s, pk["ln_s_w"], None, self.layernorm_s.eps, out_dtype=torch.bfloat16)
        return F.linear(sn, pk["w_gs"], pk["b_gs"])

    @torch.compiler.disable
    def forward(self, a: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
        """a (B, Ns, L, c_a), s (B, 1 or Ns, L, c_s) -> (B, Ns, L, c_a): bf16 under bfloat16 compute, float32 under
        float32 compute."""
        _check_inference(a)
        precise = _is_precise(compute_dtype(a), "AdaLN")
        with torch.autocast(a.device.type, enabled=False):
            samples = _sample_share(a, s)
            return F.adaln(a, self.gate_shift(s, precise), samples)


def _sample_share(a: torch.Tensor, s: torch.Tensor) -> int:
    """How many consecutive samples of `a` share one conditioning row of `s` (its sample dim is 1 or equal)."""
    if a.dim() < 3 or s.dim() != a.dim():
        return 1
    if s.shape[-3] == 1 and a.shape[-3] != 1:
        return int(a.shape[-3])
    return 1


class _ConditioningBank:
    """The conditioning projections of EVERY block of a stack from one LayerNorm and two GEMMs.

    Each AdaLN computes sigmoid-gate and shift rows from LayerNorm_s(s) with its own scale, and each block adds output
    gates Linear(s).  All of them depend on s alone, so the stack normalises s once (the per-AdaLN scale is folded into
    that AdaLN's weight columns), multiplies once by all stacked AdaLN matrices and once by all stacked gate matrices,
    and every block reads its columns of the two wide tables in place (the kernels take a row stride).
    bfloat16 compute only: folding the scale moves a bf16 rounding, which the float32-accurate path must not do."""

    def __init__(self):
        self._key = None
        self._packed = None

    def _pack(self, adalns, gates, device):
        params = [p for m in adalns for p in (m.layernorm_s.weight, m.linear_g.weight, m.linear_g.bias, m.linear_bias.weight)]
        params += [p for g in gates for p in (g.weight, g.bias)]
        key = (device,) + tuple(v for p in params for v in (p.data_ptr(), None if torch.is_inference(p) else p._version))
        if self._key != key:
            w1, b1 = [], []
            for m in adalns:
                gamma = m.layernorm_s.weight.detach().float()[None, :]
                w1 += [m.linear_g.weight.detach().float() * gamma, m.linear_bias.weight.detach().float() * gamma]
                b1 += [m.linear_g.bias.detach().float(), torch.zeros_like(m.linear_g.bias, dtype=torch.float32)]
            w2 = [g.weight.detach().float() for g in gates]
            b2 = [g.bias.detach().float() for g in gates]
            bf = torch.bfloat16
            self._packed = (torch.cat(w1).to(device, bf).contiguous(), torch.cat(b1).to(device).contiguous(),
                            torch.cat(w2).to(device, bf).contiguous(), torch.cat(b2).to(device).contiguous())
            self._key = key
        return self._packed

    def tables(self, s: torch.Tensor, adalns, gates):
        """-> (gate_shift, out_gate): lists of views, one per AdaLN (..., L, 2 c_a) and one per gate (..., L, c_a)."""
        eps = adalns[0].layernorm_s.eps
        w1, b1, w2, b2 = self._pack(adalns, gates, s.device)
        sn = F.layer_norm(s, None, None, eps, out_dtype=torch.bfloat16)
        t1 = F.linear(sn, w1, b1)
        t2 = F.linear(s, w2, b2)
        gs, off = [], 0
        for m in adalns:
            gs.append(t1[..., off: off + 2 * m.channel_a])
            off += 2 * m.channel_a
        og, off = [], 0
        for g in gates:
            og.append(t2[..., off: off + g.weight.shape[0]])
            off += g.weight.shape[0]
        return gs, og


class SelfAttentionPairBias(nn.Module, _PackedMixin):
    """Pair-bias self-attention: the single-track form (``channel_s=None``, LayerNorm prologue) and the diffusion
    form (AdaLN prologue and the sigmoid(Linear(s)) output gate), model/layers/folding/attention_pair_bias.py:70-158."""

    def __init__(self, channel_a: int, num_heads: int, channel_s: int | None, call_site: str, inf: float = 1e9,
                 kernel_backend: str = "b200") -> None:
        super().__init__()
        if call_site not in {"diffusion_global", "confidence"}:
            raise ValueError(f"Unsupported self APB call site: {call_site!r}")
        if inf != 1e9:
            raise ValueError("the kernel's key-mask offset is fixed at 1e9 (the reference default)")
        assert channel_a % num_heads == 0
        self.channel_a, self.num_heads, self.head_dim, self.inf = channel_a, num_heads, channel_a // num_heads, inf
        self.call_site, self.kernel_backend = call_site, kernel_backend
        self.use_single_conditioning = channel_s is not None
        self.linear_q = Linear(channel_a, channel_a)
        self.linear_k = LinearNoBias(channel_a, channel_a)
        self.linear_v = LinearNoBias(channel_a, channel_a)
        self.linear_g = LinearNoBias(channel_a, channel_a)
        self.linear_out = LinearNoBias(channel_a, channel_a)
        if self.use_single_conditioning:
            self.adaln_a = AdaLN(channel_a, channel_s)
            self.linear_ada_out = Linear(channel_s, channel_a)
        else:
            self.layernorm_a = LayerNorm(channel_a, create_offset=True)
        self._ada_w = None
        self._ada_key = None

    def _apb_packed(self, device, precise: bool = False):
        keys = ("linear_q.weight", "linear_q.bias", "linear_k.weight", "linear_v.weight", "linear_g.weight",
                "linear_out.weight")
        return self._packed(device, torch.float32 if precise else torch.bfloat16,
                            lambda sd, dev: packing.pack_apb({k: sd[k] for k in keys}, self.num_heads, dev, precise=precise))

    def _ada_out(self, device, precise: bool = False):
        w, b = self.linear_ada_out.weight, self.linear_ada_out.bias
        key = (device, precise, w.data_ptr(), b.data_ptr(), None if torch.is_inference(w) else (w._version, b._version))
        if self._ada_key != key:
            wd = packing.split3_weights(w).to(device) if precise else w.detach().to(device, torch.bfloat16).contiguous()
            self._ada_w = (wd, b.detach().to(device, torch.float32).contiguous())
            self._ada_key = key
        return self._ada_w

    @torch.compiler.disable
    def forward(self, a: torch.Tensor, s: torch.Tensor | None, pair_bias: torch.Tensor, mask: torch.Tensor,
                residual: bool = False, cond=None) -> torch.Tensor:
        """a (...,L,c_a); s (...,L,c_s) or None; pair_bias (...,H,L,L); mask (...,L) -> (...,L,c_a).
        With ``residual`` the result is a + update (fused into the last kernel).  ``cond``: the (gate/shift rows, output
        gate logits) of this module taken from a stack's conditioning tables (bfloat16 compute)."""
        _check_inference(a)
        precise = _is_precise(compute_dtype(a), "SelfAttentionPairBias")
        pk = self._apb_packed(a.device, precise)
        with torch.autocast(a.device.type, enabled=False):
            if cond is not None and not precise and self.use_single_conditioning:
                share = _sample_share(a, s)
                an = F.adaln(a, cond[0], share)
                return F.attention_pair_bias(an, pair_bias, mask, pk, out_dtype=a.dtype, out_gate=cond[1], gate_share=share,
                                             resid=a if residual else None)
            if precise and self.use_single_conditioning:
                assert s is not None
                share = _sample_share(a, s)
                an = F.adaln(a.float(), self.adaln_a.gate_shift(s, True), share)
                w6, b_ada = self._ada_out(a.device, True)
                gate = F.linear_fp32(s.float(), w6, b_ada)
                return F.attention_pair_bias(an, pair_bias, mask, pk, out_dtype=a.dtype, out_gate=gate, gate_share=share,
                                             resid=a if residual else None)
            if precise:
                an = F.layer_norm(a.float(), self.layernorm_a.weight, self.layernorm_a.bias, self.layernorm_a.eps,
                                  out_dtype=torch.float32)
                return F.attention_pair_bias(an, pair_bias, mask, pk, out_dtype=a.dtype, resid=a if residual else None)
            if self.use_single_conditioning:
                assert s is not None
                share = _sample_share(a, s)
                an = F.adaln(a, self.adaln_a.gate_shift(s), share)
                w_ada, b_ada = self._ada_out(a.device)
                gate = F.linear(s, w_ada, b_ada)
                return F.attention_pair_bias(an, pair_bias, mask, pk, out_dtype=a.dtype, out_gate=gate, gate_share=share,
                                             resid=a if residual else None)
            assert s is None
            an = F.layer_norm(a, self.layernorm_a.weight, self.layernorm_a.bias, self.layernorm_a.eps, out_dtype=torch.bfloat16)
            return F.attention_pair_bias(an, pair_bias, mask, pk, out_dtype=a.dtype, resid=a if residual else None)


class ConditionedTransitionBlock(nn.Module, _PackedMixin):
    """model/layers/folding/diffusion_transformer.py:45-81."""

    def __init__(self, channel_a: int, channel_s: int, expansion_factor: int = 2):
        super().__init__()
        model_dim = int(channel_a * expansion_factor)
        self.adaln = AdaLN(channel_a, channel_s)
        self.swiglu = _SwiGLU(channel_a, model_dim)
        self.linear_g = Linear(channel_s, channel_a)
        self.linear_out = LinearNoBias(model_dim, channel_a)

    @torch.compiler.disable
    def forward(self, a: torch.Tensor, s: torch.Tensor, residual: bool = False, precise: bool | None = None,
                cond=None) -> torch.Tensor:
        """``precise`` overrides the choice made from the compute dtype (for callers that already run with autocast
        switched off).  ``cond``: (gate/shift rows, output gate logits) from a stack's conditioning tables."""
        _check_inference(a)
        if precise is None:
            precise = _is_precise(compute_dtype(a), "ConditionedTransitionBlock")
        pk = self._packed(a.device, torch.float32 if precise else torch.bfloat16,
                          lambda sd, dev: packing.pack_cond_transition(sd, dev, precise=precise))
        with torch.autocast(a.device.type, enabled=False):
            share = _sample_share(a, s)
            if precise:
                an = F.adaln(a.float(), self.adaln.gate_shift(s, True), share)
                gate = F.linear_fp32(s.float(), pk["w_g"], pk["b_g"])
            elif cond is not None:
                an, gate = F.adaln(a, cond[0], share), cond[1]
            else:
                an = F.adaln(a, self.adaln.gate_shift(s), share)
                gate = F.linear(s, pk["w_g"], pk["b_g"])
            return F.conditioned_transition(an, pk, gate, share, resid=a if residual else None, out_dtype=a.dtype)


class SingleConditioning(nn.Module):
    """model/layers/folding/diffusion.py:97-152 (AF3 Algorithm 21, single part): float32 Linear(s_inputs) plus the
    float32 projection of the normalised Fourier features of the noise level, broadcast over tokens and samples, then two
    Transitions.  The two projections are float32 in the reference whatever the autocast state; they run on the
    split-operand tensor-core GEMM.  The Fourier weights are the reference's (torch.randn with generator seed 42 on
    the CPU, non-persistent buffers)."""

    def __init__(self, channel_s: int = 384, dim_fourier: int = 256):
        super().__init__()
        gen = torch.Generator()
        gen.manual_seed(42)
        self.register_buffer("fourier_w", torch.randn(size=(1, dim_fourier), generator=gen, device="cpu"), persistent=False)
        self.register_buffer("fourier_b", torch.randn(size=(1, dim_fourier), generator=gen, device="cpu"), persistent=False)
        self.layernorm_fourier = LayerNorm(dim_fourier, create_offset=False)
        self.linear_fourier = LinearNoBias(dim_fourier, channel_s)
        self.linear = LinearNoBias(channel_s, channel_s)
        self.transitions = nn.ModuleList([Transition(channel_s, expansion_factor=2) for _ in range(2)])
        self._proj = _ProjectionCache()

    @torch.compiler.disable
    def forward(self, s_inputs: torch.Tensor, c_noise: torch.Tensor) -> torch.Tensor:
        """s_inputs (B, Lt, c_s); c_noise (B, N) -> (B, N, Lt, c_s)."""
        _check_inference(s_inputs)
        with torch.autocast(s_inputs.device.type, enabled=False):
            dev = s_inputs.device
            s = F.linear_fp32(s_inputs.float(), self._proj.get(self.linear, dev, True), None)
            emb = F.fourier_embed(c_noise, self.fourier_w, self.fourier_b)
            ln = self.layernorm_fourier
            emb = F.layer_norm(emb, ln.weight, ln.bias, ln.eps, out_dtype=torch.float32)
            emb = F.linear_fp32(emb, self._proj.get(self.linear_fourier, dev, True), None)
            s = F.broadcast_add(s, emb).to(s_inputs.dtype)
        for transition in self.transitions:
            s = transition(s, residual=True)
        return s


class TokenPairBias(nn.Module):
    """The pair bias of the token transformer, ``DiffusionStack.get_pair_bias`` (model/layers/folding/diffusion.py:290-294
    and :397-416): LayerNorm(z) projected to blocks x heads values per pair, laid out (B, Nblock, H, L, L).  Parameter
    names as in DiffusionStack (``layernorm_z``, ``linear_z_to_bias``).  The result is bf16 (float32 under float32
    compute) and is what CachedGlobalTransformerStack consumes without another conversion or copy; it does not depend
    on the noise level, so one call serves all sampler steps."""

    def __init__(self, channel_z: int, token_transformer_blocks: int = 24, token_transformer_heads: int = 16):
        super().__init__()
        self.blocks, self.heads = token_transformer_blocks, token_transformer_heads
        self.layernorm_z = LayerNorm(channel_z, create_offset=False)
        self.linear_z_to_bias = LinearNoBias(channel_z, token_transformer_blocks * token_transformer_heads)
        self._cache = {}

    @torch.compiler.disable
    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return _token_pair_bias(z, self.layernorm_z, self.linear_z_to_bias, self.blocks, self.heads, self._cache)


def _token_pair_bias(z: torch.Tensor, layernorm_z, linear_z_to_bias, blocks: int, heads: int, cache: dict) -> torch.Tensor:
    """LayerNorm(z) projected to blocks x heads values per pair, laid out (B, Nblock, H, L, L)
    (model/layers/folding/diffusion.py:411-416); `cache` keeps the device copy of the projection weight."""
    _check_inference(z)
    precise = _is_precise(compute_dtype(z), "TokenPairBias")
    w = linear_z_to_bias.weight
    key = (z.device, precise, w.data_ptr(), None if torch.is_inference(w) else w._version)
    if cache.get("key") != key:
        cache["w"] = packing.split3_weights(w).to(z.device) if precise else w.detach().to(z.device, torch.bfloat16).contiguous()
        cache["key"] = key
    b, l = z.shape[0], z.shape[1]
    lp = (l + 7) // 8 * 8
    with torch.autocast(z.device.type, enabled=False):
        zz = z.float() if precise else z.to(torch.bfloat16)
        if lp != l:
            zz = torch.nn.functional.pad(zz, (0, 0, 0, lp - l, 0, lp - l))
        out = F.pair_bias(zz, layernorm_z.weight.detach().float(), None, cache["w"], layernorm_z.eps)      # (B, blocks*H, L, L)
    out = out.view(b, blocks, heads, lp, lp)
    return out if lp == l else out[..., :l, :l]


class CachedGlobalTransformerBlock(nn.Module):
    """model/layers/folding/diffusion_transformer.py:342-413: a += attention(a, s, bias, mask); a += transition(a, s)."""

    def __init__(self, channel_a: int, channel_s: int, num_heads: int, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.attention = SelfAttentionPairBias(channel_a, num_heads, channel_s, call_site="diffusion_global")
        self.transition = ConditionedTransitionBlock(channel_a, channel_s)

    def forward(self, a: torch.Tensor, s: torch.Tensor, pair_bias: torch.Tensor, mask: torch.Tensor, cond=None) -> torch.Tensor:
        """``cond``: ((attention gate/shift, attention output gate), (transition gate/shift, transition output gate)) from
        the stack's conditioning tables."""
        a = self.attention(a, s, pair_bias, mask, residual=True, cond=None if cond is None else cond[0])
        return self.transition(a, s, residual=True, cond=None if cond is None else cond[1])


class CachedGlobalTransformerStack(nn.Module):
    """model/layers/folding/diffusion_transformer.py:260-339.  pair_bias (*, Nblock, H, L, L), as produced by
    DiffusionStack.get_pair_bias; it is converted to bf16 once per tensor and reused across sampler steps."""

    def __init__(self, channel_a: int, channel_s: int, num_heads: int, num_blocks: int, blocks_per_ckpt=None,
                 kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.blocks = nn.ModuleList(
            [CachedGlobalTransformerBlock(channel_a, channel_s, num_heads) for _ in range(num_blocks)])
        self._bias_cache = None
        self._bias_key = None
        self._bias_src = None
        self._bank = _ConditioningBank()

    def _prepared_bias(self, pair_bias: torch.Tensor, precise: bool = False):
        key = _tensor_key(pair_bias) + (precise,)
        if self._bias_key != key:
            # (*, N, H, L, L) -> N tensors (*, H, L, L), contiguous: bf16 for the tensor-core kernel, float32 for the
            # fp32-accurate one
            pb = pair_bias.movedim(-4, 0).to(torch.float32 if precise else torch.bfloat16).contiguous()
            self._bias_cache, self._bias_key = pb, key
            # the conversion may have copied: keep the source alive, so that its address cannot be handed to the bias of
            # the next complex (same shape, version 0) while this entry is still in the cache
            self._bias_src = pair_bias
        return self._bias_cache

    def reset_caches(self) -> None:
        """Forget the converted pair bias (call once per complex when the bias tensor is overwritten in place under
        ``torch.inference_mode()``, where tensors carry no version counter)."""
        self._bias_cache = self._bias_key = self._bias_src = None

    @torch.compiler.disable
    def forward(self, a: torch.Tensor, s: torch.Tensor, pair_bias: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        _check_inference(a)
        precise = _is_precise(compute_dtype(a), "CachedGlobalTransformerStack")
        pb = self._prepared_bias(pair_bias, precise)
        conds = [None] * len(self.blocks)
        if not precise:
            # the conditioning projections of all blocks: one LayerNorm of s and two GEMMs
            with torch.autocast(a.device.type, enabled=False):
                gs, og = self._bank.tables(s, [m for b in self.blocks for m in (b.attention.adaln_a, b.transition.adaln)],
                                           [g for b in self.blocks for g in (b.attention.linear_ada_out, b.transition.linear_g)])
            conds = [((gs[2 * i], og[2 * i]), (gs[2 * i + 1], og[2 * i + 1])) for i in range(len(self.blocks))]
        for i, blk in enumerate(self.blocks):
            a = blk(a, s, pb[i], mask, cond=conds[i])
        return a


# --------------------------------------------------------------------------------------------
# atom-level local transformer: windows of 32 queries attending 128 keys
# --------------------------------------------------------------------------------------------
WINDOW_Q, WINDOW_K = 32, 128


def build_atom_to_qk_fn(length: int, device):
    """Window indexing of the local attention (model/layers/folding/utils.py:97-188): window w holds queries
    [32 w, 32 w + 32) and keys [32 w - 48, 32 w + 80); keys outside [0, length) are zero-filled.  Returns
    fn(x, dim) -> (x_q, x_k) that unflattens dimension `dim` into (W, 32) and gathers it into (W, 128)."""
    if length % WINDOW_Q != 0:
        raise ValueError("Length must be divisible by 32")
    windows = length // WINDOW_Q
    idx = torch.arange(windows, device=device)[:, None] * WINDOW_Q - 48 + torch.arange(WINDOW_K, device=device)[None, :]
    pad = (idx < 0) | (idx >= length)
    idx = idx.clamp(0, length - 1).reshape(-1)

    def to_qk(x: torch.Tensor, dim: int):
        dim = dim % x.ndim
        x_q = x.unflatten(dim, (windows, WINDOW_Q))
        x_k = x.index_select(dim, idx).unflatten(dim, (windows, WINDOW_K))
        shape = [1] * x_k.ndim
        shape[dim], shape[dim + 1] = windows, WINDOW_K
        return x_q, x_k.masked_fill(pad.view(shape), 0)

    return to_qk


def _bias_sharing(lead: tuple, bias_lead: tuple):
    """How a bias with leading dims `bias_lead` (1 = broadcast) is shared by a batch with leading dims `lead` ordered
    (group..., shared..., window...): (bias_div, bias_mod) for the kernels, or None when the pattern is not of that form."""
    bl = (1,) * (len(lead) - len(bias_lead)) + tuple(bias_lead)
    i = 0
    while i < len(lead) and bl[i] == lead[i]:
        i += 1
    j = i
    while j < len(lead) and bl[j] == 1:
        j += 1
    if any(bl[k] != lead[k] for k in range(j, len(lead))):
        return None
    shared = windows = 1
    for d in lead[i:j]:
        shared *= d
    for d in lead[j:]:
        windows *= d
    if shared > 1 and windows > 1:
        return shared * windows, windows
    return (shared if windows == 1 else 1), 0


def _index_share(lead: tuple, other_lead: tuple):
    """n such that entry b of a batch with leading dims `lead` uses row b // n of a tensor whose leading dims `other_lead`
    equal `lead` up to trailing 1s (those dims are shared); None for any other broadcast pattern."""
    return F._index_sharing(lead, other_lead)


class CrossAttentionPairBias(nn.Module, _PackedMixin):
    """Pair-bias cross attention of the atom windows (model/layers/folding/attention_pair_bias.py:161-260): AdaLN (or
    LayerNorm) prologues for the query and the key side, attention with `call_site="diffusion_local"`, and the
    sigmoid(Linear(s_q)) output gate."""

    def __init__(self, channel_a: int, num_heads: int, channel_s: int | None, inf: float = 1e9, kernel_backend: str = "b200"):
        super().__init__()
        if inf != 1e9:
            raise ValueError("the kernel's key-mask offset is fixed at 1e9 (the reference default)")
        assert channel_a % num_heads == 0
        self.channel_a, self.num_heads, self.head_dim, self.inf = channel_a, num_heads, channel_a // num_heads, inf
        self.kernel_backend = kernel_backend
        self.use_single_conditioning = channel_s is not None
        self.linear_q = Linear(channel_a, channel_a)
        self.linear_k = LinearNoBias(channel_a, channel_a)
        self.linear_v = LinearNoBias(channel_a, channel_a)
        self.linear_g = LinearNoBias(channel_a, channel_a)
        self.linear_out = LinearNoBias(channel_a, channel_a)
        if self.use_single_conditioning:
            self.adaln_a_q = AdaLN(channel_a, channel_s)
            self.adaln_a_k = AdaLN(channel_a, channel_s)
            self.linear_ada_out = Linear(channel_s, channel_a)
        else:
            self.layernorm_a_q = LayerNorm(channel_a, create_offset=True)
            self.layernorm_a_k = LayerNorm(channel_a, create_offset=True)
        self._ada_w = None
        self._ada_key = None

    _ada_out = SelfAttentionPairBias._ada_out

    def _cross_packed(self, device, precise: bool = False):
        keys = ("linear_q.weight", "linear_q.bias", "linear_k.weight", "linear_v.weight", "linear_g.weight", "linear_out.weight")
        return self._packed(device, torch.float32 if precise else torch.bfloat16,
                            lambda sd, dev: packing.pack_apb_cross({k: sd[k] for k in keys}, self.num_heads, dev, precise=precise))

    def normed_inputs(self, a: torch.Tensor, s: torch.Tensor | None, precise: bool, cond=None):
        """Query-side and key-side prologues on the un-windowed rows a (..., L, c_a), s (..., L, c_s), and the logits of
        the output gate (or None).  Both prologues are row-wise, so windows can be cut afterwards.  ``cond``: (query
        gate/shift rows, key gate/shift rows, output gate logits) from a stack's conditioning tables."""
        if self.use_single_conditioning:
            assert s is not None
            share = _sample_share(a, s)
            if cond is not None and not precise:
                return F.adaln(a, cond[0], share), F.adaln(a, cond[1], share), cond[2]
            af = a.float() if precise else a
            xq = F.adaln(af, self.adaln_a_q.gate_shift(s, precise), share)
            xk = F.adaln(af, self.adaln_a_k.gate_shift(s, precise), share)
            w_ada, b_ada = self._ada_out(a.device, precise)
            gate = F.linear_fp32(s.float(), w_ada, b_ada) if precise else F.linear(s, w_ada, b_ada)
            return xq, xk, gate
        assert s is None
        dt = torch.float32 if precise else torch.bfloat16
        af = a.float() if precise else a
        lq, lk = self.layernorm_a_q, self.layernorm_a_k
        return (F.layer_norm(af, lq.weight, lq.bias, lq.eps, out_dtype=dt), F.layer_norm(af, lk.weight, lk.bias, lk.eps, out_dtype=dt),
                None)

    @torch.compiler.disable
    def forward(self, a_q: torch.Tensor, a_k: torch.Tensor, s_q: torch.Tensor | None, s_k: torch.Tensor | None,
                pair_bias: torch.Tensor, mask: torch.Tensor, residual: bool = False) -> torch.Tensor:
        """The reference's signature on windowed tensors: a_q (..., W, Lq, c_a), a_k (..., W, Lk, c_a), s_q / s_k alike with
        c_s, pair_bias (..., W, H, Lq, Lk), mask (..., W, Lk) -> (..., W, Lq, c_a).  With ``residual`` the result is
        a_q + update (fused into the last kernel)."""
        _check_inference(a_q)
        precise = _is_precise(compute_dtype(a_q), "CrossAttentionPairBias")
        pk = self._cross_packed(a_q.device, precise)
        with torch.autocast(a_q.device.type, enabled=False):
            flat = lambda t: None if t is None else t.flatten(-3, -2)
            if self.use_single_conditioning:
                assert s_q is not None and s_k is not None
                aqf, akf, sqf, skf = flat(a_q), flat(a_k), flat(s_q), flat(s_k)
                cast = (lambda t: t.float()) if precise else (lambda t: t)
                xq = F.adaln(cast(aqf), self.adaln_a_q.gate_shift(sqf, precise), _sample_share(aqf, sqf)).view(a_q.shape)
                xk = F.adaln(cast(akf), self.adaln_a_k.gate_shift(skf, precise), _sample_share(akf, skf)).view(a_k.shape)
            else:
                assert s_q is None and s_k is None
                dt = torch.float32 if precise else torch.bfloat16
                lq, lk = self.layernorm_a_q, self.layernorm_a_k
                xq = F.layer_norm(a_q.float() if precise else a_q, lq.weight, lq.bias, lq.eps, out_dtype=dt)
                xk = F.layer_norm(a_k.float() if precise else a_k, lk.weight, lk.bias, lk.eps, out_dtype=dt)
            gate = None
            if self.use_single_conditioning:
                w_ada, b_ada = self._ada_out(a_q.device, precise)
                gate = F.linear_fp32(s_q.float(), w_ada, b_ada) if precise else F.linear(s_q, w_ada, b_ada)
            return F.attention_pair_bias_cross_bcast(xq, xk, pair_bias, mask, pk, out_dtype=a_q.dtype, out_gate=gate,
                                                     resid=a_q if residual else None)


class LocalTransformerBlock(nn.Module):
    """model/layers/folding/diffusion_transformer.py:515-597: a_q += attention(a_q, a_k, s_q, s_k, bias(z), mask);
    a_q += transition(a_q, s_q)."""

    def __init__(self, channel_a: int, channel_s: int, channel_z: int, num_heads: int, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.linear_z_to_bias = LinearNoBias(channel_z, num_heads)
        self.attention = CrossAttentionPairBias(channel_a, num_heads, channel_s)
        self.transition = ConditionedTransitionBlock(channel_a, channel_s)

    @torch.compiler.disable
    def forward(self, a_q: torch.Tensor, a_k: torch.Tensor, s_q: torch.Tensor, s_k: torch.Tensor, z: torch.Tensor,
                mask: torch.Tensor) -> torch.Tensor:
        """Reference signature: windowed a_q / a_k / s_q / s_k, normalised z (..., W, Lq, Lk, c_z), mask (..., W, Lk)."""
        _check_inference(a_q)
        precise = _is_precise(compute_dtype(a_q), "LocalTransformerBlock")
        with torch.autocast(a_q.device.type, enabled=False):
            dt = torch.float32 if precise else torch.bfloat16
            w = self.linear_z_to_bias.weight.detach().to(z.device, dt).contiguous()
            # z arrives normalised: projection only; (H, ..., W, Lq, Lk) -> (..., W, H, Lq, Lk)
            bias = F.window_bias(z.to(dt), None, None, w, normalise=False).movedim(0, -3)
        a_q = self.attention(a_q, a_k, s_q, s_k, bias, mask, residual=True)
        shape = a_q.shape
        out = self.transition(a_q.flatten(-3, -2), s_q.flatten(-3, -2), residual=True)
        return out.view(shape)


class LocalTransformerStack(nn.Module):
    """model/layers/folding/diffusion_transformer.py:419-512.  The whole stack works on the un-windowed atoms: the
    prologues, the projections, the output gate and the transition are row-wise, and under bfloat16 compute (head dim
    <= 32) the attention kernel walks the windows itself; the float32 path gathers the key side into windows.  The pair
    biases of all blocks come from one pass over z."""

    def __init__(self, channel_a: int, channel_s: int, channel_z: int, num_heads: int, num_blocks: int,
                 kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.num_heads = num_heads
        self.layernorm_z = LayerNorm(channel_z, create_offset=False)
        self.blocks = nn.ModuleList(
            [LocalTransformerBlock(channel_a, channel_s, channel_z, num_heads) for _ in range(num_blocks)])
        self._bias_w = None
        self._bias_w_key = None
        self._bias_all = None
        self._bias_all_key = None
        self._bias_all_src = None
        self._bank = _ConditioningBank()

    def _stacked_bias_weights(self, device, dt):
        ws = [b.linear_z_to_bias.weight for b in self.blocks]
        key = (device, dt) + tuple(v for w in ws for v in (w.data_ptr(), None if torch.is_inference(w) else w._version))
        if self._bias_w_key != key:
            self._bias_w = torch.cat([w.detach() for w in ws], dim=0).to(device, dt).contiguous()
            self._bias_w_key = key
        return self._bias_w

    def _window_biases(self, z: torch.Tensor, dt) -> torch.Tensor:
        """LayerNorm(z) projected to the heads of every block, head-major.  The window pair tensor does not change between
        the steps of a sampler run, so the result is kept for as long as z (same storage, same version) and the weights stay."""
        ln = self.layernorm_z
        w = self._stacked_bias_weights(z.device, dt)
        lw = ln.weight
        key = _tensor_key(z) + (dt, w.data_ptr(),
                                None if lw is None else (lw.data_ptr(), None if torch.is_inference(lw) else lw._version))
        if self._bias_all_key != key:
            self._bias_all = F.window_bias(z.to(dt), None if lw is None else lw.detach().float(),
                                           None if ln.bias is None else ln.bias.detach().float(), w, ln.eps)
            self._bias_all_key = key
            self._bias_all_src = z          # keeps z's storage alive so that its address cannot be reused
        return self._bias_all

    def reset_caches(self) -> None:
        """Forget the window biases (see CachedGlobalTransformerStack.reset_caches)."""
        self._bias_all = self._bias_all_key = self._bias_all_src = None

    @torch.compiler.disable
    def forward(self, a: torch.Tensor, s: torch.Tensor, z: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """a (*, L, c_a); s (*, L, c_s) (leading dims may be 1 where a's are not); z (*, W, 32, 128, c_z) likewise;
        mask (*, L) -> (*, L, c_a)."""
        _check_inference(a)
        precise = _is_precise(compute_dtype(a), "LocalTransformerStack")
        dt = torch.float32 if precise else torch.bfloat16
        length, c = a.shape[-2:]
        lead = tuple(a.shape[:-2])
        if length % WINDOW_Q != 0:
            raise ValueError("Length must be divisible by 32")
        windows = length // WINDOW_Q
        h = self.num_heads
        with torch.autocast(a.device.type, enabled=False):
            bias_all = self._window_biases(z, dt)                                        # (blocks*H, *z_lead, W, 32, 128)
            z_lead = tuple(z.shape[:-3])                                                 # includes the window dim
            # bf16 compute with head dim <= 32: the kernel walks the windows over the un-gathered atoms
            native = (not precise and c // h <= 32 and c % h == 0
                      and _index_share(lead, tuple(z.shape[:-4])) is not None and _index_share(lead, tuple(mask.shape[:-1])) is not None)
            if native:
                batch = 1
                for dd in lead:
                    batch *= dd
                bias_share = _index_share(lead, tuple(z.shape[:-4]))
                mask2 = mask.to(torch.bool).reshape(-1, length)
                bias_all = bias_all.reshape(len(self.blocks), h, -1, WINDOW_Q, WINDOW_K)
            else:
                to_qk = build_atom_to_qk_fn(length, a.device)
                _, mask_k = to_qk(mask.to(torch.bool), -1)                              # (*, W, 128)
                mask_k = mask_k.expand(*lead, windows, WINDOW_K).reshape(-1, WINDOW_K)
                sharing = _bias_sharing(lead + (windows,), z_lead)
                if sharing is None:
                    bias_all = bias_all.expand(bias_all.shape[0], *lead, windows, WINDOW_Q, WINDOW_K)
                    sharing = (1, 0)
                bias_all = bias_all.reshape(len(self.blocks), h, -1, WINDOW_Q, WINDOW_K)
                batch = mask_k.shape[0]
            conds = [None] * len(self.blocks)
            if not precise and all(b.attention.use_single_conditioning for b in self.blocks):
                # the conditioning projections of all blocks: one LayerNorm of s and two GEMMs
                gs, og = self._bank.tables(
                    s, [m for b in self.blocks for m in (b.attention.adaln_a_q, b.attention.adaln_a_k, b.transition.adaln)],
                    [g for b in self.blocks for g in (b.attention.linear_ada_out, b.transition.linear_g)])
                conds = [((gs[3 * i], gs[3 * i + 1], og[2 * i]), (gs[3 * i + 2], og[2 * i + 1])) for i in range(len(self.blocks))]
            for i, blk in enumerate(self.blocks):
                att = blk.attention
                xq, xk_flat, gate = att.normed_inputs(a, s, precise, cond=None if conds[i] is None else conds[i][0])
                if gate is not None:
                    gl = tuple(gate.shape[:-2])
                    while gl and gl[0] == 1:
                        gl = gl[1:]
                    if gl != lead[len(lead) - len(gl):]:
                        gate = gate.expand(*lead, length, c)
                pk = att._cross_packed(a.device, precise)
                if native:
                    a = F.attention_pair_bias_window(
                        xq.reshape(batch, length, c), xk_flat.reshape(batch, length, c), bias_all[i], mask2, pk,
                        bias_share=bias_share, bias_head_major=True, out_dtype=a.dtype, out_gate=gate,
                        resid=a).view(*lead, length, c)
                else:
                    _, xk = to_qk(xk_flat, -2)                                          # (*, W, 128, c)
                    a = F.attention_pair_bias_cross(
                        xq.reshape(batch, WINDOW_Q, c), xk.reshape(batch, WINDOW_K, c), bias_all[i], mask_k, pk,
                        bias_div=sharing[0], bias_mod=sharing[1], bias_head_major=True,
                        out_dtype=a.dtype, out_gate=gate, resid=a).view(*lead, length, c)
                a = blk.transition(a, s, residual=True, precise=precise, cond=None if conds[i] is None else conds[i][1])
        return a


class _ProjectionCache:
    """Device copies of plain projection weights (bf16, or the bf16 triple split for the float32-accurate path),
    re-made when the parameter changes."""

    def __init__(self):
        self._c = {}

    def get(self, lin: nn.Module, device, precise: bool) -> torch.Tensor:
        w = lin.weight
        key = (device, precise, w.data_ptr(), None if torch.is_inference(w) else w._version)
        hit = self._c.get(id(lin))
        if hit is None or hit[0] != key:
            wd = packing.split3_weights(w).to(device) if precise else w.detach().to(device, torch.bfloat16).contiguous()
            hit = (key, wd)
            self._c[id(lin)] = hit
        return hit[1]


def _project(x: torch.Tensor, w: torch.Tensor, precise: bool) -> torch.Tensor:
    return F.linear_fp32(x.float(), w, None) if precise else F.linear(x, w, None)


class AtomAttentionEncoder(nn.Module):
    """model/layers/folding/atom_transformer.py:263-389 (AF3 Algorithm 5): optional coordinate embedding, the atom-level
    local transformer, then ReLU(Linear(q)) averaged over the atoms of every token."""

    def __init__(self, channel_atom: int, channel_atompair: int, channel_token: int, channel_coords: int = 3, num_blocks=3,
                 num_heads=4, use_structure: bool = False, ckpt_atom_stack: bool = False, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend, self.use_structure, self.ckpt_atom_stack = kernel_backend, use_structure, ckpt_atom_stack
        if use_structure:
            self.linear_r_to_q = LinearNoBias(channel_coords, channel_atom)
        self.transformer = LocalTransformerStack(channel_atom, channel_atom, channel_atompair, num_heads, num_blocks)
        self.linear_q_to_a = LinearNoBias(channel_atom, channel_token)
        self._proj = _ProjectionCache()

    @torch.compiler.disable
    def forward(self, q: torch.Tensor, c: torch.Tensor, p: torch.Tensor, token_index: torch.Tensor, mask: torch.Tensor,
                num_tokens: int, r_noisy: torch.Tensor | None = None, mask_coords: bool = False):
        """q (*, La, c_atom); c (*, La, c_atom); p (*, W, 32, 128, c_atompair); token_index, mask (*, La);
        r_noisy (*, N, La, 3) -> (a (*, Lt, c_token), q_skip, c_skip, p_skip).  ``mask_coords``: the coordinates of
        padding atoms count as zero (the `r_noisy * atom_mask` of DiffusionStack.step, fused into the embedding)."""
        _check_inference(q)
        precise = _is_precise(compute_dtype(q), "AtomAttentionEncoder")
        if self.use_structure:
            assert r_noisy is not None, "r_noisy must be provided if use_structure is True"
            with torch.autocast(q.device.type, enabled=False):
                q = F.coord_embed(q, r_noisy, self.linear_r_to_q.weight, mask=mask if mask_coords else None)
        else:
            assert r_noisy is None, "r_noisy must be None if use_structure is False"
        q = self.transformer(q, c, p, mask)
        with torch.autocast(q.device.type, enabled=False):
            x = _project(q, self._proj.get(self.linear_q_to_a, q.device, precise), precise)
            a = F.aggregate_atoms_to_tokens(x, token_index, mask, num_tokens, relu=True)
        return a, q, c, p


class AtomAttentionDecoder(nn.Module):
    """model/layers/folding/atom_transformer.py:392-489 (AF3 Algorithm 6): token features projected and broadcast to their
    atoms plus the skip connection, the atom-level local transformer, LayerNorm and the float32 projection to
    coordinate updates."""

    def __init__(self, channel_a: int, channel_atom: int, channel_atompair: int, num_blocks: int = 3, num_heads: int = 4,
                 ckpt_atom_stack: bool = False, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend, self.ckpt_atom_stack = kernel_backend, ckpt_atom_stack
        self.linear_a_to_q = LinearNoBias(channel_a, channel_atom)
        self.transformer = LocalTransformerStack(channel_atom, channel_atom, channel_atompair, num_heads, num_blocks)
        self.layernorm_q = LayerNorm(channel_atom, create_offset=False)
        self.linear_q_to_r = LinearNoBias(channel_atom, 3)
        self._proj = _ProjectionCache()

    @torch.compiler.disable
    def forward(self, a: torch.Tensor, q_skip: torch.Tensor, c_skip: torch.Tensor, p_skip: torch.Tensor,
                token_index: torch.Tensor, mask: torch.Tensor, mask_out: bool = False) -> torch.Tensor:
        """a (*, Lt, c_token); q_skip, c_skip (*, La, c_atom); p_skip (*, W, 32, 128, c_atompair); token_index, mask
        (*, La) -> float32 position updates (*, La, 3).  ``mask_out``: padding atoms get a zero update (the
        `r_update * atom_mask` of DiffusionStack.step, fused into the projection)."""
        _check_inference(a)
        precise = _is_precise(compute_dtype(a), "AtomAttentionDecoder")
        with torch.autocast(a.device.type, enabled=False):
            a_to_q = _project(a, self._proj.get(self.linear_a_to_q, a.device, precise), precise)
            q = F.broadcast_tokens_to_atoms(a_to_q, token_index, add=q_skip)
        q = self.transformer(q, c_skip, p_skip, mask)
        ln = self.layernorm_q
        with torch.autocast(a.device.type, enabled=False):
            return F.ln_project(q, ln.weight, ln.bias, self.linear_q_to_r.weight, ln.eps, mask=mask if mask_out else None)


class DiffusionStack(nn.Module):
    """The time-dependent part of the AF3 diffusion module, ``DiffusionStack.step`` with ``get_single_conditioning`` and
    ``get_pair_bias`` (model/layers/folding/diffusion.py:155-600, AF3 Algorithm 20): atom attention encoder ->
    token transformer -> atom attention decoder.  Sub-module and parameter names are the reference's, so the matching
    part of a reference state dict loads by name (both the plain form and the production form with
    ``separate_endpoint_atom_encoder``).  Not included: ``pair_conditioning`` and ``atom_embedder`` (they run once per
    complex, before the sampler loop)."""

    def __init__(self, channel_a: int = 768, channel_s: int = 384, channel_z: int = 256, channel_atom: int = 128,
                 channel_atompair: int = 16, channel_coords: int = 3, separate_endpoint_atom_encoder: bool = False,
                 atom_encoder_blocks: int = 3, atom_encoder_heads: int = 4, token_transformer_blocks: int = 24,
                 token_transformer_heads: int = 16, atom_decoder_blocks: int = 3, atom_decoder_heads: int = 4,
                 blocks_per_ckpt: int | None = None, ckpt_atom_stack: bool = False, kernel_backend: str = "b200"):
        super().__init__()
        if separate_endpoint_atom_encoder and channel_coords != 6:
            raise ValueError("separate_endpoint_atom_encoder expects channel_coords=6 for [r_t, r_T] ECSI inputs.")
        self.kernel_backend = kernel_backend
        self.separate_endpoint_atom_encoder = separate_endpoint_atom_encoder
        self.token_transformer_blocks, self.token_transformer_heads = token_transformer_blocks, token_transformer_heads
        self.single_conditioning = SingleConditioning(channel_s, dim_fourier=256)
        enc_coords = 3 if separate_endpoint_atom_encoder else channel_coords
        self.atom_attention_encoder = AtomAttentionEncoder(channel_atom, channel_atompair, channel_a, enc_coords,
                                                           atom_encoder_blocks, atom_encoder_heads, use_structure=True)
        if separate_endpoint_atom_encoder:
            # the production form (model/layers/folding/diffusion.py:254-279): a second encoder reads the prior coordinates,
            # the two token streams are normalised, concatenated and fused by a float32 Linear
            self.endpoint_atom_attention_encoder = AtomAttentionEncoder(channel_atom, channel_atompair, channel_a, enc_coords,
                                                                        atom_encoder_blocks, atom_encoder_heads, use_structure=True)
            self.layernorm_a_t = LayerNorm(channel_a, create_offset=False)
            self.layernorm_a_endpoint = LayerNorm(channel_a, create_offset=False)
            self.endpoint_fusion = LinearNoBias(channel_a * 2, channel_a)
        self.layernorm_s = LayerNorm(channel_s, create_offset=False)
        self.linear_s_to_a = LinearNoBias(channel_s, channel_a)
        self.layernorm_z = LayerNorm(channel_z, create_offset=False)
        self.linear_z_to_bias = LinearNoBias(channel_z, token_transformer_blocks * token_transformer_heads)
        self.token_transformer = CachedGlobalTransformerStack(channel_a, channel_s, token_transformer_heads,
                                                              token_transformer_blocks)
        self.layernorm_a = LayerNorm(channel_a, create_offset=False)
        self.atom_attention_decoder = AtomAttentionDecoder(channel_a, channel_atom, channel_atompair, atom_decoder_blocks,
                                                           atom_decoder_heads)
        self._proj = _ProjectionCache()
        self._bias_w = {}

    def get_single_conditioning(self, s_inputs: torch.Tensor, c_noise: torch.Tensor) -> torch.Tensor:
        return self.single_conditioning(s_inputs, c_noise)

    def reset_caches(self) -> None:
        """Forget everything derived from the tensors of one complex (the converted token pair bias, the window biases of
        both atom transformers).  The caches are keyed on the source tensor's storage, shape and version; call this between
        complexes when those tensors are overwritten in place under ``torch.inference_mode()``."""
        self.token_transformer.reset_caches()
        self.atom_attention_encoder.transformer.reset_caches()
        self.atom_attention_decoder.transformer.reset_caches()
        if self.separate_endpoint_atom_encoder:
            self.endpoint_atom_attention_encoder.transformer.reset_caches()

    @staticmethod
    def check() -> None:
        """Synchronise and raise if a kernel recorded an error since the last check (a bounded wait that gave up, or a token
        index out of range): results computed since then must be discarded.  Cheap enough for once per sampler run."""
        from . import _lib
        _lib.device_status()

    def get_pair_bias(self, z: torch.Tensor) -> torch.Tensor:
        """(B, Nblock, H, Lt, Lt): bf16 under bfloat16 compute, float32 under float32 compute; time-independent."""
        return _token_pair_bias(z, self.layernorm_z, self.linear_z_to_bias, self.token_transformer_blocks,
                                self.token_transformer_heads, self._bias_w)

    @torch.compiler.disable
    def step(self, r_noisy: torch.Tensor, q: torch.Tensor, c: torch.Tensor, p: torch.Tensor, token_index: torch.Tensor,
             atom_mask: torch.Tensor, s: torch.Tensor, pair_bias: torch.Tensor, token_mask: torch.Tensor) -> torch.Tensor:
        """r_noisy (B, N, La, channel_coords); q, c (B, La, c_atom); p (B, W, 32, 128, c_atompair); token_index, atom_mask (B, La);
        s (B, N, Lt, c_s); pair_bias (B, Nblock, H, Lt, Lt); token_mask (B, Lt) -> float32 position updates (B, N, La, 3)."""
        _check_inference(r_noisy)
        q, c, p = q.unsqueeze(-3), c.unsqueeze(-3), p.unsqueeze(-5)
        atom_mask, token_mask, token_index = atom_mask.unsqueeze(-2), token_mask.unsqueeze(-2), token_index.unsqueeze(-2)
        if self.separate_endpoint_atom_encoder:
            r_t, r_T = r_noisy[..., :3].contiguous(), r_noisy[..., 3:].contiguous()
            a, q_skip, c_skip, p_skip = self.atom_attention_encoder(q, c, p, token_index, atom_mask, token_mask.shape[-1],
                                                                    r_noisy=r_t, mask_coords=True)
            a_e, _, _, _ = self.endpoint_atom_attention_encoder(q, c, p, token_index, atom_mask, token_mask.shape[-1],
                                                                r_noisy=r_T, mask_coords=True)
            with torch.autocast(a.device.type, enabled=False):
                lt, le = self.layernorm_a_t, self.layernorm_a_endpoint
                cat = torch.cat((F.layer_norm(a, lt.weight, lt.bias, lt.eps), F.layer_norm(a_e, le.weight, le.bias, le.eps)), dim=-1)
                a = F.linear_fp32(cat.float(), self._proj.get(self.endpoint_fusion, a.device, True), None)
        else:
            a, q_skip, c_skip, p_skip = self.atom_attention_encoder(q, c, p, token_index, atom_mask, token_mask.shape[-1],
                                                                    r_noisy=r_noisy, mask_coords=True)
        ln = self.layernorm_s
        with torch.autocast(a.device.type, enabled=False):
            # a.float() + linear_s_to_a(layernorm_s(s)): a float32 Linear in the reference whatever the autocast state
            w_sa = self._proj.get(self.linear_s_to_a, a.device, True)
            if s.shape[-3] == a.shape[-3]:
                a = F.ln_linear_fp32(s.float(), ln.weight, ln.bias, w_sa, None, resid=a.float(), eps=ln.eps)
            else:       # one conditioning row shared by the samples (the sampler's form): project once, add to every sample
                a = a.float() + F.ln_linear_fp32(s.float(), ln.weight, ln.bias, w_sa, None, eps=ln.eps)
        a = self.token_transformer(a, s, pair_bias.unsqueeze(-5), token_mask)
        a = self.layernorm_a(a)
        return self.atom_attention_decoder(a, q_skip, c_skip, p_skip, token_index, atom_mask, mask_out=True)


# --------------------------------------------------------------------------------------------
# blocks
# --------------------------------------------------------------------------------------------
class TriangularBlock(nn.Module):
    """K-Fold trunk block: tri-mult out, tri-mult in, transition, residual adds fused into the kernels."""

    def __init__(self, channel_z: int = 256, dropout: float = 0.25, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend, self.channel_z, self.dropout = kernel_backend, channel_z, dropout
        self.tri_mul_out = TriangleMultiplicationOutgoing(channel_z)
        self.tri_mul_in = TriangleMultiplicationIncoming(channel_z)
        self.transition_z = Transition(channel_z, expansion_factor=4)

    def forward(self, z: torch.Tensor, pair_mask: torch.Tensor) -> torch.Tensor:
        z = self.tri_mul_out(z, pair_mask, residual=True)
        z = self.tri_mul_in(z, pair_mask, residual=True)
        return self.transition_z(z, residual=True)


class PairformerBlock(nn.Module):
    """AF3-shaped Pairformer block assembled from the reference's modules: the pair track in the order of
    ``PairformerBlock.forward`` (tri-mult out/in, tri-att start/end, transition x4) and the single track of
    ``ConfidencePairSingleBlock.forward`` (pair bias from LN(z), single attention with pair bias, transition x4)."""

    def __init__(self, channel_z: int = 128, channel_s: int = 384, num_tri_heads: int = 4, num_heads: int = 16,
                 kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.tri_mul_out = TriangleMultiplicationOutgoing(channel_z)
        self.tri_mul_in = TriangleMultiplicationIncoming(channel_z)
        self.tri_att_start = TriangleAttentionStartingNode(channel_z, num_tri_heads)
        self.tri_att_end = TriangleAttentionEndingNode(channel_z, num_tri_heads)
        self.transition_z = Transition(channel_z, expansion_factor=4)
        self.layernorm_z = LayerNorm(channel_z)
        self.linear_pair_bias = LinearNoBias(channel_z, num_heads)
        self.attention = SelfAttentionPairBias(channel_s, num_heads, None, "confidence")
        self.transition = Transition(channel_s, expansion_factor=4)
        self._bias_w = None
        self._bias_key = None

    def _pair_bias(self, z: torch.Tensor) -> torch.Tensor:
        p = self.linear_pair_bias.weight
        precise = z.dtype == torch.float32
        key = (z.device, precise, p.data_ptr(), None if torch.is_inference(p) else p._version)
        if self._bias_key != key:
            self._bias_w = packing.split3_weights(p).to(z.device) if precise else p.detach().to(z.device, torch.bfloat16).contiguous()
            self._bias_key = key
        n = z.shape[1]
        if n % 8 != 0:  # rare: pad the pair tensor so that bias rows stay 16-byte aligned
            npad = (n + 7) // 8 * 8
            zp = z.new_zeros(z.shape[0], npad, npad, z.shape[-1])
            zp[:, :n, :n] = z
            return F.pair_bias(zp, self.layernorm_z.weight.detach().float(), self.layernorm_z.bias.detach().float(),
                               self._bias_w, self.layernorm_z.eps)[:, :, :n, :n]
        return F.pair_bias(z, self.layernorm_z.weight.detach().float(), self.layernorm_z.bias.detach().float(),
                           self._bias_w, self.layernorm_z.eps)

    @torch.compiler.disable
    def forward(self, z: torch.Tensor, s: torch.Tensor, pair_mask: torch.Tensor, mask: torch.Tensor):
        """z (B,N,N,c_z), s (B,N,c_s), pair_mask (B,N,N), mask (B,N) -> (z, s)."""
        _check_inference(z)
        z = self.tri_mul_out(z, pair_mask, residual=True)
        z = self.tri_mul_in(z, pair_mask, residual=True)
        z = self.tri_att_start(z, pair_mask, residual=True)
        z = self.tri_att_end(z, pair_mask, residual=True)
        z = self.transition_z(z, residual=True)
        with torch.autocast(z.device.type, enabled=False):
            bias = self._pair_bias(z if compute_dtype(z) == z.dtype else z.to(compute_dtype(z)))
        s = self.attention(s, None, bias, mask, residual=True)
        s = self.transition(s, residual=True)
        return z, s
