"""Callers of the pair stacks in K-Fold's trunk and the pair conditioning of its diffusion module.

  ParcaeRecurrence   `z = a * z + F.linear(self.layernorm_z(u_t), b)` between recycling iterations, with the discretised
                     dynamics of ``KFold._parcae_discretized_dynamics``          model/model.py:203-217, :272-277, :528
  LMToPair           outer-product features of the language-model embedding -> pair tensor        model/model.py:114-134
  PairConditioning   LayerNorm + float32 Linear over [z | relative-position features], two Transitions
                                                                                  model/layers/folding/diffusion.py:45-94

Parameter names are the reference's, so the matching entries of a reference ``state_dict`` load by name.  All three run once
per recycling iteration or once per complex, next to stacks that take milliseconds per block: they are built for
completeness of the path (no torch arithmetic on pair-sized tensors between the stacks), not tuned.
"""
from __future__ import annotations

import torch
import torch.nn.functional as tF
from torch import nn

from . import functional as F
from . import packing
from .modules import LayerNorm, Linear, LinearNoBias, Transition, _check_inference, _is_precise, compute_dtype

__all__ = ["ParcaeRecurrence", "LMToPair", "PairConditioning"]


def _param_key(*params):
    return tuple(v for p in params for v in (p.data_ptr(), None if torch.is_inference(p) else p._version))


class ParcaeRecurrence(nn.Module):
    """The pair-state recurrence of the trunk (model/model.py:523-529): ``z = a * z + Linear_b(LayerNorm(u))`` with
    a = exp(-softplus(log_delta) * exp(log_a)) per channel and b = softplus(log_delta)[:, None] * b_cont
    (``_parcae_discretized_dynamics``, :272-277).  Parameters carry the names they have on the reference's ``KFold``."""

    def __init__(self, channel_z: int, decay_init: float = 0.4472135954999579):
        super().__init__()
        import math
        self.channel_z = channel_z
        self.parcae_log_a = nn.Parameter(torch.zeros(channel_z))
        delta_init = -math.log(decay_init)
        self.parcae_log_delta = nn.Parameter(torch.full((channel_z,), math.log(math.expm1(delta_init))))
        self.parcae_b_cont = nn.Parameter(torch.eye(channel_z))
        self.layernorm_z = LayerNorm(channel_z)
        self._dyn = None
        self._dyn_key = None

    def dynamics(self, device):
        """(a float32 [C], b bf16 [C, C]) on `device`, recomputed when a parameter changes."""
        key = (device,) + _param_key(self.parcae_log_a, self.parcae_log_delta, self.parcae_b_cont)
        if self._dyn_key != key:
            delta = tF.softplus(self.parcae_log_delta.detach().float())
            a = torch.exp(-delta * torch.exp(self.parcae_log_a.detach().float()))
            b = delta[:, None] * self.parcae_b_cont.detach().float()
            # the reference casts both to the autocast dtype before use (model.py:505)
            self._dyn = (a.to(torch.bfloat16).float().to(device).contiguous(), b.to(device, torch.bfloat16).contiguous())
            self._dyn_key = key
        return self._dyn

    @torch.compiler.disable
    def forward(self, z: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
        """z, u (B, N, N, C) -> a * z + Linear_b(LayerNorm(u)), same shape and dtype as z."""
        _check_inference(z)
        if _is_precise(compute_dtype(z), "ParcaeRecurrence"):
            raise NotImplementedError("ParcaeRecurrence: bfloat16 compute only (the trunk runs under autocast(bfloat16))")
        a, b = self.dynamics(z.device)
        ln = self.layernorm_z
        with torch.autocast(z.device.type, enabled=False):
            return F.parcae_update(z, u, ln.weight, ln.bias, a, b, ln.eps)


class LMToPair(nn.Module):
    """model/model.py:114-134: [xi | xj] = Linear(LayerNorm(s_lm)); z = LayerNorm(MLP([xi * xj | xi - xj])) over all token
    pairs, the MLP being Linear(2 c_z -> c_z), GELU, Linear(c_z -> c_z)."""

    def __init__(self, channel_s: int, channel_z: int):
        super().__init__()
        self.channel_s, self.channel_z = channel_s, channel_z
        self.proj = nn.Sequential(LayerNorm(channel_s), Linear(channel_s, channel_z * 2))
        self.mlp = nn.Sequential(Linear(2 * channel_z, channel_z), nn.Identity(), Linear(channel_z, channel_z))   # [1] = GELU
        self.layernorm_pair = LayerNorm(channel_z)
        self._w = None
        self._w_key = None

    def _weights(self, device):
        lins = (self.proj[1], self.mlp[0], self.mlp[2])
        key = (device,) + _param_key(*[p for m in lins for p in (m.weight, m.bias)])
        if self._w_key != key:
            self._w = [(m.weight.detach().to(device, torch.bfloat16).contiguous(), m.bias.detach().to(device, torch.float32).contiguous())
                       for m in lins]
            self._w_key = key
        return self._w

    @torch.compiler.disable
    def forward(self, s_lm: torch.Tensor) -> torch.Tensor:
        """s_lm (B, L, c_s) -> (B, L, L, c_z) in the compute dtype (bfloat16)."""
        _check_inference(s_lm)
        if _is_precise(compute_dtype(s_lm), "LMToPair"):
            raise NotImplementedError("LMToPair: bfloat16 compute only (the trunk runs under autocast(bfloat16))")
        (wp, bp), (w0, b0), (w2, b2) = self._weights(s_lm.device)
        ln, lnp = self.proj[0], self.layernorm_pair
        with torch.autocast(s_lm.device.type, enabled=False):
            x = F.linear(F.layer_norm(s_lm, ln.weight, ln.bias, ln.eps, out_dtype=torch.bfloat16), wp, bp)      # (B, L, 2 c_z)
            feats = F.lm_pair_features(x)                                                                       # (B, L, L, 2 c_z)
            h = F.gelu(F.linear(feats, w0, b0))
            y = F.linear(h, w2, b2)
            return F.layer_norm(y, lnp.weight, lnp.bias, lnp.eps)


class PairConditioning(nn.Module):
    """model/layers/folding/diffusion.py:45-94 (AF3 Algorithm 21, pair part): z = Linear_fp32(LayerNorm([z | rel_pos])),
    then two Transitions with residual.  The relative-position features are an input here (the reference derives them from
    the FoldingInput with ``RelativePositionEncoding(32, 2)``, 139 channels, model/layers/folding/embeddings.py:25-140)."""

    def __init__(self, channel_z: int = 256, rel_pos_dim: int = 139, r_max: int = 32, s_max: int = 2):
        super().__init__()
        if rel_pos_dim != 4 * (r_max + 1) + 2 * (s_max + 1) + 1:
            raise ValueError("rel_pos_dim does not match RelativePositionEncoding(r_max, s_max)")
        self.channel_z, self.rel_pos_dim, self.r_max, self.s_max = channel_z, rel_pos_dim, r_max, s_max
        in_channel = channel_z + rel_pos_dim
        self.layernorm = LayerNorm(in_channel, create_offset=False)
        self.linear = LinearNoBias(in_channel, channel_z)
        self.transitions = nn.ModuleList([Transition(channel_z, expansion_factor=2) for _ in range(2)])
        self._w = None
        self._w_key = None

    def _weight6(self, device, k_pad: int):
        w = self.linear.weight
        key = (device, k_pad) + _param_key(w)
        if self._w_key != key:
            wp = tF.pad(w.detach().float(), (0, k_pad - w.shape[1]))          # zero columns for the padded features
            self._w = packing.split3_weights(wp).to(device)
            self._w_key = key
        return self._w

    @torch.compiler.disable
    def forward(self, rel_pos, z: torch.Tensor) -> torch.Tensor:
        """rel_pos: the relative-position features (B, L, L, rel_pos_dim), or -- the reference's own argument -- the
        FoldingInput (anything whose `.token` carries asym_id, residue_index, entity_id, token_index, sym_id), in which case
        the features are computed inside the LayerNorm kernel and never stored; z (B, L, L, c_z) -> float32 (B, L, L, c_z)."""
        _check_inference(z)
        ln = self.layernorm
        with torch.autocast(z.device.type, enabled=False):
            k = z.shape[-1] + self.rel_pos_dim
            k_pad = (k + 7) // 8 * 8          # the split-operand GEMM wants rows of a multiple of 8 elements
            if isinstance(rel_pos, torch.Tensor):
                zn = F.concat_layer_norm(z, rel_pos, ln.weight, ln.bias, k_pad, ln.eps)
            else:
                zn = F.relpos_concat_layer_norm(z, rel_pos.token, ln.weight, ln.bias, k_pad, self.r_max, self.s_max, ln.eps)
            out = F.linear_fp32(zn, self._weight6(z.device, k_pad), None)
        for transition in self.transitions:
            out = transition(out, residual=True)
        return out
