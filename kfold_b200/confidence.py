"""K-Fold's confidence head on the B200 kernels: the per-sample loop of ``ConfidenceHead`` (model/modules/confidence_head.py).

  ConfidencePairSingleBlock   TriangularBlock on z, pair bias from LayerNorm(z), single pair-bias attention, Transition (:125-175)
  ConfidencePairSingleStack   the blocks in sequence (:85-122)
  ConfidenceHead              `prepare` (:343-351), `forward_single` (:413-470) and the loop over the diffusion samples (:365-378)

Parameter names are the reference's.  What `ConfidenceHead.forward` does around the loop with the FoldingInput -- picking the
representative atoms, scattering the per-token logits into the atom layout, the final masks (:339-342, :380-399) -- is output
formatting on small tensors and stays with the caller; the loop, the stack and the four heads are here.
"""
from __future__ import annotations

import torch
from torch import nn

from . import functional as F
from .modules import (LayerNorm, LinearNoBias, SelfAttentionPairBias, Transition, TriangularBlock, _check_inference, _is_precise,
                      _ProjectionCache, compute_dtype)

__all__ = ["ConfidencePairSingleBlock", "ConfidencePairSingleStack", "ConfidenceHead"]


class ConfidencePairSingleBlock(nn.Module):
    """model/modules/confidence_head.py:125-175."""

    def __init__(self, channel_s: int, channel_z: int, num_heads: int, dropout: float = 0.25, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.pair_block = TriangularBlock(channel_z, dropout)
        self.layernorm_z = LayerNorm(channel_z)
        self.linear_pair_bias = LinearNoBias(channel_z, num_heads)
        self.attention = SelfAttentionPairBias(channel_s, num_heads, None, "confidence")
        self.transition = Transition(channel_s, expansion_factor=4)
        self._proj = _ProjectionCache()

    @torch.compiler.disable
    def forward(self, z: torch.Tensor, s: torch.Tensor, pair_mask: torch.Tensor, mask: torch.Tensor):
        _check_inference(z)
        z = self.pair_block(z, pair_mask)
        cd = compute_dtype(z)
        precise = _is_precise(cd, "ConfidencePairSingleBlock")
        ln = self.layernorm_z
        with torch.autocast(z.device.type, enabled=False):
            zz = z if z.dtype == cd else z.to(cd)
            n = zz.shape[1]
            if n % 8 != 0:      # bias rows must stay 16-byte aligned
                npad = (n + 7) // 8 * 8
                zp = zz.new_zeros(zz.shape[0], npad, npad, zz.shape[-1])
                zp[:, :n, :n] = zz
                zz = zp
            bias = F.pair_bias(zz, ln.weight.detach().float(), ln.bias.detach().float(),
                               self._proj.get(self.linear_pair_bias, z.device, precise), ln.eps)[:, :, :n, :n]
        s = self.attention(s, None, bias, mask, residual=True)
        s = self.transition(s, residual=True)
        return z, s


class ConfidencePairSingleStack(nn.Module):
    """model/modules/confidence_head.py:85-122."""

    def __init__(self, channel_s: int, channel_z: int, num_heads: int, num_blocks: int, dropout: float = 0.25,
                 blocks_per_ckpt=None, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.blocks = nn.ModuleList([ConfidencePairSingleBlock(channel_s, channel_z, num_heads, dropout) for _ in range(num_blocks)])

    def forward(self, z, s, pair_mask, mask):
        for blk in self.blocks:
            z, s = blk(z, s, pair_mask, mask)
        return z, s


class ConfidenceHead(nn.Module):
    """model/modules/confidence_head.py:178-470 (AF3 Algorithm 31): the constructor takes the reference's configuration
    fields as keyword arguments."""

    def __init__(self, channel_s: int = 384, channel_z: int = 256, num_heads_attn: int = 16, num_blocks: int = 4,
                 dropout: float = 0.25, num_bins: int = 39, min_dist: float = 3.25, max_dist: float = 50.75,
                 num_pae_bins: int = 64, num_pde_bins: int = 64, num_plddt_bins: int = 50, kernel_backend: str = "b200"):
        super().__init__()
        self.kernel_backend = kernel_backend
        self.num_bins, self.num_pae_bins, self.num_pde_bins, self.num_plddt_bins = num_bins, num_pae_bins, num_pde_bins, num_plddt_bins
        self.linear_s1 = LinearNoBias(channel_s, channel_z)
        self.linear_s2 = LinearNoBias(channel_s, channel_z)
        self.s_lm_to_s = nn.Sequential(LayerNorm(channel_s), LinearNoBias(channel_s, channel_s))
        self.register_buffer("boundaries", torch.linspace(min_dist, max_dist, num_bins - 1), persistent=False)
        self.linear_distogram = LinearNoBias(num_bins, channel_z)
        self.stack = ConfidencePairSingleStack(channel_s, channel_z, num_heads_attn, num_blocks, dropout)
        self.pae_head = nn.Sequential(LayerNorm(channel_z), LinearNoBias(channel_z, num_pae_bins))
        self.pde_head = nn.Sequential(LayerNorm(channel_z), LinearNoBias(channel_z, num_pde_bins))
        self.plddt_head = nn.Sequential(LayerNorm(channel_s), LinearNoBias(channel_s, 24 * num_plddt_bins))
        self.resolved_head = nn.Sequential(LayerNorm(channel_s), LinearNoBias(channel_s, 24 * 2))
        self._proj = _ProjectionCache()
        self._dgram_w = {}

    def _head(self, seq: nn.Sequential, x: torch.Tensor) -> torch.Tensor:
        """float32 LayerNorm + Linear (the heads run with autocast off, :461-468)."""
        ln, lin = seq[0], seq[1]
        return F.ln_linear_fp32(x.float(), ln.weight, ln.bias, self._proj.get(lin, x.device, True), None, eps=ln.eps)

    @torch.compiler.disable
    def prepare(self, s_inputs: torch.Tensor, s_lm: torch.Tensor, z: torch.Tensor):
        """:343-351 -> (z + linear_s1(s_inputs)[j] + linear_s2(s_inputs)[i], s_lm_to_s(s_lm)) in the compute dtype."""
        _check_inference(z)
        cd = compute_dtype(z)
        if _is_precise(cd, "ConfidenceHead"):
            raise NotImplementedError("ConfidenceHead: bfloat16 compute only (the head runs under autocast(bfloat16))")
        with torch.autocast(z.device.type, enabled=False):
            si = s_inputs.to(cd)
            a1 = F.linear(si, self._proj.get(self.linear_s1, z.device, False), None)
            a2 = F.linear(si, self._proj.get(self.linear_s2, z.device, False), None)
            zz = F.pair_outer_add(z.to(cd), a1, a2)
            ln = self.s_lm_to_s[0]
            s = F.linear(F.layer_norm(s_lm.to(cd), ln.weight, ln.bias, ln.eps), self._proj.get(self.s_lm_to_s[1], z.device, False), None)
        return zz, s

    @torch.compiler.disable
    def forward_single(self, z: torch.Tensor, s: torch.Tensor, x: torch.Tensor, mask: torch.Tensor):
        """:413-470.  z (B, L, L, c_z) and s (B, L, c_s) as `prepare` returns them; x (B, L, 3) coordinates of the tokens'
        representative atoms of ONE sample; mask (B, L) -> (pae, pde, plddt, resolved) logits, float32."""
        _check_inference(z)
        w = self.linear_distogram.weight
        key = (z.device, z.dtype, w.data_ptr(), None if torch.is_inference(w) else w._version)
        if self._dgram_w.get("key") != key:
            self._dgram_w = {"key": key, "w": w.detach().t().to(z.device, z.dtype).contiguous()}
        with torch.autocast(z.device.type, enabled=False):
            z = F.distogram_embed_add(z, x, self.boundaries, self._dgram_w["w"])
        pair_mask = mask[..., :, None] & mask[..., None, :]
        z, s = self.stack(z, s.clone(), pair_mask, mask)
        with torch.autocast(z.device.type, enabled=False):
            pae = self._head(self.pae_head, z)
            pde = self._head(self.pde_head, z)
            pde = pde + pde.transpose(-2, -3)
            plddt = self._head(self.plddt_head, s).unflatten(-1, (24, self.num_plddt_bins))
            resolved = self._head(self.resolved_head, s).unflatten(-1, (24, 2))
        return pae, pde, plddt, resolved

    @torch.compiler.disable
    def forward_samples(self, s_inputs: torch.Tensor, s_lm: torch.Tensor, z: torch.Tensor, x_repr: torch.Tensor, mask: torch.Tensor):
        """The loop of :365-378 over the N samples: x_repr (B, N, L, 3) -> dict of logits stacked along dim 1."""
        zz, s = self.prepare(s_inputs, s_lm, z)
        outs = [self.forward_single(zz, s, x_repr[:, i], mask) for i in range(x_repr.shape[1])]
        names = ("pae_logits", "pde_logits", "plddt_logits", "resolved_logits")
        return {n: torch.stack([o[k] for o in outs], dim=1) for k, n in enumerate(names)}
