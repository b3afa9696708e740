"""Seeded synthetic inputs and random-init weights for the hot-path operators.

K-Fold ships no public test vectors and its released weights are not available
offline, so every test and benchmark here runs on synthetic data: activations
``~ N(0,1)``, every 2-D weight ``~ N(0, 1/fan_in)`` (including the ones the
reference zero-initialises, which would make every output identically zero),
LayerNorm scales near one.  All values come from ``numpy.random.RandomState``,
whose stream is frozen across numpy versions, so the same seed gives the same
bits on every machine.  Tensors are created on the CPU in float32; callers move
them to the device.

Weight dictionaries are keyed exactly like the ``state_dict()`` of the
reference module of the same name.
"""
from __future__ import annotations

import numpy as np
import torch


class _Rng:
    def __init__(self, seed: int):
        self.rs = np.random.RandomState(seed)

    def normal(self, *shape, std: float = 1.0) -> torch.Tensor:
        return torch.from_numpy((self.rs.standard_normal(shape) * std).astype(np.float32))

    def linear(self, out_f: int, in_f: int) -> torch.Tensor:
        return self.normal(out_f, in_f, std=in_f ** -0.5)

    def ln_w(self, n: int) -> torch.Tensor:
        return 1.0 + self.normal(n, std=0.1)

    def ln_b(self, n: int) -> torch.Tensor:
        return self.normal(n, std=0.1)


def _prefixed(prefix: str, d: dict) -> dict:
    return {f"{prefix}.{k}": v for k, v in d.items()}


def trimul_weights(rng: _Rng, c: int) -> dict:
    """TriangleMultiplication{Outgoing,Incoming} (model/primitives/triangle_multiplication.py:171-177)."""
    return {
        "layernorm_in.weight": rng.ln_w(c), "layernorm_in.bias": rng.ln_b(c),
        "linear_p_in.weight": rng.linear(2 * c, c), "linear_g_in.weight": rng.linear(2 * c, c),
        "layernorm_out.weight": rng.ln_w(c), "layernorm_out.bias": rng.ln_b(c),
        "linear_p_out.weight": rng.linear(c, c), "linear_g_out.weight": rng.linear(c, c),
    }


def triatt_weights(rng: _Rng, c: int, heads: int) -> dict:
    """TriangleAttention (model/primitives/triangle_attention.py:338-373)."""
    hd = c  # c_hidden * heads == c_in
    return {
        "layer_norm.weight": rng.ln_w(c), "layer_norm.bias": rng.ln_b(c),
        "linear.weight": rng.linear(heads, c),
        "mha.linear_q.weight": rng.linear(hd, c), "mha.linear_k.weight": rng.linear(hd, c),
        "mha.linear_v.weight": rng.linear(hd, c), "mha.linear_o.weight": rng.linear(c, hd),
        "mha.linear_g.weight": rng.linear(hd, c),
    }


def transition_weights(rng: _Rng, c: int, factor: int) -> dict:
    """Transition (model/layers/folding/transition.py:27-46)."""
    return {
        "layernorm.weight": rng.ln_w(c), "layernorm.bias": rng.ln_b(c),
        "swiglu.linear.weight": rng.linear(2 * c * factor, c),
        "linear_out.weight": rng.linear(c, c * factor),
    }


def adaln_weights(rng: _Rng, c_a: int, c_s: int) -> dict:
    """AdaLN (model/primitives/normalization.py:99-115)."""
    return {
        "layernorm_s.weight": rng.ln_w(c_s),
        "linear_g.weight": rng.linear(c_a, c_s), "linear_g.bias": rng.normal(c_a, std=0.1),
        "linear_bias.weight": rng.linear(c_a, c_s),
    }


def apb_weights(rng: _Rng, c_a: int, c_s: int | None) -> dict:
    """SelfAttentionPairBias (model/layers/folding/attention_pair_bias.py:57-112)."""
    w = {
        "linear_q.weight": rng.linear(c_a, c_a), "linear_q.bias": rng.normal(c_a, std=0.1),
        "linear_k.weight": rng.linear(c_a, c_a), "linear_v.weight": rng.linear(c_a, c_a),
        "linear_g.weight": rng.linear(c_a, c_a), "linear_out.weight": rng.linear(c_a, c_a),
    }
    if c_s is None:
        w["layernorm_a.weight"] = rng.ln_w(c_a)
        w["layernorm_a.bias"] = rng.ln_b(c_a)
    else:
        w.update(_prefixed("adaln_a", adaln_weights(rng, c_a, c_s)))
        w["linear_ada_out.weight"] = rng.linear(c_a, c_s)
        w["linear_ada_out.bias"] = rng.normal(c_a, std=0.1) - 2.0
    return w


def cross_apb_weights(rng: _Rng, c_a: int, c_s: int | None) -> dict:
    """CrossAttentionPairBias (model/layers/folding/attention_pair_bias.py:161-205)."""
    w = {
        "linear_q.weight": rng.linear(c_a, c_a), "linear_q.bias": rng.normal(c_a, std=0.1),
        "linear_k.weight": rng.linear(c_a, c_a), "linear_v.weight": rng.linear(c_a, c_a),
        "linear_g.weight": rng.linear(c_a, c_a), "linear_out.weight": rng.linear(c_a, c_a),
    }
    if c_s is None:
        for side in ("q", "k"):
            w[f"layernorm_a_{side}.weight"] = rng.ln_w(c_a)
            w[f"layernorm_a_{side}.bias"] = rng.ln_b(c_a)
    else:
        w.update(_prefixed("adaln_a_q", adaln_weights(rng, c_a, c_s)))
        w.update(_prefixed("adaln_a_k", adaln_weights(rng, c_a, c_s)))
        w["linear_ada_out.weight"] = rng.linear(c_a, c_s)
        w["linear_ada_out.bias"] = rng.normal(c_a, std=0.1) - 2.0
    return w


def local_stack_weights(rng: _Rng, c_a: int, c_s: int, c_z: int, heads: int, blocks: int) -> dict:
    """LocalTransformerStack (model/layers/folding/diffusion_transformer.py:419-467)."""
    w = {"layernorm_z.weight": rng.ln_w(c_z)}
    for i in range(blocks):
        w[f"blocks.{i}.linear_z_to_bias.weight"] = rng.linear(heads, c_z)
        w.update(_prefixed(f"blocks.{i}.attention", cross_apb_weights(rng, c_a, c_s)))
        w.update(_prefixed(f"blocks.{i}.transition", conditioned_transition_weights(rng, c_a, c_s)))
    return w


def atom_encoder_weights(rng: _Rng, c_atom: int, c_pair: int, c_token: int, heads: int, blocks: int, use_structure: bool,
                         c_coords: int = 3) -> dict:
    """AtomAttentionEncoder (model/layers/folding/atom_transformer.py:263-309)."""
    w = {}
    if use_structure:
        w["linear_r_to_q.weight"] = rng.linear(c_atom, c_coords)
    w.update(_prefixed("transformer", local_stack_weights(rng, c_atom, c_atom, c_pair, heads, blocks)))
    w["linear_q_to_a.weight"] = rng.linear(c_token, c_atom)
    return w


def atom_decoder_weights(rng: _Rng, c_token: int, c_atom: int, c_pair: int, heads: int, blocks: int) -> dict:
    """AtomAttentionDecoder (model/layers/folding/atom_transformer.py:392-431)."""
    w = {"linear_a_to_q.weight": rng.linear(c_atom, c_token)}
    w.update(_prefixed("transformer", local_stack_weights(rng, c_atom, c_atom, c_pair, heads, blocks)))
    w["layernorm_q.weight"] = rng.ln_w(c_atom)
    w["linear_q_to_r.weight"] = rng.linear(3, c_atom)
    return w


def single_conditioning_weights(rng: _Rng, c_s: int, dim_fourier: int) -> dict:
    """SingleConditioning (model/layers/folding/diffusion.py:102-120)."""
    w = {"layernorm_fourier.weight": rng.ln_w(dim_fourier), "linear_fourier.weight": rng.linear(c_s, dim_fourier),
         "linear.weight": rng.linear(c_s, c_s)}
    for i in range(2):
        w.update(_prefixed(f"transitions.{i}", transition_weights(rng, c_s, 2)))
    return w


def diffusion_step_weights(rng: _Rng, c_a: int, c_s: int, c_atom: int, c_pair: int, atom_blocks: int, atom_heads: int,
                           token_blocks: int, token_heads: int, c_coords: int = 3, separate_endpoint: bool = False) -> dict:
    """The parameters DiffusionStack.step touches (model/layers/folding/diffusion.py:250-325): atom attention encoder and
    decoder, layernorm_s / linear_s_to_a, the token transformer, layernorm_a; with ``separate_endpoint`` also the second
    encoder for the prior coordinates and the fusion of the two token streams (:254-279)."""
    enc_coords = 3 if separate_endpoint else c_coords
    w = _prefixed("atom_attention_encoder", atom_encoder_weights(rng, c_atom, c_pair, c_a, atom_heads, atom_blocks, True, enc_coords))
    w["layernorm_s.weight"] = rng.ln_w(c_s)
    w["linear_s_to_a.weight"] = rng.linear(c_a, c_s)
    for i in range(token_blocks):
        w.update(_prefixed(f"token_transformer.blocks.{i}.attention", apb_weights(rng, c_a, c_s)))
        w.update(_prefixed(f"token_transformer.blocks.{i}.transition", conditioned_transition_weights(rng, c_a, c_s)))
    w["layernorm_a.weight"] = rng.ln_w(c_a)
    w.update(_prefixed("atom_attention_decoder", atom_decoder_weights(rng, c_a, c_atom, c_pair, atom_heads, atom_blocks)))
    if separate_endpoint:
        w.update(_prefixed("endpoint_atom_attention_encoder",
                           atom_encoder_weights(rng, c_atom, c_pair, c_a, atom_heads, atom_blocks, True, 3)))
        w["layernorm_a_t.weight"] = rng.ln_w(c_a)
        w["layernorm_a_endpoint.weight"] = rng.ln_w(c_a)
        w["endpoint_fusion.weight"] = rng.linear(c_a, 2 * c_a)
    return w


def conditioned_transition_weights(rng: _Rng, c_a: int, c_s: int, factor: int = 2) -> dict:
    """ConditionedTransitionBlock (model/layers/folding/diffusion_transformer.py:50-71)."""
    w = _prefixed("adaln", adaln_weights(rng, c_a, c_s))
    w["swiglu.linear.weight"] = rng.linear(2 * c_a * factor, c_a)
    w["linear_g.weight"] = rng.linear(c_a, c_s)
    w["linear_g.bias"] = rng.normal(c_a, std=0.1) - 2.0
    w["linear_out.weight"] = rng.linear(c_a, c_a * factor)
    return w


def pairformer_block_weights(seed: int, c_z: int = 128, c_s: int = 384, tri_heads: int = 4,
                             single_heads: int = 16) -> dict:
    """All weights of the composite Pairformer block (pair track + single track)."""
    rng = _Rng(seed)
    w = {}
    w.update(_prefixed("tri_mul_out", trimul_weights(rng, c_z)))
    w.update(_prefixed("tri_mul_in", trimul_weights(rng, c_z)))
    w.update(_prefixed("tri_att_start", triatt_weights(rng, c_z, tri_heads)))
    w.update(_prefixed("tri_att_end", triatt_weights(rng, c_z, tri_heads)))
    w.update(_prefixed("transition_z", transition_weights(rng, c_z, 4)))
    w["layernorm_z.weight"] = rng.ln_w(c_z)
    w["layernorm_z.bias"] = rng.ln_b(c_z)
    w["linear_pair_bias.weight"] = rng.linear(single_heads, c_z)
    w.update(_prefixed("attention", apb_weights(rng, c_s, None)))
    w.update(_prefixed("transition", transition_weights(rng, c_s, 4)))
    return w


def triangular_block_weights(seed: int, c_z: int = 256) -> dict:
    """TriangularBlock, the block of K-Fold's own trunk (model/modules/tri_stack.py:119-128)."""
    rng = _Rng(seed)
    w = {}
    w.update(_prefixed("tri_mul_out", trimul_weights(rng, c_z)))
    w.update(_prefixed("tri_mul_in", trimul_weights(rng, c_z)))
    w.update(_prefixed("transition_z", transition_weights(rng, c_z, 4)))
    return w


def lm_to_pair_weights(rng: _Rng, c_s: int, c_z: int) -> dict:
    """LMToPair (model/model.py:114-126)."""
    return {"proj.0.weight": rng.ln_w(c_s), "proj.0.bias": rng.ln_b(c_s),
            "proj.1.weight": rng.linear(2 * c_z, c_s), "proj.1.bias": rng.normal(2 * c_z, std=0.1),
            "mlp.0.weight": rng.linear(c_z, 2 * c_z), "mlp.0.bias": rng.normal(c_z, std=0.1),
            "mlp.2.weight": rng.linear(c_z, c_z), "mlp.2.bias": rng.normal(c_z, std=0.1),
            "layernorm_pair.weight": rng.ln_w(c_z), "layernorm_pair.bias": rng.ln_b(c_z)}


def pair_conditioning_weights(rng: _Rng, c_z: int, rel_pos_dim: int = 139) -> dict:
    """PairConditioning (model/layers/folding/diffusion.py:50-68)."""
    w = {"layernorm.weight": rng.ln_w(c_z + rel_pos_dim), "linear.weight": rng.linear(c_z, c_z + rel_pos_dim)}
    for i in range(2):
        w.update(_prefixed(f"transitions.{i}", transition_weights(rng, c_z, 2)))
    return w


def parcae_weights(rng: _Rng, c_z: int) -> dict:
    """The recurrence parameters of KFold (model/model.py:203-217) and its layernorm_z; perturbed around their initial
    values so that every term matters."""
    import math
    delta_init = -math.log(0.4472135954999579)
    return {"parcae_log_a": rng.normal(c_z, std=0.3), "parcae_log_delta": rng.normal(c_z, std=0.2) + math.log(math.expm1(delta_init)),
            "parcae_b_cont": torch.eye(c_z) + rng.normal(c_z, c_z, std=0.05),
            "layernorm_z.weight": rng.ln_w(c_z), "layernorm_z.bias": rng.ln_b(c_z)}


def confidence_head_weights(rng: _Rng, c_s: int, c_z: int, heads: int, blocks: int, num_bins: int = 39, pae: int = 64,
                            pde: int = 64, plddt: int = 50) -> dict:
    """ConfidenceHead (model/modules/confidence_head.py:216-296)."""
    w = {"linear_s1.weight": rng.linear(c_z, c_s), "linear_s2.weight": rng.linear(c_z, c_s),
         "s_lm_to_s.0.weight": rng.ln_w(c_s), "s_lm_to_s.0.bias": rng.ln_b(c_s), "s_lm_to_s.1.weight": rng.linear(c_s, c_s),
         "linear_distogram.weight": rng.linear(c_z, num_bins)}
    for i in range(blocks):
        p = f"stack.blocks.{i}"
        w.update(_prefixed(p + ".pair_block.tri_mul_out", trimul_weights(rng, c_z)))
        w.update(_prefixed(p + ".pair_block.tri_mul_in", trimul_weights(rng, c_z)))
        w.update(_prefixed(p + ".pair_block.transition_z", transition_weights(rng, c_z, 4)))
        w[p + ".layernorm_z.weight"], w[p + ".layernorm_z.bias"] = rng.ln_w(c_z), rng.ln_b(c_z)
        w[p + ".linear_pair_bias.weight"] = rng.linear(heads, c_z)
        w.update(_prefixed(p + ".attention", apb_weights(rng, c_s, None)))
        w.update(_prefixed(p + ".transition", transition_weights(rng, c_s, 4)))
    for name, c_in, c_out in (("pae_head", c_z, pae), ("pde_head", c_z, pde), ("plddt_head", c_s, 24 * plddt), ("resolved_head", c_s, 48)):
        w[name + ".0.weight"], w[name + ".0.bias"] = rng.ln_w(c_in), rng.ln_b(c_in)
        w[name + ".1.weight"] = rng.linear(c_out, c_in)
    return w


def token_mask(n: int, valid: int | None = None, pad_frac: float | None = None) -> torch.Tensor:
    """Boolean token mask with a trailing padding tail (how K-Fold pads, inference/data_pipeline.py:129-134)."""
    if valid is None:
        valid = n if pad_frac is None else n - int(pad_frac * n)
    m = torch.zeros(n, dtype=torch.bool)
    m[:valid] = True
    return m


def pair_inputs(seed: int, n: int, c_z: int = 128, batch: int = 1, valid: int | None = None,
                pad_frac: float | None = None):
    """z ~ N(0,1) of shape (B,N,N,C) and the outer-product pair mask (B,N,N) bool."""
    rng = _Rng(seed + 7919)
    z = rng.normal(batch, n, n, c_z)
    m = token_mask(n, valid, pad_frac)
    pm = (m[:, None] & m[None, :]).unsqueeze(0).expand(batch, n, n).contiguous()
    return z, pm, m.unsqueeze(0).expand(batch, n).contiguous()


def single_inputs(seed: int, n: int, c_s: int = 384, batch: int = 1) -> torch.Tensor:
    return _Rng(seed + 104729).normal(batch, n, c_s)


def block_mask(seed: int, batch: int, n: int) -> torch.Tensor:
    """A general, non-separable (B,N,N) mask like the Apo stack's (model/modules/apo_module.py:322-330)."""
    rs = np.random.RandomState(seed + 31)
    return torch.from_numpy(rs.rand(batch, n, n) > 0.2)
