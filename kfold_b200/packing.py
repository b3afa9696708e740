"""Weight packing for the CUDA kernels (done once per module, cached by the caller).

The tcgen05 GEMM computes 128 x 256 output tiles.  For gated projections the
epilogue needs a value column and its gate column in the SAME tile, so the two
weight matrices are interleaved in blocks of 128 rows: tile t holds value rows
[128 t, 128 t + 128) followed by the gate rows of the same channels.
"""
from __future__ import annotations

import torch

GLU_HALF = 128  # value (or gate) columns per 256-wide GEMM tile
GLU_HALF_PRECISE = 64  # the fp32-accurate GEMM variant uses 128-wide tiles


def interleave_glu(value_w: torch.Tensor, gate_w: torch.Tensor, half: int = GLU_HALF, value_scale: float = 1.0,
                   gate_scale: float = 1.0) -> torch.Tensor:
    """[n, k] value and gate weights -> [2n, k] with alternating blocks of `half` rows.  The scales implement the bf16
    kernels' gate arithmetic: sigmoid(g) = 0.5 + 0.5 tanh(g / 2), so the tensor core is handed the halved matrices
    (exact in bf16) and the epilogue needs one tanh and one fused multiply-add per gate:
      sigmoid GLU   v sigmoid(g)   = v' + v' tanh(g')     with v' = v / 2, g' = g / 2      -> glu_scales("sigmoid")
      SwiGLU        a sigmoid(a) g = (a' + a' tanh(a')) g with a' = a / 2                  -> glu_scales("swiglu")
    The fp32-accurate packing keeps the matrices as they are (exact sigmoid in the epilogue)."""
    n, k = value_w.shape
    value_w, gate_w = value_w * value_scale, gate_w * gate_scale
    assert gate_w.shape == (n, k) and n % half == 0, (value_w.shape, gate_w.shape, half)
    v = value_w.reshape(n // half, half, k)
    g = gate_w.reshape(n // half, half, k)
    return torch.stack((v, g), dim=1).reshape(2 * n, k).contiguous()


def glu_scales(kind: str, precise: bool) -> dict:
    """Keyword arguments of interleave_glu for the bf16 kernels' halved gate operands (none for the fp32-accurate mode)."""
    if precise:
        return {}
    return {"value_scale": 0.5, "gate_scale": 0.5} if kind == "sigmoid" else {"value_scale": 0.5}


# The tensor-core attention kernel keeps its logits in log2 units: the query projection carries log2(e) / sqrt(D).
LOG2E = 1.4426950408889634


def split3_weights(w: torch.Tensor) -> torch.Tensor:
    """fp32 [n, k] -> bf16 [n, 6k] = [w0 | w1 | w0 | w1 | w2 | w0] with w = w0 + w1 + w2 (bf16 parts): the B operand of
    the fp32-accurate GEMMs, matching activations stored as [x0 | x0 | x1 | x1 | x0 | x2]."""
    w = w.detach().float()
    w0 = w.to(torch.bfloat16)
    r1 = w - w0.float()
    w1 = r1.to(torch.bfloat16)
    w2 = (r1 - w1.float()).to(torch.bfloat16)
    return torch.cat([w0, w1, w0, w1, w2, w0], dim=-1).contiguous()


def _w(t: torch.Tensor, device, precise: bool) -> torch.Tensor:
    """A projection weight on the device: bf16, or its triple split for the fp32-accurate mode."""
    if precise:
        return split3_weights(t).to(device)
    return t.detach().to(device=device, dtype=torch.bfloat16).contiguous()


def _dev(t: torch.Tensor, device, dtype) -> torch.Tensor:
    return t.detach().to(device=device, dtype=dtype).contiguous()


def channel_shard_order(c: int, world: int, parts: int = 1) -> torch.Tensor:
    """Order of the 2c operand channels [a | b] for the channel-sharded exchange: `parts` groups of c / parts channels
    that are exchanged one after the other, inside each group rank q's share first for q = 0, 1, ...:
    [h][q][a, b][c / (parts * world)].  Position (h, q, s, i) holds source channel s*c + h*(c/parts) + q*cl + i, so that
    the contraction result, returned group by group and rank by rank, lies in the original channel order."""
    cl = c // (world * parts)
    h, q, s_, i = torch.meshgrid(torch.arange(parts), torch.arange(world), torch.arange(2), torch.arange(cl), indexing="ij")
    return (s_ * c + h * (c // parts) + q * cl + i).reshape(-1)


def pack_trimul(w: dict, device, dtype=torch.bfloat16, precise: bool = False, shard_world: int = 0, shard_parts: int = 1) -> dict:
    """Weights of TriangleMultiplication{Outgoing,Incoming}: keys as in the reference state_dict
    (model/primitives/triangle_multiplication.py:171-177).  LayerNorm affine stays fp32.
    ``shard_world`` > 1 orders the operand channels for the channel-sharded exchange (channel_shard_order)."""
    wp, wg = w["linear_p_in.weight"].detach().float(), w["linear_g_in.weight"].detach().float()
    if shard_world > 1:
        order = channel_shard_order(wp.shape[0] // 2, shard_world, shard_parts).to(wp.device)
        wp, wg = wp[order], wg[order]
    return {
        "ln_in_w": _dev(w["layernorm_in.weight"], device, torch.float32),
        "ln_in_b": _dev(w["layernorm_in.bias"], device, torch.float32),
        "w_in": _w(interleave_glu(wp, wg, GLU_HALF_PRECISE if precise else GLU_HALF, **glu_scales("sigmoid", precise)), device, precise),
        "w_gout": _w(w["linear_g_out.weight"], device, precise),
        "ln_out_w": _dev(w["layernorm_out.weight"], device, torch.float32),
        "ln_out_b": _dev(w["layernorm_out.bias"], device, torch.float32),
        "w_pout": _w(w["linear_p_out.weight"], device, precise),
        "c": int(w["linear_p_out.weight"].shape[0]), "precise": precise,
    }


def head_dim_pad(d: int) -> int:
    """Head dims are padded to one swizzle span of the attention kernel: 32 or 64 elements."""
    if d % 8 != 0 or d < 16 or d > 64:
        raise ValueError(f"head dim {d} is not supported (multiples of 8 in [16, 64])")
    return 32 if d <= 32 else 64


def _pad_heads(w: torch.Tensor, heads: int, d: int, dp: int, scale: float = 1.0) -> torch.Tensor:
    """[heads*d, k] (or [heads*d]) -> [heads*dp, k] with zero rows after each head's d rows."""
    tail = w.shape[1:]
    out = w.new_zeros((heads, dp) + tuple(tail))
    out[:, :d] = w.reshape((heads, d) + tuple(tail)) * scale
    return out.reshape((heads * dp,) + tuple(tail))


def pack_triatt(w: dict, heads: int, device, dtype=torch.bfloat16, precise: bool = False) -> dict:
    """Weights of TriangleAttention (model/primitives/triangle_attention.py:338-373).

    One projection matrix [q * log2(e) / sqrt(D) | k | g | v | triangle-bias] with every head padded to the
    kernel's head stride and the bias rows padded to 32.  The fp32-accurate packing keeps the heads unpadded
    and stores every matrix as its bf16 triple split.
    """
    c = int(w["mha.linear_q.weight"].shape[1])
    d = c // heads
    if precise:
        g = lambda k, s=1.0: w[k].detach().float() * s
        wz_p = torch.zeros(32, c)
        wz_p[:heads] = w["linear.weight"].detach().float()
        proj = torch.cat([g("mha.linear_q.weight", d ** -0.5), g("mha.linear_k.weight"), g("mha.linear_g.weight"),
                          g("mha.linear_v.weight"), wz_p.to(w["linear.weight"].device)], dim=0)
        return {
            "ln_w": _dev(w["layer_norm.weight"], device, torch.float32),
            "ln_b": _dev(w["layer_norm.bias"], device, torch.float32),
            "w_proj": _w(proj, device, True),
            "w_out": _w(w["mha.linear_o.weight"], device, True),
            "c": c, "heads": heads, "precise": True,
        }
    dp = head_dim_pad(d)
    f = lambda k, s=1.0: _pad_heads(w[k].detach().float(), heads, d, dp, s)
    wz = w["linear.weight"].detach().float()
    wz_pad = wz.new_zeros(32, c)
    wz_pad[:heads] = wz
    proj = torch.cat([f("mha.linear_q.weight", d ** -0.5 * LOG2E), f("mha.linear_k.weight"), f("mha.linear_g.weight"),
                      f("mha.linear_v.weight"), wz_pad], dim=0)
    return {
        "ln_w": _dev(w["layer_norm.weight"], device, torch.float32),
        "ln_b": _dev(w["layer_norm.bias"], device, torch.float32),
        "w_proj": _dev(proj, device, dtype),
        "w_out": _dev(w["mha.linear_o.weight"], device, dtype),
        "c": c, "heads": heads,
    }


def pack_apb(w: dict, heads: int, device, dtype=torch.bfloat16, precise: bool = False) -> dict:
    """Projections of AttentionPairBias (model/layers/folding/attention_pair_bias.py:30-67):
    [q * log2(e) / sqrt(D) (+ bias, same scale) | k | g | v], heads padded; output projection as is.
    The fp32-accurate packing keeps the heads unpadded and stores the matrices as bf16 triple splits."""
    c = int(w["linear_q.weight"].shape[1])
    d = c // heads
    if precise:
        qs = d ** -0.5
        g = lambda k, s=1.0: w[k].detach().float() * s
        proj = torch.cat([g("linear_q.weight", qs), g("linear_k.weight"), g("linear_g.weight"), g("linear_v.weight")], dim=0)
        pb = torch.zeros(4 * c, dtype=torch.float32)
        if w.get("linear_q.bias") is not None:
            pb[:c] = w["linear_q.bias"].detach().float().cpu() * qs
        if w.get("linear_g.bias") is not None:
            pb[2 * c: 3 * c] = w["linear_g.bias"].detach().float().cpu()
        ob = w.get("linear_out.bias")
        return {
            "w_proj": _w(proj, device, True),
            "proj_bias": _dev(pb, device, torch.float32),
            "w_out": _w(w["linear_out.weight"], device, True),
            "out_bias": None if ob is None else _dev(ob, device, torch.float32),
            "c": c, "heads": heads, "precise": True,
        }
    dp = head_dim_pad(d)
    f = lambda k, s=1.0: _pad_heads(w[k].detach().float(), heads, d, dp, s)
    qs = d ** -0.5 * LOG2E
    proj = torch.cat([f("linear_q.weight", qs), f("linear_k.weight"), f("linear_g.weight"), f("linear_v.weight")], dim=0)
    pb = torch.zeros(4 * heads * dp, dtype=torch.float32)
    if w.get("linear_q.bias") is not None:
        pb[: heads * dp] = _pad_heads(w["linear_q.bias"].detach().float(), heads, d, dp, qs)
    if w.get("linear_g.bias") is not None:
        pb[2 * heads * dp: 3 * heads * dp] = _pad_heads(w["linear_g.bias"].detach().float(), heads, d, dp)
    ob = w.get("linear_out.bias")
    return {
        "w_proj": _dev(proj, device, dtype),
        "proj_bias": _dev(pb, device, torch.float32),
        "w_out": _dev(w["linear_out.weight"], device, dtype),
        "out_bias": None if ob is None else _dev(ob, device, torch.float32),
        "c": c, "heads": heads,
    }


def pack_apb_cross(w: dict, heads: int, device, dtype=torch.bfloat16, precise: bool = False) -> dict:
    """Projections of AttentionPairBias for cross attention (queries and keys from different tensors,
    model/primitives/attention.py:75-83): the query side [q * log2(e) / sqrt(D) (+ bias) | g] and the key side [k | v]
    as two matrices, heads padded; the fp32-accurate packing keeps the heads unpadded, scales q by 1 / sqrt(D) only
    and stores bf16 triple splits."""
    c = int(w["linear_q.weight"].shape[1])
    d = c // heads
    ob = w.get("linear_out.bias")
    if precise:
        qs = d ** -0.5
        g = lambda k, s=1.0: w[k].detach().float() * s
        qb = torch.zeros(2 * c, dtype=torch.float32)
        if w.get("linear_q.bias") is not None:
            qb[:c] = w["linear_q.bias"].detach().float().cpu() * qs
        if w.get("linear_g.bias") is not None:
            qb[c:] = w["linear_g.bias"].detach().float().cpu()
        return {
            "w_q": _w(torch.cat([g("linear_q.weight", qs), g("linear_g.weight")], dim=0), device, True),
            "q_bias": _dev(qb, device, torch.float32),
            "w_kv": _w(torch.cat([g("linear_k.weight"), g("linear_v.weight")], dim=0), device, True),
            "w_out": _w(w["linear_out.weight"], device, True),
            "out_bias": None if ob is None else _dev(ob, device, torch.float32),
            "c": c, "heads": heads, "precise": True,
        }
    dp = head_dim_pad(d)
    hdp = heads * dp
    f = lambda k, s=1.0: _pad_heads(w[k].detach().float(), heads, d, dp, s)
    qs = d ** -0.5 * LOG2E
    qb = torch.zeros(2 * hdp, dtype=torch.float32)
    if w.get("linear_q.bias") is not None:
        qb[:hdp] = _pad_heads(w["linear_q.bias"].detach().float(), heads, d, dp, qs)
    if w.get("linear_g.bias") is not None:
        qb[hdp:] = _pad_heads(w["linear_g.bias"].detach().float(), heads, d, dp)
    return {
        "w_q": _dev(torch.cat([f("linear_q.weight", qs), f("linear_g.weight")], dim=0), device, dtype),
        "q_bias": _dev(qb, device, torch.float32),
        "w_kv": _dev(torch.cat([f("linear_k.weight"), f("linear_v.weight")], dim=0), device, dtype),
        "w_out": _dev(w["linear_out.weight"], device, dtype),
        "out_bias": None if ob is None else _dev(ob, device, torch.float32),
        "c": c, "heads": heads,
    }


def pack_transition(w: dict, device, dtype=torch.bfloat16, precise: bool = False) -> dict:
    """Weights of Transition (model/layers/folding/transition.py:27-46): the SwiGLU matrix is split into
    its silu half and its linear half (model/primitives/activation.py:27-29) and interleaved per GEMM tile."""
    sw = w["swiglu.linear.weight"].detach().float()
    hidden = sw.shape[0] // 2
    return {
        "ln_w": _dev(w["layernorm.weight"], device, torch.float32),
        "ln_b": _dev(w["layernorm.bias"], device, torch.float32),
        "w_swiglu": _w(interleave_glu(sw[:hidden], sw[hidden:], GLU_HALF_PRECISE if precise else GLU_HALF, **glu_scales("swiglu", precise)), device,
                       precise),
        "w_out": _w(w["linear_out.weight"], device, precise),
        "c": int(sw.shape[1]), "hidden": int(hidden), "precise": precise,
    }


def pack_adaln(w: dict, device, dtype=torch.bfloat16, precise: bool = False) -> dict:
    """AdaLN (model/primitives/normalization.py:99-115): the gate and shift projections of the conditioning
    stacked into one [2 c_a, c_s] matrix (bias only on the gate half)."""
    wg, wb = w["linear_g.weight"].detach().float(), w["linear_bias.weight"].detach().float()
    c_a = wg.shape[0]
    bias = torch.zeros(2 * c_a, dtype=torch.float32)
    bias[:c_a] = w["linear_g.bias"].detach().float()
    return {
        "ln_s_w": _dev(w["layernorm_s.weight"], device, torch.float32),
        "w_gs": _w(torch.cat([wg, wb], dim=0), device, precise),
        "b_gs": _dev(bias, device, torch.float32),
        "c_a": int(c_a), "c_s": int(wg.shape[1]), "precise": precise,
    }


def pack_cond_transition(w: dict, device, dtype=torch.bfloat16, precise: bool = False) -> dict:
    """ConditionedTransitionBlock (model/layers/folding/diffusion_transformer.py:50-71)."""
    sw = w["swiglu.linear.weight"].detach().float()
    hidden = sw.shape[0] // 2
    return {
        "adaln": pack_adaln({k[len("adaln."):]: v for k, v in w.items() if k.startswith("adaln.")}, device, dtype, precise),
        "w_swiglu": _w(interleave_glu(sw[:hidden], sw[hidden:], GLU_HALF_PRECISE if precise else GLU_HALF, **glu_scales("swiglu", precise)), device,
                       precise),
        "w_out": _w(w["linear_out.weight"], device, precise),
        "w_g": _w(w["linear_g.weight"], device, precise),
        "b_g": _dev(w["linear_g.bias"], device, torch.float32),
        "c": int(sw.shape[1]), "hidden": int(hidden), "precise": precise,
    }
