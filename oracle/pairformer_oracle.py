"""CPU oracle for the Pairformer / diffusion hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch on the CPU, the arithmetic that K-Fold's
``kernel_backend="torch"`` path performs for the operators this repository
accelerates.  Nothing under ``kfold_b200/`` may import it: it exists so that
tests, the smoke check and the CPU-baseline leg of the benchmark have an
independent result to compare the CUDA kernels against.

Parity is pinned: ``tests/golden/make_golden.py`` runs the real reference
modules (imported from the K-Fold source tree) on seeded inputs, stores their
outputs under ``tests/golden/``, and ``tests/test_oracle_golden.py`` checks every
function here against those vectors.

Every function takes a flat ``dict`` of weights keyed exactly like the
``state_dict()`` of the reference module it follows, so a reference module's
weights drop straight in.

``mode`` selects the arithmetic:
  * ``"fp32"``  -- everything in float32 (ground truth).
  * ``"bf16"``  -- rounds to bfloat16 at the points where the reference rounds
    when it runs under ``torch.autocast("cuda", dtype=torch.bfloat16)``:
    linear / matmul / einsum outputs are bf16 (fp32 accumulate), LayerNorm and
    softmax are computed in fp32 and LayerNorm is rounded back to the input
    dtype.  Used to report the reference's own bf16 noise floor.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

__all__ = [
    "layer_norm",
    "triangle_multiplication",
    "triangle_attention",
    "attention_pair_bias",
    "self_attention_pair_bias",
    "adaln",
    "transition",
    "conditioned_transition",
    "pairformer_block",
    "global_transformer_stack",
    "triangular_block",
    "sub",
]


def sub(weights: dict, prefix: str) -> dict:
    """Select ``prefix.*`` from a flat state dict and strip the prefix."""
    p = prefix + "."
    return {k[len(p):]: v for k, v in weights.items() if k.startswith(p)}


class _Mode:
    def __init__(self, mode: str):
        if mode not in ("fp32", "bf16"):
            raise ValueError(f"unknown oracle mode {mode!r}")
        self.bf16 = mode == "bf16"

    def r(self, t: torch.Tensor) -> torch.Tensor:
        """Round to the compute dtype (identity in fp32 mode), stay float32."""
        return t.to(torch.bfloat16).float() if self.bf16 else t

    def linear(self, x, w, b=None):
        # autocast casts inputs and weights to bf16, accumulates fp32, rounds the result
        out = F.linear(self.r(x), self.r(w), None if b is None else self.r(b))
        return self.r(out)


def layer_norm(x, weight, bias, eps: float = 1e-5, mode: str = "fp32"):
    """``LayerNorm.forward`` -- model/primitives/normalization.py:61-91.

    Statistics and affine in fp32 whatever the input dtype; the result is cast
    back to the input dtype (which is bf16 inside a bf16 pipeline).
    """
    m = _Mode(mode)
    out = F.layer_norm(x.float(), (x.shape[-1],), weight, bias, eps)
    return m.r(out)


def triangle_multiplication(x, mask, w: dict, direction: str, mode: str = "fp32", eps: float = 1e-5):
    """``TriangleMultiplication{Outgoing,Incoming}.forward`` --
    model/primitives/triangle_multiplication.py:179-229 and :263-313.

    x (B,N,N,C); mask (B,N,N); returns the update (the caller adds it to x).
    """
    m = _Mode(mode)
    x = m.r(x.float())
    xn = layer_norm(x, w["layernorm_in.weight"], w["layernorm_in.bias"], eps, mode)
    ab = m.r(m.linear(xn, w["linear_p_in.weight"]) * torch.sigmoid(m.linear(xn, w["linear_g_in.weight"])))
    ab = m.r(ab * mask.unsqueeze(-1).to(ab.dtype))
    a, b = torch.chunk(ab, 2, dim=-1)
    if direction == "outgoing":
        t = torch.einsum("bikd,bjkd->bijd", a, b)      # :224
    elif direction == "incoming":
        t = torch.einsum("bkid,bkjd->bijd", a, b)      # :308
    else:
        raise ValueError(f"unknown direction {direction!r}")
    t = m.r(t)  # einsum is autocast to bf16 although its inputs were .float()
    tn = layer_norm(t, w["layernorm_out.weight"], w["layernorm_out.bias"], eps, mode)
    out = m.linear(tn, w["linear_p_out.weight"]) * torch.sigmoid(m.linear(xn, w["linear_g_out.weight"]))
    return m.r(out)


def triangle_attention(x, mask, w: dict, num_heads: int, starting: bool, mode: str = "fp32",
                       inf: float = 1e9, eps: float = 1e-5, row_chunk: int | None = None):
    """``TriangleAttention.forward`` + ``MultiHeadAttention.forward`` --
    model/primitives/triangle_attention.py:375-434 and :285-335.

    x (*,I,J,C); mask (*,I,J) or None.  Ending node = starting node on the
    transposed pair representation (:400-402), transposed back (:431-432).
    ``row_chunk`` only bounds memory: the rows I are independent attention problems and
    are processed ``row_chunk`` at a time with identical arithmetic.
    """
    m = _Mode(mode)
    x = m.r(x.float())
    if mask is None:
        mask = x.new_ones(x.shape[:-1])
    if not starting:
        x = x.transpose(-2, -3)
        mask = mask.transpose(-1, -2)
    H = num_heads
    C = x.shape[-1]
    D = C // H
    xn = layer_norm(x, w["layer_norm.weight"], w["layer_norm.bias"], eps, mode)
    # bias[..., h, j, k] = linear(xn)[..., j, k, h]                (:416-422)
    tri_bias = m.linear(xn, w["linear.weight"]).movedim(-1, -3).unsqueeze(-4)
    q = m.linear(xn, w["mha.linear_q.weight"])
    k = m.linear(xn, w["mha.linear_k.weight"])
    v = m.linear(xn, w["mha.linear_v.weight"])
    q, k, v = (t.unflatten(-1, (H, D)).transpose(-2, -3) for t in (q, k, v))   # (*,I,H,J,D)
    q = m.r(q / math.sqrt(D))                                                    # :264-265
    mask_bias = -inf * (~mask.bool()).to(q.dtype)[..., :, None, None, :]        # (*,I,1,1,J)  :328

    def core(q, k, v, mask_bias):
        a = m.r(torch.matmul(q, k.transpose(-1, -2)))                           # (*,I,H,J,J)  :139
        a = m.r(a + mask_bias)
        a = m.r(a + tri_bias)
        a = a.softmax(dim=-1)   # CUDA autocast runs softmax in fp32 and keeps it fp32
        return m.r(torch.matmul(m.r(a), v))                                     # :149

    n_rows = q.shape[-4]
    if row_chunk is None or row_chunk >= n_rows:
        o = core(q, k, v, mask_bias)
    else:
        o = torch.cat([core(q[..., i:i + row_chunk, :, :, :], k[..., i:i + row_chunk, :, :, :],
                            v[..., i:i + row_chunk, :, :, :], mask_bias[..., i:i + row_chunk, :, :, :])
                       for i in range(0, n_rows, row_chunk)], dim=-4)
    o = o.transpose(-2, -3)                                                      # (*,I,J,H,D)
    g = torch.sigmoid(m.linear(xn, w["mha.linear_g.weight"])).unflatten(-1, (H, D))
    o = m.r(o * g).flatten(-2)                                                   # :269-278
    out = m.linear(o, w["mha.linear_o.weight"])                                  # :281
    if not starting:
        out = out.transpose(-2, -3)
    return out


def attention_pair_bias(x_q, x_k, pair_bias, mask, w: dict, num_heads: int, mode: str = "fp32",
                        inf: float = 1e9):
    """``attention_pair_bias`` with the torch kernel --
    model/primitives/attention.py:28-94 and ``torch_attention_pair_bias`` :239-271,
    ``_attention`` :122-168.  Inputs are already normalised.

    x_q (*,Lq,c); x_k (*,Lk,c); pair_bias broadcastable to (*,H,Lq,Lk);
    mask broadcastable to (*,Lk).  The logits and softmax are fp32 in every mode.
    """
    m = _Mode(mode)
    H = num_heads
    c = x_q.shape[-1]
    D = c // H
    x_q = m.r(x_q.float())
    x_k = m.r(x_k.float())
    q = m.linear(x_q, w["linear_q.weight"], w.get("linear_q.bias"))
    k = m.linear(x_k, w["linear_k.weight"])
    v = m.linear(x_k, w["linear_v.weight"])
    q, k, v = (t.unflatten(-1, (H, D)).transpose(-2, -3) for t in (q, k, v))    # (*,H,L,D)
    bias = pair_bias.float() - inf * (~mask.bool()).float()[..., None, None, :]  # :254-257
    scale = 1.0 / math.sqrt(D)
    attn = torch.einsum("...qc,...kc->...qk", q * scale, k) + bias              # fp32 :155-160
    attn = m.r(attn.softmax(dim=-1))                                            # .to(value.dtype) :163
    av = m.r(torch.einsum("...qk,...kc->...qc", attn, v))
    av = av.transpose(-2, -3).reshape(x_q.shape)                                # :267
    g = torch.sigmoid(m.linear(x_q, w["linear_g.weight"], w.get("linear_g.bias")))
    return m.linear(m.r(g * av), w["linear_out.weight"], w.get("linear_out.bias"))


def adaln(a, s, w: dict, mode: str = "fp32", eps: float = 1e-5):
    """``AdaLN.forward`` -- model/primitives/normalization.py:117-125."""
    m = _Mode(mode)
    a = layer_norm(a, None, None, eps, mode)
    s = layer_norm(s, w["layernorm_s.weight"], None, eps, mode)
    g = torch.sigmoid(m.linear(s, w["linear_g.weight"], w["linear_g.bias"]))
    return m.r(g * a + m.linear(s, w["linear_bias.weight"]))


def self_attention_pair_bias(a, s, pair_bias, mask, w: dict, num_heads: int, mode: str = "fp32",
                             inf: float = 1e9):
    """``SelfAttentionPairBias.forward`` -- model/layers/folding/attention_pair_bias.py:114-158.

    With ``s is None`` the prologue is a plain LayerNorm (the confidence / single
    track form); otherwise AdaLN prologue and the sigmoid(Linear(s)) output gate.
    """
    m = _Mode(mode)
    if s is None:
        an = layer_norm(a, w["layernorm_a.weight"], w["layernorm_a.bias"], 1e-5, mode)
    else:
        an = adaln(a, s, sub(w, "adaln_a"), mode)
    out = attention_pair_bias(an, an, pair_bias, mask, w, num_heads, mode, inf)
    if s is not None:
        gate = torch.sigmoid(m.linear(m.r(s.float()), w["linear_ada_out.weight"], w["linear_ada_out.bias"]))
        out = m.r(gate * out)
    return out


def transition(x, w: dict, mode: str = "fp32", eps: float = 1e-5):
    """``Transition.forward`` -- model/layers/folding/transition.py:48-68 with
    ``SwiGLU.forward`` -- model/primitives/activation.py:27-29."""
    m = _Mode(mode)
    xn = layer_norm(m.r(x.float()), w["layernorm.weight"], w["layernorm.bias"], eps, mode)
    u1, u2 = m.linear(xn, w["swiglu.linear.weight"]).chunk(2, dim=-1)
    h = m.r(F.silu(u1) * u2)
    return m.linear(h, w["linear_out.weight"])


def conditioned_transition(a, s, w: dict, mode: str = "fp32"):
    """``ConditionedTransitionBlock.forward`` --
    model/layers/folding/diffusion_transformer.py:73-81: AdaLN prologue, SwiGLU,
    output projection gated by sigmoid(Linear(s))."""
    m = _Mode(mode)
    an = adaln(a, s, sub(w, "adaln"), mode)
    u1, u2 = m.linear(an, w["swiglu.linear.weight"]).chunk(2, dim=-1)
    h = m.r(F.silu(u1) * u2)
    gate = torch.sigmoid(m.linear(m.r(s.float()), w["linear_g.weight"], w["linear_g.bias"]))
    return m.r(gate * m.linear(h, w["linear_out.weight"]))


def global_transformer_stack(a, s, pair_bias, mask, w: dict, num_heads: int, num_blocks: int, mode: str = "fp32"):
    """``CachedGlobalTransformerStack.forward`` -- model/layers/folding/diffusion_transformer.py:302-339 with the
    block of :376-413: a += SelfAttentionPairBias(a, s, bias_n, mask); a += ConditionedTransitionBlock(a, s).
    pair_bias (*, Nblock, H, L, L)."""
    m = _Mode(mode)
    a = a.float()
    for i in range(num_blocks):
        wb = sub(w, f"blocks.{i}")
        a = a + self_attention_pair_bias(a, s, pair_bias[..., i, :, :, :].unsqueeze(-4) if pair_bias.dim() == a.dim() + 1
                                         else pair_bias[..., i, :, :, :], mask, sub(wb, "attention"), num_heads, mode)
        a = a + conditioned_transition(a, s, sub(wb, "transition"), mode)
    return a


def broadcast_tokens_to_atoms(x, token_index):
    """``broadcast_tokens_to_atoms`` -- model/layers/folding/utils.py:25-51: out[..., a, :] = x[..., token_index[a], :]."""
    if x.ndim == token_index.ndim:
        return broadcast_tokens_to_atoms(x.unsqueeze(-1), token_index).squeeze(-1)
    shape = list(x.shape)
    shape[-2] = token_index.shape[-1]
    return torch.gather(x, -2, token_index.unsqueeze(-1).expand(*shape))


def aggregate_atoms_to_tokens(x, token_index, mask, num_tokens: int):
    """``aggregate_atoms_to_tokens`` -- model/layers/folding/utils.py:54-93: fp32 mean over the valid atoms of each
    token (padding atoms go to an extra slot that is dropped); tokens without atoms give zeros."""
    index = torch.where(mask, token_index, num_tokens).unsqueeze(-1).expand(*x.shape)
    shape = list(x.shape)
    shape[-2] = num_tokens + 1
    out = torch.zeros(*shape, dtype=torch.float32, device=x.device).scatter_reduce_(
        -2, index, x.float(), reduce="mean", include_self=False)
    return out[..., :num_tokens, :].to(x.dtype).contiguous()


def atom_windows(x, dim: int):
    """Window indexing of the local attention -- model/layers/folding/utils.py:97-188: queries in windows of 32,
    keys = eight half-blocks of 16 atoms around each window, i.e. atoms [32 w - 48, 32 w + 80); out-of-range keys
    are zero-filled (:140-147, :184-187)."""
    dim = dim % x.ndim
    length = x.shape[dim]
    if length % 32 != 0:
        raise ValueError("Length must be divisible by 32")
    nw = length // 32
    idx = torch.arange(nw, device=x.device)[:, None] * 32 - 48 + torch.arange(128, device=x.device)[None, :]
    pad = (idx < 0) | (idx >= length)
    x_q = x.unflatten(dim, (nw, 32))
    x_k = x.index_select(dim, idx.clamp(0, length - 1).reshape(-1)).unflatten(dim, (nw, 128))
    shape = [1] * x_k.ndim
    shape[dim], shape[dim + 1] = nw, 128
    return x_q, x_k.masked_fill(pad.view(shape), 0)


def cross_attention_pair_bias(a_q, a_k, s_q, s_k, pair_bias, mask, w: dict, num_heads: int, mode: str = "fp32"):
    """``CrossAttentionPairBias.forward`` -- model/layers/folding/attention_pair_bias.py:206-260."""
    m = _Mode(mode)
    if s_q is not None:
        x_q = adaln(a_q, s_q, sub(w, "adaln_a_q"), mode)
        x_k = adaln(a_k, s_k, sub(w, "adaln_a_k"), mode)
    else:
        x_q = layer_norm(a_q, w["layernorm_a_q.weight"], w["layernorm_a_q.bias"], 1e-5, mode)
        x_k = layer_norm(a_k, w["layernorm_a_k.weight"], w["layernorm_a_k.bias"], 1e-5, mode)
    out = attention_pair_bias(x_q, x_k, pair_bias, mask, w, num_heads, mode)
    if s_q is not None:
        gate = torch.sigmoid(m.linear(m.r(s_q.float()), w["linear_ada_out.weight"], w["linear_ada_out.bias"]))
        out = m.r(gate * out)
    return out


def local_transformer_stack(a, s, z, mask, w: dict, num_heads: int, num_blocks: int, mode: str = "fp32"):
    """``LocalTransformerStack.forward`` -- model/layers/folding/diffusion_transformer.py:469-512 with the block of
    :564-597.  a (*, L, c_a); s (*, L, c_s); z (*, W, 32, 128, c_z); mask (*, L)."""
    m = _Mode(mode)
    a = a.float()
    s_q, s_k = atom_windows(s, -2)
    _, mask_k = atom_windows(mask, -1)
    zn = layer_norm(z, w["layernorm_z.weight"], None, 1e-5, mode)
    for i in range(num_blocks):
        wb = sub(w, f"blocks.{i}")
        a_q, a_k = atom_windows(a, -2)
        bias = m.linear(zn, wb["linear_z_to_bias.weight"]).movedim(-1, -3)          # (*, W, H, 32, 128)
        a_q = a_q + cross_attention_pair_bias(a_q, a_k, s_q, s_k, bias, mask_k, sub(wb, "attention"), num_heads, mode)
        a_q = a_q + conditioned_transition(a_q, s_q, sub(wb, "transition"), mode)
        a = a_q.flatten(-3, -2)
    return a


def atom_attention_encoder(q, c, p, token_index, mask, num_tokens: int, r_noisy, w: dict, num_heads: int, num_blocks: int,
                           mode: str = "fp32"):
    """``AtomAttentionEncoder.forward`` -- model/layers/folding/atom_transformer.py:311-389 with use_structure: the
    float32 coordinate embedding (:362-367), the local transformer, ReLU(Linear(q)) averaged per token (:383-385).
    Returns (a, q_skip)."""
    m = _Mode(mode)
    if r_noisy is not None:
        q = q.float() + F.linear(r_noisy.float(), w["linear_r_to_q.weight"].float())
    q = local_transformer_stack(q, c, p, mask, sub(w, "transformer"), num_heads, num_blocks, mode)
    x = torch.relu(m.linear(m.r(q), w["linear_q_to_a.weight"]))
    idx = torch.broadcast_to(token_index, x.shape[:-1])
    return m.r(aggregate_atoms_to_tokens(x, idx, torch.broadcast_to(mask, x.shape[:-1]), num_tokens)), q


def atom_attention_decoder(a, q_skip, c_skip, p_skip, token_index, mask, w: dict, num_heads: int, num_blocks: int,
                           mode: str = "fp32"):
    """``AtomAttentionDecoder.forward`` -- model/layers/folding/atom_transformer.py:433-489: Linear(a) broadcast to the
    atoms plus the skip connection, the local transformer, LayerNorm and the float32 projection to 3 coordinates."""
    m = _Mode(mode)
    a_to_q = m.linear(m.r(a.float()), w["linear_a_to_q.weight"])
    q = broadcast_tokens_to_atoms(a_to_q, torch.broadcast_to(token_index, a_to_q.shape[:-2] + token_index.shape[-1:])) + q_skip
    q = local_transformer_stack(q, c_skip, p_skip, mask, sub(w, "transformer"), num_heads, num_blocks, mode)
    qn = F.layer_norm(q.float(), (q.shape[-1],), w["layernorm_q.weight"].float(), None, 1e-5)
    return F.linear(qn, w["linear_q_to_r.weight"].float())


def fourier_weights(dim: int):
    """The fixed random Fourier weights -- model/layers/folding/embeddings.py:149-157: two draws of torch.randn from a
    CPU generator seeded with 42."""
    gen = torch.Generator()
    gen.manual_seed(42)
    w = torch.randn(size=(1, dim), generator=gen, device="cpu")
    b = torch.randn(size=(1, dim), generator=gen, device="cpu")
    return w, b


def single_conditioning(s_inputs, c_noise, w: dict, mode: str = "fp32"):
    """``SingleConditioning.forward`` -- model/layers/folding/diffusion.py:122-152: float32 Linear(s_inputs), Fourier
    features of the noise level (embeddings.py:174) normalised and projected in float32, broadcast sum, two
    Transitions.  s_inputs (B, Lt, c_s); c_noise (B, N) -> (B, N, Lt, c_s)."""
    fw, fb = fourier_weights(w["linear_fourier.weight"].shape[1])
    fw, fb = fw.to(s_inputs.device), fb.to(s_inputs.device)
    s = F.linear(s_inputs.float(), w["linear.weight"].float())
    emb = torch.cos((2 * math.pi) * c_noise.float()[..., None] * fw + fb)
    emb = F.layer_norm(emb, (emb.shape[-1],), w["layernorm_fourier.weight"].float(), None, 1e-5)
    emb = F.linear(emb, w["linear_fourier.weight"].float())
    s = (s[:, None, :, :] + emb[:, :, None, :]).to(s_inputs.dtype)
    for i in range(2):
        s = s + transition(s, sub(w, f"transitions.{i}"), mode)
    return s


def diffusion_step(r_noisy, q, c, p, token_index, atom_mask, s, pair_bias, token_mask, w: dict, atom_heads: int,
                   atom_blocks: int, token_heads: int, token_blocks: int, mode: str = "fp32"):
    """``DiffusionStack.step`` -- model/layers/folding/diffusion.py:465-600.  With ``endpoint_atom_attention_encoder.*``
    among the weights this is the separate-endpoint variant (:521-550): the six coordinate channels split between two atom
    encoders, whose token streams are normalised, concatenated and fused by a float32 Linear."""
    m = _Mode(mode)
    q, c, p = q.unsqueeze(-3), c.unsqueeze(-3), p.unsqueeze(-5)
    atom_mask, token_mask, token_index = atom_mask.unsqueeze(-2), token_mask.unsqueeze(-2), token_index.unsqueeze(-2)
    r_noisy = r_noisy * atom_mask[..., None]
    if "endpoint_fusion.weight" in w:
        a, q_skip = atom_attention_encoder(q, c, p, token_index, atom_mask, token_mask.shape[-1], r_noisy[..., :3],
                                           sub(w, "atom_attention_encoder"), atom_heads, atom_blocks, mode)
        a_e, _ = atom_attention_encoder(q, c, p, token_index, atom_mask, token_mask.shape[-1], r_noisy[..., 3:],
                                        sub(w, "endpoint_atom_attention_encoder"), atom_heads, atom_blocks, mode)
        cat = torch.cat((layer_norm(a, w["layernorm_a_t.weight"], None, 1e-5, mode),
                         layer_norm(a_e, w["layernorm_a_endpoint.weight"], None, 1e-5, mode)), dim=-1)
        a = F.linear(cat.float(), w["endpoint_fusion.weight"].float())      # a float32 Linear whatever the autocast state
    else:
        a, q_skip = atom_attention_encoder(q, c, p, token_index, atom_mask, token_mask.shape[-1], r_noisy,
                                           sub(w, "atom_attention_encoder"), atom_heads, atom_blocks, mode)
    sn = F.layer_norm(s.float(), (s.shape[-1],), w["layernorm_s.weight"].float(), None, 1e-5)
    a = a.float() + F.linear(sn, w["linear_s_to_a.weight"].float())
    a = global_transformer_stack(a, s, pair_bias.unsqueeze(-5), token_mask, sub(w, "token_transformer"), token_heads, token_blocks,
                                 mode)
    a = layer_norm(a, w["layernorm_a.weight"], None, 1e-5, mode)
    r_update = atom_attention_decoder(a, q_skip, c, p, token_index, atom_mask, sub(w, "atom_attention_decoder"), atom_heads,
                                      atom_blocks, mode)
    return r_update * atom_mask[..., None]


def parcae_dynamics(w: dict):
    """``KFold._parcae_discretized_dynamics`` -- model/model.py:272-277."""
    delta = F.softplus(w["parcae_log_delta"].float())
    a = torch.exp(-delta * torch.exp(w["parcae_log_a"].float()))
    return a, delta[:, None] * w["parcae_b_cont"].float()


def parcae_update(z, u, w: dict, mode: str = "fp32"):
    """The trunk's recurrence between recycling iterations, ``z = a * z + F.linear(self.layernorm_z(u_t), b)`` --
    model/model.py:528 (a and b cast to the autocast dtype first, :505)."""
    m = _Mode(mode)
    a, b = parcae_dynamics(w)
    un = layer_norm(u, w["layernorm_z.weight"], w["layernorm_z.bias"], 1e-5, mode)
    return m.r(m.r(m.r(a) * m.r(z.float())) + m.linear(un, b))


def lm_to_pair(s_lm, w: dict, mode: str = "fp32"):
    """``LMToPair.forward`` -- model/model.py:127-134."""
    m = _Mode(mode)
    x = m.linear(layer_norm(s_lm, w["proj.0.weight"], w["proj.0.bias"], 1e-5, mode), w["proj.1.weight"], w["proj.1.bias"])
    xi, xj = torch.chunk(x, 2, dim=-1)
    xi, xj = xi.unsqueeze(-2), xj.unsqueeze(-3)
    feats = torch.cat([m.r(xi * xj), m.r(xi - xj)], dim=-1)
    h = m.r(F.gelu(m.linear(feats, w["mlp.0.weight"], w["mlp.0.bias"])))
    y = m.linear(h, w["mlp.2.weight"], w["mlp.2.bias"])
    return layer_norm(y, w["layernorm_pair.weight"], w["layernorm_pair.bias"], 1e-5, mode)


def pair_conditioning(rel_pos_feats, z, w: dict, mode: str = "fp32"):
    """``PairConditioning.forward`` -- model/layers/folding/diffusion.py:70-94, the relative-position features given:
    a float32 LayerNorm + Linear over [z | rel_pos], then two Transitions added in place."""
    zc = torch.cat((z.float(), rel_pos_feats.float()), dim=-1)
    zn = F.layer_norm(zc, (zc.shape[-1],), w["layernorm.weight"].float(), None, 1e-5)
    out = F.linear(zn, w["linear.weight"].float())
    for i in range(2):
        out = out + transition(out, sub(w, f"transitions.{i}"), mode)
    return out


def confidence_head(s_inputs, s_lm, z, x_repr, mask, w: dict, num_heads: int, num_blocks: int, mode: str = "fp32",
                    min_dist: float = 3.25, max_dist: float = 50.75, num_bins: int = 39):
    """``ConfidenceHead.forward`` between the representative-atom gather and the atom-layout scatter, with
    ``forward_single`` for every sample -- model/modules/confidence_head.py:343-378, :413-470; blocks :152-175."""
    m = _Mode(mode)
    s0 = m.linear(layer_norm(s_lm, w["s_lm_to_s.0.weight"], w["s_lm_to_s.0.bias"], 1e-5, mode), w["s_lm_to_s.1.weight"])
    z0 = m.r(m.r(z.float()) + m.linear(s_inputs, w["linear_s1.weight"])[..., None, :, :]
             + m.linear(s_inputs, w["linear_s2.weight"])[..., :, None, :])
    boundaries = torch.linspace(min_dist, max_dist, num_bins - 1, device=z.device)
    pair_mask = mask[..., :, None] & mask[..., None, :]
    outs = []
    for i in range(x_repr.shape[1]):
        x = x_repr[:, i].float()
        d = (x[..., :, None, :] - x[..., None, :, :]).norm(dim=-1)
        dgram = F.one_hot((d[..., None] > boundaries).sum(dim=-1), num_bins).float()
        zi, si = m.r(z0 + m.linear(dgram, w["linear_distogram.weight"])), s0
        for b in range(num_blocks):
            wb = sub(w, f"stack.blocks.{b}")
            zi = triangular_block(zi, pair_mask, sub(wb, "pair_block"), mode)
            zn = layer_norm(zi, wb["layernorm_z.weight"], wb["layernorm_z.bias"], 1e-5, mode)
            bias = m.linear(zn, wb["linear_pair_bias.weight"]).movedim(-1, -3)
            si = m.r(si + self_attention_pair_bias(si, None, bias, mask, sub(wb, "attention"), num_heads, mode))
            si = m.r(si + transition(si, sub(wb, "transition"), mode))
        zf, sf = zi.float(), si.float()

        def head(x_, name):
            xn = F.layer_norm(x_, (x_.shape[-1],), w[name + ".0.weight"].float(), w[name + ".0.bias"].float(), 1e-5)
            return F.linear(xn, w[name + ".1.weight"].float())

        pde = head(zf, "pde_head")
        outs.append((head(zf, "pae_head"), pde + pde.transpose(-2, -3), head(sf, "plddt_head").unflatten(-1, (24, -1)),
                     head(sf, "resolved_head").unflatten(-1, (24, 2))))
    names = ("pae_logits", "pde_logits", "plddt_logits", "resolved_logits")
    return {n: torch.stack([o[k] for o in outs], dim=1) for k, n in enumerate(names)}


def triangular_block(z, pair_mask, w: dict, mode: str = "fp32"):
    """``TriangularBlock.forward`` (eval) -- model/modules/tri_stack.py:130-151."""
    m = _Mode(mode)
    z = m.r(z.float())
    z = m.r(z + triangle_multiplication(z, pair_mask, sub(w, "tri_mul_out"), "outgoing", mode))
    z = m.r(z + triangle_multiplication(z, pair_mask, sub(w, "tri_mul_in"), "incoming", mode))
    z = m.r(z + transition(z, sub(w, "transition_z"), mode))
    return z


def pairformer_block(z, s, pair_mask, mask, w: dict, tri_heads: int = 4, single_heads: int = 16,
                     mode: str = "fp32", final_pair_mask: bool = False, row_chunk: int | None = None):
    """The composite AF3-shaped Pairformer block, assembled from reference modules only.

    Pair track in ``PairformerBlock.forward`` order (model/modules/apo_module.py:145-172:
    tri-mult out, tri-mult in, tri-att start, tri-att end, transition) and the single
    track of ``ConfidencePairSingleBlock.forward`` (model/modules/confidence_head.py:152-175:
    bias = Linear(LN(z)) moved to (B,H,L,L); s += SelfAttentionPairBias(s, None, bias, mask);
    s += Transition(s)).  All residual adds are the in-place eval adds of
    model/primitives/utils.py:30-50.
    """
    m = _Mode(mode)
    z = m.r(z.float())
    s = m.r(s.float())
    z = m.r(z + triangle_multiplication(z, pair_mask, sub(w, "tri_mul_out"), "outgoing", mode))
    z = m.r(z + triangle_multiplication(z, pair_mask, sub(w, "tri_mul_in"), "incoming", mode))
    z = m.r(z + triangle_attention(z, pair_mask, sub(w, "tri_att_start"), tri_heads, True, mode,
                                     row_chunk=row_chunk))
    z = m.r(z + triangle_attention(z, pair_mask, sub(w, "tri_att_end"), tri_heads, False, mode,
                                     row_chunk=row_chunk))
    z = m.r(z + transition(z, sub(w, "transition_z"), mode))
    if final_pair_mask:
        z = z * pair_mask[..., None].to(z.dtype)
    zn = layer_norm(z, w["layernorm_z.weight"], w["layernorm_z.bias"], 1e-5, mode)
    pair_bias = m.linear(zn, w["linear_pair_bias.weight"]).movedim(-1, -3)
    s = m.r(s + self_attention_pair_bias(s, None, pair_bias, mask, sub(w, "attention"), single_heads, mode))
    s = m.r(s + transition(s, sub(w, "transition"), mode))
    return z, s
