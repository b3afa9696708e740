"""Weight packing for the CUDA kernels (done once per module, cached by the caller).

The tcgen05 GEMM computes 128 x 256 output tiles.  For gated projections the
epilogue needs a value column and its gate column in the SAME tile, so the two
weight matrices are interleaved in blocks of 128 rows: tile t holds value rows
[128 t, 128 t + 128) followed by the gate rows of the same channels.
"""
from __future__ import annotations

import torch

GLU_HALF = 128  # value (or gate) columns per 256-wide GEMM tile


def interleave_glu(value_w: torch.Tensor, gate_w: torch.Tensor, half: int = GLU_HALF) -> torch.Tensor:
    """[n, k] value and gate weights -> [2n, k] with alternating blocks of `half` rows."""
    n, k = value_w.shape
    assert gate_w.shape == (n, k) and n % half == 0, (value_w.shape, gate_w.shape, half)
    v = value_w.reshape(n // half, half, k)
    g = gate_w.reshape(n // half, half, k)
    return torch.stack((v, g), dim=1).reshape(2 * n, k).contiguous()


def _dev(t: torch.Tensor, device, dtype) -> torch.Tensor:
    return t.detach().to(device=device, dtype=dtype).contiguous()


def pack_trimul(w: dict, device, dtype=torch.bfloat16) -> dict:
    """Weights of TriangleMultiplication{Outgoing,Incoming}: keys as in the reference state_dict
    (model/primitives/triangle_multiplication.py:171-177).  LayerNorm affine stays fp32."""
    return {
        "ln_in_w": _dev(w["layernorm_in.weight"], device, torch.float32),
        "ln_in_b": _dev(w["layernorm_in.bias"], device, torch.float32),
        "w_in": _dev(interleave_glu(w["linear_p_in.weight"], w["linear_g_in.weight"]), device, dtype),
        "w_gout": _dev(w["linear_g_out.weight"], device, dtype),
        "ln_out_w": _dev(w["layernorm_out.weight"], device, torch.float32),
        "ln_out_b": _dev(w["layernorm_out.bias"], device, torch.float32),
        "w_pout": _dev(w["linear_p_out.weight"], device, dtype),
        "c": int(w["linear_p_out.weight"].shape[0]),
    }
