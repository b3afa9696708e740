"""Functional entry points: torch tensors in, torch tensors out, CUDA kernels in between.

Each function checks shapes, pads the token dimension to the kernels' granularity,
takes a workspace from a per-device cache, and calls the C ABI on the current
stream.  There is no CPU path and no PyTorch fallback: inputs must be CUDA tensors
and the extension must be built.
"""
from __future__ import annotations


import torch

from . import _lib as L

_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = None
        _workspaces.pop(key, None)
        ws = torch.empty(int(nbytes * 1.05) + 4096, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def release_workspaces() -> None:
    _workspaces.clear()


def _rows(t: torch.Tensor, c: int, dtype=None):
    """(tensor, rows, row stride) of `t` (..., c) seen as rows of c contiguous elements at a constant stride: a column
    slice of a wider row-major table is passed as it lies, anything else is made contiguous first."""
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    rows = t.numel() // c
    if t.stride(-1) == 1 and t.dim() >= 2:
        ld = t.stride(-2) if t.shape[-2] > 1 else c
        ok, span = ld >= c, ld * t.shape[-2]
        for d in range(t.dim() - 3, -1, -1):
            if t.shape[d] != 1 and t.stride(d) != span:
                ok = False
            span *= t.shape[d]
        if ok and (t.data_ptr() % 16 == 0) and ld % 8 == 0:
            return t, rows, ld
    t = t.reshape(-1, c).contiguous()
    return t, rows, c


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("kfold_b200 kernels require CUDA tensors (there is no CPU path)")


def _pad_pair(x: torch.Tensor, mask: torch.Tensor, mult: int = 8):
    n = x.shape[-2]
    npad = (n + mult - 1) // mult * mult
    if npad == n:
        return x, mask, n
    xp = x.new_zeros(x.shape[0], npad, npad, x.shape[-1])
    xp[:, :n, :n] = x
    mp = mask.new_zeros(mask.shape[0], npad, npad)
    mp[:, :n, :n] = mask
    return xp, mp, n


def layer_norm(x: torch.Tensor, weight, bias, eps: float = 1e-5, out_dtype=None) -> torch.Tensor:
    """LayerNorm over the last dim (model/primitives/normalization.py:61-91)."""
    _require_cuda(x)
    c = x.shape[-1]
    x2 = x.reshape(-1, c)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty(x2.shape, dtype=out_dtype or x.dtype, device=x.device)
    w = None if weight is None else weight.detach().float().contiguous()
    b = None if bias is None else bias.detach().float().contiguous()
    with L.on_device(x.device):
        L.check(L.lib().kfb_layernorm(L.ptr(x2), L.ptr(out), L.ptr(w), L.ptr(b), x2.shape[0], c, x2.stride(0), c, eps,
                                      L.dtype_code(x2.dtype), L.dtype_code(out.dtype), L.stream_ptr()))
    return out.view(*x.shape[:-1], c)


def triangle_multiplication(x: torch.Tensor, mask: torch.Tensor, packed: dict, direction: str, eps: float = 1e-5,
                            residual: bool = False) -> torch.Tensor:
    """Triangle multiplicative update (model/primitives/triangle_multiplication.py:179-229, :263-313).

    x (B,N,N,C) bf16 or fp32; mask (B,N,N).  Returns the update, or x + update when
    ``residual`` is set (the add is fused into the last kernel).
    """
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f"unknown direction {direction!r}")
    _require_cuda(x, mask)
    if x.dim() != 4 or x.shape[1] != x.shape[2] or mask.shape != x.shape[:-1]:
        raise ValueError(f"triangle_multiplication: x {tuple(x.shape)} / mask {tuple(mask.shape)}")
    c = x.shape[-1]
    if c != packed["c"]:
        raise ValueError(f"triangle_multiplication: channel mismatch {c} vs {packed['c']}")
    xp, mp, n = _pad_pair(x.contiguous(), mask.to(torch.bool).contiguous())
    b, npad = xp.shape[0], xp.shape[1]
    mp8 = mp.view(torch.uint8)
    out = torch.empty_like(xp)
    lib = L.lib()
    precise = bool(packed.get("precise"))
    if precise and xp.dtype != torch.float32:
        raise ValueError("the fp32-accurate mode takes float32 tensors")
    with L.on_device(x.device):
        need = (lib.kfb_trimul_workspace_bytes_precise if precise else lib.kfb_trimul_workspace_bytes)(b, npad, c)
        ws = _workspace(x.device, need)
        L.check(lib.kfb_trimul_fwd(1 if direction == "incoming" else 0, L.ptr(xp), L.ptr(mp8), L.ptr(packed["ln_in_w"]),
                                   L.ptr(packed["ln_in_b"]), L.ptr(packed["w_in"]), L.ptr(packed["w_gout"]),
                                   L.ptr(packed["ln_out_w"]), L.ptr(packed["ln_out_b"]), L.ptr(packed["w_pout"]),
                                   L.ptr(out), L.ptr(xp) if residual else None, L.ptr(ws), ws.numel(), b, npad, c, eps,
                                   L.KFB_FP32_PRECISE if precise else L.dtype_code(xp.dtype), L.stream_ptr()))
    return out if npad == n else out[:, :n, :n].contiguous()


def triangle_attention(x: torch.Tensor, mask: torch.Tensor | None, packed: dict, starting: bool, eps: float = 1e-5,
                       residual: bool = False) -> torch.Tensor:
    """Triangle attention around the starting / ending node
    (model/primitives/triangle_attention.py:375-434).  x (B,N,N,C); mask (B,N,N) or None."""
    _require_cuda(x, mask)
    if x.dim() != 4 or x.shape[1] != x.shape[2]:
        raise ValueError(f"triangle_attention: x {tuple(x.shape)}")
    if mask is None:
        mask = torch.ones(x.shape[:-1], dtype=torch.bool, device=x.device)
    if mask.shape != x.shape[:-1]:
        raise ValueError(f"triangle_attention: mask {tuple(mask.shape)} vs x {tuple(x.shape)}")
    c, heads = x.shape[-1], packed["heads"]
    if c != packed["c"]:
        raise ValueError(f"triangle_attention: channel mismatch {c} vs {packed['c']}")
    xp, mp, n = _pad_pair(x.contiguous(), mask.to(torch.bool).contiguous())
    b, npad = xp.shape[0], xp.shape[1]
    out = torch.empty_like(xp)
    lib = L.lib()
    precise = bool(packed.get("precise"))
    if precise and xp.dtype != torch.float32:
        raise ValueError("the fp32-accurate mode takes float32 tensors")
    with L.on_device(x.device):
        need = (lib.kfb_triatt_workspace_bytes_precise if precise else lib.kfb_triatt_workspace_bytes)(b, npad, c, heads)
        ws = _workspace(x.device, need)
        L.check(lib.kfb_triatt_fwd(0 if starting else 1, L.ptr(xp), L.ptr(mp.view(torch.uint8)), L.ptr(packed["ln_w"]),
                                   L.ptr(packed["ln_b"]), L.ptr(packed["w_proj"]), L.ptr(packed["w_out"]), L.ptr(out),
                                   L.ptr(xp) if residual else None, L.ptr(ws), ws.numel(), b, npad, c, heads, eps,
                                   L.KFB_FP32_PRECISE if precise else L.dtype_code(xp.dtype), L.stream_ptr()))
    return out if npad == n else out[:, :n, :n].contiguous()


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """y = x w^T (+ bias) on the tensor-core GEMM.  x (..., k) bf16, w (n, k) bf16, bias fp32 (n,) or None."""
    _require_cuda(x, w)
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if x2.dtype != torch.bfloat16:
        x2 = x2.to(torch.bfloat16)
    x2 = x2.contiguous()
    n = w.shape[0]
    out = torch.empty(x2.shape[0], n, dtype=out_dtype, device=x.device)
    with L.on_device(x.device):
        L.check(L.lib().kfb_gemm_bf16(L.ptr(x2), L.ptr(w), L.ptr(out), L.ptr(bias), 1, x2.shape[0], n, k, k, k, n, 0, 0, 0,
                                      L.dtype_code(out_dtype), L.stream_ptr()))
    return out.view(*x.shape[:-1], n)


def linear_fp32(x: torch.Tensor, w6: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x w^T (+ bias) at float32 accuracy: x (..., k) float32, w6 (n, 6k) the bf16 triple split of w
    (packing.split3_weights), bias float32 (n,) or None; float32 result."""
    _require_cuda(x, w6)
    k = x.shape[-1]
    if w6.shape[1] != 6 * k:
        raise ValueError(f"linear_fp32: weight {tuple(w6.shape)} is not the triple split of a (n, {k}) matrix")
    x2 = x.reshape(-1, k).float().contiguous()
    n = w6.shape[0]
    out = torch.empty(x2.shape[0], n, dtype=torch.float32, device=x.device)
    lib = L.lib()
    with L.on_device(x.device):
        ws = _workspace(x.device, lib.kfb_linear_fp32_workspace_bytes(x2.shape[0], k))
        L.check(lib.kfb_linear_fp32(L.ptr(x2), L.ptr(w6), L.ptr(bias), L.ptr(out), L.ptr(ws), ws.numel(), x2.shape[0], n, k,
                                    L.stream_ptr()))
    return out.view(*x.shape[:-1], n)


def ln_linear_fp32(x: torch.Tensor, ln_w: torch.Tensor | None, ln_b: torch.Tensor | None, w6: torch.Tensor,
                   bias: torch.Tensor | None = None, resid: torch.Tensor | None = None, eps: float = 1e-5) -> torch.Tensor:
    """resid + LayerNorm(x) w^T (+ bias) at float32 accuracy (model/layers/folding/diffusion.py:568): x (..., k) float32,
    w6 (n, 6k) the bf16 triple split of w; float32 result."""
    _require_cuda(x, w6)
    k = x.shape[-1]
    if w6.shape[1] != 6 * k:
        raise ValueError(f"ln_linear_fp32: weight {tuple(w6.shape)} is not the triple split of a (n, {k}) matrix")
    x2 = x.reshape(-1, k).float().contiguous()
    n = w6.shape[0]
    out = torch.empty(x2.shape[0], n, dtype=torch.float32, device=x.device)
    res = None if resid is None else resid.expand(*x.shape[:-1], n).reshape(-1, n).float().contiguous()
    f32 = lambda t: None if t is None else t.detach().float().contiguous()
    lw, lb = f32(ln_w), f32(ln_b)
    lib = L.lib()
    with L.on_device(x.device):
        ws = _workspace(x.device, lib.kfb_linear_fp32_workspace_bytes(x2.shape[0], k))
        L.check(lib.kfb_ln_linear_fp32(L.ptr(x2), L.ptr(lw), L.ptr(lb), L.ptr(w6), L.ptr(bias), L.ptr(res), L.ptr(out), L.ptr(ws),
                                       ws.numel(), x2.shape[0], n, k, eps, 1, L.stream_ptr()))
    return out.view(*x.shape[:-1], n)


def adaln(a: torch.Tensor, gate_shift: torch.Tensor, samples: int, eps: float = 1e-5) -> torch.Tensor:
    """sigmoid(g) * LayerNorm(a) + v  (model/primitives/normalization.py:117-125).
    a (groups * samples, L, c) flattened as rows; gate_shift (groups, L, 2c) bf16 = [g | v]."""
    _require_cuda(a, gate_shift)
    c, l = a.shape[-1], a.shape[-2]
    a2 = a.reshape(-1, c).contiguous()
    precise = gate_shift.dtype == torch.float32     # float32 gate / shift rows: everything stays float32
    if precise:
        a2 = a2.float()
    out = torch.empty(a2.shape, dtype=torch.float32 if precise else torch.bfloat16, device=a.device)
    gs, _, gs_ld = _rows(gate_shift, 2 * c)
    with L.on_device(a.device):
        L.check(L.lib().kfb_adaln_fwd(L.ptr(a2), L.ptr(gs), gs_ld, L.ptr(out), a2.shape[0], c, samples, l, eps,
                                      L.KFB_FP32_PRECISE if precise else L.dtype_code(a2.dtype), L.stream_ptr()))
    return out.view(a.shape)


def conditioned_transition(x_normed: torch.Tensor, packed: dict, out_gate: torch.Tensor, samples: int,
                           resid: torch.Tensor | None = None, out_dtype=None) -> torch.Tensor:
    """sigmoid(gate) * Linear_out(SwiGLU(x)) (+ resid)  (model/layers/folding/diffusion_transformer.py:73-81).
    x_normed (rows, L, c) bf16 AdaLN output; out_gate (rows / samples, L, c) bf16 logits."""
    _require_cuda(x_normed, out_gate)
    c, hidden, l = packed["c"], packed["hidden"], x_normed.shape[-2]
    x2 = x_normed.reshape(-1, c).contiguous()
    rows = x2.shape[0]
    precise = bool(packed.get("precise"))
    want = out_dtype or (resid.dtype if resid is not None else x_normed.dtype)
    out = torch.empty(rows, c, dtype=torch.float32 if precise else want, device=x2.device)
    r2 = None if resid is None else resid.reshape(-1, c).contiguous()
    g2, _, g_ld = _rows(out_gate, c, torch.float32 if precise else None)
    if precise:
        x2 = x2.float()
        r2 = None if r2 is None else r2.float()
    lib = L.lib()
    with L.on_device(x2.device):
        need = (lib.kfb_cond_transition_workspace_bytes_precise(rows, c, hidden) if precise
                else lib.kfb_cond_transition_workspace_bytes(rows, hidden))
        ws = _workspace(x2.device, need)
        L.check(lib.kfb_cond_transition_fwd(L.ptr(x2), L.ptr(packed["w_swiglu"]), L.ptr(packed["w_out"]), L.ptr(g2), g_ld, L.ptr(out),
                                            L.ptr(r2), L.ptr(ws), ws.numel(), rows, c, hidden, samples, l,
                                            L.KFB_FP32_PRECISE if precise else L.dtype_code(out.dtype), L.stream_ptr()))
    return out.view(x_normed.shape).to(want)


def attention_pair_bias(x: torch.Tensor, pair_bias: torch.Tensor, mask: torch.Tensor, packed: dict,
                        out_dtype=None, out_gate: torch.Tensor | None = None, gate_share: int = 1,
                        resid: torch.Tensor | None = None) -> torch.Tensor:
    """Gated self-attention with pair bias on already-normalised inputs
    (model/primitives/attention.py:28-94 with x_q is x_k).

    x (*, L, c); pair_bias broadcastable to (*, H, L, L) -- entries that share a bias (the
    diffusion samples) must be adjacent in the flattened batch; mask broadcastable to (*, L).
    ``out_gate``: bf16 logits (batch / gate_share, L, c), the result is multiplied by their sigmoid (the
    AdaLN-Zero output gate); ``resid``: tensor like the result that is added (fused residual).
    """
    _require_cuda(x, pair_bias, mask)
    c, heads = x.shape[-1], packed["heads"]
    l = x.shape[-2]
    lead = x.shape[:-2]
    batch = 1
    for s in lead:
        batch *= s
    pb = pair_bias
    # leading dims of the bias that are 1 where x's are not -> shared bias
    pb_lead = pb.shape[:-3]
    pb_lead = (1,) * (len(lead) - len(pb_lead)) + tuple(pb_lead)
    nb = 1
    for s in pb_lead:
        nb *= s
    # sharing must be over trailing leading-dims so that sharers are adjacent
    k = len(lead)
    while k > 0 and pb_lead[k - 1] == 1:
        k -= 1
    if tuple(pb_lead[:k]) != tuple(lead[:k]):
        pb = pb.expand(*lead, heads, l, l)
        pb_lead, nb = tuple(lead), batch
    bias_div = batch // nb
    lp = (l + 7) // 8 * 8
    precise = bool(packed.get("precise"))
    act = torch.float32 if precise else torch.bfloat16     # dtype of the activations handed to the kernels
    xb = x.reshape(batch, l, c).to(act)
    pbb = pb.reshape(nb, heads, l, l).to(act)
    mb = mask.to(torch.bool).expand(*lead, l).reshape(batch, l)
    if lp != l:
        xb = torch.nn.functional.pad(xb, (0, 0, 0, lp - l))
        pbb = torch.nn.functional.pad(pbb, (0, lp - l, 0, lp - l))
        mb = torch.nn.functional.pad(mb, (0, lp - l))
    gate, gate_ld = None, 0
    if out_gate is not None:
        if lp != l:
            gate = torch.nn.functional.pad(out_gate.reshape(-1, l, c).to(act), (0, 0, 0, lp - l)).contiguous()
        else:
            gate, _, gate_ld = _rows(out_gate, c, act)
    res = None
    if resid is not None:
        res = resid.reshape(batch, l, c)
        if precise:
            res = res.float()
        if lp != l:
            res = torch.nn.functional.pad(res, (0, 0, 0, lp - l))
        res = res.contiguous()
    xb, pbb, mb = xb.contiguous(), pbb.contiguous(), mb.contiguous()
    want = out_dtype or (resid.dtype if resid is not None else x.dtype)
    out = torch.empty(batch, lp, c, dtype=torch.float32 if precise else want, device=x.device)
    lib = L.lib()
    with L.on_device(x.device):
        need = lib.kfb_apb_workspace_bytes_precise(batch, lp, c) if precise else lib.kfb_apb_workspace_bytes(batch, lp, c, heads)
        ws = _workspace(x.device, need)
        L.check(lib.kfb_apb_fwd(L.ptr(xb), L.ptr(pbb), L.ptr(mb.view(torch.uint8)), L.ptr(packed["w_proj"]),
                                L.ptr(packed["proj_bias"]), L.ptr(packed["w_out"]), L.ptr(packed["out_bias"]), L.ptr(gate),
                                gate_share, gate_ld, L.ptr(out), L.ptr(res), L.ptr(ws), ws.numel(), batch, lp, c, heads, bias_div,
                                L.KFB_FP32_PRECISE if precise else L.dtype_code(out.dtype), L.stream_ptr()))
    return out[:, :l].reshape(*lead, l, c).to(want)


def window_bias(z: torch.Tensor, ln_w: torch.Tensor | None, ln_b: torch.Tensor | None, w: torch.Tensor,
                eps: float = 1e-5, normalise: bool = True) -> torch.Tensor:
    """Pair bias of the atom windows for all blocks of a local transformer at once
    (model/layers/folding/diffusion_transformer.py:496 and :590-591 with the blocks' weights stacked).
    z (..., Lq, Lk, c_z) bf16 or float32; w (heads_total, c_z) of the same dtype -> (heads_total, ..., Lq, Lk).
    ``normalise=False`` skips the LayerNorm (z already normalised): projection only."""
    _require_cuda(z, w)
    c = z.shape[-1]
    if z.dtype not in (torch.bfloat16, torch.float32) or w.dtype != z.dtype:
        raise TypeError("window_bias: z and w must both be bfloat16 or both float32")
    z2 = z.reshape(-1, c).contiguous()
    nh = w.shape[0]
    out = torch.empty((nh,) + tuple(z.shape[:-1]), dtype=z.dtype, device=z.device)
    with L.on_device(z.device):
        L.check(L.lib().kfb_window_bias_fwd(L.ptr(z2), L.ptr(ln_w), L.ptr(ln_b), L.ptr(w.contiguous()), L.ptr(out), z2.shape[0], c,
                                            nh, eps, 1 if normalise else 0, L.dtype_code(z.dtype), L.stream_ptr()))
    return out


def attention_pair_bias_cross(x_q: torch.Tensor, x_k: torch.Tensor, pair_bias: torch.Tensor, mask: torch.Tensor, packed: dict,
                              bias_div: int = 1, bias_mod: int = 0, bias_head_major: bool = False, out_dtype=None,
                              out_gate: torch.Tensor | None = None, resid: torch.Tensor | None = None) -> torch.Tensor:
    """Gated cross attention with pair bias on already-normalised inputs (model/primitives/attention.py:28-94 with
    x_q and x_k different tensors, as CrossAttentionPairBias.forward calls it on the atom windows).

    Flattened form: x_q (batch, Lq, c); x_k (batch, Lk, c); mask (batch, Lk); Lq, Lk multiples of 8;
    pair_bias (bias batches, H, Lq, Lk), or (H, bias batches, Lq, Lk) with ``bias_head_major``.  Batch entry b uses
    bias batch b // bias_div, or with ``bias_mod`` > 0 (batch ordered (group, sample, window), bias_mod windows,
    bias_div = samples * windows) (b // bias_div) * bias_mod + b % bias_mod.
    ``out_gate``: logits (gate_rows, c); query row r is multiplied by sigmoid(out_gate[r % gate_rows]).
    ``resid``: (batch, Lq, c), added.  With a float32 packing every tensor is float32."""
    _require_cuda(x_q, x_k, pair_bias, mask)
    batch, lq, c = x_q.shape
    lk = x_k.shape[1]
    heads = packed["heads"]
    precise = bool(packed.get("precise"))
    act = torch.float32 if precise else torch.bfloat16
    if x_k.shape[0] != batch or x_k.shape[2] != c or tuple(mask.shape) != (batch, lk):
        raise ValueError(f"attention_pair_bias_cross: x_q {tuple(x_q.shape)}, x_k {tuple(x_k.shape)}, mask {tuple(mask.shape)}")
    if lq % 8 or lk % 8:
        raise ValueError("attention_pair_bias_cross: Lq and Lk must be multiples of 8")
    nbb = pair_bias.shape[1] if bias_head_major else pair_bias.shape[0]
    want_nbb = (batch + bias_div - 1) // bias_div * (bias_mod if bias_mod > 0 else 1)
    exp_shape = (heads, nbb, lq, lk) if bias_head_major else (nbb, heads, lq, lk)
    if tuple(pair_bias.shape) != exp_shape or nbb < want_nbb:
        raise ValueError(f"attention_pair_bias_cross: pair_bias {tuple(pair_bias.shape)}, expected {exp_shape} with at least "
                         f"{want_nbb} bias batches")
    xq, xk = x_q.to(act).contiguous(), x_k.to(act).contiguous()
    pb = pair_bias.to(act).contiguous()
    mb = mask.to(torch.bool).contiguous().view(torch.uint8)
    gate, gate_rows, gate_ld = None, 0, 0
    if out_gate is not None:
        gate, gate_rows, gate_ld = _rows(out_gate, c, act)
    res = None
    if resid is not None:
        res = resid.reshape(batch, lq, c)
        res = (res.float() if precise else res).contiguous()
    want = out_dtype or (resid.dtype if resid is not None else x_q.dtype)
    out = torch.empty(batch, lq, c, dtype=torch.float32 if precise else want, device=x_q.device)
    if res is not None and res.dtype != out.dtype:
        res = res.to(out.dtype)
    lib = L.lib()
    with L.on_device(x_q.device):
        need = (lib.kfb_apb_cross_workspace_bytes_precise(batch, lq, lk, c) if precise
                else lib.kfb_apb_cross_workspace_bytes(batch, lq, lk, c, heads))
        ws = _workspace(x_q.device, need)
        L.check(lib.kfb_apb_cross_fwd(L.ptr(xq), L.ptr(xk), L.ptr(pb), L.ptr(mb), L.ptr(packed["w_q"]), L.ptr(packed["q_bias"]),
                                      L.ptr(packed["w_kv"]), L.ptr(packed["w_out"]), L.ptr(packed["out_bias"]), L.ptr(gate),
                                      gate_rows, gate_ld, L.ptr(out), L.ptr(res), L.ptr(ws), ws.numel(), batch, lq, lk, c, heads,
                                      bias_div, bias_mod, nbb if bias_head_major else 0,
                                      L.KFB_FP32_PRECISE if precise else L.dtype_code(out.dtype), L.stream_ptr()))
    return out.to(want)


def attention_pair_bias_window(x_q: torch.Tensor, x_k: torch.Tensor, pair_bias: torch.Tensor, mask: torch.Tensor, packed: dict,
                               bias_share: int = 1, bias_head_major: bool = False, out_dtype=None,
                               out_gate: torch.Tensor | None = None, resid: torch.Tensor | None = None) -> torch.Tensor:
    """The windowed cross attention of the atom transformers on UN-windowed atoms (bf16 compute, head dim <= 32): query
    atom q attends atoms 32 (q // 32) - 48 ... + 79 (model/layers/folding/utils.py:97-188); the kernel walks the windows.

    x_q, x_k (batch, L, c), L a multiple of 32; mask (batch // mask_share, L) atom validity; pair_bias one (32, 128) bias
    per window and head: (groups * L/32, H, 32, 128) or head-major (H, n, 32, 128); ``bias_share`` consecutive batch
    entries (samples) use the same biases.  out_gate / resid as in attention_pair_bias_cross."""
    _require_cuda(x_q, x_k, pair_bias, mask)
    batch, l, c = x_q.shape
    heads = packed["heads"]
    if packed.get("precise"):
        raise ValueError("attention_pair_bias_window: bfloat16 compute only (the float32 path gathers the windows)")
    if tuple(x_k.shape) != (batch, l, c) or l % 32 or mask.shape[-1] != l or batch % mask.shape[0] or batch % bias_share:
        raise ValueError(f"attention_pair_bias_window: x_q {tuple(x_q.shape)}, x_k {tuple(x_k.shape)}, mask {tuple(mask.shape)}")
    windows = l // 32
    nbb = pair_bias.shape[1] if bias_head_major else pair_bias.shape[0]
    exp_shape = (heads, nbb, 32, 128) if bias_head_major else (nbb, heads, 32, 128)
    if tuple(pair_bias.shape) != exp_shape or nbb < batch // bias_share * windows:
        raise ValueError(f"attention_pair_bias_window: pair_bias {tuple(pair_bias.shape)}, expected {exp_shape} with at least "
                         f"{batch // bias_share * windows} window biases")
    bf = torch.bfloat16
    xq, xk, pb = x_q.to(bf).contiguous(), x_k.to(bf).contiguous(), pair_bias.to(bf).contiguous()
    mb = mask.to(torch.bool).contiguous().view(torch.uint8)
    gate, gate_rows, gate_ld = None, 0, 0
    if out_gate is not None:
        gate, gate_rows, gate_ld = _rows(out_gate, c, bf)
    want = out_dtype or (resid.dtype if resid is not None else x_q.dtype)
    out = torch.empty(batch, l, c, dtype=want, device=x_q.device)
    res = None if resid is None else resid.reshape(batch, l, c).to(want).contiguous()
    lib = L.lib()
    with L.on_device(x_q.device):
        ws = _workspace(x_q.device, lib.kfb_apb_window_workspace_bytes(batch, l, c, heads))
        L.check(lib.kfb_apb_window_fwd(L.ptr(xq), L.ptr(xk), L.ptr(pb), L.ptr(mb), L.ptr(packed["w_q"]), L.ptr(packed["q_bias"]),
                                       L.ptr(packed["w_kv"]), L.ptr(packed["w_out"]), L.ptr(packed["out_bias"]), L.ptr(gate),
                                       gate_rows, gate_ld, L.ptr(out), L.ptr(res), L.ptr(ws), ws.numel(), batch, l, c, heads, bias_share,
                                       batch // mask.shape[0], nbb if bias_head_major else 0, L.dtype_code(out.dtype),
                                       L.stream_ptr()))
    return out


def attention_pair_bias_cross_bcast(x_q: torch.Tensor, x_k: torch.Tensor, pair_bias: torch.Tensor, mask: torch.Tensor,
                                    packed: dict, out_dtype=None, out_gate: torch.Tensor | None = None,
                                    resid: torch.Tensor | None = None) -> torch.Tensor:
    """The reference's calling convention (model/primitives/attention.py:28-60): x_q (*, Lq, c), x_k (*, Lk, c),
    pair_bias broadcastable to (*, H, Lq, Lk), mask broadcastable to (*, Lk).  A bias whose missing or size-1 leading
    dimensions form one block (the sample dimension of the sampler: bias (B, 1, W, H, Lq, Lk) against x (B, S, W, ...))
    is shared without being expanded; any other broadcast pattern is expanded.  ``out_gate``: logits broadcastable to
    x_q's shape; the result is multiplied by their sigmoid.  ``resid``: tensor like x_q that is added."""
    lead = tuple(x_q.shape[:-2])
    lq, c = x_q.shape[-2:]
    lk = x_k.shape[-2]
    heads = packed["heads"]
    batch = 1
    for d in lead:
        batch *= d
    pl = tuple(pair_bias.shape[:-3])
    pl = (1,) * (len(lead) - len(pl)) + pl
    # split the leading dims as (group..., shared..., window...): bias has the group and window dims, 1 in the shared ones
    i = 0
    while i < len(lead) and pl[i] == lead[i]:
        i += 1
    j = i
    while j < len(lead) and pl[j] == 1:
        j += 1
    if all(pl[k] == lead[k] for k in range(j, len(lead))):
        shared = 1
        for d in lead[i:j]:
            shared *= d
        windows = 1
        for d in lead[j:]:
            windows *= d
        pb = pair_bias.reshape(-1, heads, lq, lk)
        bias_div, bias_mod = shared * windows, (windows if shared > 1 and windows > 1 else 0)
        if bias_mod == 0:
            bias_div = shared if windows == 1 else 1
    else:
        pb = pair_bias.expand(*lead, heads, lq, lk).reshape(batch, heads, lq, lk)
        bias_div, bias_mod = 1, 0
    lqp, lkp = (lq + 7) // 8 * 8, (lk + 7) // 8 * 8
    xq = x_q.reshape(batch, lq, c)
    xk = x_k.expand(*lead, lk, c).reshape(batch, lk, c)
    mb = mask.to(torch.bool).expand(*lead, lk).reshape(batch, lk)
    gate = None if out_gate is None else out_gate.expand(*lead, lq, c).reshape(batch, lq, c)
    res = None if resid is None else resid.reshape(batch, lq, c)
    if lqp != lq or lkp != lk:
        pad = torch.nn.functional.pad
        xq, xk = pad(xq, (0, 0, 0, lqp - lq)), pad(xk, (0, 0, 0, lkp - lk))
        pb, mb = pad(pb, (0, lkp - lk, 0, lqp - lq)), pad(mb, (0, lkp - lk))
        gate = None if gate is None else pad(gate, (0, 0, 0, lqp - lq))
        res = None if res is None else pad(res, (0, 0, 0, lqp - lq))
    out = attention_pair_bias_cross(xq, xk, pb, mb, packed, bias_div=bias_div, bias_mod=bias_mod, out_dtype=out_dtype or x_q.dtype,
                                    out_gate=gate, resid=res)
    return out[:, :lq].reshape(*lead, lq, c)


def transition(x: torch.Tensor, packed: dict, eps: float = 1e-5, residual: bool = False) -> torch.Tensor:
    """Transition layer (model/layers/folding/transition.py:48-68).  x (..., C)."""
    _require_cuda(x)
    c, hidden = packed["c"], packed["hidden"]
    if x.shape[-1] != c:
        raise ValueError(f"transition: channel mismatch {x.shape[-1]} vs {c}")
    x2 = x.reshape(-1, c).contiguous()
    rows = x2.shape[0]
    out = torch.empty_like(x2)
    lib = L.lib()
    precise = bool(packed.get("precise"))
    if precise and x2.dtype != torch.float32:
        raise ValueError("the fp32-accurate mode takes float32 tensors")
    with L.on_device(x.device):
        need = (lib.kfb_transition_workspace_bytes_precise if precise else lib.kfb_transition_workspace_bytes)(rows, c, hidden)
        ws = _workspace(x.device, need)
        L.check(lib.kfb_transition_fwd(L.ptr(x2), L.ptr(packed["ln_w"]), L.ptr(packed["ln_b"]), L.ptr(packed["w_swiglu"]),
                                       L.ptr(packed["w_out"]), L.ptr(out), L.ptr(x2) if residual else None, L.ptr(ws),
                                       ws.numel(), rows, c, hidden, eps,
                                       L.KFB_FP32_PRECISE if precise else L.dtype_code(x2.dtype), L.stream_ptr()))
    return out.view(x.shape)


def pair_bias(z: torch.Tensor, ln_w: torch.Tensor, ln_b: torch.Tensor, w: torch.Tensor, eps: float = 1e-5,
              transposed: bool = False) -> torch.Tensor:
    """bias = Linear(LayerNorm(z)) moved to (B, H, N, N), bf16
    (model/modules/confidence_head.py:162-163; model/layers/folding/diffusion.py:411-416).
    z (B,N,N,C); w (H,C) already on the device in bf16; N must be a multiple of 8.
    ``transposed`` swaps the last two dims of the result."""
    _require_cuda(z, w)
    b, n, _, c = z.shape
    if n % 8 != 0:
        raise ValueError("pair_bias: N must be a multiple of 8")
    heads = w.shape[0]
    precise = w.shape[1] == 6 * c          # the weight as a bf16 triple split (packing.split3_weights)
    if precise and z.dtype != torch.float32:
        raise ValueError("the fp32-accurate mode takes float32 tensors")
    out = torch.empty(b, heads, n, n, dtype=torch.float32 if precise else torch.bfloat16, device=z.device)
    zc = z.contiguous()
    lib = L.lib()
    with L.on_device(z.device):
        need = (lib.kfb_pair_bias_workspace_bytes_precise if precise else lib.kfb_pair_bias_workspace_bytes)(b, n, c)
        ws = _workspace(z.device, need)
        L.check(lib.kfb_pair_bias_fwd(L.ptr(zc), L.ptr(ln_w), L.ptr(ln_b), L.ptr(w), L.ptr(out), L.ptr(ws), ws.numel(), b, n,
                                      c, heads, 1 if transposed else 0, eps,
                                      L.KFB_FP32_PRECISE if precise else L.dtype_code(zc.dtype), L.stream_ptr()))
    return out


def pair_bias_rows(z_rows: torch.Tensor, ln_w: torch.Tensor, ln_b: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """pair_bias on a row shard: z_rows (rows, N, C) -> (H, rows, N) bf16."""
    _require_cuda(z_rows, w)
    rows, n, c = z_rows.shape
    heads = w.shape[0]
    out = torch.empty(heads, rows, n, dtype=torch.bfloat16, device=z_rows.device)
    zc = z_rows.contiguous()
    lib = L.lib()
    with L.on_device(zc.device):
        ws = _workspace(zc.device, rows * n * c * 2 + 256)
        L.check(lib.kfb_pair_bias_rows_fwd(L.ptr(zc), L.ptr(ln_w), L.ptr(ln_b), L.ptr(w), L.ptr(out), L.ptr(ws), ws.numel(), rows,
                                           n, c, heads, eps, L.dtype_code(zc.dtype), L.stream_ptr()))
    return out


def _index_sharing(lead: tuple, index_lead: tuple):
    """index_div such that batch entry b of a tensor with leading dims `lead` uses index row b // index_div, for an
    index tensor whose leading dims equal `lead` up to trailing 1s; None otherwise."""
    il = (1,) * (len(lead) - len(index_lead)) + tuple(index_lead)
    k = len(lead)
    div = 1
    while k > 0 and il[k - 1] == 1:
        div *= lead[k - 1]
        k -= 1
    return div if tuple(il[:k]) == tuple(lead[:k]) else None


def broadcast_tokens_to_atoms(x: torch.Tensor, token_index: torch.Tensor, add: torch.Tensor | None = None) -> torch.Tensor:
    """Token features gathered to their atoms (model/layers/folding/utils.py:25-51): x (*, Ntoken[, D]) bf16 or
    float32, token_index (*, Natom) int64 (leading dims may be 1 where x's are not) -> (*, Natom[, D]).
    ``add``: a tensor like the result that is added in the same pass (the decoder's skip connection,
    model/layers/folding/atom_transformer.py:468-470); the result then has the promoted dtype."""
    if x.ndim == token_index.ndim:
        if add is not None:
            raise ValueError("broadcast_tokens_to_atoms: `add` needs feature vectors")
        return broadcast_tokens_to_atoms(x.unsqueeze(-1), token_index).squeeze(-1)
    _require_cuda(x, token_index)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("broadcast_tokens_to_atoms: bfloat16 or float32 features")
    lead, n_token, d = tuple(x.shape[:-2]), x.shape[-2], x.shape[-1]
    n_atom = token_index.shape[-1]
    div = _index_sharing(lead, tuple(token_index.shape[:-1]))
    idx = token_index.to(torch.int64)
    if div is None:
        idx, div = idx.expand(*lead, n_atom), 1
    idx = idx.reshape(-1, n_atom).contiguous()
    x2 = x.reshape(-1, n_token, d).contiguous()
    out_dtype = x.dtype if add is None else torch.promote_types(x.dtype, add.dtype)
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("broadcast_tokens_to_atoms: bfloat16 or float32 addend")
    add2 = None if add is None else add.expand(*lead, n_atom, d).reshape(-1, n_atom, d).to(out_dtype).contiguous()
    out = torch.empty(x2.shape[0], n_atom, d, dtype=out_dtype, device=x.device)
    with L.on_device(x.device):
        L.check(L.lib().kfb_tokens_to_atoms(L.ptr(x2), L.ptr(idx), L.ptr(add2), L.ptr(out), x2.shape[0], n_token, n_atom, d, div,
                                            L.dtype_code(x.dtype), L.dtype_code(out_dtype), L.stream_ptr()))
    return out.view(*lead, n_atom, d)


def aggregate_atoms_to_tokens(x: torch.Tensor, token_index: torch.Tensor, mask: torch.Tensor, num_tokens: int,
                              relu: bool = False) -> torch.Tensor:
    """Masked mean of the atom features of every token (model/layers/folding/utils.py:54-93): x (*, Natom, D) bf16 or
    float32, token_index and mask (*, Natom) -> (*, num_tokens, D); fp32 accumulation in atom order.  ``relu`` applies
    max(., 0) to the features as they are read (model/layers/folding/atom_transformer.py:384)."""
    _require_cuda(x, token_index, mask)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("aggregate_atoms_to_tokens: bfloat16 or float32 features")
    lead, n_atom, d = tuple(x.shape[:-2]), x.shape[-2], x.shape[-1]
    idx, mk = torch.broadcast_tensors(token_index.to(torch.int64), mask.to(torch.bool))
    div = _index_sharing(lead, tuple(idx.shape[:-1]))
    if div is None:
        idx, mk, div = idx.expand(*lead, n_atom), mk.expand(*lead, n_atom), 1
    idx = idx.reshape(-1, n_atom).contiguous()
    mk = mk.reshape(-1, n_atom).contiguous().view(torch.uint8)
    x2 = x.reshape(-1, n_atom, d).contiguous()
    out = torch.empty(x2.shape[0], num_tokens, d, dtype=x.dtype, device=x.device)
    lib = L.lib()
    with L.on_device(x.device):
        ws = _workspace(x.device, lib.kfb_atoms_to_tokens_workspace_bytes(x2.shape[0], num_tokens, div))
        L.check(lib.kfb_atoms_to_tokens(L.ptr(x2), L.ptr(idx), L.ptr(mk), L.ptr(out), L.ptr(ws), ws.numel(), x2.shape[0], n_atom,
                                        num_tokens, d, div,
                                            1 if relu else 0, L.dtype_code(x.dtype), L.stream_ptr()))
    return out.view(*lead, num_tokens, d)


def _shared_mask(mask: torch.Tensor | None, lead: tuple, l: int, share: int):
    """The atom mask as bytes with one row per `share` consecutive batch entries, or None."""
    if mask is None:
        return None
    m = mask.to(torch.bool)
    if _index_sharing(lead, tuple(m.shape[:-1])) != share:
        m = m.expand(*lead, l)
        if share != 1:
            raise ValueError("the atom mask must be shared like the atom features")
    return m.reshape(-1, l).contiguous().view(torch.uint8)


def coord_embed(q: torch.Tensor, r: torch.Tensor, w: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
    """q + Linear_fp32(r) (model/layers/folding/atom_transformer.py:362-367): q (*, [1 or N,] La, c) bf16 or float32,
    r (*, N, La, k) coordinates, w (c, k) -> float32 (*, N, La, c).  q's sample dimension may be 1 (shared).
    ``mask`` (atom validity, shared like q): the coordinates of padding atoms count as zero."""
    _require_cuda(q, r, w)
    c, kc = w.shape
    lead, l = tuple(r.shape[:-2]), r.shape[-2]
    if q.dtype not in (torch.bfloat16, torch.float32):
        q = q.float()
    if q.dim() == r.dim() - 1:
        q = q.unsqueeze(-3)
    share = _index_sharing(lead, tuple(q.shape[:-2]))
    if share is None:
        q, share = q.expand(*lead, l, c), 1
    q2 = q.reshape(-1, c).contiguous()
    r2 = r.reshape(-1, kc).float().contiguous()
    out = torch.empty(r2.shape[0], c, dtype=torch.float32, device=r.device)
    mk = _shared_mask(mask, lead, l, share)
    with L.on_device(r.device):
        L.check(L.lib().kfb_coord_embed(L.ptr(q2), L.ptr(r2), L.ptr(w.detach().float().contiguous()), L.ptr(mk), L.ptr(out), r2.shape[0], c, kc,
                                        share, l, L.dtype_code(q2.dtype), L.stream_ptr()))
    return out.view(*lead, l, c)


def ln_project(x: torch.Tensor, ln_w: torch.Tensor | None, ln_b: torch.Tensor | None, w: torch.Tensor,
               eps: float = 1e-5, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Linear_fp32(LayerNorm(x.float())) to a handful of outputs (model/layers/folding/atom_transformer.py:487-488):
    x (*, L, c) bf16 or float32, w (n_out <= 8, c) -> float32 (*, L, n_out).  ``mask`` (*, L), leading dims 1 where
    shared: rows of padding atoms give zeros."""
    _require_cuda(x, w)
    c, n_out = x.shape[-1], w.shape[0]
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    x2 = x.reshape(-1, c).contiguous()
    out = torch.empty(x2.shape[0], n_out, dtype=torch.float32, device=x.device)
    f32 = lambda t: None if t is None else t.detach().float().contiguous()
    lw, lb, ww = f32(ln_w), f32(ln_b), f32(w)
    mk, share, l = None, 1, 1
    if mask is not None:
        lead, l = tuple(x.shape[:-2]), x.shape[-2]
        share = _index_sharing(lead, tuple(mask.shape[:-1])) or 1
        mk = _shared_mask(mask, lead, l, share)
    with L.on_device(x.device):
        L.check(L.lib().kfb_ln_project(L.ptr(x2), L.ptr(lw), L.ptr(lb), L.ptr(ww), L.ptr(mk), L.ptr(out), x2.shape[0], c, n_out, eps,
                                       share, l, L.dtype_code(x2.dtype), L.stream_ptr()))
    return out.view(*x.shape[:-1], n_out)


def fourier_embed(t: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """cos(2 pi t w + b), float32 (model/layers/folding/embeddings.py:159-174): t (*,), w and b (dim,) -> (*, dim)."""
    _require_cuda(t, w, b)
    t2 = t.reshape(-1).float().contiguous()
    w2, b2 = w.reshape(-1).float().contiguous(), b.reshape(-1).float().contiguous()
    out = torch.empty(t2.shape[0], w2.shape[0], dtype=torch.float32, device=t.device)
    with L.on_device(t.device):
        L.check(L.lib().kfb_fourier_embed(L.ptr(t2), L.ptr(w2), L.ptr(b2), L.ptr(out), t2.shape[0], w2.shape[0], L.stream_ptr()))
    return out.view(*t.shape, w2.shape[0])


def broadcast_add(s: torch.Tensor, f: torch.Tensor) -> torch.Tensor:
    """s[:, None] + f[:, :, None], float32 (model/layers/folding/diffusion.py:146): s (B, L, c), f (B, N, c) -> (B, N, L, c)."""
    _require_cuda(s, f)
    b, l, c = s.shape
    n = f.shape[1]
    s2, f2 = s.float().contiguous(), f.float().contiguous()
    out = torch.empty(b, n, l, c, dtype=torch.float32, device=s.device)
    with L.on_device(s.device):
        L.check(L.lib().kfb_broadcast_add(L.ptr(s2), L.ptr(f2), L.ptr(out), b, n, l, c, L.stream_ptr()))
    return out


# ------------------------------------------------------------------------------------------------
# coordinate-space steps of the sampler loop (model/modules/ecsi.py:498-560)
# ------------------------------------------------------------------------------------------------
def _coord_sets(x: torch.Tensor, mask: torch.Tensor):
    """(n sets, l atoms, sets per mask row, mask bytes) of coordinates x (*, L, 3) with an atom mask (*, L) whose leading
    dims equal x's up to trailing 1s (the samples of a complex share their mask)."""
    if x.dtype != torch.float32 or x.shape[-1] != 3:
        raise ValueError(f"coordinates must be float32 (*, L, 3), got {x.dtype} {tuple(x.shape)}")
    lead, l = tuple(x.shape[:-2]), x.shape[-2]
    div = _index_sharing(lead, tuple(mask.shape[:-1]))
    m = mask.to(torch.bool)
    if div is None:
        m, div = m.expand(*lead, l), 1
    n = 1
    for d in lead:
        n *= d
    return n, l, div, m.reshape(-1, l).contiguous().view(torch.uint8)


def coords_augment(coords: list, normals: torch.Tensor, trans: torch.Tensor | None, mask: torch.Tensor) -> list:
    """x <- x R + trans on the valid atoms, 0 on padding (CenterRandomAugmentation with centering=False,
    utils/geometry/random_augment.py:463-513) for one or two coordinate tensors (*, L, 3) that share R and trans.
    normals (n, 4): the standard normals of the rotation quaternions; trans (*, 1, 3) or None.  Returns new tensors."""
    _require_cuda(*coords, normals, mask)
    if not 1 <= len(coords) <= 2:
        raise ValueError("coords_augment takes one or two coordinate tensors")
    n, l, div, mk = _coord_sets(coords[0], mask)
    out = [x.contiguous().clone() for x in coords]
    nr = normals.reshape(n, 4).float().contiguous()
    tr = None if trans is None else trans.reshape(n, 3).float().contiguous()
    with L.on_device(out[0].device):
        L.check(L.lib().kfb_coords_augment(L.ptr(out[0]), L.ptr(out[1]) if len(out) > 1 else None, L.ptr(nr), L.ptr(tr), L.ptr(mk),
                                           n, l, div, L.stream_ptr()))
    return out


def sampler_prepare(x_t: torch.Tensor, x_T: torch.Tensor, mask: torch.Tensor, c_in: float, sigma_T: float,
                    churn: tuple | None = None, noise: torch.Tensor | None = None):
    """Churn and input preconditioning (model/modules/ecsi.py:670-732, :624-633): with ``churn = (a, b, c)`` and ``noise``,
    x_hat = a x_t + b x_T + c noise (noise zero on padding), else x_hat = x_t; returns (x_hat, r6) with
    r6 = [c_in x_hat | x_T / sigma_T] (*, L, 6)."""
    _require_cuda(x_t, x_T, mask)
    n, l, div, mk = _coord_sets(x_t, mask)
    xt, xT = x_t.contiguous(), x_T.contiguous()
    x_hat = torch.empty_like(xt)
    r6 = torch.empty(*xt.shape[:-1], 6, dtype=torch.float32, device=xt.device)
    a, b, c = churn if churn is not None else (1.0, 0.0, 0.0)
    nz = None
    if churn is not None:
        if noise is None or noise.shape != x_t.shape:
            raise ValueError("Sigma-matched churn noise must match x_t shape.")
        nz = noise.float().contiguous()
    with L.on_device(xt.device):
        L.check(L.lib().kfb_sampler_prepare(L.ptr(xt), L.ptr(xT), L.ptr(nz), L.ptr(mk), a, b, c, c_in, 1.0 / sigma_T, L.ptr(x_hat),
                                            L.ptr(r6), n, l, div, L.stream_ptr()))
    return x_hat, r6


def sampler_update(x_noisy: torch.Tensor, r_update: torch.Tensor, x_T: torch.Tensor, mask: torch.Tensor, c_skip: float,
                   c_out: float, coef: tuple, noise: torch.Tensor | None = None, return_x0: bool = False):
    """Output preconditioning, rotation-only rigid alignment onto x_noisy, centring and the SI / ECSI update in one kernel
    (model/modules/ecsi.py:666-667, :535-550): x0 = c_skip x_noisy + c_out r_update aligned and centred;
    x_next = A x_noisy + B x0 + C x_T + D noise with ``coef = (A, B, C, D)``."""
    _require_cuda(x_noisy, r_update, x_T, mask)
    n, l, div, mk = _coord_sets(x_noisy, mask)
    xn, ru, xT = x_noisy.contiguous(), r_update.float().contiguous(), x_T.contiguous()
    A, B, C, D = coef
    nz = None
    if D != 0.0:
        if noise is None or noise.shape != x_noisy.shape:
            raise ValueError("the stochastic update needs noise of the coordinates' shape")
        nz = noise.float().contiguous()
    x_next = torch.empty_like(xn)
    x0 = torch.empty_like(xn) if return_x0 else None
    with L.on_device(xn.device):
        L.check(L.lib().kfb_sampler_update(L.ptr(xn), L.ptr(ru), L.ptr(xT), L.ptr(nz), L.ptr(mk), c_skip, c_out, A, B, C, D,
                                           L.ptr(x_next), L.ptr(x0), n, l, div, L.stream_ptr()))
    return (x_next, x0) if return_x0 else x_next


def rigid_align(coords: torch.Tensor, target: torch.Tensor, mask: torch.Tensor, rotation_only: bool = False) -> torch.Tensor:
    """custom_rigid_align with output_mask = mask (model/modules/ecsi.py:59-103): the weighted Kabsch fit of `coords`
    onto `target` over the masked atoms, applied to them; padding atoms give zeros."""
    _require_cuda(coords, target, mask)
    n, l, div, mk = _coord_sets(coords, mask)
    c, t = coords.float().contiguous(), target.float().contiguous()
    out = torch.empty_like(c)
    with L.on_device(c.device):
        L.check(L.lib().kfb_rigid_align(L.ptr(c), L.ptr(t), L.ptr(mk), 1 if rotation_only else 0, L.ptr(out), n, l, div, L.stream_ptr()))
    return out.to(coords.dtype)


def center_coords(coords: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """do_centering (utils/geometry/random_augment.py:90-130): subtract the mean position of the valid atoms, zero padding."""
    _require_cuda(coords, mask)
    n, l, div, mk = _coord_sets(coords, mask)
    c = coords.contiguous()
    out = torch.empty_like(c)
    with L.on_device(c.device):
        L.check(L.lib().kfb_center_coords(L.ptr(c), L.ptr(mk), L.ptr(out), n, l, div, L.stream_ptr()))
    return out


# ------------------------------------------------------------------------------------------------
# callers of the pair stacks in the trunk (model/model.py:477-534)
# ------------------------------------------------------------------------------------------------
def parcae_update(z: torch.Tensor, u: torch.Tensor, ln_w, ln_b, a: torch.Tensor, b_w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """a * z + Linear_b(LayerNorm(u)) (model/model.py:528): z, u (..., C) bf16 or float32; a float32 (C,); b_w bf16 (C, C)."""
    _require_cuda(z, u, a, b_w)
    c = z.shape[-1]
    z2, u2 = z.reshape(-1, c).contiguous(), u.reshape(-1, c).to(z.dtype).contiguous()
    out = torch.empty_like(z2)
    f32 = lambda t: None if t is None else t.detach().float().contiguous()
    lw, lb, af = f32(ln_w), f32(ln_b), f32(a)
    lib = L.lib()
    with L.on_device(z.device):
        ws = _workspace(z.device, lib.kfb_parcae_workspace_bytes(z2.shape[0], c))
        L.check(lib.kfb_parcae_fwd(L.ptr(z2), L.ptr(u2), L.ptr(lw), L.ptr(lb), L.ptr(af), L.ptr(b_w), L.ptr(out), L.ptr(ws), ws.numel(),
                                   z2.shape[0], c, eps, L.dtype_code(z2.dtype), L.stream_ptr()))
    return out.view(z.shape)


def lm_pair_features(x: torch.Tensor) -> torch.Tensor:
    """[xi * xj | xi - xj] for every token pair (model/model.py:128-131): x (B, L, 2 D) = [xi | xj] -> bf16 (B, L, L, 2 D)."""
    _require_cuda(x)
    b, n, d2 = x.shape
    xc = x.contiguous()
    out = torch.empty(b, n, n, d2, dtype=torch.bfloat16, device=x.device)
    with L.on_device(x.device):
        L.check(L.lib().kfb_lm_pair_features(L.ptr(xc), L.ptr(out), b, n, d2 // 2, L.dtype_code(xc.dtype), L.stream_ptr()))
    return out


def gelu(x: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """erf GELU, element-wise (torch.nn.GELU() of model/model.py:122)."""
    _require_cuda(x)
    xc = x.contiguous()
    out = torch.empty(xc.shape, dtype=out_dtype or x.dtype, device=x.device)
    with L.on_device(x.device):
        L.check(L.lib().kfb_gelu(L.ptr(xc), L.ptr(out), xc.numel(), L.dtype_code(xc.dtype), L.dtype_code(out.dtype), L.stream_ptr()))
    return out


def concat_layer_norm(z: torch.Tensor, rel: torch.Tensor, ln_w, ln_b, k_pad: int, eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm(cat([z, rel], -1)) in one pass (model/layers/folding/diffusion.py:84-90): float32 (..., k_pad), the columns past
    c_z + c_rel zero.  z and rel bf16 or float32, same leading shape."""
    _require_cuda(z, rel)
    if z.shape[:-1] != rel.shape[:-1]:
        raise ValueError(f"concat_layer_norm: leading shapes {tuple(z.shape[:-1])} and {tuple(rel.shape[:-1])} differ")
    c1, c2 = z.shape[-1], rel.shape[-1]
    fix = lambda t: (t if t.dtype in (torch.bfloat16, torch.float32) else t.float()).contiguous()
    zc, rc = fix(z), fix(rel)
    f32 = lambda t: None if t is None else t.detach().float().contiguous()
    lw, lb = f32(ln_w), f32(ln_b)
    rows = zc.numel() // c1
    out = torch.empty(*z.shape[:-1], k_pad, dtype=torch.float32, device=z.device)
    with L.on_device(z.device):
        L.check(L.lib().kfb_concat_layernorm(L.ptr(zc), L.dtype_code(zc.dtype), L.ptr(rc), L.dtype_code(rc.dtype), L.ptr(lw), L.ptr(lb),
                                             L.ptr(out), rows, c1, c2, k_pad, eps, L.stream_ptr()))
    return out


def relpos_concat_layer_norm(z: torch.Tensor, token, ln_w, ln_b, k_pad: int, r_max: int = 32, s_max: int = 2,
                             eps: float = 1e-5) -> torch.Tensor:
    """LayerNorm(cat([z, RelativePositionEncoding(token)], -1)) without the one-hot tensor
    (model/layers/folding/embeddings.py:58-130 + diffusion.py:84-90): `token` carries asym_id, residue_index, entity_id,
    token_index and sym_id, (B, L) integer tensors; z (B, L, L, c_z).  float32 (B, L, L, k_pad)."""
    _require_cuda(z)
    b, n, _, c1 = z.shape
    zc = (z if z.dtype in (torch.bfloat16, torch.float32) else z.float()).contiguous()
    ids = [getattr(token, k).to(device=z.device, dtype=torch.int64).reshape(b, n).contiguous()
           for k in ("asym_id", "residue_index", "entity_id", "token_index", "sym_id")]
    f32 = lambda t: None if t is None else t.detach().float().contiguous()
    lw, lb = f32(ln_w), f32(ln_b)
    out = torch.empty(b, n, n, k_pad, dtype=torch.float32, device=z.device)
    with L.on_device(z.device):
        L.check(L.lib().kfb_relpos_concat_layernorm(L.ptr(zc), L.dtype_code(zc.dtype), *[L.ptr(t) for t in ids], r_max, s_max,
                                                    L.ptr(lw), L.ptr(lb), L.ptr(out), b, n, c1, k_pad, eps, L.stream_ptr()))
    return out


def pair_outer_add(z: torch.Tensor, row_add: torch.Tensor, col_add: torch.Tensor) -> torch.Tensor:
    """z[b, i, j] + row_add[b, j] + col_add[b, i] (model/modules/confidence_head.py:347-351): z (B, L, L, C), the addends (B, L, C)."""
    _require_cuda(z, row_add, col_add)
    b, n, _, c = z.shape
    zc = z.contiguous()
    ra, ca = row_add.to(z.dtype).contiguous(), col_add.to(z.dtype).contiguous()
    out = torch.empty_like(zc)
    with L.on_device(z.device):
        L.check(L.lib().kfb_pair_outer_add(L.ptr(zc), L.ptr(ra), L.ptr(ca), L.ptr(out), b, n, c, L.dtype_code(zc.dtype), L.stream_ptr()))
    return out


def distogram_embed_add(z: torch.Tensor, x: torch.Tensor, boundaries: torch.Tensor, w_t: torch.Tensor) -> torch.Tensor:
    """z + Linear(one_hot(distance bin of |x_i - x_j|)) (model/modules/confidence_head.py:449-455): z (B, L, L, C), x (B, L, 3),
    boundaries (bins - 1,), w_t (bins, C) = the embedding weight transposed, in z's dtype."""
    _require_cuda(z, x, boundaries, w_t)
    b, n, _, c = z.shape
    zc = z.contiguous()
    xc, bd, wt = x.float().contiguous(), boundaries.float().contiguous(), w_t.to(z.dtype).contiguous()
    out = torch.empty_like(zc)
    with L.on_device(z.device):
        L.check(L.lib().kfb_distogram_embed_add(L.ptr(zc), L.ptr(xc), L.ptr(bd), bd.numel(), L.ptr(wt), L.ptr(out), b, n, c,
                                                L.dtype_code(zc.dtype), L.stream_ptr()))
    return out
