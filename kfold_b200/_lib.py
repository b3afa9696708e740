"""ctypes binding of the C ABI in include/kfold_b200.h.

The shared library is built in-tree by ``python -m kfold_b200.build``.  There is no
fallback: if the library is missing, importing this module's ``lib()`` raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "_C", "libkfold_b200.so")

KFB_BF16, KFB_FP32, KFB_FP32_PRECISE = 0, 1, 2
_lib = None

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class KfbError(RuntimeError):
    pass


# name -> argtypes; every function returns int except where noted
_SIGNATURES = {
    "kfb_version": [],
    "kfb_device_status": [ctypes.POINTER(c_int)],
    "kfb_profile_enable": [c_int],
    "kfb_profile_report": [ctypes.c_char_p, ctypes.c_size_t],
    "kfb_layernorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_float, c_int, c_int, c_void_p],
    "kfb_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll,
                      c_ll, c_int, c_void_p],
    "kfb_trimul_fwd": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_triatt_fwd": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       ctypes.c_size_t, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_apb_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_ll, c_void_p, c_void_p,
                    c_void_p, ctypes.c_size_t, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_apb_cross_fwd": [c_void_p] * 10 + [c_ll, c_ll, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_void_p],
    "kfb_apb_window_fwd": [c_void_p] * 10 + [c_ll, c_ll, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_int, c_int, c_int, c_int, c_int,
                           c_int, c_int, c_int, c_void_p],
    "kfb_window_bias_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "kfb_tokens_to_atoms": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_atoms_to_tokens": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_void_p],
    "kfb_fourier_embed": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "kfb_broadcast_add": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_coord_embed": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_ln_project": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_float, c_int, c_int, c_int,
                       c_void_p],
    "kfb_ln_linear_fp32": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_ll,
                           c_int, c_int, c_float, c_int, c_void_p],
    "kfb_trimul_contract_cs": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_trimul_project": [c_void_p] * 9 + [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_trimul_contract": [c_void_p, c_void_p, c_int, c_ll, c_void_p, c_int, c_int, c_int, c_void_p],
    "kfb_layernorm_exchange": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_trimul_finish": [c_void_p, c_void_p, c_int, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_triatt_project": [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_triatt_finish": [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_pair_bias_rows_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_int, c_int,
                               c_int, c_int, c_float, c_int, c_void_p],
    "kfb_linear_fp32": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_ll, c_int, c_int, c_void_p],
    "kfb_adaln_fwd": [c_void_p, c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_cond_transition_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_ll,
                                c_int, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_transition_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t,
                           c_ll, c_int, c_int, c_float, c_int, c_void_p],
    "kfb_pair_bias_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_int, c_int, c_int,
                          c_int, c_int, c_float, c_int, c_void_p],
    "kfb_parcae_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_size_t, c_ll, c_int,
                       c_float, c_int, c_void_p],
    "kfb_lm_pair_features": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_gelu": [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
    "kfb_relpos_concat_layernorm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "kfb_concat_layernorm": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_float, c_void_p],
    "kfb_pair_outer_add": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_distogram_embed_add": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "kfb_coords_augment": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "kfb_sampler_prepare": [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float, c_float, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_void_p],
    "kfb_sampler_update": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float, c_float, c_float, c_float, c_float,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "kfb_rigid_align": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
    "kfb_center_coords": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "kfb_transition_fwd_static": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int,
                                  c_float, c_int, c_void_p],
}
_SIZE_FUNCS = {
    "kfb_triatt_workspace_bytes_precise": [c_int, c_int, c_int, c_int],
    "kfb_apb_workspace_bytes_precise": [c_int, c_int, c_int],
    "kfb_pair_bias_workspace_bytes_precise": [c_int, c_int, c_int],
    "kfb_trimul_workspace_bytes_precise": [c_int, c_int, c_int],
    "kfb_transition_workspace_bytes_precise": [c_ll, c_int, c_int],
    "kfb_cond_transition_workspace_bytes": [c_ll, c_int],
    "kfb_cond_transition_workspace_bytes_precise": [c_ll, c_int, c_int],
    "kfb_linear_fp32_workspace_bytes": [c_ll, c_int],
    "kfb_transition_static_max_bytes": [],
    "kfb_pair_bias_workspace_bytes": [c_int, c_int, c_int],
    "kfb_transition_workspace_bytes": [c_ll, c_int, c_int],
    "kfb_triatt_workspace_bytes": [c_int, c_int, c_int, c_int],
    "kfb_apb_workspace_bytes": [c_int, c_int, c_int, c_int],
    "kfb_atoms_to_tokens_workspace_bytes": [c_int, c_int, c_int],
    "kfb_apb_cross_workspace_bytes": [c_int, c_int, c_int, c_int, c_int],
    "kfb_apb_window_workspace_bytes": [c_int, c_int, c_int, c_int],
    "kfb_apb_cross_workspace_bytes_precise": [c_int, c_int, c_int, c_int],
    "kfb_trimul_workspace_bytes": [c_int, c_int, c_int],
    "kfb_parcae_workspace_bytes": [c_ll, c_int],
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise KfbError(
                f"{LIB_PATH} not found: the CUDA extension is not built "
                "(run `python -m kfold_b200.build`); there is no fallback path")
        l = ctypes.CDLL(LIB_PATH)
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = c_int
        for name, args in _SIZE_FUNCS.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = ctypes.c_size_t
        l.kfb_launch_count.argtypes = []
        l.kfb_launch_count.restype = c_ll
        l.kfb_last_error.argtypes = []
        l.kfb_last_error.restype = ctypes.c_char_p
        _lib = l
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = lib().kfb_last_error().decode()
        if status == 1:
            raise ValueError(f"kfold_b200: {msg}")
        raise KfbError(f"kfold_b200 (status {status}): {msg}")


def ptr(t: torch.Tensor | None):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class on_device:
    """``with on_device(t.device):`` -- makes the tensor's GPU current for the calls inside, like ``torch.cuda.device``,
    but does nothing at all when that GPU already is current (the usual case: one process per GPU), which keeps the
    per-call host cost of the wrappers down."""

    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index
        self.prev = -1

    def __enter__(self):
        if self.idx is not None:
            cur = torch.cuda.current_device()
            if cur != self.idx:
                self.prev = cur
                torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return KFB_BF16
    if dt == torch.float32:
        return KFB_FP32
    raise ValueError(f"kfold_b200 supports bfloat16 and float32 activations, got {dt}")


def device_status() -> int:
    """Synchronise and return the device-side status word (0 = ok); raises if a bounded wait gave up."""
    code = c_int(0)
    check(lib().kfb_device_status(ctypes.byref(code)))
    return code.value


def launch_count() -> int:
    """Number of kernels this library has launched in this process."""
    return int(lib().kfb_launch_count())


def profile_enable(on: bool) -> None:
    """Start (and clear) or stop per-launch CUDA-event timing inside the library."""
    check(lib().kfb_profile_enable(1 if on else 0))


def profile_report(detail: bool = False) -> dict:
    """{tag: (launches, total_ms)} for the launches recorded since profile_enable(True); with `detail`
    {tag: (launches, total_ms, large launches, their total_ms)}, "large" = at least half as long as the tag's upper-quartile launch
    (tags shared by the pair tensor and the single track: the pair-sized launches)."""
    buf = ctypes.create_string_buffer(16384)
    check(lib().kfb_profile_report(buf, len(buf)))
    out = {}
    for line in buf.value.decode().splitlines():
        tag, n, ms, nl, msl = line.split()
        out[tag] = (int(n), float(ms), int(nl), float(msl)) if detail else (int(n), float(ms))
    return out
