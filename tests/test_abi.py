"""The C-ABI library loads and exports every symbol that include/kfold_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kfold_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"KFB_API[^;(]*?\b(kfb_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def library():
    from kfold_b200 import _lib, build
    build.build()
    return ctypes.CDLL(_lib.LIB_PATH)


def test_header_declares_the_entry_points():
    syms = declared_symbols()
    for need in ("kfb_trimul_fwd", "kfb_triatt_fwd", "kfb_apb_fwd", "kfb_transition_fwd", "kfb_layernorm",
                 "kfb_pair_bias_fwd", "kfb_gemm_bf16", "kfb_version", "kfb_last_error", "kfb_device_status"):
        assert need in syms


def test_library_exports_every_declared_symbol(library):
    for name in declared_symbols():
        assert hasattr(library, name), f"{name} is declared in the header but not exported"


def test_version_and_error_string(library):
    library.kfb_version.restype = ctypes.c_int
    assert library.kfb_version() >= 100
    library.kfb_last_error.restype = ctypes.c_char_p
    assert isinstance(library.kfb_last_error(), bytes)


def test_workspace_queries_need_no_gpu(library):
    library.kfb_trimul_workspace_bytes.restype = ctypes.c_size_t
    library.kfb_trimul_workspace_bytes.argtypes = [ctypes.c_int] * 3
    b768 = library.kfb_trimul_workspace_bytes(1, 768, 128)
    # xn + ab(2x) + gl + t, each N*N*C bf16
    assert b768 >= 5 * 768 * 768 * 128 * 2
    assert b768 < 5 * 768 * 768 * 128 * 2 + 8192
    library.kfb_triatt_workspace_bytes.restype = ctypes.c_size_t
    library.kfb_triatt_workspace_bytes.argtypes = [ctypes.c_int] * 4
    assert library.kfb_triatt_workspace_bytes(1, 384, 128, 4) > 0


def test_invalid_arguments_are_rejected_without_a_gpu(library):
    """Argument validation happens before any CUDA call."""
    library.kfb_trimul_fwd.restype = ctypes.c_int
    vp = ctypes.c_void_p
    library.kfb_trimul_fwd.argtypes = [ctypes.c_int] + [vp] * 12 + [ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                                    ctypes.c_float, ctypes.c_int, vp]
    st = library.kfb_trimul_fwd(0, *([None] * 12), 0, 1, 64, 128, 1e-5, 0, None)
    assert st == 1  # KFB_ERR_INVALID_ARGUMENT
    library.kfb_last_error.restype = ctypes.c_char_p
    assert b"null" in library.kfb_last_error()
