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


def test_ctypes_signatures_match_the_header():
    """Every prototype bound in kfold_b200/_lib.py has as many parameters as its declaration in the header, pointers where
    the header has pointers and 64-bit integers where it has `long long` / `size_t` (a mismatch would corrupt the call)."""
    from kfold_b200 import _lib
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    protos = {m.group(1): m.group(2) for m in re.finditer(r"KFB_API[^;(]*?\b(kfb_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)}
    bound = dict(_lib._SIGNATURES)
    bound.update(_lib._SIZE_FUNCS)
    assert bound, "no bound prototypes found"
    for name, args in bound.items():
        assert name in protos, f"{name} is bound but not declared"
        params = [p.strip() for p in protos[name].split(",")] if protos[name].strip() not in ("", "void") else []
        assert len(params) == len(args), f"{name}: header has {len(params)} parameters, the binding {len(args)}"
        for i, (par, ct) in enumerate(zip(params, args)):
            if "*" in par:
                assert ct in (ctypes.c_void_p, ctypes.c_char_p) or issubclass(ct, ctypes._Pointer), f"{name} parameter {i} ({par}) is a pointer"
            elif "long long" in par:
                assert ct is ctypes.c_longlong, f"{name} parameter {i} ({par}) is 64-bit"
            elif "size_t" in par:
                assert ct is ctypes.c_size_t, f"{name} parameter {i} ({par}) is size_t"
            elif "float" in par:
                assert ct is ctypes.c_float, f"{name} parameter {i} ({par}) is float"
            else:
                assert ct is ctypes.c_int, f"{name} parameter {i} ({par}) is int"
