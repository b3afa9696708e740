"""The workspace-free transition entry point, checked against the regular one through the C ABI.

`kfb_transition_fwd_static` serves hosts that may not allocate device memory while they run (a
server with a memory pool frozen at start-up, a callback that must not trigger cudaMalloc's device
synchronisation): its temporaries live in a fixed array inside the library.  The test calls it twice
in a row on different inputs -- the second call sees the first call's leftovers in the array -- and
compares both results with `kfb_transition_fwd` on a caller-provided workspace.  Same kernels, same
arithmetic order, so the results must be identical.  This file sorts last on purpose: if it fails,
a run that stops at the first failure has already covered everything else.
"""
import pytest
import torch

from oracle import pairformer_oracle as O

pytestmark = pytest.mark.gpu


def _call_both(L, x, pk, rows, c, hidden, dtype_code):
    lib = L.lib()
    out_ws = torch.empty_like(x)
    out_static = torch.empty_like(x)
    need = lib.kfb_transition_workspace_bytes(rows, c, hidden)
    ws = torch.empty(need, dtype=torch.uint8, device=x.device)
    L.check(lib.kfb_transition_fwd(L.ptr(x), L.ptr(pk["ln_w"]), L.ptr(pk["ln_b"]), L.ptr(pk["w_swiglu"]), L.ptr(pk["w_out"]),
                                   L.ptr(out_ws), None, L.ptr(ws), ws.numel(), rows, c, hidden, 1e-5, dtype_code, L.stream_ptr()))
    L.check(lib.kfb_transition_fwd_static(L.ptr(x), L.ptr(pk["ln_w"]), L.ptr(pk["ln_b"]), L.ptr(pk["w_swiglu"]),
                                          L.ptr(pk["w_out"]), L.ptr(out_static), None, rows, c, hidden, 1e-5, dtype_code,
                                          L.stream_ptr()))
    torch.cuda.synchronize()
    return out_ws, out_static


def test_static_scratch_transition_matches_workspace_version_twice():
    from kfold_b200 import _lib as L
    from kfold_b200 import packing
    import synth

    dev = torch.device("cuda:0")
    c, factor = 384, 4
    hidden = c * factor
    rng = synth._Rng(4242)
    pk = packing.pack_transition(synth.transition_weights(rng, c, factor), dev)
    w = synth.transition_weights(synth._Rng(4242), c, factor)
    with torch.no_grad():
        for rows, scale in ((768, 1.0), (1000, 3.0)):  # second call: other size, other data, dirty scratch
            x = (rng.normal(rows, c) * scale).to(dev, torch.bfloat16)
            ref, got = _call_both(L, x, pk, rows, c, hidden, L.KFB_BF16)
            assert torch.isfinite(got.float()).all()
            assert torch.equal(got, ref), f"rows={rows}: max diff {(got.float() - ref.float()).abs().max().item():.3e}"
            # and against the CPU oracle directly, at the tolerance of the other bf16 parity tests
            oref = O.transition(x.float().cpu(), w)
            d = got.float().cpu() - oref
            rel = float(d.pow(2).mean().sqrt() / oref.pow(2).mean().sqrt())
            assert rel <= 1e-2, f"rows={rows}: RMS error {rel:.3e} of RMS(oracle)"
    assert L.device_status() == 0


def test_static_scratch_transition_allocates_no_device_memory():
    """What the entry point is for: the call leaves the device's free memory where it was.  The first call on a device
    looks up the scratch array's address; it is made before the measurement, as a host would make it at start-up."""
    from kfold_b200 import _lib as L
    from kfold_b200 import packing
    import synth

    dev = torch.device("cuda:0")
    c, hidden, rows = 384, 1536, 512
    rng = synth._Rng(4343)
    pk = packing.pack_transition(synth.transition_weights(rng, c, 4), dev)
    lib = L.lib()
    for dt, code in ((torch.bfloat16, L.KFB_BF16), (torch.float32, L.KFB_FP32)):
        x = rng.normal(rows, c).to(dev, dt)
        out = torch.empty_like(x)
        args = (L.ptr(x), L.ptr(pk["ln_w"]), L.ptr(pk["ln_b"]), L.ptr(pk["w_swiglu"]), L.ptr(pk["w_out"]), L.ptr(out), None,
                rows, c, hidden, 1e-5, code, L.stream_ptr())
        L.check(lib.kfb_transition_fwd_static(*args))      # set-up call
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info(dev)
        reserved0 = torch.cuda.memory_reserved(dev)
        for _ in range(3):
            L.check(lib.kfb_transition_fwd_static(*args))
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info(dev)
        assert free1 == free0, f"device free memory moved by {free0 - free1} bytes across the calls"
        assert torch.cuda.memory_reserved(dev) == reserved0
        assert torch.isfinite(out.float()).all()
    assert L.device_status() == 0


def test_static_scratch_transition_refuses_oversize():
    from kfold_b200 import _lib as L

    lib = L.lib()
    limit = lib.kfb_transition_static_max_bytes()
    assert limit == 8 << 20
    rows, c, hidden = 768 * 768, 128, 512          # the pair-track transition: far beyond the array
    assert lib.kfb_transition_workspace_bytes(rows, c, hidden) > limit
    x = torch.zeros(8, device="cuda:0")            # never dereferenced: the size check comes first
    st = lib.kfb_transition_fwd_static(L.ptr(x), None, None, L.ptr(x), L.ptr(x), L.ptr(x), None, rows, c, hidden, 1e-5,
                                       L.KFB_BF16, L.stream_ptr())
    assert st == 2  # KFB_ERR_UNSUPPORTED
    msg = lib.kfb_last_error().decode()
    assert "built-in array holds" in msg and str(limit) in msg
    # the fp32-accurate mode keeps six bf16 parts of each temporary: a size that fits in bf16 is refused there, with
    # the same status and a message that says why
    rows = 1000
    assert lib.kfb_transition_workspace_bytes(rows, 384, 1536) <= limit < lib.kfb_transition_workspace_bytes_precise(rows, 384, 1536)
    st = lib.kfb_transition_fwd_static(L.ptr(x), None, None, L.ptr(x), L.ptr(x), L.ptr(x), None, rows, 384, 1536, 1e-5,
                                       L.KFB_FP32_PRECISE, L.stream_ptr())
    assert st == 2 and "fp32-accurate" in lib.kfb_last_error().decode()
    st = lib.kfb_transition_fwd_static(L.ptr(x), None, None, L.ptr(x), L.ptr(x), L.ptr(x), None, rows, 384, 1536, 1e-5, 7,
                                       L.stream_ptr())
    assert st == 1  # KFB_ERR_INVALID_ARGUMENT: unknown dtype
