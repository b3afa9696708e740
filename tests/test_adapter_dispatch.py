"""install()/convert() against the REAL K-Fold sources (skipped where the reference tree is absent).

No GPU is needed: the CUDA calls are replaced by recorders, so what is checked is the dispatch itself --
which reference modules route to the backend, with which tensors, and that the other backends still work.
"""
import pytest
import torch

import ref_shim

pytestmark = pytest.mark.skipif(ref_shim.reference_root() is None, reason="K-Fold reference tree not present")


@pytest.fixture(scope="module")
def ref():
    ns = ref_shim.load_reference()
    from kfold_b200 import adapter
    adapter.install()
    adapter.install()  # idempotent
    return ns


@pytest.fixture()
def recorder(monkeypatch):
    from kfold_b200 import adapter
    calls = []
    monkeypatch.setattr(adapter, "_check", lambda x, what: None)
    monkeypatch.setattr(adapter, "_cached_pack", lambda module, x, dt, slot, fn: {"slot": slot})

    def rec(name):
        def f(*a, **k):
            calls.append((name, a, k))
            return torch.zeros_like(a[0])
        return f

    monkeypatch.setattr(adapter.F, "triangle_multiplication", rec("trimul"))
    monkeypatch.setattr(adapter.F, "triangle_attention", rec("triatt"))
    monkeypatch.setattr(adapter.F, "attention_pair_bias", rec("apb"))
    monkeypatch.setattr(adapter.F, "attention_pair_bias_cross_bcast", rec("apb_cross"))
    return calls


def test_select_kernel_backend_accepts_b200(ref, monkeypatch):
    import kfold.utils.runtime as rt
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    assert rt.select_kernel_backend("b200") == "b200"
    assert rt.select_kernel_backend("torch") == "torch"
    with pytest.raises(ValueError):
        rt.select_kernel_backend("nonsense")


def test_triangle_multiplication_routes(ref, recorder):
    x = torch.randn(1, 8, 8, 128)
    m = torch.ones(1, 8, 8, dtype=torch.bool)
    for cls, direction in ((ref.TriangleMultiplicationOutgoing, "outgoing"), (ref.TriangleMultiplicationIncoming, "incoming")):
        mod = cls(128, kernel_backend="b200")
        with torch.no_grad():
            out = mod(x, m)
        name, a, k = recorder[-1]
        assert name == "trimul" and a[3] == direction and a[0] is x and out.shape == x.shape
    # the torch backend is untouched
    n = len(recorder)
    with torch.no_grad():
        ref.TriangleMultiplicationOutgoing(128)(x, m)
    assert len(recorder) == n


def test_triangle_attention_receives_untransposed_input(ref, recorder):
    x = torch.randn(1, 8, 8, 128)
    m = torch.ones(1, 8, 8, dtype=torch.bool)
    for cls, starting in ((ref.TriangleAttentionStartingNode, True), (ref.TriangleAttentionEndingNode, False)):
        mod = cls(128, 4, kernel_backend="b200")
        with torch.no_grad():
            mod(x, m)
        name, a, k = recorder[-1]
        assert name == "triatt" and a[3] is starting
        assert a[0].data_ptr() == x.data_ptr() and a[0].is_contiguous()   # no transposed view reaches the kernels


def test_attention_pair_bias_routes_after_convert(ref, recorder):
    from kfold_b200 import adapter
    mod = ref.SelfAttentionPairBias(384, 16, None, "confidence", kernel_backend="sdpa")
    holder = torch.nn.ModuleList([mod, ref.TriangleMultiplicationOutgoing(128), ref.TriangleAttentionEndingNode(128, 4),
                                  ref.SelfAttentionPairBias(768, 16, 384, "diffusion_global", kernel_backend="sdpa"),
                                  ref.TriangleAttentionStartingNode(64, 4)])
    assert adapter.convert(holder) == 4          # the float32 diffusion attention stays as it was unless asked for
    assert holder[3].kernel_backend == "sdpa" and holder[4].kernel_backend == "b200"   # D=16 tri-att is taken
    assert adapter.convert(holder, diffusion=True) == 5
    s = torch.randn(1, 12, 384)
    bias = torch.randn(1, 16, 12, 12)
    mask = torch.ones(1, 12, dtype=torch.bool)
    with torch.no_grad():
        out = mod(s, None, bias, mask)
    name, a, k = recorder[-1]
    assert name == "apb" and a[1] is bias and out.shape == s.shape


def test_cross_attention_routes_for_the_atom_windows(ref, recorder):
    """CrossAttentionPairBias (call site "diffusion_local") is converted together with the sampler's other attention
    modules and hands the windowed query / key tensors to the cross-attention entry."""
    from kfold_b200 import adapter
    mod = ref.CrossAttentionPairBias(128, 4, 128, kernel_backend="sdpa")
    holder = torch.nn.ModuleList([mod])
    assert adapter.convert(holder) == 0 and mod.kernel_backend == "sdpa"
    assert adapter.convert(holder, diffusion=True) == 1 and mod.kernel_backend == "b200"
    a_q, a_k = torch.randn(1, 2, 3, 32, 128), torch.randn(1, 2, 3, 128, 128)
    s_q, s_k = torch.randn(1, 1, 3, 32, 128), torch.randn(1, 1, 3, 128, 128)
    bias = torch.randn(1, 1, 3, 4, 32, 128)
    mask = torch.ones(1, 1, 3, 128, dtype=torch.bool)
    with torch.no_grad():
        out = mod(a_q, a_k, s_q, s_k, bias, mask)
    name, a, k = recorder[-1]
    assert name == "apb_cross" and a[0].shape == a_q.shape and a[1].shape == a_k.shape and a[2] is bias and a[3] is mask
    assert a[4] == {"slot": "apb_cross"} and out.shape == a_q.shape


def test_backend_refuses_cpu_and_grad(ref):
    mod = ref.TriangleMultiplicationOutgoing(128, kernel_backend="b200")
    x = torch.randn(1, 8, 8, 128)
    m = torch.ones(1, 8, 8, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="inference-only"):
        mod(x, m)
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        mod(x, m)
