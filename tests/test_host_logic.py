"""Host-side logic that needs no GPU: weight packing, module/state-dict compatibility, error behaviour."""
import pytest
import torch

from kfold_b200 import functional as F
from kfold_b200 import modules as M
from kfold_b200 import packing
import synth


def test_interleave_glu_layout():
    v = torch.arange(256 * 4, dtype=torch.float32).reshape(256, 4)
    g = -v
    p = packing.interleave_glu(v, g)
    assert p.shape == (512, 4)
    assert torch.equal(p[:128], v[:128]) and torch.equal(p[128:256], g[:128])
    assert torch.equal(p[256:384], v[128:]) and torch.equal(p[384:], g[128:])
    # the bf16 kernels' halved gate operands; none in the fp32-accurate packing
    ps = packing.interleave_glu(v, g, **packing.glu_scales("sigmoid", False))
    assert torch.equal(ps, 0.5 * p)
    pw = packing.interleave_glu(v, g, **packing.glu_scales("swiglu", False))
    assert torch.equal(pw[:128], 0.5 * v[:128]) and torch.equal(pw[128:256], g[:128])
    assert torch.equal(packing.interleave_glu(v, g, **packing.glu_scales("swiglu", True)), p)


def test_pad_heads_scales_and_zero_fills():
    w = torch.ones(16 * 24, 8)
    p = packing._pad_heads(w, 16, 24, 32, 0.5)
    assert p.shape == (16 * 32, 8)
    p = p.reshape(16, 32, 8)
    assert torch.all(p[:, :24] == 0.5) and torch.all(p[:, 24:] == 0)


def test_head_dim_pad():
    assert packing.head_dim_pad(16) == 32 and packing.head_dim_pad(24) == 32 and packing.head_dim_pad(32) == 32
    assert packing.head_dim_pad(48) == 64 and packing.head_dim_pad(64) == 64
    with pytest.raises(ValueError):
        packing.head_dim_pad(20)


def test_pack_triatt_projection_matches_unpacked_math():
    w = synth.triatt_weights(synth._Rng(3), 128, 4)
    pk = packing.pack_triatt(w, 4, "cpu", torch.float32)
    x = torch.randn(5, 128)
    y = x @ pk["w_proj"].T
    q = (x @ w["mha.linear_q.weight"].T) / 32 ** 0.5 * packing.LOG2E   # the kernel keeps logits in log2 units
    assert torch.allclose(y[:, :128], q, atol=1e-5)
    assert torch.allclose(y[:, 128:256], x @ w["mha.linear_k.weight"].T, atol=1e-5)
    assert torch.allclose(y[:, 256:384], x @ w["mha.linear_g.weight"].T, atol=1e-5)
    assert torch.allclose(y[:, 384:512], x @ w["mha.linear_v.weight"].T, atol=1e-5)
    assert torch.allclose(y[:, 512:516], x @ w["linear.weight"].T, atol=1e-5)
    assert torch.all(y[:, 516:] == 0)


def test_pack_apb_pads_d24_to_32():
    w = synth.apb_weights(synth._Rng(4), 384, None)
    pk = packing.pack_apb(w, 16, "cpu", torch.float32)
    assert pk["w_proj"].shape == (4 * 16 * 32, 384)
    assert pk["proj_bias"].shape == (4 * 16 * 32,)
    x = torch.randn(3, 384)
    y = (x @ pk["w_proj"].T + pk["proj_bias"]).reshape(3, 4, 16, 32)
    q = ((x @ w["linear_q.weight"].T + w["linear_q.bias"]) / 24 ** 0.5 * packing.LOG2E).reshape(3, 16, 24)
    assert torch.allclose(y[:, 0, :, :24], q, atol=1e-5)
    assert torch.all(y[:, 0, :, 24:] == 0)


@pytest.mark.parametrize("cls,gen", [
    (lambda: M.TriangleMultiplicationOutgoing(128), lambda r: synth.trimul_weights(r, 128)),
    (lambda: M.TriangleMultiplicationIncoming(128), lambda r: synth.trimul_weights(r, 128)),
    (lambda: M.TriangleAttentionStartingNode(128, 4), lambda r: synth.triatt_weights(r, 128, 4)),
    (lambda: M.TriangleAttentionEndingNode(128, 4), lambda r: synth.triatt_weights(r, 128, 4)),
    (lambda: M.Transition(128, 4), lambda r: synth.transition_weights(r, 128, 4)),
    (lambda: M.SelfAttentionPairBias(384, 16, None, "confidence"), lambda r: synth.apb_weights(r, 384, None)),
    (lambda: M.SelfAttentionPairBias(768, 16, 384, "diffusion_global"), lambda r: synth.apb_weights(r, 768, 384)),
    (lambda: M.ConditionedTransitionBlock(768, 384), lambda r: synth.conditioned_transition_weights(r, 768, 384)),
])
def test_modules_accept_reference_state_dicts(cls, gen):
    """synth.*_weights are keyed like the reference modules' state_dict(); strict loading must succeed."""
    mod = cls()
    mod.load_state_dict(gen(synth._Rng(0)), strict=True)


def test_block_state_dict_keys():
    blk = M.PairformerBlock()
    blk.load_state_dict(synth.pairformer_block_weights(0), strict=True)


def test_inference_only_and_cuda_only():
    mod = M.TriangleMultiplicationOutgoing(128)
    x = torch.zeros(1, 8, 8, 128)
    m = torch.ones(1, 8, 8, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="inference-only"):
        mod(x, m)
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        mod(x, m)


def test_functional_rejects_cpu_tensors_and_bad_shapes():
    pk = {"c": 128}
    with pytest.raises(RuntimeError, match="CUDA"):
        F.triangle_multiplication(torch.zeros(1, 8, 8, 128), torch.ones(1, 8, 8, dtype=torch.bool), pk, "outgoing")
    with pytest.raises(ValueError):
        F.triangle_multiplication(torch.zeros(1, 8, 8, 128), torch.ones(1, 8, 8, dtype=torch.bool), pk, "sideways")


def test_unsupported_variants_fail_loudly():
    with pytest.raises(ValueError):
        M.SelfAttentionPairBias(768, 16, None, "somewhere")


def test_missing_extension_fails_loudly(monkeypatch, tmp_path):
    from kfold_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.KfbError, match="no fallback"):
        _lib.lib()


def test_pad_pair():
    x = torch.randn(2, 10, 10, 4)
    m = torch.ones(2, 10, 10, dtype=torch.bool)
    xp, mp, n = F._pad_pair(x, m)
    assert xp.shape == (2, 16, 16, 4) and mp.shape == (2, 16, 16) and n == 10
    assert torch.equal(xp[:, :10, :10], x) and not mp[:, 10:].any() and not mp[:, :, 10:].any()


def test_atom_window_indexing_matches_the_oracle():
    """Windows of 32 queries and 128 keys [32 w - 48, 32 w + 80), zero-filled outside (model/layers/folding/utils.py:97-188)."""
    from kfold_b200.modules import build_atom_to_qk_fn
    from oracle import pairformer_oracle as O
    x = torch.arange(1, 96 * 3 + 1, dtype=torch.float32).view(1, 96, 3)
    to_qk = build_atom_to_qk_fn(96, "cpu")
    q, k = to_qk(x, -2)
    oq, ok = O.atom_windows(x, -2)
    assert torch.equal(q, oq) and torch.equal(k, ok) and k.shape == (1, 3, 128, 3)
    assert (k[0, 0, :48] == 0).all() and torch.equal(k[0, 0, 48:], x[0, :80])      # first window: 48 keys before atom 0
    assert torch.equal(k[0, 1], torch.cat([torch.zeros(16, 3), x[0, :96], torch.zeros(16, 3)]))   # second: atoms -16 .. 111
    m = torch.ones(1, 96, dtype=torch.bool)
    assert to_qk(m, -1)[1].sum() == O.atom_windows(m, -1)[1].sum() == 80 + 96 + 80
    with pytest.raises(ValueError):
        build_atom_to_qk_fn(40, "cpu")


def test_bias_sharing_patterns():
    from kfold_b200.modules import _bias_sharing
    assert _bias_sharing((1, 5, 188), (1, 1, 188)) == (5 * 188, 188)     # samples share the per-window bias
    assert _bias_sharing((2, 5, 188), (2, 1, 188)) == (5 * 188, 188)
    assert _bias_sharing((1, 5, 188), (188,)) == (5 * 188, 188)
    assert _bias_sharing((1, 5, 188), (1, 5, 188)) == (1, 0)             # nothing shared
    assert _bias_sharing((1, 5), (1, 1)) == (5, 0)                       # plain sharing by consecutive entries
    assert _bias_sharing((1, 1, 188), (1, 1, 188)) == (1, 0)
    assert _bias_sharing((2, 5, 188), (1, 5, 188)) == (2 * 5 * 188, 5 * 188)
    assert _bias_sharing((2, 5, 188), (2, 5, 1)) == (188, 0)
    assert _bias_sharing((2, 5, 188), (1, 5, 1)) is None                 # shared dims not in one block


def test_pack_apb_cross_layout():
    from kfold_b200 import packing
    import synth
    w = synth.cross_apb_weights(synth._Rng(3), 128, 128)
    keys = ("linear_q.weight", "linear_q.bias", "linear_k.weight", "linear_v.weight", "linear_g.weight", "linear_out.weight")
    pk = packing.pack_apb_cross({k: w[k] for k in keys}, 4, "cpu")
    assert pk["w_q"].shape == (256, 128) and pk["w_kv"].shape == (256, 128) and pk["q_bias"].shape == (256,)
    scale = 32 ** -0.5 * packing.LOG2E
    assert torch.allclose(pk["w_q"][:128].float(), (w["linear_q.weight"] * scale).bfloat16().float())
    assert torch.allclose(pk["q_bias"][:128], w["linear_q.bias"] * scale) and (pk["q_bias"][128:] == 0).all()
    assert torch.equal(pk["w_kv"][128:].float(), w["linear_v.weight"].bfloat16().float())
    pkp = packing.pack_apb_cross({k: w[k] for k in keys}, 4, "cpu", precise=True)
    assert pkp["w_q"].shape == (256, 6 * 128) and pkp["w_kv"].shape == (256, 6 * 128) and pkp["precise"]


def test_rows_helper_passes_column_slices_as_they_lie():
    """A column slice of a wide row-major table reaches the kernels as (pointer, rows, row stride) without a copy; layouts
    that are not rows at a constant stride are made contiguous."""
    from kfold_b200.functional import _rows
    table = torch.zeros(2, 1, 40, 96, dtype=torch.bfloat16)
    sl = table[..., 32:64]
    t, rows, ld = _rows(sl, 32)
    assert t.data_ptr() == sl.data_ptr() and rows == 80 and ld == 96
    t, rows, ld = _rows(table, 96)
    assert rows == 80 and ld == 96
    t, rows, ld = _rows(sl.expand(2, 3, 40, 32), 32)             # a broadcast dimension: copied
    assert t.is_contiguous() and rows == 240 and ld == 32
    t, rows, ld = _rows(table[..., 4:36], 32)                     # misaligned start: copied
    assert t.is_contiguous() and ld == 32
    t, rows, ld = _rows(sl, 32, torch.float32)                    # dtype change: converted, then dense
    assert t.dtype == torch.float32 and rows == 80


def test_conditioning_tables_fold_the_layernorm_scale():
    """The stacked, scale-folded AdaLN matrices of a stack reproduce every AdaLN's gate / shift rows:
    LN(s) (W * gamma)^T + b == (LN(s) * gamma) W^T + b, and the gate table is the plain stack of the gate Linears."""
    from kfold_b200 import modules as M
    torch.manual_seed(3)
    c_a, c_s = 64, 48
    adalns = [M.AdaLN(c_a, c_s) for _ in range(3)]
    gates = [M.Linear(c_s, c_a) for _ in range(2)]
    for m in adalns:
        m.layernorm_s.weight.data = 1.0 + 0.2 * torch.randn(c_s)
        m.linear_g.bias.data = torch.randn(c_a)
    for g in gates:
        g.bias.data = torch.randn(c_a)
    w1, b1, w2, b2 = M._ConditioningBank()._pack(adalns, gates, torch.device("cpu"))
    assert w1.shape == (3 * 2 * c_a, c_s) and w2.shape == (2 * c_a, c_s) and w1.dtype == torch.bfloat16
    s = torch.randn(10, c_s)
    sn = torch.nn.functional.layer_norm(s, (c_s,))
    t1 = sn @ w1.float().t() + b1
    t2 = s @ w2.float().t() + b2
    for i, m in enumerate(adalns):
        sm = sn * m.layernorm_s.weight
        ref = torch.cat([sm @ m.linear_g.weight.t() + m.linear_g.bias, sm @ m.linear_bias.weight.t()], dim=-1)
        assert (t1[:, i * 2 * c_a:(i + 1) * 2 * c_a] - ref).abs().max() < 0.05            # bf16 weights
    for i, g in enumerate(gates):
        assert (t2[:, i * c_a:(i + 1) * c_a] - (s @ g.weight.t() + g.bias)).abs().max() < 0.05


def test_index_sharing_patterns():
    """Which batch entries share an index / mask row: trailing size-1 leading dims are shared, anything else is not."""
    from kfold_b200.functional import _index_sharing, _shared_mask
    assert _index_sharing((1, 5), (1, 1)) == 5
    assert _index_sharing((2, 5), (2, 1)) == 5
    assert _index_sharing((2, 5), (2, 5)) == 1
    assert _index_sharing((1, 5), (1,)) == 5              # fewer leading dims: padded with 1 on the left
    assert _index_sharing((2, 5), (2,)) is None           # (1, 2) against (2, 5): not a trailing-share pattern
    assert _index_sharing((2, 5), (1, 5)) is None
    assert _index_sharing((), ()) == 1
    m = torch.tensor([[[True, False, True, True]]])       # (1, 1, 4) shared by 3 samples
    mk = _shared_mask(m, (1, 3), 4, 3)
    assert mk.dtype == torch.uint8 and mk.shape == (1, 4) and mk.tolist() == [[1, 0, 1, 1]]
    full = _shared_mask(m.expand(1, 3, 4), (1, 3), 4, 1)
    assert full.shape == (3, 4)
    with pytest.raises(ValueError):
        _shared_mask(m.expand(1, 3, 4), (1, 3), 4, 3)     # per-sample mask with shared features


def test_modules_refuse_what_they_do_not_cover():
    from kfold_b200 import modules as M
    with pytest.raises(ValueError):
        M.DiffusionStack(separate_endpoint_atom_encoder=True, token_transformer_blocks=1)      # needs channel_coords=6
    sep = M.DiffusionStack(channel_a=64, channel_s=32, channel_z=32, channel_atom=32, channel_atompair=16, channel_coords=6,
                           separate_endpoint_atom_encoder=True, atom_encoder_blocks=1, atom_encoder_heads=2,
                           token_transformer_blocks=1, token_transformer_heads=2, atom_decoder_blocks=1, atom_decoder_heads=2)
    assert {"endpoint_fusion.weight", "layernorm_a_t.weight", "layernorm_a_endpoint.weight",
            "endpoint_atom_attention_encoder.linear_r_to_q.weight"} <= set(sep.state_dict())
    assert sep.atom_attention_encoder.linear_r_to_q.weight.shape == (32, 3)
    with pytest.raises(ValueError):
        M.CrossAttentionPairBias(128, 4, 128, inf=1e6)
    with pytest.raises(ValueError):
        M.build_atom_to_qk_fn(100, "cpu")
    ds = M.DiffusionStack(channel_a=64, channel_s=32, channel_z=32, channel_atom=32, channel_atompair=16, atom_encoder_blocks=1,
                          atom_encoder_heads=2, token_transformer_blocks=1, token_transformer_heads=2, atom_decoder_blocks=1,
                          atom_decoder_heads=2)
    keys = set(ds.state_dict())
    for k in ("layernorm_s.weight", "linear_s_to_a.weight", "layernorm_z.weight", "linear_z_to_bias.weight", "layernorm_a.weight",
              "atom_attention_encoder.linear_r_to_q.weight", "atom_attention_encoder.transformer.blocks.0.attention.adaln_a_q.linear_g.bias",
              "token_transformer.blocks.0.attention.linear_ada_out.bias", "atom_attention_decoder.linear_q_to_r.weight",
              "single_conditioning.transitions.1.linear_out.weight"):
        assert k in keys, k
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        ds.get_pair_bias(torch.zeros(1, 8, 8, 32))
