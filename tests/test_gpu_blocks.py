"""GPU parity of whole blocks, of the backend entry points a K-Fold maintainer would call, and of the production shapes.

Same tolerances as tests/test_gpu_parity.py: bf16 compute is accepted at RMS error <= 1e-2 x RMS(reference), the
fp32-accurate path at max-abs <= 2e-4 and RMS <= 5e-5 x RMS(reference).  Large cases compare against the oracle run on
the GPU in float32 (TF32 off); small ones against the golden vectors of the real reference modules.
"""
import pytest
import torch

import cases
from helpers import compare_pair_output, err_stats, load_golden
from oracle import pairformer_oracle as O
from test_gpu_parity import MAX_TOL, PRECISE_MAX_TOL, PRECISE_RMS_TOL, RMS_TOL, _check, _oracle_on

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _no_grad_and_status():
    from kfold_b200 import _lib as L
    with torch.no_grad():
        yield
    assert L.device_status() == 0


# ----------------------------------------------------------------------------- K-Fold's own trunk block
@pytest.mark.parametrize("name", ["tri_block_c256", "tri_block_c128"])
def test_triangular_block_against_reference_golden(dev, name):
    """modules.TriangularBlock (model/modules/tri_stack.py:130-151) against the output of the reference class: bf16
    compute within bf16 noise, float32 compute at float32 accuracy."""
    from kfold_b200 import modules as M
    inp = cases.build_inputs(name)
    gold = load_golden(name)["out"]
    blk = M.TriangularBlock(inp["case"]["c_z"]).to(dev)
    blk.load_state_dict(inp["w"], strict=True)
    z, pm = inp["z"].to(dev), inp["pair_mask"].to(dev)
    out = blk(z.bfloat16(), pm)
    assert out.dtype == torch.bfloat16
    _check(*err_stats(out.float().cpu(), gold), name + " bf16")
    out = blk(z, pm)
    assert out.dtype == torch.float32
    mx, r = err_stats(out.cpu(), gold)
    assert mx < PRECISE_MAX_TOL and r < PRECISE_RMS_TOL, f"{name} fp32: {mx:.3e} {r:.3e}"


def test_triangular_block_production_width(dev):
    """The production trunk block (channel_z = 256, configs/kfold.yaml:2-3) at N=256 against the oracle on the GPU."""
    from kfold_b200 import modules as M
    import synth
    n, c = 256, 256
    z, pm, _ = synth.pair_inputs(61, n, c, 1, pad_frac=0.1)
    w = synth.triangular_block_weights(61, c)
    blk = M.TriangularBlock(c).to(dev)
    blk.load_state_dict(w, strict=True)
    zb = z.bfloat16()
    out = blk(zb.to(dev), pm.to(dev)).float().cpu()
    ref = _oracle_on(dev, O.triangular_block, zb.float(), pm, w)
    _check(*err_stats(out, ref), "TriangularBlock C=256 N=256")
    # the update alone (what the kernels compute), not only the residual stream it is added to
    _check(*err_stats(out - zb.float(), ref - zb.float()), "TriangularBlock C=256 N=256, update")


# ----------------------------------------------------------------------------- the benchmarked composite block
@pytest.mark.parametrize("n", [256, 768])
def test_pairformer_block_at_benchmark_size(dev, n):
    """The composite Pairformer block the benchmark times (N=768, c_z=128, c_s=384, 10 % padding tail, seed 3) and a
    smaller one, whole, against the oracle run on the GPU in float32."""
    from kfold_b200 import modules as M
    import synth
    z, pm, m = synth.pair_inputs(3, n, 128, 1, pad_frac=0.1)
    s = synth.single_inputs(3, n, 384, 1)
    w = synth.pairformer_block_weights(3, 128, 384)
    blk = M.PairformerBlock(128, 384).to(dev)
    blk.load_state_dict(w, strict=True)
    zb, sb = z.bfloat16(), s.bfloat16()
    zo, so = blk(zb.to(dev), sb.to(dev), pm.to(dev), m.to(dev))
    zo, so = zo.float().cpu(), so.float().cpu()
    assert torch.isfinite(zo).all() and torch.isfinite(so).all()

    def run(z_, s_, pm_, m_, w_):
        zr, sr = O.pairformer_block(z_, s_, pm_, m_, w_, row_chunk=32)
        return torch.cat([zr.reshape(-1), sr.reshape(-1)])

    ref = _oracle_on(dev, run, zb.float(), sb.float(), pm, m, w)
    zr, sr = ref[: zo.numel()].view_as(zo), ref[zo.numel():].view_as(so)
    valid = pm[0]
    _check(*err_stats(zo[0][valid], zr[0][valid]), f"block N={n} z, valid region")
    _check(*err_stats(so[0][m[0]], sr[0][m[0]]), f"block N={n} s, valid tokens")
    _check(*err_stats(zo, zr), f"block N={n} z")
    _check(*err_stats(so, sr), f"block N={n} s")
    # the five pair updates together, without the residual stream that dilutes their error
    _check(*err_stats(zo - zb.float(), zr - zb.float()), f"block N={n} z update")


# ----------------------------------------------------------------------------- backend entry points of the adapter
def test_adapter_entry_points_on_the_gpu(dev):
    """adapter.b200_triangular_mult / b200_triangular_attn / b200_attention_pair_bias -- the functions the reference's
    dispatch calls once `install()` ran -- from module state dict to kernels, against the oracle.  A module of this
    package stands in for the reference module (same parameter names and attributes)."""
    from kfold_b200 import adapter
    from kfold_b200 import modules as M
    import synth
    n, b = 40, 2
    rng = synth._Rng(91)
    x = rng.normal(b, n, n, 128).bfloat16()
    mask = synth.block_mask(91, b, n)
    for direction, cls in (("outgoing", M.TriangleMultiplicationOutgoing), ("incoming", M.TriangleMultiplicationIncoming)):
        w = synth.trimul_weights(rng, 128)
        mod = cls(128).to(dev)
        mod.load_state_dict(w, strict=True)
        out = adapter.b200_triangular_mult(mod, x.to(dev), mask.to(dev), direction)
        assert out.dtype == torch.bfloat16 and "trimul" in mod._b200_cache
        _check(*err_stats(out.float().cpu(), O.triangle_multiplication(x.float(), mask, w, direction)), f"adapter trimul {direction}")
        with torch.autocast("cuda", dtype=torch.bfloat16):      # fp32 input under autocast: bf16 compute, fp32 result
            out = adapter.b200_triangular_mult(mod, x.float().to(dev), mask.to(dev), direction)
        assert out.dtype == torch.float32
        _check(*err_stats(out.cpu(), O.triangle_multiplication(x.float(), mask, w, direction)), f"adapter trimul {direction} autocast")
    for starting, cls in ((True, M.TriangleAttentionStartingNode), (False, M.TriangleAttentionEndingNode)):
        w = synth.triatt_weights(rng, 128, 4)
        mod = cls(128, 4).to(dev)
        mod.load_state_dict(w, strict=True)
        out = adapter.b200_triangular_attn(mod, x.to(dev), mask.to(dev), starting)
        _check(*err_stats(out.float().cpu(), O.triangle_attention(x.float(), mask, w, 4, starting)), f"adapter triatt {starting}")
        out32 = adapter.b200_triangular_attn(mod, x.float().to(dev), mask.to(dev), starting)      # float32 compute
        mx, r = err_stats(out32.cpu(), O.triangle_attention(x.float(), mask, w, 4, starting))
        assert out32.dtype == torch.float32 and mx < PRECISE_MAX_TOL and r < PRECISE_RMS_TOL
    # token-level self attention (call site "confidence") and windowed cross attention ("diffusion_local")
    l = 72
    w = synth.apb_weights(rng, 384, None)
    mod = M.SelfAttentionPairBias(384, 16, None, "confidence").to(dev)
    mod.load_state_dict(w, strict=True)
    a = rng.normal(1, l, 384).bfloat16()
    an = O.layer_norm(a.float(), w["layernorm_a.weight"], w["layernorm_a.bias"]).bfloat16()
    bias = rng.normal(1, 16, l, l)
    tmask = synth.token_mask(l, valid=65).unsqueeze(0)
    and_ = an.to(dev)        # `x_q is x_k` selects the self-attention path, as at the reference's call sites
    out = adapter.b200_attention_pair_bias(mod, and_, and_, bias.to(dev), tmask.to(dev), call_site="confidence")
    ref = O.attention_pair_bias(an.float(), an.float(), bias, tmask, w, 16)
    _check(*err_stats(out.float().cpu(), ref), "adapter apb confidence")
    wc = synth.cross_apb_weights(rng, 128, 128)
    modc = M.CrossAttentionPairBias(128, 4, 128).to(dev)
    modc.load_state_dict(wc, strict=True)
    xq, xk = rng.normal(1, 2, 3, 32, 128).bfloat16(), rng.normal(1, 2, 3, 128, 128).bfloat16()
    wbias = rng.normal(1, 1, 3, 4, 32, 128)
    wmask = torch.ones(1, 1, 3, 128, dtype=torch.bool)
    wmask[..., 100:] = False
    out = adapter.b200_attention_pair_bias(modc, xq.to(dev), xk.to(dev), wbias.to(dev), wmask.to(dev), call_site="diffusion_local")
    ref = O.attention_pair_bias(xq.float(), xk.float(), wbias, wmask, wc, 4)
    _check(*err_stats(out.float().cpu(), ref), "adapter apb diffusion_local")


# ----------------------------------------------------------------------------- torch.inference_mode(), how the reference runs
def test_stacks_run_under_inference_mode(dev):
    """The reference decorates inference() / predict() with torch.inference_mode() (model/model.py:294, :361); tensors
    made there carry no version counter.  DiffusionStack.step (token and atom stacks, their per-complex caches) must
    run there, twice, and agree with the torch.no_grad() result."""
    from kfold_b200 import modules as M
    inp = cases.build_inputs("diffusion_step")
    cs = inp["case"]
    mod = M.DiffusionStack(channel_a=cs["c_a"], channel_s=cs["c_s"], channel_z=cs["c_z"], channel_atom=cs["c_atom"],
                           channel_atompair=cs["c_pair"], atom_encoder_blocks=cs["atom_blocks"], atom_encoder_heads=cs["atom_heads"],
                           token_transformer_blocks=cs["token_blocks"], token_transformer_heads=cs["token_heads"],
                           atom_decoder_blocks=cs["atom_blocks"], atom_decoder_heads=cs["atom_heads"]).to(dev)
    mod.load_state_dict(inp["w"], strict=False)
    names = ("r_noisy", "q", "c", "p", "token_index", "atom_mask", "s", "pair_bias", "token_mask")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        base = mod.step(*[inp[k].to(dev) for k in names]).clone()
    mod.reset_caches()
    with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
        args = [inp[k].to(dev) for k in names]          # inference tensors
        assert torch.is_inference(args[0])
        out1 = mod.step(*args)
        out2 = mod.step(*args)
        assert torch.equal(out1, out2) and torch.equal(out1, base)
        # the pair-bias attention of the single track and a stand-alone local stack
        inp2 = cases.build_inputs("local_stack")
        c2 = inp2["case"]
        stack = M.LocalTransformerStack(c2["c"], c2["c_s"], c2["c_z"], c2["heads"], c2["blocks"]).to(dev)
        stack.load_state_dict(inp2["w"], strict=True)
        out = stack(*[inp2[k].to(dev) for k in ("a", "s", "z", "mask")])
        valid = inp2["mask"].reshape(-1)
        _check(*err_stats(out.float().cpu()[..., valid, :], load_golden("local_stack")["out"][..., valid, :]), "local stack, inference mode")
    mod.check()


def test_pair_bias_cache_keeps_its_source_alive(dev):
    """The converted pair bias is cached per source tensor; the cache holds the source, so a freed source's address
    cannot be handed to the bias of the next complex and hit the stale entry."""
    from kfold_b200 import modules as M
    import synth
    rng = synth._Rng(17)
    l, blocks = 24, 2
    w = {}
    for i in range(blocks):
        w.update(synth._prefixed(f"blocks.{i}.attention", synth.apb_weights(rng, 768, 384)))
        w.update(synth._prefixed(f"blocks.{i}.transition", synth.conditioned_transition_weights(rng, 768, 384)))
    stack = M.CachedGlobalTransformerStack(768, 384, 16, blocks).to(dev)
    stack.load_state_dict(w, strict=True)
    a, s = rng.normal(1, 2, l, 768).to(dev), rng.normal(1, 1, l, 384).to(dev)
    mask = torch.ones(1, 1, l, dtype=torch.bool, device=dev)
    outs = []
    for seed in (1, 2):
        bias = synth._Rng(seed).normal(1, blocks, 16, l, l).to(dev)        # fp32 source -> a bf16 copy is cached
        with torch.autocast("cuda", dtype=torch.bfloat16):
            outs.append(stack(a, s, bias, mask).clone())
        assert stack._bias_src is bias
        del bias
    assert not torch.equal(outs[0], outs[1])


# ----------------------------------------------------------------------------- production shapes of the sampler
def test_token_transformer_production_width(dev):
    """K-Fold's production token transformer width: channel_a = 1024, 16 heads x 64 (configs/kfold.yaml:61-76),
    2 blocks, L=256, 3 samples sharing the pair bias, against the oracle on the GPU."""
    from kfold_b200 import modules as M
    import synth
    rng = synth._Rng(1024)
    blocks, l, ns, c, cs = 2, 256, 3, 1024, 384
    w = {}
    for i in range(blocks):
        w.update(synth._prefixed(f"blocks.{i}.attention", synth.apb_weights(rng, c, cs)))
        w.update(synth._prefixed(f"blocks.{i}.transition", synth.conditioned_transition_weights(rng, c, cs)))
    a, s = rng.normal(1, ns, l, c), rng.normal(1, 1, l, cs)
    bias = rng.normal(1, blocks, 16, l, l)
    mask = synth.token_mask(l, pad_frac=0.1).view(1, 1, l)
    stack = M.CachedGlobalTransformerStack(c, cs, 16, blocks).to(dev)
    stack.load_state_dict(w, strict=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = stack(a.to(dev), s.to(dev), bias.to(dev), mask.to(dev)).cpu()
    ref = _oracle_on(dev, O.global_transformer_stack, a, s, bias, mask, w, 16, blocks)
    _check(*err_stats(out, ref), "token transformer c=1024")


def test_tolerances_are_the_stated_ones():
    assert RMS_TOL == 1e-2 and MAX_TOL == 0.15


def test_host_pipeline_matches_direct_calls(dev):
    """host_pipeline.HostPipeline: five different host-resident inputs through a Transition with the copies overlapped;
    every result equals the one of the plain call on that input, and unpinned buffers are refused."""
    from kfold_b200 import modules as M
    from kfold_b200.host_pipeline import HostPipeline
    import synth
    c = 128
    mod = M.Transition(c, 4).to(dev)
    mod.load_state_dict(synth.transition_weights(synth._Rng(5), c, 4), strict=True)
    g = torch.Generator().manual_seed(9)
    xs = [torch.randn(1, 96, 96, c, generator=g).bfloat16().pin_memory() for _ in range(5)]
    outs = [(torch.empty_like(x).pin_memory(),) for x in xs]
    pipe = HostPipeline(lambda x: mod(x, residual=True), dev, depth=2)
    pipe.run([(x,) for x in xs], outs)
    torch.cuda.synchronize()
    for x, (o,) in zip(xs, outs):
        assert torch.equal(o, mod(x.to(dev), residual=True).cpu())
    with pytest.raises(ValueError):
        pipe.run([(torch.zeros(1, 8, 8, c),)], [(torch.zeros(1, 8, 8, c),)])
