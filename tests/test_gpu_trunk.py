"""GPU parity of the callers either side of the pair stacks: the trunk's recurrence and language-model pair embedding, the
diffusion module's pair conditioning, and the confidence head's per-sample loop -- each against the golden vectors of the
reference's own classes (tests/golden/make_golden.py).

bf16 compute is accepted at RMS error <= 1e-2 x RMS(reference); float32 compute at max-abs <= 2e-4 and
RMS <= 5e-5 x RMS(reference) -- the tolerances of tests/test_gpu_parity.py.
"""
import pytest
import torch

import cases
from helpers import err_stats, load_golden
from test_gpu_parity import PRECISE_MAX_TOL, PRECISE_RMS_TOL, _check

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


def test_parcae_recurrence(dev):
    """z = a * z + Linear_b(LayerNorm(u)) with the discretised dynamics (model/model.py:272-277, :528)."""
    from kfold_b200.trunk import ParcaeRecurrence
    inp = cases.build_inputs("parcae_c128")
    gold = load_golden("parcae_c128")["out"]
    mod = ParcaeRecurrence(inp["case"]["c"]).to(dev)
    mod.load_state_dict(inp["w"], strict=True)
    out = mod(inp["z"].to(dev).bfloat16(), inp["u"].to(dev).bfloat16())
    assert out.dtype == torch.bfloat16 and out.shape == gold.shape
    _check(*err_stats(out.float().cpu(), gold), "parcae bf16")
    # float32 state under autocast(bfloat16): the trunk keeps z in float32 between iterations on request
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = mod(inp["z"].to(dev), inp["u"].to(dev))
    assert out.dtype == torch.float32
    _check(*err_stats(out.cpu(), gold), "parcae fp32 state")
    with pytest.raises(NotImplementedError):
        mod(inp["z"].to(dev), inp["u"].to(dev))
    # a parameter update is picked up (the dynamics are cached per parameter version)
    mod.parcae_log_a.add_(0.25)
    out2 = mod(inp["z"].to(dev).bfloat16(), inp["u"].to(dev).bfloat16())
    assert (out2.float() - out.float()).abs().max() > 1e-3


def test_lm_to_pair(dev):
    """LMToPair (model/model.py:114-134)."""
    from kfold_b200.trunk import LMToPair
    inp = cases.build_inputs("lm_to_pair")
    cs = inp["case"]
    gold = load_golden("lm_to_pair")["out"]
    mod = LMToPair(cs["c_s"], cs["c_z"]).to(dev)
    mod.load_state_dict(inp["w"], strict=True)
    out = mod(inp["s_lm"].to(dev).bfloat16())
    assert out.shape == gold.shape
    _check(*err_stats(out.float().cpu(), gold), "lm_to_pair bf16")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = mod(inp["s_lm"].to(dev))
    _check(*err_stats(out.float().cpu(), gold), "lm_to_pair autocast")


def test_pair_conditioning(dev):
    """PairConditioning (model/layers/folding/diffusion.py:45-94): float32 compute at float32 accuracy, bf16 compute and
    autocast within bf16 noise."""
    from kfold_b200.trunk import PairConditioning
    inp = cases.build_inputs("pair_conditioning")
    g = load_golden("pair_conditioning")
    gold, rel = g["out"], g["rel_pos_feats"].to(dev)
    mod = PairConditioning(inp["case"]["c_z"], rel.shape[-1]).to(dev)
    w = {k: v for k, v in inp["w"].items()}
    mod.load_state_dict(w, strict=True)
    out = mod(rel, inp["z"].to(dev))
    assert out.dtype == torch.float32
    mx, r = err_stats(out.cpu(), gold)
    assert mx < PRECISE_MAX_TOL and r < PRECISE_RMS_TOL, f"pair_conditioning fp32: {mx:.3e} {r:.3e}"
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = mod(rel, inp["z"].to(dev))
    _check(*err_stats(out.float().cpu(), gold), "pair_conditioning autocast")
    out = mod(rel.bfloat16(), inp["z"].to(dev).bfloat16())
    _check(*err_stats(out.float().cpu(), gold), "pair_conditioning bf16")
    # the reference's own call form: the FoldingInput instead of ready-made features (computed inside the kernel)
    import types
    f_input = types.SimpleNamespace(token=types.SimpleNamespace(**{k: inp[k].to(dev) for k in
                                                                   ("asym_id", "entity_id", "sym_id", "residue_index", "token_index")}))
    out2 = mod(f_input, inp["z"].to(dev))
    assert torch.equal(out2, mod(rel, inp["z"].to(dev)))
    mx, r = err_stats(out2.cpu(), gold)
    assert mx < PRECISE_MAX_TOL and r < PRECISE_RMS_TOL, f"pair_conditioning from token attributes: {mx:.3e} {r:.3e}"


def test_confidence_preparation_kernels(dev):
    """pair_outer_add and distogram_embed_add against plain torch, both dtypes, a ragged L."""
    from kfold_b200 import functional as F
    g = torch.Generator().manual_seed(11)
    b, l, c, bins = 2, 37, 128, 39
    z = torch.randn(b, l, l, c, generator=g).to(dev)
    r, q = torch.randn(b, l, c, generator=g).to(dev), torch.randn(b, l, c, generator=g).to(dev)
    x = (torch.randn(b, l, 3, generator=g) * 9.0).to(dev)
    bd = torch.linspace(3.25, 50.75, bins - 1, device=dev)
    w_t = torch.randn(bins, c, generator=g).to(dev)
    ref = z + r[:, None, :, :] + q[:, :, None, :]
    assert torch.equal(F.pair_outer_add(z, r, q), ref)
    d = (x[:, :, None] - x[:, None, :]).norm(dim=-1)
    idx = (d[..., None] > bd).sum(-1)
    ref = z + w_t[idx]
    got = F.distogram_embed_add(z, x, bd, w_t)
    # a distance within float rounding of a boundary may fall either side: allow a handful of pairs to differ
    bad = ((got - ref).abs().amax(-1) > 0).sum().item()
    assert bad <= 2, bad
    zb = z.bfloat16()
    got = F.pair_outer_add(zb, r.bfloat16(), q.bfloat16()).float()
    ref = zb.float() + r.bfloat16().float()[:, None] + q.bfloat16().float()[:, :, None]
    assert (got - ref).abs().max() <= 2 ** -6 * ref.abs().max()
    got = F.distogram_embed_add(zb, x, bd, w_t.bfloat16()).float()
    ref = zb.float() + w_t.bfloat16().float()[idx]
    assert ((got - ref.bfloat16().float()).abs().amax(-1) > 0).sum().item() <= 2


def test_confidence_head_against_reference_golden(dev):
    """ConfidenceHead.prepare + forward_single per sample (model/modules/confidence_head.py:343-378, :413-470) against
    the reference's own class run in float32: 2 blocks, 2 samples, 24 tokens of which 21 valid.  The head computes in bf16
    (the reference runs it under autocast(bfloat16)); logits are compared on the valid tokens."""
    from kfold_b200.confidence import ConfidenceHead
    inp = cases.build_inputs("confidence_head")
    cs = inp["case"]
    gold = load_golden("confidence_head")
    head = ConfidenceHead(cs["c_s"], cs["c_z"], cs["heads"], cs["blocks"]).to(dev)
    head.load_state_dict(inp["w"], strict=True)
    mask = inp["mask"].to(dev)
    args = [inp[k].to(dev) for k in ("s_inputs", "s_lm", "z", "x_repr")]
    v = cs["valid"]
    for label, call in (("bf16", lambda: head.forward_samples(*[a.bfloat16() if i < 3 else a for i, a in enumerate(args)], mask)),
                        ("autocast", None)):
        if call is None:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = head.forward_samples(*args, mask)
        else:
            out = call()
        for k in ("pae_logits", "pde_logits"):
            assert out[k].dtype == torch.float32 and out[k].shape == gold[k].shape
            _check(*err_stats(out[k][:, :, :v, :v].cpu(), gold[k][:, :, :v, :v]), f"confidence {k} {label}")
        for k in ("plddt_logits", "resolved_logits"):
            assert out[k].shape == gold[k].shape
            _check(*err_stats(out[k][:, :, :v].cpu(), gold[k][:, :, :v]), f"confidence {k} {label}")
    with pytest.raises(NotImplementedError):
        head.forward_samples(*args, mask)
