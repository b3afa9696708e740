"""GPU parity of the sampler loop: the coordinate-space kernels against the oracle, the production form of the score
network's step and the whole loop against golden vectors produced by the real reference (KFoldECSI.sample_structure with
its normal draws read from a tape).

Tolerances: float32 compute must reproduce the reference's final coordinates to an RMSD of 1e-3 Angstrom; bfloat16 compute
is held to the bound stated for the full sampler, RMSD <= 0.05 Angstrom.
"""
import types

import pytest
import torch

import cases
from helpers import err_stats, load_golden
from oracle import pairformer_oracle as O
from oracle import sampler_oracle as SO
from test_gpu_parity import PRECISE_MAX_TOL, PRECISE_RMS_TOL, _check

pytestmark = pytest.mark.gpu

RMSD_FP32 = 1e-3
RMSD_BF16 = 0.05


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _no_grad_and_status():
    from kfold_b200 import _lib as L
    with torch.no_grad():
        yield
    assert L.device_status() == 0


def _rmsd(a: torch.Tensor, b: torch.Tensor, mask: torch.Tensor) -> float:
    d = (a.double().cpu() - b.double().cpu()).pow(2).sum(-1)[..., mask.reshape(-1).cpu()]
    return float(d.mean().sqrt())


def test_coordinate_kernels_against_the_oracle(dev):
    """Random augmentation, rigid alignment (full and rotation only) and centring on 3 x 4 coordinate sets of 333 atoms with
    a padding tail, against the oracle's restatement of the reference functions (SVD-based Kabsch there, quaternion here)."""
    from kfold_b200 import functional as F
    tape = SO.NoiseTape(77)
    b, n, l = 3, 4, 333
    mask = torch.ones(b, 1, l, dtype=torch.bool)
    mask[0, :, 300:] = False
    mask[2, :, 17:] = False
    x = tape.randn((b, n, l, 3)) * 9.0 + 3.0
    y = tape.randn((b, n, l, 3)) * 9.0 - 1.0
    # augmentation with the same normals on both sides
    t1, t2 = SO.NoiseTape(5), SO.NoiseTape(5)
    ref = SO.random_augmentation([x, y], mask, t1)
    from kfold_b200.sampler import CenterRandomAugmentation
    got = CenterRandomAugmentation()(x.to(dev), y.to(dev), mask=mask.to(dev), rng=t2)
    for g, r in zip(got, ref):
        assert err_stats(g, r)[0] < 1e-5
    assert t1.calls == t2.calls == 2
    # alignment of a rotated, shifted, noisy copy back onto the original
    (moved,) = SO.random_augmentation([x], mask, SO.NoiseTape(6))
    moved = moved + tape.randn((b, n, l, 3)) * 0.3
    for rot_only in (False, True):
        ref = SO.custom_rigid_align(moved, x, mask, rotation_only=rot_only)
        got = F.rigid_align(moved.to(dev), x.to(dev), mask.to(dev), rotation_only=rot_only)
        assert err_stats(got, ref)[0] < 2e-5, f"rigid_align rotation_only={rot_only}"
    assert err_stats(F.center_coords(x.to(dev), mask.to(dev)), SO.do_centering(x, mask))[0] < 1e-6
    # the fused update against its parts
    ru = tape.randn((b, n, l, 3))
    noise = tape.randn((b, n, l, 3))
    c_skip, c_out, coef = 0.37, 4.2, (0.9, 0.05, 0.03, 0.7)
    x0 = SO.do_centering(SO.custom_rigid_align(c_skip * x + c_out * ru, x, mask, rotation_only=True), mask)
    ref = coef[0] * x + coef[1] * x0 + coef[2] * y + coef[3] * noise.masked_fill(~mask[..., None], 0.0)
    got, got_x0 = F.sampler_update(x.to(dev), ru.to(dev), y.to(dev), mask.to(dev), c_skip, c_out, coef, noise=noise.to(dev),
                                   return_x0=True)
    assert err_stats(got_x0, x0)[0] < 2e-5 and err_stats(got, ref)[0] < 2e-5


def _stack_for(cs, dev, w):
    from kfold_b200 import modules as M
    mod = M.DiffusionStack(channel_a=cs["c_a"], channel_s=cs["c_s"], channel_z=cs["c_z"], channel_atom=cs["c_atom"],
                           channel_atompair=cs["c_pair"], channel_coords=cs.get("coords", 3),
                           separate_endpoint_atom_encoder=cs.get("separate_endpoint", False),
                           atom_encoder_blocks=cs["atom_blocks"], atom_encoder_heads=cs["atom_heads"],
                           token_transformer_blocks=cs["token_blocks"], token_transformer_heads=cs["token_heads"],
                           atom_decoder_blocks=cs["atom_blocks"], atom_decoder_heads=cs["atom_heads"]).to(dev)
    missing, unexpected = mod.load_state_dict(w, strict=False)
    assert not unexpected, unexpected
    return mod, missing


def test_production_form_of_the_step_against_reference_golden(dev):
    """DiffusionStack.step with six coordinate channels split between two atom encoders (configs/kfold.yaml:61-76) against
    the output of the reference class: float32 compute at float32 accuracy, bfloat16 compute within bf16 noise."""
    inp = cases.build_inputs("diffusion_step_sep")
    gold = load_golden("diffusion_step_sep")["out"]
    mod, missing = _stack_for(inp["case"], dev, inp["w"])
    assert all(k.startswith(("single_conditioning.", "layernorm_z.", "linear_z_to_bias.")) for k in missing)
    args = [inp[k].to(dev) for k in ("r_noisy", "q", "c", "p", "token_index", "atom_mask", "s", "pair_bias", "token_mask")]
    out = mod.step(*args)
    mx, r = err_stats(out.cpu(), gold)
    assert out.dtype == torch.float32 and mx < PRECISE_MAX_TOL and r < PRECISE_RMS_TOL, f"{mx:.3e} {r:.3e}"
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out = mod.step(*args)
    _check(*err_stats(out.cpu(), gold), "separate-endpoint step, bf16")


def _sampler_inputs(dev):
    inp = cases.build_inputs("sampler_small")
    gold = load_golden("sampler_small")
    cs = inp["case"]
    mod, _ = _stack_for(cs, dev, inp["w"])
    atom = types.SimpleNamespace(pad_mask=inp["atom_mask"].to(dev), token_index=inp["token_index"].to(dev),
                                 prior_coords=inp["x_apo"].permute(0, 2, 1, 3).contiguous().to(dev))
    token = types.SimpleNamespace(pad_mask=inp["token_mask"].to(dev))
    f_input = types.SimpleNamespace(atom=atom, token=token)
    pre = {k: gold[k].to(dev) for k in ("q", "c", "p", "pair_bias")}
    return inp, gold, cs, mod, f_input, pre


def test_sampler_loop_against_reference_golden(dev):
    """KFoldECSI.sample_structure (6 steps: churn + ECSI SDE, SDE, SI ODE; 2 samples) with the normals of the tape the
    reference consumed: same number of draws, final coordinates within 1e-3 Angstrom in float32 compute and within
    0.05 Angstrom in bfloat16 compute; the CUDA-graph replay of the network equals the eager loop."""
    from kfold_b200.sampler import KFoldECSI
    inp, gold, cs, mod, f_input, pre = _sampler_inputs(dev)
    sampler = KFoldECSI(KFoldECSI.Config(), mod)
    assert sampler.get_sampling_schedule(cs["steps"]) == SO.sampling_schedule(SO.DEFAULTS, cs["steps"])
    s_in = inp["s_inputs"].to(dev)
    tape = SO.NoiseTape(cs["tape"])
    out = sampler.sample_structure(f_input, s_in, None, num_steps=cs["steps"], num_samples=cs["samples"], precomputed=pre, rng=tape)
    assert tape.calls == int(gold["draws"])
    assert err_stats(out["init_coordinates"].cpu(), gold["x_T"])[0] < 1e-5
    r32 = _rmsd(out["coordinates"], gold["coordinates"], inp["atom_mask"])
    assert r32 < RMSD_FP32, f"float32 compute: RMSD {r32:.3e} A"
    pad = ~inp["atom_mask"].reshape(-1)
    assert (out["coordinates"].cpu()[..., pad, :] == 0).all()
    res = {}
    for graph in (False, True):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            o = sampler.sample_structure(f_input, s_in, None, num_steps=cs["steps"], num_samples=cs["samples"], precomputed=pre,
                                         rng=SO.NoiseTape(cs["tape"]), cuda_graph=graph)
        res[graph] = o["coordinates"].clone()
    rb = _rmsd(res[False], gold["coordinates"], inp["atom_mask"])
    print(f"sampler RMSD vs the reference: float32 compute {r32:.2e} A, bfloat16 compute {rb:.2e} A")
    assert rb < RMSD_BF16, f"bfloat16 compute: RMSD {rb:.3e} A"
    assert torch.equal(res[False], res[True])


def test_sampler_default_generator_is_reproducible(dev):
    """Without an injected source the normals come from the device generator: the same seed gives the same structure."""
    from kfold_b200.sampler import KFoldECSI
    inp, gold, cs, mod, f_input, pre = _sampler_inputs(dev)
    sampler = KFoldECSI(KFoldECSI.Config(), mod)
    outs = []
    for _ in range(2):
        torch.manual_seed(1234)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            outs.append(sampler.sample_structure(f_input, inp["s_inputs"].to(dev), None, num_steps=4, num_samples=3,
                                                 precomputed=pre)["coordinates"].clone())
    assert torch.equal(outs[0], outs[1]) and torch.isfinite(outs[0]).all()
