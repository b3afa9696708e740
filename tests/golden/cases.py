"""The list of golden cases: which reference module, which sizes, which seed.

Shared by ``make_golden.py`` (runs the real reference) and by the tests (run the
oracle / the CUDA path on the same seeded inputs and compare with the stored
reference output).  Inputs and weights are regenerated from the seed with
``kfold_b200.synth``; only reference *outputs* are stored.
"""
from __future__ import annotations

import numpy as np
import torch

import synth

# pair outputs with N >= 48 are stored as out[:, ::SUB_STRIDE, ::SUB_STRIDE] plus checksums
SUB_STRIDE = 3

# name -> dict(kind=..., seed=..., dims...)
CASES = {
    # triangle multiplication: ragged N with a padding tail, and batch>1 with a general block mask
    "trimul_out_n24": dict(kind="trimul", direction="outgoing", seed=11, n=24, c=128, batch=1, valid=20),
    "trimul_in_n24": dict(kind="trimul", direction="incoming", seed=12, n=24, c=128, batch=1, valid=20),
    "trimul_out_b2": dict(kind="trimul", direction="outgoing", seed=13, n=16, c=128, batch=2, blockmask=True),
    "trimul_in_b2": dict(kind="trimul", direction="incoming", seed=14, n=16, c=128, batch=2, blockmask=True),
    "trimul_out_n64": dict(kind="trimul", direction="outgoing", seed=15, n=64, c=128, batch=1, valid=58),
    "trimul_in_n64": dict(kind="trimul", direction="incoming", seed=16, n=64, c=128, batch=1, valid=58),
    # production trunk width (configs/kfold.yaml:2-3, channel_z 256) and the apo stack's width (configs/kfold.yaml:15-20)
    "trimul_out_c256": dict(kind="trimul", direction="outgoing", seed=17, n=24, c=256, batch=1, valid=21),
    "trimul_in_c256": dict(kind="trimul", direction="incoming", seed=18, n=24, c=256, batch=1, valid=21),
    "trimul_out_c64": dict(kind="trimul", direction="outgoing", seed=19, n=32, c=64, batch=2, blockmask=True),
    "trimul_in_c64": dict(kind="trimul", direction="incoming", seed=20, n=32, c=64, batch=2, blockmask=True),
    # triangle attention
    "triatt_start_n24": dict(kind="triatt", starting=True, seed=21, n=24, c=128, heads=4, batch=1, valid=20),
    "triatt_end_n24": dict(kind="triatt", starting=False, seed=22, n=24, c=128, heads=4, batch=1, valid=20),
    "triatt_start_b2": dict(kind="triatt", starting=True, seed=23, n=16, c=128, heads=4, batch=2, blockmask=True),
    "triatt_end_b2": dict(kind="triatt", starting=False, seed=24, n=16, c=128, heads=4, batch=2, blockmask=True),
    "triatt_start_n64": dict(kind="triatt", starting=True, seed=25, n=64, c=128, heads=4, batch=1, valid=58),
    "triatt_end_n64": dict(kind="triatt", starting=False, seed=26, n=64, c=128, heads=4, batch=1, valid=58),
    "triatt_start_c64": dict(kind="triatt", starting=True, seed=27, n=32, c=64, heads=4, batch=1, valid=30),
    # pair-bias attention (single track, LayerNorm prologue) and diffusion form (AdaLN + shared bias)
    "apb_single": dict(kind="apb", seed=31, l=40, c=384, heads=16, c_s=None, batch=1, samples=1, valid=36),
    "apb_diffusion": dict(kind="apb", seed=32, l=24, c=768, heads=16, c_s=384, batch=1, samples=3, valid=20),
    # transitions
    "transition_pair": dict(kind="transition", seed=41, rows=96, c=128, factor=4),
    "transition_single": dict(kind="transition", seed=42, rows=40, c=384, factor=4),
    "cond_transition": dict(kind="cond_transition", seed=43, rows=24, c=768, c_s=384, samples=2),
    # two blocks of the diffusion token transformer (AdaLN attention + conditioned transition), shared bias over 3 samples
    "diffusion_stack": dict(kind="diffusion_stack", seed=44, l=24, c=768, c_s=384, heads=16, blocks=2, samples=3, valid=20),
    # atom-level local transformer: 3 blocks over 5 windows of 32 atoms (keys: 128 per window), 2 samples sharing z and s
    "local_stack": dict(kind="local_stack", seed=45, l=160, c=128, c_s=128, c_z=16, heads=4, blocks=3, samples=2, valid=150),
    # token <-> atom maps: 40 tokens, 160 atoms (1 to 8 atoms per token, one token without atoms), 2 samples
    "atom_token_maps": dict(kind="atom_token_maps", seed=46, tokens=40, atoms=160, d=96, samples=2, valid=150),
    # atom attention encoder (with coordinate embedding) and decoder around a 2-block local transformer: 96 atoms, 24 tokens
    "atom_encoder": dict(kind="atom_encoder", seed=47, tokens=24, atoms=96, c=128, c_z=16, c_token=256, heads=4, blocks=2,
                         samples=2, valid=90),
    "atom_decoder": dict(kind="atom_decoder", seed=48, tokens=24, atoms=96, c=128, c_z=16, c_token=256, heads=4, blocks=2,
                         samples=2, valid=90),
    # single conditioning of the sampler: 40 tokens, 3 noise levels
    "single_conditioning": dict(kind="single_conditioning", seed=49, l=40, c_s=384, dim_fourier=256, samples=3),
    # DiffusionStack.step: encoder (2 blocks) -> token transformer (2 blocks) -> decoder (2 blocks); 24 tokens, 96 atoms, 2 samples
    "diffusion_step": dict(kind="diffusion_step", seed=50, tokens=24, atoms=96, c_a=256, c_s=384, c_z=128, c_atom=128, c_pair=16,
                           atom_blocks=2, atom_heads=4, token_blocks=2, token_heads=8, samples=2, valid_atoms=90, valid_tokens=23),
    # the production form of the step (configs/kfold.yaml:61-76): six coordinate channels [c_in x_t | x_T / sigma_T], split
    # between two atom encoders whose token streams are normalised, concatenated and fused by a float32 Linear
    "diffusion_step_sep": dict(kind="diffusion_step", seed=52, tokens=24, atoms=96, c_a=256, c_s=384, c_z=128, c_atom=128, c_pair=16,
                               atom_blocks=2, atom_heads=4, token_blocks=2, token_heads=8, samples=2, valid_atoms=90, valid_tokens=23,
                               coords=6, separate_endpoint=True),
    # the sampler loop around the step (model/modules/ecsi.py:498-560): 6 steps, 2 samples, 16 tokens, 64 atoms, every normal
    # draw taken from a tape (seed in `tape`): steps 0-2 churn + ECSI SDE, step 3 SDE, steps 4-5 SI ODE
    "sampler_small": dict(kind="sampler", seed=53, tape=5301, tokens=16, atoms=64, priors=2, c_a=256, c_s=384, c_z=128, c_atom=128,
                          c_pair=16, atom_blocks=1, atom_heads=4, token_blocks=2, token_heads=8, samples=2, steps=6, valid_atoms=60,
                          valid_tokens=15, coords=6),
    # callers of the pair stacks in the trunk (model/model.py:114-134, :523-529) and the diffusion module's pair conditioning
    "parcae_c128": dict(kind="parcae", seed=54, n=24, c=128),
    "lm_to_pair": dict(kind="lm_to_pair", seed=55, l=24, c_s=256, c_z=128),
    "pair_conditioning": dict(kind="pair_conditioning", seed=56, l=24, c_z=128),
    # confidence head: z / s preparation, then forward_single for each of 2 samples (2 blocks, 24 tokens, 21 valid)
    "confidence_head": dict(kind="confidence_head", seed=57, l=24, c_s=384, c_z=128, heads=16, blocks=2, samples=2, valid=21),
    # layer norm
    "layernorm_c128": dict(kind="layernorm", seed=51, rows=50, c=128),
    # composite block: benchmark config 1 (N=64, fp32, all-ones mask, seed 0) and a padded N=32 one
    "block_cfg1_n64": dict(kind="block", seed=0, n=64, c_z=128, c_s=384, valid=64),
    "block_n32": dict(kind="block", seed=5, n=32, c_z=128, c_s=384, valid=28),
    # K-Fold's own trunk block (tri-mult out + in + transition x4), at the production width and at the benchmark's
    "tri_block_c256": dict(kind="tri_block", seed=6, n=24, c_z=256, valid=21),
    "tri_block_c128": dict(kind="tri_block", seed=7, n=40, c_z=128, valid=36),
}


def build_inputs(name: str) -> dict:
    """Seeded inputs + weights of one case (all float32 / bool CPU tensors)."""
    cs = CASES[name]
    kind, seed = cs["kind"], cs["seed"]
    rng = synth._Rng(seed)
    out: dict = {"case": cs}
    if kind in ("trimul", "triatt"):
        x, pm, _ = synth.pair_inputs(seed, cs["n"], cs["c"], cs["batch"], valid=cs.get("valid"))
        if cs.get("blockmask"):
            pm = synth.block_mask(seed, cs["batch"], cs["n"])
        out["x"], out["mask"] = x, pm
        out["w"] = synth.trimul_weights(rng, cs["c"]) if kind == "trimul" else synth.triatt_weights(rng, cs["c"], cs["heads"])
    elif kind == "apb":
        l, c, h = cs["l"], cs["c"], cs["heads"]
        out["w"] = synth.apb_weights(rng, c, cs["c_s"])
        out["a"] = rng.normal(cs["batch"], cs["samples"], l, c)
        out["s"] = None if cs["c_s"] is None else rng.normal(cs["batch"], 1, l, cs["c_s"])
        out["pair_bias"] = rng.normal(cs["batch"], 1, h, l, l)
        out["mask"] = synth.token_mask(l, cs["valid"]).view(1, 1, l).expand(cs["batch"], 1, l).contiguous()
    elif kind == "transition":
        out["w"] = synth.transition_weights(rng, cs["c"], cs["factor"])
        out["x"] = rng.normal(cs["rows"], cs["c"])
    elif kind == "cond_transition":
        out["w"] = synth.conditioned_transition_weights(rng, cs["c"], cs["c_s"])
        out["a"] = rng.normal(1, cs["samples"], cs["rows"], cs["c"])
        out["s"] = rng.normal(1, 1, cs["rows"], cs["c_s"])
    elif kind == "diffusion_stack":
        w = {}
        for i in range(cs["blocks"]):
            w.update(synth._prefixed(f"blocks.{i}.attention", synth.apb_weights(rng, cs["c"], cs["c_s"])))
            w.update(synth._prefixed(f"blocks.{i}.transition", synth.conditioned_transition_weights(rng, cs["c"], cs["c_s"])))
        out["w"] = w
        out["a"] = rng.normal(1, cs["samples"], cs["l"], cs["c"])
        out["s"] = rng.normal(1, 1, cs["l"], cs["c_s"])
        out["pair_bias"] = rng.normal(1, cs["blocks"], cs["heads"], cs["l"], cs["l"])
        out["mask"] = synth.token_mask(cs["l"], cs["valid"]).view(1, 1, cs["l"]).contiguous()
    elif kind == "local_stack":
        l, w_ = cs["l"], cs["l"] // 32
        out["w"] = synth.local_stack_weights(rng, cs["c"], cs["c_s"], cs["c_z"], cs["heads"], cs["blocks"])
        out["a"] = rng.normal(1, cs["samples"], l, cs["c"])
        out["s"] = rng.normal(1, 1, l, cs["c_s"])
        out["z"] = rng.normal(1, 1, w_, 32, 128, cs["c_z"])
        out["mask"] = synth.token_mask(l, cs["valid"]).view(1, 1, l).contiguous()
    elif kind == "atom_token_maps":
        nt, na = cs["tokens"], cs["atoms"]
        # atoms sorted by token, token nt - 2 left without atoms, sizes 1..8
        sizes = rng.rs.randint(1, 9, size=nt)
        sizes[nt - 2] = 0
        index = np.repeat(np.arange(nt), sizes)[:na]
        index = np.concatenate([index, np.full(na - len(index), nt - 1)]).astype(np.int64)
        out["token_index"] = torch.from_numpy(index).view(1, 1, na)
        out["mask"] = synth.token_mask(na, cs["valid"]).view(1, 1, na)
        out["x_token"] = rng.normal(1, cs["samples"], nt, cs["d"])
        out["x_atom"] = rng.normal(1, cs["samples"], na, cs["d"])
    elif kind in ("atom_encoder", "atom_decoder"):
        nt, na, c = cs["tokens"], cs["atoms"], cs["c"]
        index = np.sort(rng.rs.randint(0, nt, size=na)).astype(np.int64)
        out["token_index"] = torch.from_numpy(index).view(1, 1, na)
        out["mask"] = synth.token_mask(na, cs["valid"]).view(1, 1, na)
        out["c"] = rng.normal(1, 1, na, c)
        out["p"] = rng.normal(1, 1, na // 32, 32, 128, cs["c_z"])
        if kind == "atom_encoder":
            out["w"] = synth.atom_encoder_weights(rng, c, cs["c_z"], cs["c_token"], cs["heads"], cs["blocks"], True)
            out["q"] = rng.normal(1, 1, na, c)
            out["r_noisy"] = rng.normal(1, cs["samples"], na, 3) * 4.0
        else:
            out["w"] = synth.atom_decoder_weights(rng, cs["c_token"], c, cs["c_z"], cs["heads"], cs["blocks"])
            out["a"] = rng.normal(1, cs["samples"], nt, cs["c_token"])
            out["q_skip"] = rng.normal(1, cs["samples"], na, c)
    elif kind == "single_conditioning":
        out["w"] = synth.single_conditioning_weights(rng, cs["c_s"], cs["dim_fourier"])
        out["s_inputs"] = rng.normal(1, cs["l"], cs["c_s"])
        out["c_noise"] = rng.normal(1, cs["samples"]) * 1.5       # 1/4 log(t_hat / sigma_data) spans about +-2
    elif kind == "diffusion_step":
        nt, na, ns = cs["tokens"], cs["atoms"], cs["samples"]
        out["w"] = synth.diffusion_step_weights(rng, cs["c_a"], cs["c_s"], cs["c_atom"], cs["c_pair"], cs["atom_blocks"],
                                                cs["atom_heads"], cs["token_blocks"], cs["token_heads"], cs.get("coords", 3),
                                                cs.get("separate_endpoint", False))
        out["r_noisy"] = rng.normal(1, ns, na, cs.get("coords", 3)) * 4.0
        out["q"], out["c"] = rng.normal(1, na, cs["c_atom"]), rng.normal(1, na, cs["c_atom"])
        out["p"] = rng.normal(1, na // 32, 32, 128, cs["c_pair"])
        out["token_index"] = torch.from_numpy(np.sort(rng.rs.randint(0, cs["valid_tokens"], size=na)).astype(np.int64)).view(1, na)
        out["atom_mask"] = synth.token_mask(na, cs["valid_atoms"]).view(1, na)
        out["s"] = rng.normal(1, ns, nt, cs["c_s"])
        out["pair_bias"] = rng.normal(1, cs["token_blocks"], cs["token_heads"], nt, nt)
        out["token_mask"] = synth.token_mask(nt, cs["valid_tokens"]).view(1, nt)
    elif kind == "sampler":
        nt, na = cs["tokens"], cs["atoms"]
        out["w"] = synth.diffusion_step_weights(rng, cs["c_a"], cs["c_s"], cs["c_atom"], cs["c_pair"], cs["atom_blocks"],
                                                cs["atom_heads"], cs["token_blocks"], cs["token_heads"], cs["coords"], False)
        out["w"].update(synth._prefixed("single_conditioning", synth.single_conditioning_weights(rng, cs["c_s"], 256)))
        out["x_apo"] = rng.normal(1, cs["priors"], na, 3) * 8.0                       # (B, Nprior, La, 3)
        out["s_inputs"] = rng.normal(1, nt, cs["c_s"])
        out["z"] = rng.normal(1, nt, nt, cs["c_z"])
        out["token_index"] = torch.from_numpy(np.sort(rng.rs.randint(0, cs["valid_tokens"], size=na)).astype(np.int64)).view(1, na)
        out["atom_mask"] = synth.token_mask(na, cs["valid_atoms"]).view(1, na)
        out["token_mask"] = synth.token_mask(nt, cs["valid_tokens"]).view(1, nt)
        # the remaining fields of the duck-typed FoldingInput the reference's embedders read (reference-side only)
        out["ref_pos"] = rng.normal(1, na, 3) * 2.0
        out["ref_charge"] = torch.from_numpy(rng.rs.randint(-1, 2, size=(1, na)).astype(np.float32))
        out["ref_element"] = torch.nn.functional.one_hot(torch.from_numpy(rng.rs.randint(0, 20, size=(1, na))), 128).float()
        out["ref_atom_name_chars"] = torch.nn.functional.one_hot(torch.from_numpy(rng.rs.randint(0, 64, size=(1, na, 4))), 64).float()
        out["ref_space_uid"] = out["token_index"].clone()
    elif kind == "parcae":
        out["w"] = synth.parcae_weights(rng, cs["c"])
        out["z"] = rng.normal(1, cs["n"], cs["n"], cs["c"])
        out["u"] = rng.normal(1, cs["n"], cs["n"], cs["c"]) * 2.0 + 0.5
    elif kind == "lm_to_pair":
        out["w"] = synth.lm_to_pair_weights(rng, cs["c_s"], cs["c_z"])
        out["s_lm"] = rng.normal(1, cs["l"], cs["c_s"])
    elif kind == "pair_conditioning":
        l = cs["l"]
        out["w"] = synth.pair_conditioning_weights(rng, cs["c_z"])
        out["z"] = rng.normal(1, l, l, cs["c_z"])
        # two chains (12 + 12 tokens) of one entity, the second a symmetric copy: every relative-position feature is exercised
        half = l // 2
        out["asym_id"] = torch.cat([torch.zeros(half), torch.ones(l - half)]).long().view(1, l)
        out["entity_id"] = torch.zeros(1, l, dtype=torch.long)
        out["sym_id"] = out["asym_id"].clone()
        out["residue_index"] = torch.cat([torch.arange(half), torch.arange(l - half)]).view(1, l)
        out["token_index"] = torch.arange(l).view(1, l)
    elif kind == "confidence_head":
        l = cs["l"]
        out["w"] = synth.confidence_head_weights(rng, cs["c_s"], cs["c_z"], cs["heads"], cs["blocks"])
        out["s_inputs"], out["s_lm"] = rng.normal(1, l, cs["c_s"]), rng.normal(1, l, cs["c_s"])
        out["z"] = rng.normal(1, l, l, cs["c_z"])
        out["x_repr"] = rng.normal(1, cs["samples"], l, 3) * 9.0          # pairwise distances span the 3.25 .. 50.75 A bins
        out["mask"] = synth.token_mask(l, cs["valid"]).view(1, l)
    elif kind == "layernorm":
        out["x"] = rng.normal(cs["rows"], cs["c"]) * 3.0 + 1.5
        out["w"] = {"weight": rng.ln_w(cs["c"]), "bias": rng.ln_b(cs["c"])}
    elif kind == "block":
        z, pm, m = synth.pair_inputs(seed, cs["n"], cs["c_z"], 1, valid=cs["valid"])
        out["z"], out["pair_mask"], out["mask"] = z, pm, m
        out["s"] = synth.single_inputs(seed, cs["n"], cs["c_s"], 1)
        out["w"] = synth.pairformer_block_weights(seed, cs["c_z"], cs["c_s"])
    elif kind == "tri_block":
        z, pm, _ = synth.pair_inputs(seed, cs["n"], cs["c_z"], 1, valid=cs["valid"])
        out["z"], out["pair_mask"] = z, pm
        out["w"] = synth.triangular_block_weights(seed, cs["c_z"])
    else:
        raise ValueError(kind)
    return out
