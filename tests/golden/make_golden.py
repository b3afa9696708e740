"""Generate tests/golden/*.npz by running the REAL K-Fold reference modules.

Run in a container where the reference source tree is present:

    python tests/golden/make_golden.py

For every case in ``cases.py`` the reference module (torch backend, CPU, fp32,
eval mode, no grad) is instantiated at the case's sizes, loaded with the seeded
synthetic weights via ``load_state_dict(strict=True)``, run on the seeded inputs,
and its output stored.  The composite Pairformer block has no single reference
class; it is assembled here from reference modules only, in the order of
``PairformerBlock.forward`` (model/modules/apo_module.py:145-172) followed by the
single track of ``ConfidencePairSingleBlock.forward``
(model/modules/confidence_head.py:152-175).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))          # tests/: synth.py

import cases  # noqa: E402
import ref_shim  # noqa: E402
from oracle.pairformer_oracle import sub  # noqa: E402  (prefix helper only)


def _load(mod, w):
    mod.load_state_dict(w, strict=True)
    return mod.eval()


@torch.no_grad()
def run_reference(ns, name: str) -> dict:
    inp = cases.build_inputs(name)
    cs = inp["case"]
    kind = cs["kind"]
    if kind == "trimul":
        cls = ns.TriangleMultiplicationOutgoing if cs["direction"] == "outgoing" else ns.TriangleMultiplicationIncoming
        return {"out": _load(cls(cs["c"]), inp["w"])(inp["x"], inp["mask"])}
    if kind == "triatt":
        cls = ns.TriangleAttentionStartingNode if cs["starting"] else ns.TriangleAttentionEndingNode
        return {"out": _load(cls(cs["c"], cs["heads"]), inp["w"])(inp["x"], inp["mask"])}
    if kind == "apb":
        site = "confidence" if cs["c_s"] is None else "diffusion_global"
        mod = _load(ns.SelfAttentionPairBias(cs["c"], cs["heads"], cs["c_s"], site, kernel_backend="torch"), inp["w"])
        return {"out": mod(inp["a"], inp["s"], inp["pair_bias"], inp["mask"])}
    if kind == "transition":
        return {"out": _load(ns.Transition(cs["c"], cs["factor"]), inp["w"])(inp["x"])}
    if kind == "cond_transition":
        import importlib
        dt = importlib.import_module("kfold.model.layers.folding.diffusion_transformer")
        return {"out": _load(dt.ConditionedTransitionBlock(cs["c"], cs["c_s"]), inp["w"])(inp["a"], inp["s"])}
    if kind == "diffusion_stack":
        import importlib
        dt = importlib.import_module("kfold.model.layers.folding.diffusion_transformer")
        stack = dt.CachedGlobalTransformerStack(cs["c"], cs["c_s"], cs["heads"], cs["blocks"])
        for blk in stack.blocks:
            blk.attention.kernel_backend = "torch"      # the oracle path; the constructor hard-codes "sdpa"
        _load(stack, inp["w"])
        return {"out": stack(inp["a"].clone(), inp["s"], inp["pair_bias"], inp["mask"])}
    if kind == "local_stack":
        import importlib
        dt = importlib.import_module("kfold.model.layers.folding.diffusion_transformer")
        stack = dt.LocalTransformerStack(cs["c"], cs["c_s"], cs["c_z"], cs["heads"], cs["blocks"])
        for blk in stack.blocks:
            blk.attention.kernel_backend = "torch"      # the oracle path; the constructor hard-codes "sdpa"
        _load(stack, inp["w"])
        return {"out": stack(inp["a"].clone(), inp["s"], inp["z"], inp["mask"])}
    if kind == "atom_token_maps":
        import importlib
        ut = importlib.import_module("kfold.model.layers.folding.utils")
        idx = inp["token_index"].expand(1, cs["samples"], cs["atoms"])
        return {"atoms": ut.broadcast_tokens_to_atoms(inp["x_token"], idx),
                "tokens": ut.aggregate_atoms_to_tokens(inp["x_atom"], idx, inp["mask"].expand_as(idx), cs["tokens"])}
    if kind in ("atom_encoder", "atom_decoder"):
        import importlib
        at = importlib.import_module("kfold.model.layers.folding.atom_transformer")
        if kind == "atom_encoder":
            mod = at.AtomAttentionEncoder(cs["c"], cs["c_z"], cs["c_token"], num_blocks=cs["blocks"], num_heads=cs["heads"],
                                          use_structure=True)
        else:
            mod = at.AtomAttentionDecoder(cs["c_token"], cs["c"], cs["c_z"], num_blocks=cs["blocks"], num_heads=cs["heads"])
        for blk in mod.transformer.blocks:
            blk.attention.kernel_backend = "torch"      # the oracle path; the constructor hard-codes "sdpa"
        _load(mod, inp["w"])
        if kind == "atom_encoder":
            a, q_skip, _, _ = mod(inp["q"], inp["c"], inp["p"], inp["token_index"], inp["mask"], cs["tokens"], inp["r_noisy"])
            return {"a": a, "q_skip": q_skip}
        return {"out": mod(inp["a"], inp["q_skip"].clone(), inp["c"], inp["p"], inp["token_index"], inp["mask"])}
    if kind == "single_conditioning":
        import importlib
        df = importlib.import_module("kfold.model.layers.folding.diffusion")
        mod = _load(df.SingleConditioning(cs["c_s"], cs["dim_fourier"]), inp["w"])
        return {"out": mod(inp["s_inputs"], inp["c_noise"]), "fourier_w": mod.fourier_embed.w, "fourier_b": mod.fourier_embed.b}
    if kind == "diffusion_step":
        import importlib
        df = importlib.import_module("kfold.model.layers.folding.diffusion")
        mod = df.DiffusionStack(channel_a=cs["c_a"], channel_s=cs["c_s"], channel_z=cs["c_z"], channel_atom=cs["c_atom"],
                                channel_atompair=cs["c_pair"], channel_coords=cs.get("coords", 3),
                                separate_endpoint_atom_encoder=cs.get("separate_endpoint", False),
                                atom_encoder_blocks=cs["atom_blocks"],
                                atom_encoder_heads=cs["atom_heads"], token_transformer_blocks=cs["token_blocks"],
                                token_transformer_heads=cs["token_heads"], atom_decoder_blocks=cs["atom_blocks"],
                                atom_decoder_heads=cs["atom_heads"], kernel_backend="torch")
        missing, unexpected = mod.load_state_dict(inp["w"], strict=False)   # the time-independent parts are not used by step()
        assert not unexpected, unexpected
        mod.eval()
        for m in mod.modules():
            if getattr(m, "kernel_backend", None) == "sdpa":
                m.kernel_backend = "torch"      # the oracle path; the constructors hard-code "sdpa"
        return {"out": mod.step(inp["r_noisy"], inp["q"], inp["c"], inp["p"], inp["token_index"], inp["atom_mask"], inp["s"],
                                inp["pair_bias"], inp["token_mask"])}
    if kind == "sampler":
        return run_reference_sampler(inp)
    if kind == "confidence_head":
        import importlib
        ch = importlib.import_module("kfold.model.modules.confidence_head")
        head = ch.ConfidenceHead(ch.ConfidenceHead.Config(channel_s=cs["c_s"], channel_z=cs["c_z"], num_heads_attn=cs["heads"],
                                                          num_blocks=cs["blocks"]), kernel_backend="torch")
        _load(head, inp["w"])
        for m in head.modules():
            if getattr(m, "kernel_backend", None) == "sdpa":
                m.kernel_backend = "torch"      # the oracle path; the constructor hard-codes "sdpa"
        # the part of ConfidenceHead.forward between the representative-atom gather and the atom-layout scatter
        # (model/modules/confidence_head.py:343-378), float32
        s = head.s_lm_to_s(inp["s_lm"])
        z = inp["z"] + head.linear_s1(inp["s_inputs"])[..., None, :, :] + head.linear_s2(inp["s_inputs"])[..., :, None, :]
        outs = [head.forward_single(z, s, inp["x_repr"][:, i], mask=inp["mask"]) for i in range(cs["samples"])]
        names = ("pae_logits", "pde_logits", "plddt_logits", "resolved_logits")
        return {n: torch.stack([o[k] for o in outs], dim=1) for k, n in enumerate(names)}
    if kind == "parcae":
        import types
        model = ref_shim.load_reference_model()
        w = inp["w"]
        holder = types.SimpleNamespace(parcae_log_a=w["parcae_log_a"], parcae_log_delta=w["parcae_log_delta"],
                                       parcae_b_cont=w["parcae_b_cont"])
        a, b = model.KFold._parcae_discretized_dynamics(holder)          # model/model.py:272-277
        ln = _load(ns.LayerNorm(cs["c"]), sub(w, "layernorm_z"))
        return {"out": a * inp["z"] + torch.nn.functional.linear(ln(inp["u"]), b)}   # model/model.py:528
    if kind == "lm_to_pair":
        model = ref_shim.load_reference_model()
        return {"out": _load(model.LMToPair(cs["c_s"], cs["c_z"]), inp["w"])(inp["s_lm"])}
    if kind == "pair_conditioning":
        import importlib
        import types
        df = importlib.import_module("kfold.model.layers.folding.diffusion")
        mod = _load(df.PairConditioning(cs["c_z"]), inp["w"])
        token = types.SimpleNamespace(**{k: inp[k] for k in ("asym_id", "entity_id", "sym_id", "residue_index", "token_index")})
        f_input = types.SimpleNamespace(token=token)
        rel = mod.rel_pos_encoding(f_input, torch.float32)
        return {"out": mod(f_input, inp["z"].clone()), "rel_pos_feats": rel}
    if kind == "layernorm":
        return {"out": _load(ns.LayerNorm(cs["c"]), inp["w"])(inp["x"])}
    if kind == "tri_block":
        import importlib
        ts = importlib.import_module("kfold.model.modules.tri_stack")
        return {"out": _load(ts.TriangularBlock(cs["c_z"], kernel_backend="torch"), inp["w"])(inp["z"].clone(), inp["pair_mask"])}
    if kind == "block":
        z, s = ref_shim.build_reference_block(ns, inp["w"], cs["c_z"], cs["c_s"])(
            inp["z"].clone(), inp["s"].clone(), inp["pair_mask"], inp["mask"])
        res = {"s": s, "z_sum": z.double().sum().reshape(1), "z_sumsq": (z.double() ** 2).sum().reshape(1)}
        if cs["n"] > 32:
            res["z_sub"] = z[:, ::cases.SUB_STRIDE, ::cases.SUB_STRIDE].contiguous()
        else:
            res["z"] = z
        return res
    raise ValueError(kind)


class _TapeRandn:
    """Stands in for torch.randn / torch.randn_like while the reference sampler runs: every draw comes from the tape."""

    def __init__(self, tape):
        self.tape = tape

    def randn(self, *size, dtype=None, device=None, generator=None, **kw):
        if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
            size = tuple(size[0])
        return self.tape.randn(size).to(dtype or torch.float32)

    def randn_like(self, t, **kw):
        return self.tape.randn(tuple(t.shape)).to(t.dtype)


@torch.no_grad()
def run_reference_sampler(inp: dict) -> dict:
    """``KFoldECSI.sample_structure`` (model/modules/ecsi.py:468-560) of the real reference on a duck-typed FoldingInput,
    its normal draws taken from a NoiseTape.  Stored besides the final coordinates: what the time-independent precompute
    of the reference (pair conditioning, atom embedder -- not part of the accelerated path) hands to the loop."""
    import importlib
    import types

    from oracle.sampler_oracle import NoiseTape
    cs = inp["case"]
    sm = importlib.import_module("kfold.model.modules.score_model")
    ecsi = importlib.import_module("kfold.model.modules.ecsi")
    cfg = sm.DiffusionModule.Config(channel_a=cs["c_a"], channel_s=cs["c_s"], channel_z=cs["c_z"], channel_atom=cs["c_atom"],
                                    channel_atompair=cs["c_pair"], channel_coords=cs["coords"],
                                    atom_encoder_blocks=cs["atom_blocks"], atom_encoder_heads=cs["atom_heads"],
                                    token_transformer_blocks=cs["token_blocks"], token_transformer_heads=cs["token_heads"],
                                    atom_decoder_blocks=cs["atom_blocks"], atom_decoder_heads=cs["atom_heads"])
    model = sm.DiffusionModule(cfg, kernel_backend="torch")
    # the reference-only parts (pair conditioning, atom embedder) get seeded random weights: zero-initialised ones would
    # make their outputs trivial
    rs = np.random.RandomState(cs["seed"] + 1000)
    for name, prm in sorted(model.named_parameters()):
        if prm.dim() >= 2:
            prm.copy_(torch.from_numpy((rs.standard_normal(tuple(prm.shape)) * prm.shape[-1] ** -0.5).astype(np.float32)))
    missing, unexpected = model.diffusion_stack.load_state_dict(inp["w"], strict=False)
    assert not unexpected, unexpected
    model.eval()
    for m in model.modules():
        if getattr(m, "kernel_backend", None) == "sdpa":
            m.kernel_backend = "torch"
    atom = types.SimpleNamespace(pad_mask=inp["atom_mask"], token_index=inp["token_index"],
                                 prior_coords=inp["x_apo"].permute(0, 2, 1, 3).contiguous(), ref_pos=inp["ref_pos"],
                                 ref_charge=inp["ref_charge"], ref_element=inp["ref_element"],
                                 ref_atom_name_chars=inp["ref_atom_name_chars"], ref_space_uid=inp["ref_space_uid"])
    nt = cs["tokens"]
    ar = torch.arange(nt).view(1, nt)
    token = types.SimpleNamespace(pad_mask=inp["token_mask"], asym_id=torch.zeros(1, nt, dtype=torch.long),
                                  entity_id=torch.zeros(1, nt, dtype=torch.long), sym_id=torch.zeros(1, nt, dtype=torch.long),
                                  residue_index=ar.clone(), token_index=ar.clone())
    f_input = types.SimpleNamespace(atom=atom, token=token, num_atoms=cs["atoms"], device=torch.device("cpu"))
    z_cond = model.get_pair_conditioning(f_input, inp["z"])
    q, c, p = model.get_atom_embeddings(f_input, z_cond)
    pair_bias = model.get_pair_bias(z_cond)
    sampler = ecsi.KFoldECSI(ecsi.KFoldECSI.Config(), model)
    stand_in = _TapeRandn(NoiseTape(cs["tape"]))
    real_randn, real_randn_like = torch.randn, torch.randn_like
    torch.randn, torch.randn_like = stand_in.randn, stand_in.randn_like
    try:
        out = sampler.sample_structure(f_input, inp["s_inputs"], inp["z"], num_steps=cs["steps"], num_samples=cs["samples"])
    finally:
        torch.randn, torch.randn_like = real_randn, real_randn_like
    return {"q": q, "c": c, "p": p, "pair_bias": pair_bias, "x_T": out["init_coordinates"], "coordinates": out["coordinates"],
            "draws": torch.tensor([stand_in.tape.calls])}


def _thin(res: dict) -> dict:
    """Keep big pair outputs small: a strided sample plus float64 checksums."""
    out = res.get("out")
    if out is not None and out.dim() == 4 and out.shape[1] >= 48:
        return {"out_sub": out[:, ::cases.SUB_STRIDE, ::cases.SUB_STRIDE].contiguous(),
                "out_sum": out.double().sum().reshape(1),
                "out_sumsq": (out.double() ** 2).sum().reshape(1)}
    return res


def main() -> None:
    ns = ref_shim.load_reference()
    torch.manual_seed(0)
    for name in cases.CASES:
        res = _thin(run_reference(ns, name))
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **{k: v.detach().cpu().numpy() for k, v in res.items()})
        print(f"{name}: " + ", ".join(f"{k}{tuple(v.shape)}" for k, v in res.items()),
              f"-> {os.path.getsize(path) / 1024:.0f} KB")


if __name__ == "__main__":
    main()
