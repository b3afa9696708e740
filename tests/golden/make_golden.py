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
                                channel_atompair=cs["c_pair"], atom_encoder_blocks=cs["atom_blocks"],
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
