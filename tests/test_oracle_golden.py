"""The CPU oracle against the golden vectors produced by the real reference modules."""
import pytest
import torch

import cases
from helpers import compare_pair_output, err_stats, load_golden
from oracle import pairformer_oracle as O

FP32_TOL = 2e-5  # max-abs / RMS(ref); both sides are fp32 CPU, only op order differs


def run_oracle(name: str, mode: str = "fp32") -> dict:
    inp = cases.build_inputs(name)
    cs, w = inp["case"], inp.get("w")
    kind = cs["kind"]
    if kind == "trimul":
        return {"out": O.triangle_multiplication(inp["x"], inp["mask"], w, cs["direction"], mode)}
    if kind == "triatt":
        return {"out": O.triangle_attention(inp["x"], inp["mask"], w, cs["heads"], cs["starting"], mode)}
    if kind == "apb":
        return {"out": O.self_attention_pair_bias(inp["a"], inp["s"], inp["pair_bias"], inp["mask"], w, cs["heads"], mode)}
    if kind == "transition":
        return {"out": O.transition(inp["x"], w, mode)}
    if kind == "cond_transition":
        return {"out": O.conditioned_transition(inp["a"], inp["s"], w, mode)}
    if kind == "diffusion_stack":
        return {"out": O.global_transformer_stack(inp["a"], inp["s"], inp["pair_bias"], inp["mask"], w, cs["heads"],
                                                  cs["blocks"], mode)}
    if kind == "local_stack":
        return {"out": O.local_transformer_stack(inp["a"], inp["s"], inp["z"], inp["mask"], w, cs["heads"], cs["blocks"], mode)}
    if kind == "atom_token_maps":
        idx = inp["token_index"].expand(1, cs["samples"], cs["atoms"])
        return {"atoms": O.broadcast_tokens_to_atoms(inp["x_token"], idx),
                "tokens": O.aggregate_atoms_to_tokens(inp["x_atom"], idx, inp["mask"].expand_as(idx), cs["tokens"])}
    if kind == "atom_encoder":
        a, q_skip = O.atom_attention_encoder(inp["q"], inp["c"], inp["p"], inp["token_index"], inp["mask"], cs["tokens"],
                                             inp["r_noisy"], w, cs["heads"], cs["blocks"], mode)
        return {"a": a, "q_skip": q_skip}
    if kind == "atom_decoder":
        return {"out": O.atom_attention_decoder(inp["a"], inp["q_skip"], inp["c"], inp["p"], inp["token_index"], inp["mask"], w,
                                                cs["heads"], cs["blocks"], mode)}
    if kind == "single_conditioning":
        return {"out": O.single_conditioning(inp["s_inputs"], inp["c_noise"], w, mode)}
    if kind == "diffusion_step":
        return {"out": O.diffusion_step(inp["r_noisy"], inp["q"], inp["c"], inp["p"], inp["token_index"], inp["atom_mask"], inp["s"],
                                        inp["pair_bias"], inp["token_mask"], w, cs["atom_heads"], cs["atom_blocks"],
                                        cs["token_heads"], cs["token_blocks"], mode)}
    if kind == "sampler":
        from oracle import sampler_oracle as SO
        gold = load_golden(name)
        step = SO.diffusion_step_fn(gold["q"], gold["c"], gold["p"], inp["token_index"], inp["atom_mask"], gold["pair_bias"],
                                    inp["token_mask"], w, cs["atom_heads"], cs["atom_blocks"], cs["token_heads"],
                                    cs["token_blocks"], mode)
        tape = SO.NoiseTape(cs["tape"])
        x_T, x = SO.sample_loop(inp["x_apo"], inp["atom_mask"], step, inp["s_inputs"], cs["steps"], cs["samples"], tape,
                                single_conditioning=lambda s_in, cn: O.single_conditioning(s_in, cn, O.sub(w, "single_conditioning"), mode))
        return {"x_T": x_T, "coordinates": x, "draws": torch.tensor([tape.calls])}
    if kind == "confidence_head":
        return O.confidence_head(inp["s_inputs"], inp["s_lm"], inp["z"], inp["x_repr"], inp["mask"], w, cs["heads"], cs["blocks"], mode)
    if kind == "parcae":
        return {"out": O.parcae_update(inp["z"], inp["u"], w, mode)}
    if kind == "lm_to_pair":
        return {"out": O.lm_to_pair(inp["s_lm"], w, mode)}
    if kind == "pair_conditioning":
        return {"out": O.pair_conditioning(load_golden(name)["rel_pos_feats"], inp["z"], w, mode)}
    if kind == "layernorm":
        return {"out": O.layer_norm(inp["x"], w["weight"], w["bias"], 1e-5, mode)}
    if kind == "tri_block":
        return {"out": O.triangular_block(inp["z"], inp["pair_mask"], w, mode)}
    if kind == "block":
        z, s = O.pairformer_block(inp["z"], inp["s"], inp["pair_mask"], inp["mask"], w, mode=mode)
        return {"z": z, "s": s}
    raise ValueError(kind)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_oracle_matches_reference_golden(name):
    gold = load_golden(name)
    got = run_oracle(name)
    if cases.CASES[name]["kind"] == "block":
        assert err_stats(got["s"], gold["s"])[0] < 5 * FP32_TOL
        assert compare_pair_output(got["z"], gold, "z")[0] < 5 * FP32_TOL
        zs = float(got["z"].double().sum())
        assert abs(zs - float(gold["z_sum"])) <= 1e-3 * float(gold["z_sumsq"]) ** 0.5
    elif cases.CASES[name]["kind"] == "sampler":
        # same tape, same number of draws, same coordinates: the restated loop consumes the normals in the reference's order
        assert int(got["draws"]) == int(gold["draws"])
        assert err_stats(got["x_T"], gold["x_T"])[0] < FP32_TOL
        d = (got["coordinates"] - gold["coordinates"]).pow(2).sum(-1)
        rmsd = float(d.mean().sqrt())
        assert rmsd < 1e-3, f"sampler: coordinate RMSD {rmsd:.3e} A between the oracle and the reference"
    elif cases.CASES[name]["kind"] == "confidence_head":
        for k in ("pae_logits", "pde_logits", "plddt_logits", "resolved_logits"):
            assert err_stats(got[k], gold[k])[0] < 5 * FP32_TOL, k
    elif cases.CASES[name]["kind"] == "atom_encoder":
        assert err_stats(got["a"], gold["a"])[0] < FP32_TOL and err_stats(got["q_skip"], gold["q_skip"])[0] < FP32_TOL
    elif cases.CASES[name]["kind"] == "atom_token_maps":
        assert torch.equal(got["atoms"], gold["atoms"])                 # a gather: exact
        assert err_stats(got["tokens"], gold["tokens"])[0] < FP32_TOL
        assert (got["tokens"][..., cases.CASES[name]["tokens"] - 2, :] == 0).all()   # the token without atoms
    else:
        out = got["out"]
        if out.dim() == 4 and ("out" not in gold):
            mx, _ = compare_pair_output(out, gold)
            assert abs(float(out.double().sum()) - float(gold["out_sum"])) <= 1e-3 * float(gold["out_sumsq"]) ** 0.5
        else:
            mx, _ = err_stats(out, gold["out"])
        assert mx < FP32_TOL, f"{name}: max-abs/RMS {mx:.3e}"


@pytest.mark.parametrize("name", ["trimul_out_n24", "triatt_start_n24", "transition_pair", "apb_single"])
def test_oracle_bf16_mode_is_within_bf16_noise(name):
    """bf16-emulating mode stays within the reference's own bf16-vs-fp32 noise (RMS error < 2e-2 RMS)."""
    gold = load_golden(name)
    inp_mode = run_oracle(name, "bf16")["out"]
    _, r = err_stats(inp_mode, gold["out"])
    assert r < 2e-2
    assert r > 1e-4  # it really rounds
