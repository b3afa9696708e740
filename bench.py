"""Benchmark of the hot path: one composite Pairformer block forward at N=768, bf16.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_triton]

One step = one forward of the AF3-shaped Pairformer block (triangle multiplication out/in,
triangle attention start/end, pair transition, single-track pair-bias attention, single
transition) on synthetic z ~ N(0,1) (1,768,768,128), s ~ N(0,1) (1,768,384), 10 % padding tail,
random-init weights -- the unit the headline metric "Pairformer-block fwd ms @N=768 bf16" names.

With N > 1 ranks (launched by torch.distributed.run) every rank runs its own block on its own
GPU -- independent complexes, the way the reference distributes work across GPUs
(src/kfold/cli/multigpu.py:22-77) -- with no data-path collective; `value` is then the
whole-job time per block (step time / blocks processed by all ranks).

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):   # synth.py, ref_shim.py
    if _p not in sys.path:
        sys.path.insert(0, _p)

N_TOKENS = 768
N_TOKENS_DEFAULT = 768
C_Z, C_S = 128, 384
PAD_FRAC = 0.1
SEED = 3
METRIC = "pairformer_block_fwd_ms_n768_bf16"


# ------------------------------------------------------------------------------------------------
# algorithmic work per launch tag at N=768, C=128 (2 flops per multiply-add; bf16 bytes, each tensor touched once)
# ------------------------------------------------------------------------------------------------
def algorithmic_work(n: int | None = None, c: int = C_Z, h: int = 4, cs: int = C_S, hs: int = 16) -> dict:
    n = N_TOKENS if n is None else n
    p = n * n
    d = c // h
    return {
        # tensor-bound kernels: flops per launch
        "trimul_contraction": ("tensor", 2.0 * n * n * n * c),
        "triatt_attention": ("tensor", 4.0 * n * n * n * h * d),
        # the pair transition (hidden = 4c): 0.23 TFLOP against 755 MB / 906 MB of traffic: the HBM floor is the higher one
        "transition_swiglu": ("hbm", 1.0 * p * c * 2 + 1.0 * p * 4 * c * 2),       # read x~, write the hidden
        "transition_out": ("hbm", 1.0 * p * 4 * c * 2 + 2.0 * p * c * 2),          # read the hidden and the residual, write out
        "apb_proj": ("tensor", 2.0 * n * cs * 4 * cs),
        "apb_attention": ("tensor", 4.0 * n * n * cs),
        "apb_out_proj": ("tensor", 2.0 * n * cs * cs),
        # HBM-bound kernels: bytes per launch (every tensor read or written once, bf16).  The K = c projections do
        # 8 tensor-core instructions per 128-row tile: their time is the traffic of the tensors around them.
        # (8 launches per block share this tag: 6 over the pair tensor and 2 over the single track; the figures of the
        # pair-sized ones are reported)
        "layernorm_rows": ("hbm", 2.0 * p * c * 2),
        "layernorm_cm": ("hbm", 2.0 * p * c * 2),
        "layernorm_cm_stats": ("hbm", 1.0 * p * c * 2 + p * 8),   # read t, write (mean, rstd) per position
        "trimul_in_proj": ("hbm", 3.0 * p * c * 2),            # read x~, write a and b
        "trimul_gate_proj": ("hbm", 2.0 * p * c * 2),          # read x~, write the gate logits
        "trimul_out_proj": ("hbm", 4.0 * p * c * 2),           # read LN(t), gate logits, residual; write out
        "triatt_proj": ("hbm", 5.0 * p * c * 2 + p * h * 2),   # read x~; write q, k, g, v^T and the bias
        "triatt_out_proj": ("hbm", 3.0 * p * c * 2),           # read gated o, residual; write out
        "pair_bias_proj": ("hbm", p * c * 2 + p * hs * 2),
    }


# DRAM traffic of the triangle-attention kernel from its ncu capture at N=384 (dram__bytes_read.sum +
# dram__bytes_write.sum of one launch: 144.9 MB + 23.9 MB); it grows with the number of pair positions.
NCU_TRAFFIC = {"triatt_attention": {"n": 384, "bytes": 144.919040e6 + 23.904512e6,
                                     "source": "ncu capture at N=384 scaled by pair positions (profiles/triatt_attention_n384_ncu.md)"}}


def ncu_traffic(tag: str, n: int):
    ent = NCU_TRAFFIC.get(tag)
    if ent is None:
        return None
    return round(ent["bytes"] * (n / ent["n"]) ** 2)


def load_peaks() -> dict:
    """Roofline denominators: the copy bandwidth and the two cuBLAS bf16 figures measured on this pool's B200s (burst =
    a kernel timed alone at the full SM clock, sustained = inside a seconds-long loop under the power cap)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops_burst": d["bf16_tflops"],
                "tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def pick_tensor_peak(peaks: dict, region_s: float, clocks: dict) -> tuple[float, str]:
    """Which bf16 peak a timed region is compared with: the burst figure when the region is short (under a second) and the
    sampled SM clock sat at its maximum, the sustained one otherwise."""
    sm, smax = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
    at_max = sm is not None and smax is not None and sm >= 0.97 * smax
    if region_s < 1.0 and at_max:
        return peaks["tflops_burst"], "burst"
    return peaks["tflops_sustained"], "sustained"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the two timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.strip().split(", ") for r in open(self.path).read().splitlines() if r.strip()]
            os.unlink(self.path)
            sm = [float(r[0]) for r in rows if len(r) >= 6]
            if sm:
                out["sm_mhz"] = statistics.median(sm)
                out["sm_max_mhz"] = float(rows[0][1])
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                out["reasons"] = [nm for i, nm in enumerate(names) if any(r[2 + i].strip() == "Active" for r in rows if len(r) >= 6)]
                out["samples"] = len(sm)
        except Exception:
            pass
        return out


def make_inputs():
    import synth
    z, pm, m = synth.pair_inputs(SEED, N_TOKENS, C_Z, 1, pad_frac=PAD_FRAC)
    s = synth.single_inputs(SEED, N_TOKENS, C_S, 1)
    w = synth.pairformer_block_weights(SEED, C_Z, C_S)
    return z, s, pm, m, w


def config_dict(n_gpus: int, sharded_mode: bool = False) -> dict:
    return {
        "workload": f"composite Pairformer block forward (BASELINE config 4's block): N_token={N_TOKENS}, c_z=128, c_s=384, "
                    "tri-mult out+in, tri-att start+end (4x32), transition x4, single pair-bias attention (16x24), transition x4",
        "n_token": N_TOKENS, "c_z": C_Z, "c_s": C_S, "padding_tail": PAD_FRAC, "seed": SEED,
        "blocks_per_step": 1 if sharded_mode else n_gpus,
        "parallelism": ("one pair tensor row-sharded over the GPUs: all-gather for triangle multiplication and the "
                        "triangle bias, all-to-all transposes for the incoming / ending-node operators") if sharded_mode
        else ("independent blocks, one per GPU, no collective" if n_gpus > 1 else "single GPU"),
        "l2": "not flushed between steps: the pair tensor alone (151 MB bf16) and every intermediate exceed the 126 MB L2",
    }


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own torch modules on the host cores (the oracle port where the reference is absent)
# ------------------------------------------------------------------------------------------------
def cpu_block_runner(n: int):
    """-> (run, kind, what): `run()` executes one composite block at `n` tokens in float32 on the CPU and returns nothing.
    kind "reference": the block assembled from the reference's own modules (kernel_backend="torch"), imported from the
    installed copy under baseline/_ref; kind "port": the oracle's restatement, when no reference copy is on the machine."""
    import synth
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    z, pm, m = synth.pair_inputs(SEED, n, C_Z, 1, pad_frac=PAD_FRAC)
    s = synth.single_inputs(SEED, n, C_S, 1)
    w = synth.pairformer_block_weights(SEED, C_Z, C_S)
    try:
        import ref_shim
        block = ref_shim.build_reference_block(ref_shim.load_reference(), w, C_Z, C_S)

        def run():
            block(z.clone(), s.clone(), pm, m)      # the reference adds in place

        return run, "reference", f"the reference's torch modules (float32, kernel_backend=\"torch\", {cores} threads)", cores
    except Exception as exc:      # no reference copy on this machine
        from oracle import pairformer_oracle as O
        why = f"{type(exc).__name__}: {exc}"

        def run():
            with torch.no_grad():
                O.pairformer_block(z, s, pm, m, w, row_chunk=64)

        return run, "port", f"CPU port of the reference torch path (float32, {cores} threads; reference not importable: {why})", cores


def time_cpu_block(run, repeats: int, warmup: int) -> list:
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        run()
        dt = (time.perf_counter() - t0) * 1e3
        if i >= warmup:
            times.append(dt)
    return times


def block_flops(n: int, c: int = C_Z, h: int = 4, cs: int = C_S, hs: int = 16) -> float:
    """Algorithmic flops of one composite block (2 per multiply-add), every GEMM and both attention cores."""
    p = n * n
    d = c // h
    trimul = 2.0 * n * n * n * c + 2.0 * p * c * 4 * c + 2 * (2.0 * p * c * c)
    triatt = 2.0 * p * c * (4 * c + h) + 4.0 * n * n * n * h * d + 2.0 * p * c * c
    transition_z = 2.0 * p * c * 8 * c + 2.0 * p * 4 * c * c
    single = 2.0 * p * c * hs + 2.0 * n * cs * 4 * cs + 4.0 * n * n * cs + 2.0 * n * cs * cs + 2.0 * n * cs * 12 * cs
    return 2 * trimul + 2 * triatt + transition_z + single


# The reference arm runs the block at the benchmark's own size.  One block takes several seconds on the host cores, so the
# arm bounds its run time by the NUMBER of steps it measures, never by the work per step: at most this many seconds of
# measured steps (at least two), after one warm-up step; the line reports the steps and warm-ups actually done.
REFERENCE_BUDGET_S = 120.0


def run_reference_arm(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    run, kind, what, cores = cpu_block_runner(N_TOKENS)
    # warm-up steps as asked, cut short once they have taken 30 s
    warm, t0 = 0, time.perf_counter()
    while warm < args.warmup and (warm == 0 or time.perf_counter() - t0 < 30.0):
        run()
        warm += 1
    first = time.perf_counter() - t0
    times = []
    while len(times) < args.steps and (len(times) < 2 or sum(times) / 1e3 + (times[-1] / 1e3) < REFERENCE_BUDGET_S):
        times += time_cpu_block(run, 1, 0)
    value = sum(times) / len(times)
    sample = (f"{what}: one block at N={N_TOKENS} per step, {len(times)} measured steps of {args.steps} asked "
              f"(run time bounded at {REFERENCE_BUDGET_S:.0f} s of measured steps), {warm} warm-up steps of {args.warmup} asked"
              + (f" ({first:.1f} s)" if warm else ""))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "ms", "n_gpus": args.gpus, "steps": len(times),
        "warmup": warm, "steps_requested": args.steps, "warmup_requested": args.warmup, "ms_per_step": value,
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config_dict(1),
        "cpu_baseline": {"value": value, "unit": "ms", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def run_reference_triton_arm(args, rank: int) -> None:
    """Report only (not the headline): the reference's GPU incumbent, its Triton backend, on this GPU.  The four pair
    operators of the block at N=768 through the reference's own modules with kernel_backend="triton" (stock code path,
    bf16 under autocast, as its inference runs them), each timed with CUDA events.  Any failure to import, JIT or run
    prints the `unavailable` line with the message."""
    if rank != 0:
        return
    try:
        import ref_shim
        import synth
        ns = ref_shim.load_reference()
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        z, pm, _ = synth.pair_inputs(SEED, N_TOKENS, C_Z, 1, pad_frac=PAD_FRAC)
        w = synth.pairformer_block_weights(SEED, C_Z, C_S)
        zd, pmd = z.to(dev, torch.bfloat16), pm.to(dev)
        mods = {}
        for name, cls, extra in (("tri_mul_out", ns.TriangleMultiplicationOutgoing, ()), ("tri_mul_in", ns.TriangleMultiplicationIncoming, ()),
                                 ("tri_att_start", ns.TriangleAttentionStartingNode, (4,)), ("tri_att_end", ns.TriangleAttentionEndingNode, (4,))):
            mod = cls(C_Z, *extra, kernel_backend="triton")
            mod.load_state_dict(ref_shim._sub(w, name), strict=True)
            mods[name] = mod.to(dev).eval()
        stream = torch.cuda.current_stream()
        per_op = {}
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            for name, mod in mods.items():
                for _ in range(max(args.warmup, 3)):      # the first call JIT-compiles (and autotunes) the kernels
                    mod(zd, pmd)
                per_op[name] = round(_event_time(lambda: mod(zd, pmd), args.steps, stream, torch.cuda.synchronize), 4)
        total = sum(per_op.values())
        emit({"impl": "reference_triton", "metric": "pair_operators_fwd_ms_n768_bf16", "value": total, "unit": "ms", "n_gpus": 1,
              "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": total, "higher_is_better": False, "dtype": "bf16",
              "data": "synthetic", "per_op_ms": per_op,
              "config": {"workload": "the reference's Triton backend: tri-mult out + in, tri-att start + end, N_token=768, c_z=128, "
                                     "4 heads x 32; updates only (no residual add, no transition, no single track)"},
              "note": "report only: a GPU anchor for the per-operator numbers, not the block metric"})
    except Exception as exc:      # Triton refused to JIT, or the reference copy did not travel
        emit({"impl": "reference_triton", "unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"})


# ------------------------------------------------------------------------------------------------
# optional second workload (--diffusion-step): one pass of the sampler's token transformer of benchmark config 4
# (24 conditioned blocks, c=768, 16 heads x 48, L=768 tokens, 5 samples sharing the pair bias), bf16 compute.
# Not the headline metric; printed as its own JSON line when asked for.
# ------------------------------------------------------------------------------------------------
def run_diffusion_step(args) -> None:
    from kfold_b200 import _lib as L
    from kfold_b200 import modules as M
    import synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    blocks, l, ns, c, cs, heads = 24, N_TOKENS, 5, 768, 384, 16
    rng = synth._Rng(SEED)
    w = {}
    for i in range(blocks):
        w.update(synth._prefixed(f"blocks.{i}.attention", synth.apb_weights(rng, c, cs)))
        w.update(synth._prefixed(f"blocks.{i}.transition", synth.conditioned_transition_weights(rng, c, cs)))
    a = rng.normal(1, ns, l, c).to(dev)
    s = rng.normal(1, 1, l, cs).to(dev)
    bias = rng.normal(1, blocks, heads, l, l).to(dev)
    mask = synth.token_mask(l, pad_frac=PAD_FRAC).view(1, 1, l).to(dev)
    stack = M.CachedGlobalTransformerStack(c, cs, heads, blocks).to(dev)
    stack.load_state_dict(w, strict=True)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for _ in range(max(args.warmup, 3)):
            stack(a, s, bias, mask)
        torch.cuda.synchronize()
        launches0 = L.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            stack(a, s, bias, mask)
        e1.record()
        torch.cuda.synchronize()
        launches_per_step = (L.launch_count() - launches0) // max(args.steps, 1)
        ms_eager = e0.elapsed_time(e1) / args.steps
        # the same pass captured once into a CUDA graph and replayed: the 24 x ~9 launches are issued by the driver
        # without the Python layer in between (the library allocates nothing and never synchronises)
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            stack(a, s, bias, mask)
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            out_g = stack(a, s, bias, mask)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_graph = e0.elapsed_time(e1) / args.steps
        graph_ok = bool(torch.isfinite(out_g.float()).all())
    ms = min(ms_eager, ms_graph) if graph_ok else ms_eager
    # per block: projections 4 c^2 + c^2, AdaLN / gate projections of the conditioning (per token, not per sample),
    # attention 4 L c per row, conditioned transition 3 * 2c * c
    rows = ns * l
    flops = blocks * (2.0 * rows * c * 5 * c + 4.0 * ns * l * l * c + 2.0 * rows * c * 6 * c + 2.0 * l * cs * 6 * c)
    emit({"metric": f"diffusion_token_transformer_step_ms_l{l}_s{ns}_bf16", "value": ms, "unit": "ms", "n_gpus": 1,
          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
          "config": {"workload": f"sampler token transformer (BASELINE config 4): {blocks} blocks, c={c}, {heads} heads, "
                                 f"L={l}, {ns} samples sharing the pair bias, one pass = one sampler step"},
          "tflops": round(flops / (ms * 1e-3) / 1e12, 1), "gpu_launches": launches_per_step * args.steps,
          "ms_eager": round(ms_eager, 3), "ms_cuda_graph": round(ms_graph, 3), "launches_per_step": launches_per_step,
          "device_status": L.device_status()})


# ------------------------------------------------------------------------------------------------
# optional third workload (--atom-step): one pass of an atom-level local transformer of benchmark config 4
# (3 blocks, 6 016 atoms = 188 windows of 32 queries x 128 keys, c=128, 4 heads x 32, pair channels 16, 5 samples
# sharing the window pair tensor and the conditioning), bf16 compute.  Its own JSON line.
# ------------------------------------------------------------------------------------------------
def run_atom_step(args) -> None:
    from kfold_b200 import _lib as L
    from kfold_b200 import modules as M
    import synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    blocks, l, ns, c, c_z, heads = 3, 6016, 5, 128, 16, 4
    rng = synth._Rng(SEED)
    w = synth.local_stack_weights(rng, c, c, c_z, heads, blocks)
    a = rng.normal(1, ns, l, c).to(dev)
    s = rng.normal(1, 1, l, c).to(dev)
    z = rng.normal(1, 1, l // 32, 32, 128, c_z).to(dev)
    mask = synth.token_mask(l, pad_frac=0.02).view(1, 1, l).to(dev)
    stack = M.LocalTransformerStack(c, c, c_z, heads, blocks).to(dev)
    stack.load_state_dict(w, strict=True)
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for _ in range(max(args.warmup, 3)):
            stack(a, s, z, mask)
        torch.cuda.synchronize()
        L.profile_enable(True)
        launches0 = L.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            stack(a, s, z, mask)
        e1.record()
        torch.cuda.synchronize()
        launches_per_step = (L.launch_count() - launches0) // max(args.steps, 1)
        prof = L.profile_report()
        L.profile_enable(False)
        ms_eager = e0.elapsed_time(e1) / args.steps
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            stack(a, s, z, mask)
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            out_g = stack(a, s, z, mask)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_graph = e0.elapsed_time(e1) / args.steps
        graph_ok = bool(torch.isfinite(out_g.float()).all())
    ms = min(ms_eager, ms_graph) if graph_ok else ms_eager
    kernels = {tag: {"launches": cnt, "avg_ms": round(t / cnt, 5)} for tag, (cnt, t) in sorted(prof.items(), key=lambda kv: -kv[1][1])}
    emit({"metric": f"atom_local_transformer_pass_ms_l{l}_s{ns}_bf16", "value": ms, "unit": "ms", "n_gpus": 1,
          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
          "config": {"workload": f"atom-level local transformer (BASELINE config 4): {blocks} blocks, {l} atoms in windows of 32 "
                                 f"queries x 128 keys, c={c}, {heads} heads, {ns} samples sharing the window pair tensor"},
          "gpu_launches": launches_per_step * args.steps, "ms_eager": round(ms_eager, 3), "ms_cuda_graph": round(ms_graph, 3),
          "launches_per_step": launches_per_step, "kernels": kernels, "device_status": L.device_status()})


# ------------------------------------------------------------------------------------------------
# optional fourth workload (--sampler-step): one call of DiffusionStack.step at benchmark config 4's shape (atom attention
# encoder, 24-block token transformer, atom attention decoder; 768 tokens, 6 016 atoms, 5 samples), bf16 compute.
# ------------------------------------------------------------------------------------------------
def run_sampler_step(args) -> None:
    from kfold_b200 import _lib as L
    from kfold_b200 import modules as M
    import synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nt, na, ns = N_TOKENS, 6016, 5
    c_a, c_s, c_atom, c_pair, tb, th = 768, 384, 128, 16, 24, 16
    rng = synth._Rng(SEED)
    w = synth.diffusion_step_weights(rng, c_a, c_s, c_atom, c_pair, 3, 4, tb, th)
    mod = M.DiffusionStack(channel_a=c_a, channel_s=c_s, channel_z=128, channel_atom=c_atom, channel_atompair=c_pair,
                           token_transformer_blocks=tb, token_transformer_heads=th).to(dev)
    mod.load_state_dict(w, strict=False)
    r = (rng.normal(1, ns, na, 3) * 4.0).to(dev)
    q, c = rng.normal(1, na, c_atom).to(dev), rng.normal(1, na, c_atom).to(dev)
    p = rng.normal(1, na // 32, 32, 128, c_pair).to(dev)
    import numpy as np
    token_index = torch.from_numpy(np.sort(rng.rs.randint(0, nt, size=na)).astype(np.int64)).view(1, na).to(dev)
    atom_mask = synth.token_mask(na, pad_frac=0.02).view(1, na).to(dev)
    s = rng.normal(1, ns, nt, c_s).to(dev)
    pair_bias = rng.normal(1, tb, th, nt, nt).to(dev, torch.bfloat16)
    token_mask = synth.token_mask(nt, pad_frac=PAD_FRAC).view(1, nt).to(dev)

    def step():
        return mod.step(r, q, c, p, token_index, atom_mask, s, pair_bias, token_mask)

    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        L.profile_enable(True)
        launches0 = L.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        launches_per_step = (L.launch_count() - launches0) // max(args.steps, 1)
        prof = L.profile_report()
        L.profile_enable(False)
        ms_eager = e0.elapsed_time(e1) / args.steps
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            out_g = step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ms_graph = e0.elapsed_time(e1) / args.steps
        graph_ok = bool(torch.isfinite(out_g.float()).all())
    ms = min(ms_eager, ms_graph) if graph_ok else ms_eager
    top = sorted(prof.items(), key=lambda kv: -kv[1][1])[:8]
    emit({"metric": f"diffusion_stack_step_ms_l{nt}_a{na}_s{ns}_bf16", "value": ms, "unit": "ms", "n_gpus": 1,
          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": False,
          "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
          "config": {"workload": f"DiffusionStack.step (BASELINE config 4): atom encoder 3 blocks, token transformer {tb} blocks "
                                 f"c={c_a}, atom decoder 3 blocks; {nt} tokens, {na} atoms, {ns} samples; one call = one sampler step"},
          "gpu_launches": launches_per_step * args.steps, "ms_eager": round(ms_eager, 3), "ms_cuda_graph": round(ms_graph, 3),
          "launches_per_step": launches_per_step,
          "top_kernels": {tag: {"launches": cnt, "total_ms": round(t, 3)} for tag, (cnt, t) in top},
          "device_status": L.device_status()})


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def _event_time(fn, steps: int, stream, barrier) -> float:
    """ms per call of `fn`, CUDA events on `stream`, a barrier + device synchronisation on both sides."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    barrier()
    return e0.elapsed_time(e1) / steps


def _rel_rms(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).pow(2).mean().sqrt() / (b.pow(2).mean().sqrt() + 1e-30))


def sharded_bytes_out(n: int, c: int, h: int, cs: int, p: int, channel: bool) -> int:
    """Bytes one rank sends to its peers during one row-sharded block (bf16): the operand exchanges of the two triangle
    multiplications (incoming: always the channel form; outgoing: the channel form from four ranks on, else the all-gather
    of b), the two shard transposes of the ending-node operator, the gathered triangle biases and the gathered rows of the
    single track.  An all-gathered piece leaves the GPU once per peer."""
    shard = n * n * c * 2 // p                       # one rank's rows of a pair-sized tensor
    out_frac = (p - 1) / p
    channel_form = (2 * shard + shard) * out_frac    # a and b out, t back: all-to-all
    trimul = channel_form + (channel_form if channel else shard * (p - 1))
    transposes = 2 * shard * out_frac                # the normalised rows and the update of the ending node
    gathers = 2 * h * (n * n * 2 // p) * (p - 1) + (n * cs * 2 // p) * (p - 1)   # two triangle biases; the single track's rows
    return int(trimul + transposes + gathers)


def measure_sharded(args, rank: int, world: int, dev, blk, barrier) -> dict:
    """Benchmark config 5's unit on the ranks of this run: ONE Pairformer block at N=2048 (5 % padding tail, seed 4), its
    pair tensor row-sharded over the GPUs; beside it the same block on one GPU, so that the speed-up is measured inside
    one process group.  With one rank only the plain block runs."""
    import torch.distributed as dist
    from kfold_b200 import _lib as L
    import synth
    n = 2048
    steps = 3
    z, pm, m = synth.pair_inputs(4, n, C_Z, 1, pad_frac=0.05)
    s = synth.single_inputs(4, n, C_S, 1)
    stream = torch.cuda.current_stream()
    zd, sd, pmd, md = z.to(dev, torch.bfloat16), s.to(dev, torch.bfloat16), pm.to(dev), m.to(dev)
    del z
    for _ in range(2):
        blk(zd, sd, pmd, md)
    ms_1gpu = _event_time(lambda: blk(zd, sd, pmd, md), steps, stream, barrier)

    def trunk_1gpu():
        zt, st = zd, sd
        for _ in range(48):
            zt, st = blk(zt, st, pmd, md)

    # the 48-block trunk of benchmark config 5 on one GPU: one pass (about three seconds)
    ms_trunk_1gpu = _event_time(trunk_1gpu, 1, stream, barrier)
    res = {"n_token": n, "ms_1gpu": round(ms_1gpu, 3), "trunk48_ms_1gpu": round(ms_trunk_1gpu, 2)}
    if world == 1:
        res.update(ms=round(ms_1gpu, 3), speedup_vs_1gpu=1.0, trunk48_ms=round(ms_trunk_1gpu, 2),
                   exchange="none (one GPU: the plain block)")
        return res
    from kfold_b200 import sharded as SH
    r0, r1 = SH.shard_rows(n, world, rank)
    z_loc, pm_loc = zd[0, r0:r1].contiguous(), pmd[0, r0:r1].contiguous()
    del zd
    from kfold_b200 import functional as F
    F.release_workspaces()
    torch.cuda.empty_cache()
    sblk = SH.ShardedPairformerBlock(blk)
    channel = world >= 4 and C_Z % world == 0
    for _ in range(2):
        sblk(z_loc, sd, pm_loc, md)
    L.profile_enable(True)
    ms = _event_time(lambda: sblk(z_loc, sd, pm_loc, md), steps, stream, barrier)
    prof = L.profile_report()
    L.profile_enable(False)
    kernel_ms = sum(t for _, t in prof.values()) / steps

    def trunk_sharded():      # 48 sharded blocks back to back: the transposed mask is exchanged once and reused
        zt, st = z_loc, sd
        for _ in range(48):
            zt, st = sblk(zt, st, pm_loc, md)

    ms_trunk = _event_time(trunk_sharded, 1, stream, barrier)
    # a plain NCCL all-to-all of the size of one shard transpose, for the bandwidth the exchanges could reach
    probe = torch.empty(n * n * C_Z // world, dtype=torch.bfloat16, device=dev)
    probe_out = torch.empty_like(probe)
    for _ in range(2):
        dist.all_to_all_single(probe_out, probe)
    ms_probe = _event_time(lambda: dist.all_to_all_single(probe_out, probe), 5, stream, barrier)
    sent = probe.numel() * 2 * (world - 1) / world
    a2a_gbs = sent / (ms_probe * 1e-3) / 1e9
    t = torch.tensor([ms, kernel_ms, ms_1gpu, ms_probe, ms_trunk, ms_trunk_1gpu], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, kernel_ms, ms_1gpu, ms_probe, ms_trunk, ms_trunk_1gpu = (float(v) for v in t)
    out_bytes = sharded_bytes_out(n, C_Z, 4, C_S, world, channel)
    bound_ms = out_bytes / (a2a_gbs * 1e9) * 1e3
    res.update(ms=round(ms, 3), ms_1gpu=round(ms_1gpu, 3), kernel_ms=round(kernel_ms, 3), comm_ms=round(ms - kernel_ms, 3),
               exchange="channel all-to-all" if channel else "outgoing: all-gather of b; incoming: channel all-to-all",
               speedup_vs_1gpu=round(ms_1gpu / ms, 3), trunk48_ms=round(ms_trunk, 2), trunk48_ms_1gpu=round(ms_trunk_1gpu, 2),
               trunk48_speedup=round(ms_trunk_1gpu / ms_trunk, 3), bytes_sent_per_rank=out_bytes,
               nccl_all_to_all_gbs_per_rank=round(a2a_gbs, 1), comm_bound_ms=round(bound_ms, 3),
               note="comm_ms = step time - kernel time: collectives, reorder copies and host gaps not hidden under kernels")
    return res


def measure_sampler(rank: int, world: int, dev, barrier, steps: int = 200, samples: int = 5, nt: int = N_TOKENS_DEFAULT,
                    na: int = 6016, seed_offset: int | None = None) -> dict:
    """Benchmark config 4's diffusion part: the 200-step ECSI sampler (kfold_b200.sampler.KFoldECSI.sample_structure) over
    5 samples of a 768-token, 6 016-atom complex, score network = atom encoder (3 blocks), 24-block token transformer
    (c=768, 16 heads), atom decoder (3 blocks), bf16 compute, the network replayed as a CUDA graph.  With several ranks
    every rank samples its own seed (the data-parallel form of config 5); the time is the maximum over the ranks."""
    import types

    import numpy as np
    import torch.distributed as dist
    from kfold_b200 import _lib as L
    from kfold_b200 import modules as M
    from kfold_b200.sampler import KFoldECSI
    import synth
    c_a, c_s, c_atom, c_pair, tb, th = 768, 384, 128, 16, 24, 16
    rng = synth._Rng(SEED)
    w = synth.diffusion_step_weights(rng, c_a, c_s, c_atom, c_pair, 3, 4, tb, th, 6, False)
    w.update(synth._prefixed("single_conditioning", synth.single_conditioning_weights(rng, c_s, 256)))
    mod = M.DiffusionStack(channel_a=c_a, channel_s=c_s, channel_z=C_Z, channel_atom=c_atom, channel_atompair=c_pair, channel_coords=6,
                           token_transformer_blocks=tb, token_transformer_heads=th).to(dev)
    mod.load_state_dict(w, strict=False)
    pre = {"q": rng.normal(1, na, c_atom).to(dev), "c": rng.normal(1, na, c_atom).to(dev),
           "p": rng.normal(1, na // 32, 32, 128, c_pair).to(dev),
           "pair_bias": rng.normal(1, tb, th, nt, nt).to(dev, torch.bfloat16)}
    token_index = torch.from_numpy(np.sort(rng.rs.randint(0, nt, size=na)).astype(np.int64)).view(1, na).to(dev)
    atom = types.SimpleNamespace(pad_mask=synth.token_mask(na, pad_frac=0.02).view(1, na).to(dev), token_index=token_index,
                                 prior_coords=(rng.normal(1, na, 1, 3) * 10.0).to(dev))
    f_input = types.SimpleNamespace(atom=atom, token=types.SimpleNamespace(pad_mask=synth.token_mask(nt, pad_frac=PAD_FRAC).view(1, nt).to(dev)))
    s_inputs = rng.normal(1, nt, c_s).to(dev)
    sampler = KFoldECSI(KFoldECSI.Config(), mod)
    stream = torch.cuda.current_stream()
    res = {}
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        torch.manual_seed(SEED + (rank if seed_offset is None else seed_offset))
        launches0 = L.launch_count()
        if samples > 0:
            sampler.sample_structure(f_input, s_inputs, None, num_steps=4, num_samples=samples, precomputed=pre, cuda_graph=True)   # warm-up
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        finite = True
        if samples > 0:      # a rank that was dealt no sample only joins the barriers
            out = sampler.sample_structure(f_input, s_inputs, None, num_steps=steps, num_samples=samples, precomputed=pre,
                                           cuda_graph=True)
        e1.record(stream)
        barrier()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1)
        if samples > 0:
            finite = bool(torch.isfinite(out["coordinates"]).all())
    if world > 1:
        t = torch.tensor([ms, wall], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1])
    res.update(steps=steps, samples=samples, tokens=nt, atoms=na, seconds=round(ms / 1e3, 4), ms_per_step=round(ms / steps, 3),
               wall_seconds=round(wall, 4), structures_per_s=round(world * samples / (ms / 1e3), 3), seeds=world, finite=finite,
               ms=ms,
               device_status=L.device_status(),
               note="eager launches counted by the library (the graph-replayed network launches are not): "
                    f"{L.launch_count() - launches0}; includes the one-off graph capture of the network")
    return res


def measure_config5(rank: int, world: int, dev, barrier, sharded_res: dict) -> dict:
    """Benchmark config 5 assembled: N=2048 tokens (16 064 atoms), the 48-block trunk plus the 200-step sampler for 5 samples.
    One GPU: the plain trunk, then the five samples as one batch.  N ranks: the row-sharded trunk (measure_sharded), then
    the five samples dealt out to the ranks (sample i on rank i mod N), every rank with the full pair bias.  The one-GPU
    figures are measured in this same run (every rank runs them; maximum over the ranks)."""
    import torch.distributed as dist
    nt, na = 2048, 16064
    one = measure_sampler(rank, 1, dev, barrier, samples=5, nt=nt, na=na, seed_offset=0)
    res = {"n_token": nt, "n_atom": na, "samples": 5, "steps": 200, "trunk48_s_1gpu": round(sharded_res["trunk48_ms_1gpu"] / 1e3, 3),
           "sampler_s_1gpu": round(one["ms"] / 1e3, 3), "finite": one["finite"]}
    res["total_s_1gpu"] = round(res["trunk48_s_1gpu"] + res["sampler_s_1gpu"], 3)
    if world == 1:
        res.update(trunk48_s=res["trunk48_s_1gpu"], sampler_s=res["sampler_s_1gpu"], total_s=res["total_s_1gpu"], speedup=1.0)
        return res
    mine = len(range(rank, 5, world))
    part = measure_sampler(rank, world, dev, barrier, samples=mine, nt=nt, na=na, seed_offset=0)
    t = torch.tensor([one["ms"], part["ms"], 0.0 if (one["finite"] and part["finite"]) else 1.0], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res.update(sampler_s_1gpu=round(float(t[0]) / 1e3, 3), trunk48_s=round(sharded_res["trunk48_ms"] / 1e3, 3),
               sampler_s=round(float(t[1]) / 1e3, 3), samples_per_rank=[len(range(r, 5, world)) for r in range(world)],
               finite=bool(t[2] == 0))
    res["total_s_1gpu"] = round(res["trunk48_s_1gpu"] + res["sampler_s_1gpu"], 3)
    res["total_s"] = round(res["trunk48_s"] + res["sampler_s"], 3)
    res["speedup"] = round(res["total_s_1gpu"] / res["total_s"], 3)
    return res


def measure_sharded_parity(rank: int, world: int, dev, blk, w) -> dict:
    """The row-sharded block at N=512 on the ranks of this run, both exchange forms, against (i) the one-GPU block on
    the same rank and (ii) the oracle run on this GPU in float32 (the checker; TF32 off).  Relative RMS errors, maximum
    over the ranks; each rank compares its own rows of z and the replicated s."""
    import torch.distributed as dist
    from kfold_b200 import sharded as SH
    from oracle import pairformer_oracle as O
    import synth
    n = 512
    z, pm, m = synth.pair_inputs(4, n, C_Z, 1, pad_frac=0.05)
    s = synth.single_inputs(4, n, C_S, 1)
    zb, sb = z.bfloat16(), s.bfloat16()
    zd, sd, pmd, md = zb.to(dev), sb.to(dev), pm.to(dev), m.to(dev)
    z1, s1 = blk(zd, sd, pmd, md)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        wd = {k: v.to(dev) for k, v in w.items()}
        zo, so = O.pairformer_block(zd.float(), sd.float(), pmd, md, wd, row_chunk=64)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    r0, r1 = SH.shard_rows(n, world, rank)
    out = {"n_token": n, "rms_1gpu_vs_oracle": round(_rel_rms(z1[0, r0:r1].float(), zo[0, r0:r1]), 5)}
    for exchange in ("gather", "channel"):
        if exchange == "channel" and C_Z % world != 0:
            continue
        sblk = SH.ShardedPairformerBlock(blk, exchange=exchange)
        zs, ss = sblk(zd[0, r0:r1].contiguous(), sd, pmd[0, r0:r1].contiguous(), md)
        errs = torch.tensor([_rel_rms(zs.float(), z1[0, r0:r1].float()), _rel_rms(zs.float(), zo[0, r0:r1]),
                             _rel_rms(ss.float(), s1.float()), _rel_rms(ss.float(), so)], device=dev, dtype=torch.float64)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        out[exchange] = {"z_rms_vs_1gpu": round(float(errs[0]), 5), "z_rms_vs_oracle": round(float(errs[1]), 5),
                         "s_rms_vs_1gpu": round(float(errs[2]), 5), "s_rms_vs_oracle": round(float(errs[3]), 5)}
    return out


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import torch.distributed as dist
    from kfold_b200 import _lib as L
    from kfold_b200 import modules as M

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        from kfold_b200 import sharded as _sh
        _sh.apply_nccl_env_defaults()
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    z, s, pm, m, w = make_inputs()
    blk = M.PairformerBlock(C_Z, C_S).to(dev)
    blk.load_state_dict(w, strict=True)
    sharded_mode = args.sharded and world > 1
    if sharded_mode:
        # strong scaling: all ranks share ONE pair tensor, row-sharded (benchmark config 5's layout)
        from kfold_b200 import sharded as SH
        r0, r1 = SH.shard_rows(N_TOKENS, world, rank)
        z, pm = z[:, r0:r1].contiguous(), pm[:, r0:r1].contiguous()
        sblk = SH.ShardedPairformerBlock(blk)
    z_host = z.bfloat16().pin_memory()
    s_host = s.bfloat16().pin_memory()
    z_dev, s_dev = z_host.to(dev), s_host.to(dev)
    pm_dev, m_dev = pm.to(dev), m.to(dev)
    z_out_host = torch.empty_like(z_host).pin_memory()
    s_out_host = torch.empty_like(s_host).pin_memory()
    stream = torch.cuda.current_stream()

    def run_block(zd, sd):
        if sharded_mode:
            return sblk(zd[0], sd, pm_dev[0], m_dev)
        return blk(zd, sd, pm_dev, m_dev)

    def step_resident():
        return run_block(z_dev, s_dev)

    from kfold_b200.host_pipeline import HostPipeline
    pipe = HostPipeline(run_block, dev, depth=2)

    def run_e2e(k: int):
        """k steps through the public host-side call: every step copies its own inputs in from pinned host memory and its
        own result out; the copies of neighbouring steps run under the compute on separate streams."""
        pipe.run([(z_host, s_host)] * k, [(z_out_host, s_out_host)] * k)

    trunk = None
    sampler_run = None
    sharded_n2048 = None
    parity = None
    config5 = None
    with torch.no_grad():
        # ---- device-resident timing (with per-launch events recorded by the library)
        for _ in range(args.warmup):
            step_resident()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        L.profile_enable(True)
        launches0 = L.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step_resident()
        e1.record(stream)
        barrier()
        launches = L.launch_count() - launches0
        ms_step = e0.elapsed_time(e1) / args.steps
        prof = L.profile_report(detail=True)
        L.profile_enable(False)
        status = L.device_status()
        # ---- end to end: host buffers in, host buffers out, copies inside the timed region
        # warm-up of the copy path: the PCIe link of an idle GPU trains up under load (the first process on a box saw
        # 12 ms per step where the next saw 4.8), so the untimed steps run until two rounds agree or a second has passed
        run_e2e(max(2, min(args.warmup, 3)))
        barrier()
        t_warm, prev = time.perf_counter(), None
        while time.perf_counter() - t_warm < 1.0:
            e0.record(stream)
            run_e2e(4)
            e1.record(stream)
            barrier()
            cur = e0.elapsed_time(e1)
            if prev is not None and abs(cur - prev) < 0.05 * prev:
                break
            prev = cur
        e0.record(stream)
        run_e2e(args.steps)
        e1.record(stream)
        barrier()
        ms_e2e = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop() if rank == 0 else {}

        if not sharded_mode and args.tokens == N_TOKENS_DEFAULT and not args.headline_only:
            # ---- a longer region: 48 blocks back to back on one pair tensor (each block's output feeds the next), the
            # trunk depth of benchmark config 4; the same block weights serve all 48 (1.4 MB of weights: no cache effect)
            def trunk_pass():
                zt, st = z_dev, s_dev
                for _ in range(48):
                    zt, st = blk(zt, st, pm_dev, m_dev)
                return zt, st

            trunk_pass()
            barrier()
            tsampler = ClockSampler(local_rank)
            if rank == 0:
                tsampler.start()
            passes = 3
            ms_trunk = _event_time(trunk_pass, passes, stream, barrier)
            zt, _ = trunk_pass()
            finite = bool(torch.isfinite(zt.float()).all())
            tclocks = tsampler.stop() if rank == 0 else {}
            if world > 1:
                t = torch.tensor([ms_trunk], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_trunk = float(t[0])
            trunk = {"ms": round(ms_trunk, 3), "blocks": 48, "passes_timed": passes, "ms_per_block": round(ms_trunk / 48, 4),
                     "region_s": round(ms_trunk * passes / 1e3, 3), "clocks": tclocks, "finite": finite,
                     "ms_x_sm_mhz": round(ms_trunk * tclocks["sm_mhz"], 1) if tclocks.get("sm_mhz") else None}
            del zt
            # ---- benchmark config 5's block: N=2048, row-sharded over the ranks of this run (plain block with one rank)
            sampler_run = measure_sampler(rank, world, dev, barrier)
            sharded_n2048 = measure_sharded(args, rank, world, dev, blk, barrier)
            if world > 1:
                parity = measure_sharded_parity(rank, world, dev, blk, w)
            from kfold_b200 import functional as _F
            _F.release_workspaces()
            torch.cuda.empty_cache()
            config5 = measure_config5(rank, world, dev, barrier, sharded_n2048)
        status = status or L.device_status()

    if world > 1:
        t = torch.tensor([ms_step, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        peaks = load_peaks()
        region_s = ms_step * args.steps / 1e3
        tensor_peak, peak_kind = pick_tensor_peak(peaks, region_s, clocks)
        work = algorithmic_work()
        total_ms = sum(v[1] for v in prof.values()) or 1.0
        kernels = {}
        for tag, (cnt, ms, cnt_large, ms_large) in sorted(prof.items(), key=lambda kv: -kv[1][1]):
            # a tag that serves the pair tensor and the single track (LayerNorm, transition): the roofline figures are those
            # of the pair-sized launches (at least half as long as the tag's longest launch), `avg_ms` is theirs
            avg_ms = ms_large / max(cnt_large, 1)
            ent = {"launches": cnt, "total_ms": round(ms, 4), "avg_ms": round(avg_ms, 5), "share": round(ms / total_ms, 4)}
            if cnt_large != cnt:
                ent.update(pair_sized_launches=cnt_large, small_launches=cnt - cnt_large,
                           small_avg_ms=round((ms - ms_large) / (cnt - cnt_large), 5))
            if tag in work:
                kind, amount = work[tag]
                if kind == "tensor":
                    ach = amount / (avg_ms * 1e-3) / 1e12
                    ent.update(bound="tensor", achieved=round(ach, 2), unit="TFLOP/s", frac=round(ach / tensor_peak, 4),
                               frac_burst=round(ach / peaks["tflops_burst"], 4),
                               frac_sustained=round(ach / peaks["tflops_sustained"], 4))
                else:
                    ent.update(bound="hbm", achieved=round(amount / (avg_ms * 1e-3) / 1e9, 1), unit="GB/s",
                               frac=round(amount / (avg_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4))
            kernels[tag] = ent
        top = next(iter(kernels)) if kernels else None
        roofline = None
        if top and "bound" in kernels[top]:
            k = kernels[top]
            roofline = {"kernel": top, "bound": k["bound"], "achieved": k["achieved"],
                        "peak": tensor_peak if k["bound"] == "tensor" else peaks["hbm_gbs"], "unit": k["unit"],
                        "frac": k["frac"], "traffic": ncu_traffic(top, N_TOKENS),
                        "traffic_source": NCU_TRAFFIC.get(top, {}).get("source"), "peak_source": peaks["source"],
                        "share_of_step": k["share"]}
            if k["bound"] == "tensor":
                roofline.update(peak_kind=f"{peak_kind} bf16 (timed region {region_s:.2f} s, median SM clock {clocks.get('sm_mhz')} MHz)",
                                frac_burst=k["frac_burst"], frac_sustained=k["frac_sustained"])
        # CPU baseline: the reference's own modules on this box's host cores, one bounded sample at the benchmark's size
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            run, kind, what, cores = cpu_block_runner(N_TOKENS)
            t_cpu = time_cpu_block(run, 1, 0)[0]
            cpu = {"value": t_cpu, "unit": "ms", "cores": cores, "kind": kind,
                   "sample": f"{what}: ONE block at N={N_TOKENS}, a single run without warm-up"}
        h2d = z_host.numel() * 2 + s_host.numel() * 2
        d2h = z_out_host.numel() * 2 + s_out_host.numel() * 2
        bf = block_flops(N_TOKENS) / (ms_step * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": ms_step if sharded_mode else ms_step / world, "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False,
            "scaling": "strong" if sharded_mode else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(world, sharded_mode),
            "block_tflops": round(bf, 2),
            "block_frac_of_tensor_peak": round(bf / tensor_peak, 4),
            "block_frac_burst": round(bf / peaks["tflops_burst"], 4), "block_frac_sustained": round(bf / peaks["tflops_sustained"], 4),
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": ms_e2e / world, "unit": "ms", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "kfold_b200.host_pipeline.HostPipeline: every step copies its inputs in from pinned host memory and "
                           "its result out; copies of neighbouring steps overlap the compute on three streams, two steps in flight"},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
            "trunk48_ms": None if trunk is None else trunk["ms"], "trunk48": trunk,
            "sampler_200x5": sampler_run,
            "config4_s": None if trunk is None or sampler_run is None else round(trunk["ms"] / 1e3 + sampler_run["seconds"], 4),
            "sharded_n2048": sharded_n2048, "sharded_parity": parity, "config5_n2048": config5, "kernels": kernels,
        }
        if trunk is not None and trunk["clocks"].get("sm_mhz"):
            tp, tk = pick_tensor_peak(peaks, trunk["region_s"], trunk["clocks"])
            tf = 48 * block_flops(N_TOKENS) / (trunk["ms"] * 1e-3) / 1e12
            trunk.update(tflops=round(tf, 1), frac_of_tensor_peak=round(tf / tp, 4), peak_kind=tk)
        emit(line)
    if world > 1:
        dist.destroy_process_group()


_REAL_STDOUT = None


def _protect_stdout() -> None:
    """Libraries (NCCL prints its version) write to fd 1; the contract is ONE JSON line there.  Everything
    else is sent to stderr and the line goes out through the saved descriptor."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _REAL_STDOUT if _REAL_STDOUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main() -> None:
    _protect_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_triton"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the side measurements (48-block trunk, N=2048 sharded block and its parity check)")
    ap.add_argument("--sharded", action="store_true",
                    help="with N > 1 ranks: row-shard ONE pair tensor over the GPUs (strong scaling) instead of one block per GPU")
    ap.add_argument("--tokens", type=int, default=N_TOKENS,
                    help="profiling aid: run the block at another N (the reported line is then NOT the benchmark workload)")
    ap.add_argument("--sampler-step", action="store_true",
                    help="fourth workload: one DiffusionStack.step at benchmark config 4's shape (its own JSON line)")
    ap.add_argument("--atom-step", action="store_true",
                    help="third workload: one pass of an atom-level local transformer of benchmark config 4 (its own JSON line)")
    ap.add_argument("--diffusion-step", action="store_true",
                    help="second workload: one pass of the sampler's token transformer of benchmark config 4 (its own JSON line)")
    args = ap.parse_args()
    if args.diffusion_step:
        run_diffusion_step(args)
        return
    if args.atom_step:
        run_atom_step(args)
        return
    if args.sampler_step:
        run_sampler_step(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and args.tokens == N_TOKENS else args.warmup
    if args.tokens != N_TOKENS:
        globals()["N_TOKENS"] = args.tokens
        globals()["METRIC"] = f"pairformer_block_fwd_ms_n{args.tokens}_bf16_PROFILING_SIZE"
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if args.impl == "reference_triton":
        run_reference_triton_arm(args, rank)
        return
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch multi-GPU runs with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
