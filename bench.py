#!/usr/bin/env python
"""Benchmark of the palettized-LUT decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one greedy decode step (one token per sequence) of a random-init,
4-bit palettized model -- every palettized GEMV of the model once, plus the
decode glue.  Default workload: the Qwen2.5-72B architecture (80 layers, hidden
8192, 64/8 heads, intermediate 29568, vocab 152064), batch 1, decoding after a
512-token prompt, tensor-parallel over N GPUs (column/row-sharded linears,
all-reduce over NVLink).  Weights are seeded synthetic tensors generated on the
device (no checkpoint is available offline); total work is fixed as N grows
(strong scaling).  The JSON line printed by rank 0 follows the driver's
contract; beside the headline it carries, each with its own roofline / e2e /
clocks:

  batch8, batch32   the same model and context at decode batches 8 and 32 (every N)
  breakdown         GEMV-only, attention-only and reduction-only passes of a step (every N)
  tp_parity         N > 1: a small model decoded under tensor parallelism against one GPU
  token_checksum    CRC of the first 32 greedy tokens of the timed model (compare across N)
  config3           N = 1: Qwen2.5-0.5B decode, 128-token prompt, 256 generated tokens
  config4           N = 1: the six prefill GEMMs of a Qwen2.5-7B layer, M = 2048, N(0,1) activations
  config4_2bit      N = 1: the same six GEMMs with 2-bit indices and a 4-entry palette per row
  lut_gemv_0p5b_shapes   N = 1: GEMV / fused gate-up / MLP at the 4864x896 shapes, working set > L2
  lut_gemv_decode_shapes N = 1: the five GEMV launch shapes of the workload's decode step, each timed alone
  cpu_baseline      N = 1: the CPU restatement of the reference's path on the host cores (a sample)

`--impl reference` times the CPU restatement of the reference's own path (the
oracle) on the host cores for the same workload; each of its steps is a bounded
SAMPLE of a decode step, extrapolated, and the line says so.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (architecture dict key, prompt context)
    "qwen2.5-72b-decode": ("QWEN25_72B", 512),
    "qwen2.5-0.5b-decode": ("QWEN25_0P5B", 128),
    # prefill: the palettized linears of one Qwen2.5-7B layer on M = 2048 tokens (tensor-core GEMM)
    "qwen2.5-7b-prefill-gemm": ("QWEN25_7B", 2048),
}
METRIC = "decode_tokens_per_s"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0
TOY = dict(num_layers=3, hidden_size=128, num_heads=8, num_kv_heads=8, head_dim=32, intermediate_size=512,
           vocab_size=1024, norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 1400.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return self

        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()
        return self

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                pw.append(float(r[3]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


def arch_dict(name):
    import prism_engine_b200 as p

    return dict(getattr(p, WORKLOADS[name][0]))


# --------------------------------------------------------------------------------------------
# CPU arm: the restatement of the reference's path, all host threads, on a bounded sample
# --------------------------------------------------------------------------------------------
class CpuSample:
    """Bounded sample of one decode step for the host cores.  One estimate = the seven palettized GEMVs
    of `n_sets` DISTINCT layers (separately generated weights, so no estimate re-reads cache-warm
    weights of the previous one) plus the LM head on 1/head_frac of its rows; the token time is the mean
    layer time x num_layers + the head time x head_frac.  Glue ops (norm, rope, attention) are not in the
    sample: on the CPU path they are < 1 % of a step."""

    def __init__(self, arch, threads, n_sets=3, head_frac=4):
        from prism_engine_b200 import synth

        self.arch, self.threads, self.n_sets = arch, threads, n_sets
        H, I, V = arch["hidden_size"], arch["intermediate_size"], arch["vocab_size"]
        qd = arch["num_heads"] * arch["head_dim"]
        kvd = arch["num_kv_heads"] * arch["head_dim"]
        self.shapes = [(qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I)]
        self.pay = [[synth.make_payload(m, k, 4, seed=100 * s + i) for i, (m, k) in enumerate(self.shapes)]
                    for s in range(n_sets)]
        self.xs = {k: synth.make_activation(k, seed=k) for _, k in self.shapes}
        self.vrows = max(64, V // head_frac // 64 * 64)
        self.head = synth.make_payload(self.vrows, H, 4, seed=99)
        self.sample = (f"SAMPLE, extrapolated: 7 palettized GEMVs of {n_sets} distinct layers (mean x {arch['num_layers']} layers) + "
                       f"{self.vrows}/{V} LM-head rows (scaled), lut_gemv restatement over {threads} threads")

    def estimate(self):
        """(extrapolated seconds per token, seconds actually spent)."""
        from oracle import oracle as orc

        a = self.arch
        t_all0 = time.perf_counter()
        layer_times = []
        for s in range(self.n_sets):
            t0 = time.perf_counter()
            for (m, k), pl in zip(self.shapes, self.pay[s]):
                orc.lut_gemv(self.xs[k], pl, m, k, threads=self.threads)
            layer_times.append(time.perf_counter() - t0)
        t0 = time.perf_counter()
        orc.lut_gemv(self.xs[a["hidden_size"]], self.head, self.vrows, a["hidden_size"], threads=self.threads)
        t_head = (time.perf_counter() - t0) * (a["vocab_size"] / self.vrows)
        spent = time.perf_counter() - t_all0
        return statistics.mean(layer_times) * a["num_layers"] + t_head, spent


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle as orc

    arch = arch_dict(args.workload)
    threads = orc.max_threads()
    cs = CpuSample(arch, threads)
    per_tok, spent = [], []
    for i in range(args.warmup + args.steps):
        t, s = cs.estimate()
        if i >= args.warmup:
            per_tok.append(t)
            spent.append(s)
    tok_s = statistics.median(per_tok)
    value = args.batch / tok_s
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # what a step of THIS arm took on the clock: one bounded sample, not a whole decode step
        "ms_per_step": statistics.mean(spent) * 1e3,
        "extrapolated_ms_per_token": tok_s * 1e3, "value_is_extrapolated_from_a_sample": True,
        "spread": {"min_tok_s": args.batch / max(per_tok), "max_tok_s": args.batch / min(per_tok), "estimates": len(per_tok)},
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights / f32 accumulate",
        "data": "synthetic", "config": workload_config(args, arch),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": cs.sample + f"; median of {len(per_tok)} estimates"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)
    return 0


def workload_config(args, arch):
    return {"workload": f"{args.workload}: batch {args.batch}, {WORKLOADS[args.workload][1]}-token prompt context, "
                        f"4-bit indices + 16-entry fp16 palette per row, greedy, fp16 KV",
            "layers": arch["num_layers"], "hidden": arch["hidden_size"], "intermediate": arch["intermediate_size"],
            "vocab": arch["vocab_size"], "batch": args.batch, "parallelism": f"tp{args.gpus}",
            "l2_policy": "inputs larger than L2: every step streams all weights of the model from HBM"}


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
class Env:
    """Process-wide state of a run: ranks, barrier, reductions over ranks."""

    def __init__(self, args):
        import torch

        self.torch = torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("cpu:gloo,cuda:nccl", rank=self.rank, world_size=self.world,
                                    device_id=torch.device("cuda", self.local))
            self.dist = dist

    def barrier(self, be):
        be.synchronize()
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()

    def max_over_ranks(self, v):
        if self.dist is None:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def measure_decode(env, be, eng, arch, B, ctx_len, steps, warmup, want_tokens=False):
    """Prefill `ctx_len` tokens for B sequences (untimed), then time `steps` decode steps twice: replayed on the
    device (CUDA events, no host traffic between steps) and end to end (one public-API call per step with the
    token copied in from pinned host memory and the greedy token copied back).  Max over ranks."""
    torch = env.torch
    from prism_engine_b200 import synth

    prompts = np.stack([synth.make_prompt(ctx_len, arch["vocab_size"], seed=b) for b in range(B)])
    eng.generate(prompts, 0)  # prefill: one step per prompt token
    tok_pinned = torch.from_numpy(prompts[:, -1].astype(np.int64)).to(torch.int32).pin_memory()
    out_pinned = torch.empty(B * max(steps, warmup, 32), dtype=torch.int32).pin_memory()  # [B][n_steps] of each call
    first = None
    if want_tokens:
        eng.decode(None, 32, tokens_ptr=tok_pinned.data_ptr(), out_ptr=out_pinned.data_ptr())
        first = out_pinned[:B * 32].numpy().astype(np.uint32).reshape(B, 32).copy()
    if warmup:
        eng.decode(None, warmup, tokens_ptr=tok_pinned.data_ptr(), out_ptr=out_pinned.data_ptr())
    sampler = ClockSampler(env.local) if env.rank == 0 else None
    env.barrier(be)
    if sampler:
        sampler.start()
    l0 = be.launch_count()
    eng.decode(None, steps, tokens_ptr=tok_pinned.data_ptr(), out_ptr=out_pinned.data_ptr())
    env.barrier(be)
    dev_ms = env.max_over_ranks(eng.last_device_ms())
    graph_launches = be.launch_count() - l0
    nxt = torch.empty(B, dtype=torch.int32).pin_memory()
    L = eng.L
    for _ in range(warmup):
        eng._ck(L.prism_cuda_engine_step(eng.h, tok_pinned.data_ptr(), nxt.data_ptr(), None))
        tok_pinned.copy_(nxt)
    env.barrier(be)
    t0 = time.perf_counter()
    for _ in range(steps):
        eng._ck(L.prism_cuda_engine_step(eng.h, tok_pinned.data_ptr(), nxt.data_ptr(), None))
        tok_pinned.copy_(nxt)
    env.barrier(be)
    e2e_s = env.max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if sampler else None
    step_bytes = eng.step_bytes()
    peak, _ = measured_peaks()
    ms = dev_ms / steps
    return {
        "value": B * steps / (dev_ms * 1e-3), "unit": UNIT, "batch": B, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "kernels_per_step": eng.kernels_per_step(), "graph_launches": graph_launches,
        "step_roofline": {"algorithmic_bytes_per_step_per_gpu": step_bytes, "achieved_gbs_per_gpu": step_bytes / (ms * 1e-3) / 1e9,
                          "frac": step_bytes / (ms * 1e-3) / 1e9 / peak},
        "e2e": {"value": B * steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
                "ms_per_step": e2e_s / steps * 1e3},
        "clocks": clocks,
    }, first


def tp_parity_check(env, be):
    """A small model decoded under tensor parallelism on all ranks against the same seeded model on one GPU
    (rank 0, a second context without a group): greedy tokens must be identical."""
    import prism_engine_b200 as p
    from prism_engine_b200 import synth

    mc = p.model_config(**TOY, max_seq=64, max_batch=2, profile="baseline")
    prompts = np.stack([synth.make_prompt(6, TOY["vocab_size"], seed=s) for s in (11, 12)])
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=21)
    got = eng.generate(prompts, 24)
    eng.close()
    res = None
    if env.rank == 0:
        ref_be = p.CudaBackend(device=env.local)
        ref = p.PrismEngine(ref_be, mc)
        ref.synth_weights(seed=21)
        want = ref.generate(prompts, 24)
        ref.close()
        ref_be.close()
        n_same = int(np.sum(got == want))
        res = {"ok": bool(np.array_equal(got, want)), "tokens_compared": int(got.size), "tokens_equal": n_same,
               "model": "3 layers, hidden 128, 8 heads, intermediate 512, vocab 1024, 2 sequences x 24 greedy tokens",
               "against": "the same seeded weights on one GPU", "peer_all_reduce": be.tp_peer_ready(),
               "peer_reason": be.tp_peer_reason()}
    env.barrier(be)
    return res


def run_ours(args):
    import prism_engine_b200 as p

    env = Env(args)
    torch = env.torch
    be = p.CudaBackend(device=env.local)
    for kv in args.option:
        key, val = kv.split("=")
        be.set_option(key, int(val))
    if env.world > 1:
        from prism_engine_b200 import tp

        uid = tp.exchange_unique_id(p.CudaBackend.tp_unique_id)
        be.tp_init(env.world, env.rank, uid)
    parity = tp_parity_check(env, be) if env.world > 1 else None
    arch = arch_dict(args.workload)
    if args.layers:
        arch["num_layers"] = args.layers
    ctx_len = WORKLOADS[args.workload][1] if args.ctx < 0 else args.ctx
    B = args.batch
    big = args.workload == "qwen2.5-72b-decode"
    extra = [b for b in (8, 32) if big and not args.no_batches and b != B]
    sub_steps, sub_warm = 16, 3
    max_seq = ctx_len + 40 + 2 * (max(args.warmup, sub_warm) + max(args.steps, sub_steps)) + 16
    mc = p.model_config(**arch, max_seq=max_seq, max_batch=max([B] + extra), profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=1)

    main, first = measure_decode(env, be, eng, arch, B, ctx_len, args.steps, args.warmup, want_tokens=True)
    # ---- each kind of launch of the step alone, between events on the context stream
    gemv_ms, gemv_bytes, gemv_launches = eng.profile_gemv(reps=2)
    gemv_ms = env.max_over_ranks(gemv_ms)
    attn_ms, attn_launches = eng.profile_part(1, reps=2)
    attn_ms = env.max_over_ranks(attn_ms)
    red_ms, red_launches = eng.profile_part(2, reps=2)
    red_ms = env.max_over_ranks(red_ms)
    peak, peak_kind = measured_peaks()
    achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": main["value"], "unit": UNIT, "n_gpus": env.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights / f32 accumulate", "data": "synthetic",
        "config": workload_config(args, arch),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8tbs_nominal": achieved / 8000.0,
                     "kernel": "lut_gemv_ws_kernel (lut_gemv_cl_kernel / lut_gemv_sk_kernel for small matrices)", "launches_timed": gemv_launches,
                     "avg_launch_us": gemv_ms * 1e3 / max(gemv_launches, 1),
                     "algorithmic_bytes_per_launch": gemv_bytes / max(gemv_launches, 1),
                     "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE and TRAFFIC_PER_ALGORITHMIC_BYTE * gemv_bytes / max(gemv_launches, 1)},
        "step_roofline": main["step_roofline"],
        "e2e": main["e2e"],
        "gpu_launches": main["kernels_per_step"] * args.steps, "kernels_per_step": main["kernels_per_step"],
        "graph_launches": main["graph_launches"], "clocks": main["clocks"],
        "breakdown": {"what": "one step's launches of each kind, alone and back to back between CUDA events (ms per step, max over ranks)",
                      "gemv_ms": gemv_ms / 2, "gemv_launches": gemv_launches // 2,
                      "attention_ms": attn_ms / 2, "attention_launches": attn_launches // 2,
                      "tp_reduction_ms": red_ms / 2, "tp_reduction_launches": red_launches // 2,
                      "step_ms": main["ms_per_step"]},
        "token_checksum": {"crc32_first_32_greedy_tokens": zlib.crc32(first[0].tobytes()) & 0xFFFFFFFF,
                           "first_8_tokens": [int(t) for t in first[0][:8]]},
    }
    if parity is not None:
        line["tp_parity"] = parity
    for b in extra:
        sub, _ = measure_decode(env, be, eng, arch, b, ctx_len, sub_steps, sub_warm)
        line[f"batch{b}"] = sub
    eng.close()
    if env.rank == 0 and env.world == 1:
        if not args.no_configs:
            line["config3"] = config3_decode(env, be)
            line["config4"] = config4_gemm(env, be)
            line["config4_2bit"] = config4_gemm(env, be, bits=2)
        if not args.no_gemv_shapes:
            line["lut_gemv_0p5b_shapes"] = small_shape_bandwidth(env, be, peak)
            line["lut_gemv_decode_shapes"] = decode_shape_bandwidth(env, be, arch, peak)
        if not args.no_cpu_baseline:
            from oracle import oracle as orc

            threads = orc.max_threads()
            cs = CpuSample(arch_dict(args.workload), threads)
            cs.estimate()
            est = [cs.estimate()[0] for _ in range(5)]
            per_tok = statistics.median(est)
            line["cpu_baseline"] = {"value": B / per_tok, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": cs.sample + "; median of 5 estimates",
                                    "min": B / max(est), "max": B / min(est)}
    if env.rank == 0:
        emit(line)
    be.close()
    if env.dist is not None:
        env.dist.barrier()
        env.dist.destroy_process_group()
    return 0


# DRAM bytes per algorithmic byte of the GEMV launches of a 72B decode step, from the ncu capture
# summarised in profiles/lut_gemv_ws_kernel_qwen72b_shapes.md (the five launch shapes together:
# 1083.3 MB of DRAM traffic for 1069.8 MB of algorithmic bytes).
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0126


def config3_decode(env, be):
    """Qwen2.5-0.5B architecture, batch 1: 128-token prompt, 256 greedy tokens, fp16 KV -- through
    prism_cuda_engine_generate (host prompt in, host tokens out), repeated so the clock sampler sees the run."""
    import prism_engine_b200 as p
    from prism_engine_b200 import synth

    arch = dict(p.QWEN25_0P5B)
    n_prompt, n_new, reps = 128, 256, 8
    mc = p.model_config(**arch, max_seq=n_prompt + n_new + 8, max_batch=1, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=3)
    prompt = synth.make_prompt(n_prompt, arch["vocab_size"], seed=5)
    for _ in range(3):
        eng.generate(prompt, n_new)  # warm-up: eager pass, graph capture, replay
    sampler = ClockSampler(env.local).start()
    be.synchronize()
    dec_ms, wall = 0.0, 0.0
    l0 = be.launch_count()
    for _ in range(reps):
        t0 = time.perf_counter()
        eng.generate(prompt, n_new)
        wall += time.perf_counter() - t0
        dec_ms += eng.last_device_ms()
    launches = be.launch_count() - l0
    clocks = sampler.stop()
    step_bytes = eng.step_bytes()
    peak, kind = measured_peaks()
    ms = dec_ms / (reps * n_new)
    out = {
        "workload": "qwen2.5-0.5b-decode: batch 1, 128-token prompt, 256 generated tokens, 4-bit palettized, fp16 KV",
        "metric": METRIC, "value": reps * n_new / (dec_ms * 1e-3), "unit": UNIT, "ms_per_step": ms,
        "kernels_per_step": eng.kernels_per_step(), "graph_launches": launches,
        "roofline": {"bound": "hbm", "achieved": step_bytes / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": step_bytes / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}",
                     "algorithmic_bytes_per_step": step_bytes, "what": "whole decode step (weights + KV read) / step time"},
        "e2e": {"value": reps * n_new / wall, "unit": "generated tok/s over the whole prism_cuda_engine_generate call (its 128 prefill steps included)",
                "h2d_bytes_per_step": 4 * n_prompt / n_new, "d2h_bytes_per_step": 4},
        "clocks": clocks, "l2_policy": "261 MB of weights per step exceed L2",
    }
    eng.close()
    return out


def config4_gemm(env, be, bits=4):
    """The six palettized linears of one Qwen2.5-7B layer on M = 2048 tokens of seeded N(0,1) fp16 activations
    through the tensor-core GEMM; every shape timed for >= 0.3 s with the clock sampler running across all."""
    torch = env.torch
    import prism_engine_b200 as p
    from prism_engine_b200 import synth

    arch = dict(p.QWEN25_7B)
    H, I = arch["hidden_size"], arch["intermediate_size"]
    kvd = arch["num_kv_heads"] * arch["head_dim"]
    m_tok = 2048
    shapes = [("q", H, H), ("k", kvd, H), ("v", kvd, H), ("gate", I, H), ("up", I, H), ("down", H, I)]
    hs = {n: be.synth(f"c4.{bits}.{n}", m, k, bits=bits, seed=50 + i) for i, (n, m, k) in enumerate(shapes)}
    X = {k: torch.from_numpy(synth.make_activation((m_tok, k), seed=k).view(np.int16)).cuda() for k in (H, I)}
    torch.cuda.synchronize()
    est = {}
    for n, m, k in shapes:
        be.bench_gemm(hs[n], X[k].data_ptr(), m_tok, 3)
        est[n] = be.bench_gemm(hs[n], X[k].data_ptr(), m_tok, 3) / 3
    sampler = ClockSampler(env.local).start()
    per, total_ms, total_flop = {}, 0.0, 0.0
    l0 = be.launch_count()
    t_wall0 = time.perf_counter()
    for n, m, k in shapes:
        reps = max(5, int(math.ceil(300.0 / max(est[n], 1e-3))))
        ms = be.bench_gemm(hs[n], X[k].data_ptr(), m_tok, reps) / reps
        flop = 2.0 * m_tok * m * k
        per[n] = {"shape": f"{m}x{k}", "ms": ms, "tflops": flop / ms / 1e9, "reps": reps}
        total_ms += ms
        total_flop += flop
    timed_s = time.perf_counter() - t_wall0
    launches = be.launch_count() - l0
    clocks = sampler.stop()
    sustained, burst, kind = measured_tensor_peak()
    value = total_flop / total_ms / 1e9
    big = per["gate"]["tflops"]
    # end to end: host activations in, host result out, through the public GEMM call
    Xh = synth.make_activation((m_tok, H), seed=1)
    be.gemm(hs["gate"], Xh)
    t0 = time.perf_counter()
    for _ in range(3):
        be.gemm(hs["gate"], Xh)
    e2e_s = (time.perf_counter() - t0) / 3
    for h in hs.values():
        be.free(h)
    return {
        "workload": f"qwen2.5-7b-prefill-gemm: q/k/v/gate/up/down of one layer, M = {m_tok} tokens of N(0,1) fp16 activations, "
                    f"{bits}-bit indices + {1 << bits}-entry fp16 palette per row",
        "metric": "prefill_gemm_tflops", "value": value, "unit": "TFLOP/s", "ms_per_step": total_ms, "timed_seconds": timed_s,
        "roofline": {"bound": "tensor", "achieved": big, "peak": sustained, "unit": "TFLOP/s", "frac": big / sustained,
                     "frac_of_burst": big / burst, "layer_frac": value / sustained, "layer_frac_of_burst": value / burst,
                     "peak_kind": f"of {kind} sustained bf16 cuBLAS {sustained} (burst {burst}); each shape ran >= 0.3 s back to back",
                     "kernel": "lut_gemm_tc5_kernel", "launch": "gate 18944x3584, M=2048",
                     # DRAM read + write bytes of one gate launch in the ncu capture summarised under profiles/
                     "traffic": 164.3e6 if bits == 4 else None, "traffic_unit": "bytes per gate launch (algorithmic 126.8e6)"},
        "per_gemm": per,
        "e2e": {"value": 2.0 * m_tok * I * H / e2e_s / 1e12, "unit": "TFLOP/s (gate GEMM through prism_cuda_gemm, host buffers)",
                "h2d_bytes_per_step": int(Xh.nbytes), "d2h_bytes_per_step": m_tok * I * 2},
        "gpu_launches": launches, "clocks": clocks, "l2_policy": "operands of a GEMM exceed L2 (X 14.7 MB + Y up to 77.6 MB + weights up to 34 MB per launch, 148 MB rolling)",
    }


def small_shape_bandwidth(env, be, peak):
    """LUT-GEMV bandwidth at the Qwen2.5-0.5B MLP shapes (4864x896 / 896x4864).  A single 2.3 MB GEMV
    is launch-bound and L2-resident, so each measurement cycles through 160 distinct weight sets
    (> 126 MB of L2) inside one CUDA graph."""
    torch = env.torch
    from prism_engine_b200 import synth

    n_sets, reps = 160, 5
    gate = [be.synth(f"bw.gate{i}", 4864, 896, seed=1000 + i) for i in range(n_sets)]
    up = [be.synth(f"bw.up{i}", 4864, 896, seed=2000 + i) for i in range(n_sets)]
    down = [be.synth(f"bw.down{i}", 896, 4864, seed=3000 + i) for i in range(n_sets)]
    x = torch.from_numpy(synth.make_activation(896, seed=7).view(np.int16)).cuda()
    torch.cuda.synchronize()
    out = {}
    b1 = synth.gemv_algorithmic_bytes(4864, 896)
    b2 = 2 * b1 - 2 * 896
    b3 = b2 + synth.gemv_algorithmic_bytes(896, 4864)
    for name, kind, hs, nbytes in (("gemv_4864x896", 0, gate, b1),
                                   ("fused_gate_up_swiglu", 1, list(zip(gate, up)), b2),
                                   ("mlp_gate_up_down", 2, list(zip(gate, up, down)), b3)):
        ms = be.bench_cycle(kind, np.array(hs, np.int32), reps, x.data_ptr())
        gbs = nbytes * n_sets * reps / (ms * 1e-3) / 1e9
        out[name] = {"gbs": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_8tbs_nominal": gbs / 8000.0,
                     "us_per_call": ms * 1e3 / (n_sets * reps), "algorithmic_bytes": nbytes}
    for h in gate + up + down:
        be.free(h)
    return out


def decode_shape_bandwidth(env, be, arch, peak):
    """The five GEMV launch shapes of the decode step (stacked q+k+v, o, fused gate+up, down, LM head), each
    timed alone: more than 1 GB of distinct weight sets of the shape cycle inside one CUDA graph, so every
    launch streams from HBM and follows a launch of its own kind."""
    torch = env.torch
    from prism_engine_b200 import synth

    H, I, V = arch["hidden_size"], arch["intermediate_size"], arch["vocab_size"]
    qkv_rows = (arch["num_heads"] + 2 * arch["num_kv_heads"]) * arch["head_dim"]
    shapes = (("qkv", qkv_rows, H, 0), ("o", H, arch["num_heads"] * arch["head_dim"], 0), ("gate_up_swiglu", I, H, 1),
              ("down", H, I, 0), ("lm_head", V, H, 0))
    out = {}
    for name, m, k, kind in shapes:
        nbytes = synth.gemv_algorithmic_bytes(m, k)
        n_sets = min(64, max(2, int(1.2e9 // nbytes)))
        if kind == 1:
            n_sets = max(2, n_sets // 2 * 2)
        hs = [be.synth(f"shape.{name}{i}", m, k, seed=5000 + i) for i in range(n_sets)]
        x = torch.from_numpy(synth.make_activation(k, seed=9).view(np.int16)).cuda()
        torch.cuda.synchronize()
        calls = n_sets // 2 if kind == 1 else n_sets
        per_call = 2 * nbytes - 2 * k if kind == 1 else nbytes
        arr = np.array(list(zip(hs[0::2], hs[1::2])) if kind == 1 else hs, np.int32)
        reps = 6
        be.bench_cycle(kind, arr, 2, x.data_ptr())
        ms = be.bench_cycle(kind, arr, reps, x.data_ptr())
        us = ms * 1e3 / (calls * reps)
        gbs = per_call / us / 1e3
        out[name] = {"rows": m * (2 if kind == 1 else 1), "k": k, "us_per_call": us, "gbs": gbs, "frac_of_measured_peak": gbs / peak,
                     "algorithmic_bytes": per_call}
        for h in hs:
            be.free(h)
    return out


def run_gemm(args):
    """Stand-alone prefill GEMM workload (the `config4` key of the default run, as its own line)."""
    import prism_engine_b200 as p

    env = Env(args)
    be = p.CudaBackend(device=0)
    for kv in args.option:
        key, val = kv.split("=")
        be.set_option(key, int(val))
    c4 = config4_gemm(env, be, bits=args.bits)
    line = {"metric": c4["metric"], "value": c4["value"], "unit": c4["unit"], "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": c4["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 operands / f32 accumulate", "data": "synthetic",
            "config": {"workload": c4["workload"], "l2_policy": c4["l2_policy"]},
            "roofline": c4["roofline"], "per_gemm": c4["per_gemm"], "e2e": c4["e2e"], "gpu_launches": c4["gpu_launches"],
            "clocks": c4["clocks"]}
    emit(line)
    be.close()
    return 0


_RESULT_FD = None


def emit(line):
    """Writes the result line to the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    # Libraries loaded by the run (NCCL prints its version banner) write to file descriptor 1;
    # the contract is ONE JSON line on stdout, so everything else is routed to stderr.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen2.5-72b-decode", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--bits", type=int, default=4, choices=[2, 4], help="palette width of the prefill-GEMM workload")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling/debugging only)")
    ap.add_argument("--ctx", type=int, default=-1, help="override the prompt context length (profiling/debugging only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemv-shapes", action="store_true")
    ap.add_argument("--no-batches", action="store_true", help="skip the batch 8 / batch 32 sub-measurements")
    ap.add_argument("--no-configs", action="store_true", help="skip the config3 / config4 sub-measurements")
    ap.add_argument("--option", action="append", default=[], metavar="KEY=INT",
                    help="backend tunable (gemv_variant, gemm_variant, fuse, pdl); profiling/debugging only")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.workload.endswith("prefill-gemm"):
        if args.impl == "reference":
            emit({"impl": "reference", "unavailable": "the reference arm times decode; run the decode workloads"})
            return 0
        return run_gemm(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
