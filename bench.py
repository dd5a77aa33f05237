#!/usr/bin/env python
"""Benchmark of the palettized-LUT decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one greedy decode step (one token per sequence) of a random-init,
4-bit palettized model -- every palettized GEMV of the model once, plus the
decode glue.  Default workload: the Qwen2.5-72B architecture (80 layers, hidden
8192, 64/8 heads, intermediate 29568, vocab 152064), batch 1, decoding after a
512-token prompt, tensor-parallel over N GPUs (column/row-sharded linears, NCCL
all-reduce).  Weights are seeded synthetic tensors generated on the device
(no checkpoint is available offline); total work is fixed as N grows (strong
scaling).  The JSON line printed by rank 0 follows the driver's contract; see
the keys below.  `--impl reference` times the CPU restatement of the
reference's own path (the oracle) on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (architecture dict key, prompt context, description)
    "qwen2.5-72b-decode": ("QWEN25_72B", 512),
    "qwen2.5-0.5b-decode": ("QWEN25_0P5B", 128),
    # prefill: the palettized linears of one Qwen2.5-7B layer on M = 2048 tokens (tensor-core GEMM)
    "qwen2.5-7b-prefill-gemm": ("QWEN25_7B", 2048),
}
METRIC = "decode_tokens_per_s"
UNIT = "tok/s"
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (read-only query)."""

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
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def arch_dict(name):
    import prism_engine_b200 as p

    return dict(getattr(p, WORKLOADS[name][0]))


# --------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's path, all host threads
# --------------------------------------------------------------------------------------------
class CpuSample:
    """Bounded sample of one decode step for the host: the seven palettized GEMVs of ONE
    transformer layer (x num_layers) plus the LM head on 1/head_frac of its rows.  Glue ops
    (norm, rope, attention) are not in the sample; on the CPU path they are < 1 % of a step."""

    def __init__(self, arch, threads, head_frac=8):
        from prism_engine_b200 import synth

        self.arch, self.threads = arch, threads
        H, I, V = arch["hidden_size"], arch["intermediate_size"], arch["vocab_size"]
        qd = arch["num_heads"] * arch["head_dim"]
        kvd = arch["num_kv_heads"] * arch["head_dim"]
        self.shapes = [(qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I)]
        self.pay = [synth.make_payload(m, k, 4, seed=i) for i, (m, k) in enumerate(self.shapes)]
        self.xs = {k: synth.make_activation(k, seed=k) for _, k in self.shapes}
        self.vrows = max(64, V // head_frac // 64 * 64)
        self.head = synth.make_payload(self.vrows, H, 4, seed=99)
        self.sample = (f"7 palettized GEMVs of one layer (extrapolated x{arch['num_layers']} layers) + "
                       f"{self.vrows}/{V} LM-head rows, lut_gemv restatement over {threads} threads")

    def token_seconds(self):
        from oracle import oracle as orc

        a = self.arch
        t0 = time.perf_counter()
        for (m, k), p in zip(self.shapes, self.pay):
            orc.lut_gemv(self.xs[k], p, m, k, threads=self.threads)
        t_layer = time.perf_counter() - t0
        t0 = time.perf_counter()
        orc.lut_gemv(self.xs[a["hidden_size"]], self.head, self.vrows, a["hidden_size"], threads=self.threads)
        t_head = (time.perf_counter() - t0) * (a["vocab_size"] / self.vrows)
        return t_layer * a["num_layers"] + t_head


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import oracle as orc

    arch = arch_dict(args.workload)
    threads = orc.max_threads()
    cs = CpuSample(arch, threads)
    sample = cs.sample
    times = []
    for i in range(args.warmup + args.steps):
        t = cs.token_seconds()
        if i >= args.warmup:
            times.append(t)
    per_tok = statistics.mean(times)
    value = args.batch / per_tok
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_tok * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights / f32 accumulate", "data": "synthetic",
        "config": workload_config(args, arch),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
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
def run_ours(args):
    import torch

    import prism_engine_b200 as p

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", local))
    be = p.CudaBackend(device=local)
    for kv in args.option:
        key, val = kv.split("=")
        be.set_option(key, int(val))
    if world > 1:
        from prism_engine_b200 import tp

        uid = tp.exchange_unique_id(p.CudaBackend.tp_unique_id)
        be.tp_init(world, rank, uid)
    arch = arch_dict(args.workload)
    if args.layers:
        arch["num_layers"] = args.layers
    ctx_len = WORKLOADS[args.workload][1] if args.ctx < 0 else args.ctx
    B = args.batch
    total_steps = ctx_len + 2 * (args.warmup + args.steps) + 8
    mc = p.model_config(**arch, max_seq=total_steps, max_batch=B, profile="baseline")
    eng = p.PrismEngine(be, mc)
    eng.synth_weights(seed=1)
    from prism_engine_b200 import synth

    prompts = np.stack([synth.make_prompt(ctx_len, arch["vocab_size"], seed=b) for b in range(B)])
    eng.generate(prompts, 0)  # prefill: one step per prompt token (untimed)

    def barrier():
        be.synchronize()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    tok_pinned = torch.from_numpy(prompts[:, -1].astype(np.int64)).to(torch.int32).pin_memory()
    out_pinned = torch.empty((B, max(args.steps, args.warmup, 1)), dtype=torch.int32).pin_memory()
    # ---- device-resident throughput: K steps replayed on the device, no host traffic in between
    if args.warmup:
        eng.decode(None, args.warmup, tokens_ptr=tok_pinned.data_ptr(), out_ptr=out_pinned.data_ptr())
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    l0 = be.launch_count()
    eng.decode(None, args.steps, tokens_ptr=tok_pinned.data_ptr(), out_ptr=out_pinned.data_ptr())
    barrier()
    dev_ms = max_over_ranks(eng.last_device_ms())
    graph_launches = be.launch_count() - l0
    kps = eng.kernels_per_step()
    # ---- end to end: one public-API call per step, token in from pinned host memory, token out
    nxt = torch.empty(B, dtype=torch.int32).pin_memory()
    L = eng.L
    for _ in range(args.warmup):
        eng._ck(L.prism_cuda_engine_step(eng.h, tok_pinned.data_ptr(), nxt.data_ptr(), None))
        tok_pinned.copy_(nxt)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        eng._ck(L.prism_cuda_engine_step(eng.h, tok_pinned.data_ptr(), nxt.data_ptr(), None))
        tok_pinned.copy_(nxt)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if sampler else None
    step_bytes = eng.step_bytes()
    # ---- dominant kernel alone: every palettized GEMV of the model, back to back, between events
    gemv_ms, gemv_bytes, gemv_launches = eng.profile_gemv(reps=2)
    gemv_ms = max_over_ranks(gemv_ms)
    peak, peak_kind = measured_peaks()
    achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9
    value = B * args.steps / (dev_ms * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 weights / f32 accumulate", "data": "synthetic",
        "config": workload_config(args, arch),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8tbs_nominal": achieved / 8000.0,
                     "kernel": "lut_gemv_ws_kernel (lut_gemv_sk_kernel for small matrices)", "launches_timed": gemv_launches,
                     "avg_launch_us": gemv_ms * 1e3 / max(gemv_launches, 1),
                     "algorithmic_bytes_per_launch": gemv_bytes / max(gemv_launches, 1),
                     "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE and TRAFFIC_PER_ALGORITHMIC_BYTE * gemv_bytes / max(gemv_launches, 1)},
        "step_roofline": {"algorithmic_bytes_per_step_per_gpu": step_bytes,
                          "achieved_gbs_per_gpu": step_bytes / (dev_ms / args.steps * 1e-3) / 1e9,
                          "frac": step_bytes / (dev_ms / args.steps * 1e-3) / 1e9 / peak},
        "e2e": {"value": B * args.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": 4 * B,
                "d2h_bytes_per_step": 4 * B, "ms_per_step": e2e_s / args.steps * 1e3},
        "gpu_launches": kps * args.steps, "kernels_per_step": kps, "graph_launches": graph_launches,
        "clocks": clocks,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as orc

            threads = orc.max_threads()
            cs = CpuSample(arch_dict(args.workload), threads)
            cs.token_seconds()
            per_tok = statistics.median([cs.token_seconds() for _ in range(3)])
            line["cpu_baseline"] = {"value": B / per_tok, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": cs.sample + "; median of 3"}
        if world == 1 and not args.no_gemv_shapes:
            line["lut_gemv_0p5b_shapes"] = small_shape_bandwidth(be, peak)
        emit(line)
    eng.close()
    be.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# DRAM bytes per algorithmic byte of the GEMV launches of a 72B decode step, from the ncu capture
# summarised in profiles/lut_gemv_ws_kernel_qwen72b_shapes.md (the five launch shapes together:
# 1083.3 MB of DRAM traffic for 1069.8 MB of algorithmic bytes).
TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0126


def small_shape_bandwidth(be, peak):
    """LUT-GEMV bandwidth at the Qwen2.5-0.5B MLP shapes (4864x896 / 896x4864).  A single 2.3 MB GEMV
    is launch-bound and L2-resident, so each measurement cycles through 160 distinct weight sets
    (> 126 MB of L2) inside one CUDA graph."""
    from prism_engine_b200 import synth

    n_sets, reps = 160, 5
    gate = [be.synth(f"bw.gate{i}", 4864, 896, seed=1000 + i) for i in range(n_sets)]
    up = [be.synth(f"bw.up{i}", 4864, 896, seed=2000 + i) for i in range(n_sets)]
    down = [be.synth(f"bw.down{i}", 896, 4864, seed=3000 + i) for i in range(n_sets)]
    out = {}
    b1 = synth.gemv_algorithmic_bytes(4864, 896)
    b2 = 2 * b1 - 2 * 896
    b3 = b2 + synth.gemv_algorithmic_bytes(896, 4864)
    for name, kind, hs, nbytes in (("gemv_4864x896", 0, gate, b1),
                                   ("fused_gate_up_swiglu", 1, list(zip(gate, up)), b2),
                                   ("mlp_gate_up_down", 2, list(zip(gate, up, down)), b3)):
        ms = be.bench_cycle(kind, np.array(hs, np.int32), reps)
        gbs = nbytes * n_sets * reps / (ms * 1e-3) / 1e9
        out[name] = {"gbs": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_8tbs_nominal": gbs / 8000.0,
                     "us_per_call": ms * 1e3 / (n_sets * reps), "algorithmic_bytes": nbytes}
    for h in gate + up + down:
        be.free(h)
    return out


def measured_tensor_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 1400.0, 1590.0, "fallback"


def run_gemm(args):
    """Prefill GEMM workload: q, k, v, gate, up, down of one Qwen2.5-7B layer, 4-bit palettized, on
    M = 2048 tokens of fp16 activations.  A step is the six GEMMs once; the metric is TFLOP/s."""
    import torch

    import prism_engine_b200 as p

    torch.cuda.set_device(0)
    be = p.CudaBackend(device=0)
    for kv in args.option:
        key, val = kv.split("=")
        be.set_option(key, int(val))
    arch = arch_dict(args.workload)
    H, I = arch["hidden_size"], arch["intermediate_size"]
    kvd = arch["num_kv_heads"] * arch["head_dim"]
    m_tok = WORKLOADS[args.workload][1]
    shapes = [("q", H, H), ("k", kvd, H), ("v", kvd, H), ("gate", I, H), ("up", I, H), ("down", H, I)]
    sampler = ClockSampler(0)
    per = {}
    total_ms, total_flop = 0.0, 0.0
    hs = {n: be.synth(f"gemm.{n}", m, k, seed=i) for i, (n, m, k) in enumerate(shapes)}
    for n, m, k in shapes:
        be.bench_gemm(hs[n], m_tok, max(args.warmup, 3))
    sampler.start()
    l0 = be.launch_count()
    for n, m, k in shapes:
        ms = be.bench_gemm(hs[n], m_tok, args.steps) / args.steps
        flop = 2.0 * m_tok * m * k
        per[n] = {"shape": f"{m}x{k}", "ms": ms, "tflops": flop / ms / 1e9}
        total_ms += ms
        total_flop += flop
    launches = be.launch_count() - l0
    clocks = sampler.stop()
    sustained, burst, kind = measured_tensor_peak()
    value = total_flop / total_ms / 1e9
    big = per["gate"]["tflops"]
    # end to end: host activations in, host result out, through the public GEMM call
    from prism_engine_b200 import synth

    X = synth.make_activation((m_tok, H), seed=1)
    be.gemm(hs["gate"], X)
    t0 = time.perf_counter()
    reps = 3
    for _ in range(reps):
        be.gemm(hs["gate"], X)
    e2e_s = (time.perf_counter() - t0) / reps
    line = {
        "metric": "prefill_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands / f32 accumulate", "data": "synthetic",
        "config": {"workload": f"{args.workload}: q/k/v/gate/up/down of one layer, M = {m_tok} tokens, 4-bit indices + "
                               "16-entry fp16 palette per row", "l2_policy": "operands of consecutive GEMMs exceed L2"},
        "roofline": {"bound": "tensor", "achieved": big, "peak": sustained, "unit": "TFLOP/s", "frac": big / sustained,
                     "peak_kind": f"of {kind} (sustained bf16 cuBLAS; burst {burst})", "kernel": "lut_gemm_tc5_kernel",
                     "launch": "gate 18944x3584, M=2048", "traffic": None},
        "per_gemm": per,
        "e2e": {"value": 2.0 * m_tok * I * H / e2e_s / 1e12, "unit": "TFLOP/s (gate GEMM through prism_cuda_gemm, host buffers)",
                "h2d_bytes_per_step": int(X.nbytes), "d2h_bytes_per_step": m_tok * I * 2},
        "gpu_launches": launches, "clocks": clocks,
    }
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
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling/debugging only)")
    ap.add_argument("--ctx", type=int, default=-1, help="override the prompt context length (profiling/debugging only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemv-shapes", action="store_true")
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
