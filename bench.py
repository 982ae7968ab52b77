#!/usr/bin/env python
"""Benchmark driver: BERT-base (seq 128, batch 1, fp32) forward passes per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass of the seeded BERT-base ONNX model over one sequence.

  ours        the model is compiled with Executor.make_dp_greedy (DP layout search + greedy
              arena) and replayed as a CUDA graph.
                value  sequences/s with inputs resident in HBM: Executor epoch = K, CUDA events
                       on the launching stream around the K replays;
                e2e    sequences/s through Executor.invoke with pinned HOST buffers, one call
                       per step, host-to-device and device-to-host copies inside the timed
                       region (host clock around K calls; each call returns after its own
                       synchronisation).
              N > 1: one process per GPU (torchrun), each an independent replica of the same
              model on its own sequences; no data-path collective.  value = N / max-over-ranks
              time per step.
  reference   FluidML's CPU execution of the same graph: the oracle's unfused, single-thread
              restatement (the reference itself needs LLVM/MLIR 18 and cannot be built here).
              Each step runs a bounded sample of the encoder layers and is scaled to 12.

Synthetic data: weights N(0, 0.02) from PCG64(0), input_ids uniform from PCG64(1), mask ones.
The 342 MB of weights exceed the 126 MB L2, so every pass streams them from HBM; no explicit
L2 flush is needed between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bert_base_s128_sequences_per_sec"
UNIT = "sequences/s"
LAYERS, HIDDEN, HEADS, FFN, SEQ = 12, 768, 12, 3072, 128


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def gemm_algorithmic_bytes():
    """Bytes every tensor-core GEMM launch of one forward pass must move (each operand once,
    result once, bias/residual once), and the launch count: four per layer (the attention
    products run inside the fused attention kernel, the pooler on the skinny kernel)."""
    S, H, F = SEQ, HIDDEN, FFN
    f4 = 4
    proj = lambda k, n, extra=0: (S * k + k * n + S * n + n + extra) * f4
    per_layer = [proj(H, 3 * H)]                       # q, k, v merged into one product (+bias)
    per_layer += [proj(H, H, S * H)]                   # out-proj + bias + residual
    per_layer += [proj(H, F)]                          # FFN1 + bias + GELU
    per_layer += [proj(F, H, S * H)]                   # FFN2 + bias + residual
    return sum(per_layer) * LAYERS, len(per_layer) * LAYERS


class ClockSampler:
    """nvidia-smi clock / throttle samples during the timed region."""

    def __init__(self, device: int):
        self.rows, self.proc = [], None
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={device}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def dist_setup(n):
    if n <= 1:
        return None, 0, 0
    import torch
    import torch.distributed as dist
    rank, local = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    try:
        torch.cuda.set_device(local)
        dist.init_process_group("nccl")
        backend = "nccl"
    except Exception:
        dist.init_process_group("gloo")
        backend = "gloo"
    return (dist, backend), rank, local


def dist_max(ctx, local, value: float) -> float:
    if ctx is None:
        return value
    import torch
    dist, backend = ctx
    t = torch.tensor([value], dtype=torch.float64, device=f"cuda:{local}" if backend == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def dist_barrier(ctx):
    if ctx is not None:
        ctx[0].barrier()


def host_threads() -> int:
    """Host threads the CPU arm uses: all the process may run on."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_baseline(sample_layers: int, repeats: int = 1):
    """Oracle (unfused, i-k-j matmul loops; the rows of every matrix product spread over all host
    threads, which changes no bit) on `sample_layers` encoder layers, scaled to 12 layers.
    Returns (sequences/s, seconds per sample)."""
    from fluidml_b200 import models
    from oracle import oracle as orc
    orc.set_threads(host_threads())
    m = models.build_bert(layers=sample_layers)
    x = models.bert_inputs()
    best = None
    for _ in range(repeats):
        t = time.perf_counter()
        orc.run_model(m, x, acc64=False, order=1)
        dt = time.perf_counter() - t
        best = dt if best is None else min(best, dt)
    full = best * LAYERS / sample_layers
    return 1.0 / full, best


def concurrent_streams(onnx_bytes, model, seeds, steps, n_streams=4):
    """Extra figure beside the headline: `n_streams` executors (each with its own stream, arena
    and graph) replaying at once on one GPU.  A single batch-1 pass leaves most SMs idle, so
    independent requests overlap; the headline `value` stays the single-stream latency figure."""
    from fluidml_b200.executor import Executor, pinned_empty
    exs = []
    for _ in range(n_streams):
        ex = Executor.make_dp_greedy("bert", steps).compile(onnx_bytes)
        host = {vi.name: pinned_empty(vi.shape, {1: np.float32, 7: np.int64}[vi.dtype])
                for vi in (*model.inputs, *model.outputs)}
        for k, v in seeds.items():
            host[k][...] = v
        ex.invoke(host)
        exs.append((ex, host))
    res = [0.0] * n_streams

    def run(i):
        res[i] = exs[i][0].invoke(exs[i][1])

    t0 = time.perf_counter()
    threads = [threading.Thread(target=run, args=(i,)) for i in range(n_streams)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    return {"streams": n_streams, "value": n_streams * steps / wall, "unit": UNIT,
            "timing": "wall clock over all streams' replays, host threads included",
            "ms_per_pass_per_stream": [r * 1e-6 for r in res]}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    # bound the whole run to a few minutes: ~0.7 s of CPU work per encoder layer on one thread
    budget = 150.0
    per_layer = 0.7 / min(8, host_threads()) + 0.05
    sample = int(max(1, min(LAYERS, budget / (per_layer * (args.steps + args.warmup)))))
    from fluidml_b200 import models
    from oracle import oracle as orc
    orc.set_threads(host_threads())
    m = models.build_bert(layers=sample)
    x = models.bert_inputs()
    for _ in range(args.warmup):
        orc.run_model(m, x, order=1)
    t = time.perf_counter()
    for _ in range(args.steps):
        orc.run_model(m, x, order=1)
    per_step = (time.perf_counter() - t) / args.steps * LAYERS / sample
    value = 1.0 / per_step
    desc = (f"{sample} of {LAYERS} encoder layers (+ embeddings and pooler) per step, time scaled by "
            f"{LAYERS}/{sample}; oracle port of the reference's unfused execution, i-k-j matmul loops, matrix-product "
            f"rows over {host_threads()} host threads (the reference itself runs on one)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BERT-base encoder+pooler fp32, batch 1, seq 128 (configs[0])"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": host_threads(), "kind": "port", "sample": desc,
                         "host_cores_available": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    ctx, rank, local = dist_setup(args.gpus)
    os.environ["FLUIDML_DEVICE"] = str(local)
    from fluidml_b200 import models
    from fluidml_b200.executor import Executor, pinned_empty

    model = models.build_bert()
    onnx_bytes = model.to_bytes()
    seeds = models.bert_inputs(seed=1 + rank)

    # host buffers in pinned memory, as a serving front end would hold them
    host = {}
    for vi in (*model.inputs, *model.outputs):
        host[vi.name] = pinned_empty(vi.shape, {1: np.float32, 7: np.int64}[vi.dtype])
    for k, v in seeds.items():
        host[k][...] = v
    h2d = sum(host[v.name].nbytes for v in model.inputs)
    d2h = sum(host[v.name].nbytes for v in model.outputs)

    ex_loop = Executor.make_dp_greedy("bert", args.steps).compile(onnx_bytes)  # K replays per invoke
    ex_one = Executor.make_dp_greedy("bert", 1).compile(onnx_bytes)
    stats = ex_one.stats()

    # warm-up
    for _ in range(args.warmup):
        ex_one.invoke(host)
    ex_loop.invoke(host)

    dist_barrier(ctx)
    sampler = ClockSampler(local) if rank == 0 else None
    # ---- device-timed: K graph replays between two events, inputs already in HBM
    ns = ex_loop.invoke(host)
    dev_s = dist_max(ctx, local, ns * 1e-9)
    dist_barrier(ctx)
    # ---- end to end: K public-API calls with host buffers
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ex_one.invoke(host)
    e2e_s = dist_max(ctx, local, (time.perf_counter() - t0) / args.steps)
    dist_barrier(ctx)
    clocks = sampler.stop() if sampler else None

    if ctx is not None:
        ctx[0].destroy_process_group()
    if rank != 0:
        return
    value = args.gpus / dev_s
    e2e = args.gpus / e2e_s

    # ---- roofline of the dominant kernel (the tcgen05 GEMM), measured live
    peak, peak_kind = measured_peaks()
    prof = ex_one.profile({k: host[k] for k in seeds}, passes=3)
    # FusedGemmKernel launches: 48 tensor-core GEMMs per pass + the pooler (skinny kernel, ~1 % of
    # the time); MatMulKernel appears only when the attention fusion is off
    gemm_us = sum(v["us"] for k, v in prof.items() if k in ("FusedGemmKernel", "MatMulKernel"))
    gemm_launches = sum(v["launches"] for k, v in prof.items() if k in ("FusedGemmKernel", "MatMulKernel"))
    alg_bytes, alg_launches = gemm_algorithmic_bytes()
    passes = max(1, gemm_launches // max(1, alg_launches))
    achieved = (alg_bytes * passes) / (gemm_us * 1e-6) / 1e9 if gemm_us else None
    total_us = sum(v["us"] for k, v in prof.items() if not k.startswith("("))
    empty_us = prof.get("(empty event pair)", {"us": 0, "launches": 1})
    roofline = {
        "bound": "hbm", "kernel": "gemm_tc_kernel (FusedGemmKernel launches)",
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if achieved else None,
        "peak_source": peak_kind,
        # DRAM bytes per launch: the ncu capture of the FFN2 shape (profiles/) read 11.069 MB and
        # wrote 0 for 11.403 MB of algorithmic bytes; scaled to the average launch by that ratio.
        "traffic": 0.9707 * alg_bytes / alg_launches,
        "traffic_source": "ncu dram__bytes_read+write of one shape, scaled by algorithmic bytes",
        "algorithmic_bytes_per_launch": alg_bytes / alg_launches,
        "avg_launch_us": gemm_us / gemm_launches if gemm_launches else None,
        "share_of_kernel_time": gemm_us / total_us if total_us else None,
        "empty_event_pair_us": empty_us["us"] / max(1, empty_us["launches"]),
    }
    # whole-model roofline: every byte the fused plan must move / HBM peak (weights dominate)
    model_bytes = 513.9e6
    model_roofline = {"t_roof_us": model_bytes / (peak * 1e9) * 1e6, "t_measured_us": dev_s * 1e6,
                      "frac": (model_bytes / (peak * 1e9)) / dev_s}

    cpu_value, cpu_secs = cpu_baseline(sample_layers=LAYERS, repeats=8) if args.gpus == 1 else (None, None)
    streams = concurrent_streams(onnx_bytes, model, seeds, args.steps) if args.gpus == 1 else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BERT-base encoder+pooler fp32, batch 1, seq 128 (configs[0]); one replica per GPU",
                   "executor": "make_dp_greedy", "gemm": "tcgen05 3xTF32",
                   "l2": "342 MB of weights per pass exceed the 126 MB L2; no flush between iterations"},
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(stats["launches"]) * args.steps,
        "launches_per_step": int(stats["launches"]),
        "clocks": clocks,
        "roofline": roofline,
        "model_roofline": model_roofline,
        "peak_arena_bytes": stats["peak_arena_bytes"],
        "reference_arena_bytes_greedy": stats["reference_arena_bytes_greedy"],
        "kernel_time_us_per_pass": {k: v["us"] / 3 for k, v in prof.items()},
    }
    if streams is not None:
        line["concurrent_streams"] = streams
    if cpu_value is not None:
        line["cpu_baseline"] = {"value": cpu_value, "unit": UNIT, "cores": host_threads(), "kind": "port",
                                "host_cores_available": os.cpu_count(),
                                "sample": f"the whole model (12 encoder layers, embeddings, pooler), best of 8 passes of "
                                          f"{cpu_secs:.1f} s; oracle port of the reference's unfused execution, "
                                          "matrix-product rows over all host threads (the reference itself runs on one)"}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
