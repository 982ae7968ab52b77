#!/usr/bin/env python
"""Benchmark driver.  Headline: BERT-base (seq 128, batch 1, fp32) forward passes per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config bert_b1|vgg16_b1|vgg16_b32|effnet_b1|effnet_b64|convbert_b8|gptneox_b4s512]
                    [--repeats R]

One "step" is one forward pass of the seeded ONNX model of the chosen configuration (the
default, bert_b1, is the configuration the metric is quoted on).

  ours        the model is compiled with Executor.make_dp_greedy (DP layout search + greedy
              arena) and replayed as a CUDA graph.
                value  units/s with inputs resident in HBM: Executor epoch = K, CUDA events on the
                       launching stream around the K replays; that measurement is repeated R
                       times (default 25) and `ms_per_step` is the median, with the minimum and
                       maximum beside it;
                e2e    units/s through Executor.invoke with pinned HOST buffers, one call per
                       step, host-to-device and device-to-host copies inside the timed region
                       (host clock around K calls; each call returns after its own
                       synchronisation).
              N > 1: one process per GPU (torchrun), each an independent replica of the same
              model on its own inputs; no data-path collective.  value = N x units per step /
              max-over-ranks time per step.
  reference   FluidML's CPU execution of the same graph: the oracle's unfused restatement (the
              reference itself needs LLVM/MLIR 18 and cannot be built here), matrix-product rows
              spread over all host threads.  Each step runs a bounded sample and is scaled.

Roofline entry.  The dominant kernel's time is taken INSIDE the replayed graph, from the
kernel-start stamps every kernel of the library writes when a trace buffer is set
(Executor.trace): a launch's period runs from its start to the next launch's start, so the
periods of a pass add up to the pass.  `traffic` scales the DRAM bytes of the committed ncu
capture named in `traffic_source` (read from that file at run time) by algorithmic bytes.

Synthetic data: weights and inputs are drawn from PCG64 seeds by fluidml_b200.models.  BERT's
342 MB of weights exceed the 126 MB L2, so every pass streams them from HBM; configurations whose
working set fits in L2 say so in `config.l2`.
"""
from __future__ import annotations

import argparse
import contextlib
import io
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, HIDDEN, HEADS, FFN, SEQ = 12, 768, 12, 3072, 128
NP_OF = {1: np.float32, 7: np.int64}


def configs():
    from fluidml_b200 import models as M
    return {
        "bert_b1": dict(build=lambda: M.build_bert(), inputs=lambda s: M.bert_inputs(seed=s), units=1,
                        metric="bert_base_s128_sequences_per_sec", unit="sequences/s",
                        workload="BERT-base encoder+pooler fp32, batch 1, seq 128 (configs[0])",
                        cpu=lambda layers: M.build_bert(layers=layers), cpu_scale=("layers", LAYERS)),
        "vgg16_b1": dict(build=lambda: M.build_vgg16(batch=1), inputs=lambda s: M.vgg_inputs(seed=s, batch=1), units=1,
                         metric="vgg16_b1_images_per_sec", unit="images/s", workload="VGG-16 fp32, 224x224, batch 1 (configs[1])"),
        "vgg16_b32": dict(build=lambda: M.build_vgg16(batch=32), inputs=lambda s: M.vgg_inputs(seed=s, batch=32), units=32,
                          metric="vgg16_b32_images_per_sec", unit="images/s", workload="VGG-16 fp32, 224x224, batch 32 (configs[1])"),
        "effnet_b1": dict(build=lambda: M.build_efficientnet_b0(batch=1), inputs=lambda s: M.efficientnet_inputs(seed=s, batch=1), units=1,
                          metric="efficientnet_b0_b1_images_per_sec", unit="images/s",
                          workload="EfficientNet-B0 fp32, 224x224, batch 1 (configs[2])"),
        "effnet_b64": dict(build=lambda: M.build_efficientnet_b0(batch=64), inputs=lambda s: M.efficientnet_inputs(seed=s, batch=64), units=64,
                           metric="efficientnet_b0_b64_images_per_sec", unit="images/s",
                           workload="EfficientNet-B0 fp32, 224x224, batch 64 (configs[2])"),
        "convbert_b8": dict(build=lambda: M.build_convbert(batch=8, seq=128), inputs=lambda s: M.convbert_inputs(seed=s, batch=8, seq=128), units=8,
                            metric="convbert_base_b8_s128_sequences_per_sec", unit="sequences/s",
                            workload="ConvBERT-base fp32, batch 8, seq 128 (configs[3])"),
        "gptneox_b4s512": dict(build=lambda: M.build_gpt_neox(batch=4, seq=512), inputs=lambda s: M.gpt_neox_inputs(seed=s, batch=4, seq=512), units=4,
                               metric="gpt_neox_410m_prefill_b4_s512_sequences_per_sec", unit="sequences/s",
                               workload="GPT-NeoX (Pythia-410M shape) fp32 prefill, batch 4, seq 512 (configs[4])"),
    }


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------ algorithmic work of a model
CONTRACTIONS = ("MatMul", "Gemm", "Conv")
ROW_OPS = ("LayerNormalization", "Softmax", "MaxPool", "AveragePool", "GlobalAveragePool", "ReduceMean", "Gather")


def model_work(model):
    """Per ONNX node class: flops (2 per multiply-add, counted once whatever the TF32 split) and
    compulsory bytes (operands read once, result written once).  Element-wise operators ride in
    the epilogues of the plan and count nothing; reshapes and transposes are addressing."""
    def shape(name):
        vi = model.info(name)
        return tuple(vi.shape) if vi is not None else ()

    def nbytes(name):
        vi = model.info(name)
        if vi is None:
            return 0
        return int(np.prod(vi.shape, dtype=np.int64)) * (8 if vi.dtype == 7 else 1 if vi.dtype == 9 else 4)

    rows = []
    for n in model.nodes:
        if n.op_type not in CONTRACTIONS and n.op_type not in ROW_OPS:
            continue
        out = shape(n.outputs[0])
        flops = 0
        if n.op_type == "MatMul":
            k = shape(n.inputs[0])[-1]
            flops = 2 * int(np.prod(out, dtype=np.int64)) * k
        elif n.op_type == "Gemm":
            a = shape(n.inputs[0])
            k = a[0] if n.attrs.get("transA", 0) else a[-1]
            flops = 2 * int(np.prod(out, dtype=np.int64)) * k
        elif n.op_type == "Conv":
            w = shape(n.inputs[1])  # [OC, IC / group, k...]
            flops = 2 * int(np.prod(out, dtype=np.int64)) * int(np.prod(w[1:], dtype=np.int64))
        b = sum(nbytes(i) for i in n.inputs if i) + sum(nbytes(o) for o in n.outputs)
        if n.op_type == "Gather":  # only the gathered rows move
            b = 2 * nbytes(n.outputs[0]) + nbytes(n.inputs[1])
        op = n.op_type
        if op == "Conv":  # the two kernel classes of the reference: padded or not
            op = "ConvWithPadding" if any(int(v) for v in n.attrs.get("pads", [])) else "ConvWithoutPadding"
        rows.append((op, flops, b))
    return rows


def roofline_time_us(rows, p_tc_tflops, bw_gbs):
    """T_roof = sum over kernels of max(F / P_tc, B / BW)."""
    t = 0.0
    for _, f, b in rows:
        t += max(f / (p_tc_tflops * 1e12), b / (bw_gbs * 1e9))
    return t * 1e6


def gemm_algorithmic_bytes():
    """Bytes every tensor-core GEMM launch of one BERT forward pass must move (each operand once,
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


def captured_traffic_ratio():
    """DRAM bytes per algorithmic byte of the tensor-core GEMM, read from the committed ncu summary
    (first capture column): (dram read + dram write) / (A + B + C bytes of that launch)."""
    path = os.path.join(ROOT, "profiles", "gemm_tc_kernel_ffn2_m128_k3072_n768.md")
    try:
        text = open(path).read()
        rd = re.search(r"`dram__bytes_read\.sum`\s*\|\s*([0-9.]+)\s*MB", text)
        wr = re.search(r"`dram__bytes_write\.sum`\s*\|\s*([0-9.]+)\s*(MB|B)", text)
        alg = re.search(r"=\s*([0-9.]+)\s*MB; DRAM traffic", text)
        if not (rd and wr and alg):
            return None, path
        w = float(wr.group(1)) * (1.0 if wr.group(2) == "MB" else 1e-6)
        return (float(rd.group(1)) + w) / float(alg.group(1)), os.path.relpath(path, ROOT)
    except OSError:
        return None, path


class ClockSampler:
    """nvidia-smi clock / throttle samples during the timed region (every 20 ms)."""

    def __init__(self, device: int):
        self.rows, self.proc = [], None
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={device}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
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
        time.sleep(0.1)
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


def cpu_time(model, inputs, repeats: int = 1) -> float:
    """Seconds of one oracle pass (unfused, i-k-j matmul loops; the rows of every matrix product
    spread over all host threads, which changes no bit): best of `repeats`."""
    from oracle import oracle as orc
    orc.set_threads(host_threads())
    best = None
    for _ in range(repeats):
        t = time.perf_counter()
        orc.run_model(model, inputs, acc64=False, order=1)
        dt = time.perf_counter() - t
        best = dt if best is None else min(best, dt)
    return best


def cpu_sample(name, cfg, budget_s: float):
    """(model, inputs, scale, description) of a bounded CPU sample of configuration `name`."""
    from fluidml_b200 import models as M
    if name == "bert_b1":
        return M.build_bert(), M.bert_inputs(), 1.0, "the whole model (12 encoder layers, embeddings, pooler)"
    if name.startswith("vgg16"):
        return M.build_vgg16(batch=1), M.vgg_inputs(batch=1), float(cfg["units"]), "one image (batch 1); images are independent, time scaled by the batch"
    if name.startswith("effnet"):
        return M.build_efficientnet_b0(batch=1), M.efficientnet_inputs(batch=1), float(cfg["units"]), "one image (batch 1); images are independent, time scaled by the batch"
    if name == "convbert_b8":
        return (M.build_convbert(layers=2, batch=1, seq=128), M.convbert_inputs(batch=1, seq=128), 6.0 * 8.0,
                "2 of 12 layers of one sequence; time scaled by 6 x 8 (layers x batch)")
    return (M.build_gpt_neox(layers=2, batch=1, seq=512), M.gpt_neox_inputs(batch=1, seq=512), 12.0 * 4.0,
            "2 of 24 layers of one sequence; time scaled by 12 x 4 (layers x batch)")


def concurrent_streams(onnx_bytes, model, seeds, steps, n_streams=4):
    """Extra figure beside the headline: `n_streams` executors (each with its own stream, arena
    and graph) replaying at once on one GPU.  A single batch-1 pass leaves most SMs idle, so
    independent requests overlap; the headline `value` stays the single-stream latency figure."""
    from fluidml_b200.executor import Executor, pinned_empty
    exs = []
    for _ in range(n_streams):
        ex = Executor.make_dp_greedy("bert", steps).compile(onnx_bytes)
        host = {vi.name: pinned_empty(vi.shape, NP_OF[vi.dtype]) for vi in (*model.inputs, *model.outputs)}
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
    return {"streams": n_streams, "value": n_streams * steps / wall, "unit": "sequences/s",
            "timing": "wall clock over all streams' replays, host threads included",
            "ms_per_pass_per_stream": [r * 1e-6 for r in res]}


def tf32_peak_tflops():
    """Dense TF32 tensor throughput of this GPU, measured once with the library's own single-pass
    tcgen05 GEMM at M = 8192, K = N = 4096 (a stand-in for a vendor-library figure: it is what
    this code base reaches, about half of the bf16 cuBLAS figure)."""
    import ctypes
    from fluidml_b200 import cabi
    from fluidml_b200.cabi import DeviceTensor as DT
    M, K, N = 8192, 4096, 4096
    a, b, c = DT((M, K), np.float32), DT((K, N), np.float32), DT((M, N), np.float32)
    a.buf.zero(); b.buf.zero()
    p = cabi.gemm_autotune(a, b, c, cabi.gemm_params(precision=cabi.GEMM_TF32))  # the library's own tile search
    L = cabi.lib()
    e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
    cabi.check(L.fml_event_create(ctypes.byref(e0)))
    cabi.check(L.fml_event_create(ctypes.byref(e1)))
    for _ in range(3):
        cabi.gemm(a, b, c, params=p)
    best = None
    for _ in range(5):
        cabi.check(L.fml_event_record(e0, None))
        cabi.gemm(a, b, c, params=p)
        cabi.check(L.fml_event_record(e1, None))
        cabi.sync()
        ms = ctypes.c_float()
        cabi.check(L.fml_event_elapsed_ms(e0, e1, ctypes.byref(ms)))
        best = ms.value if best is None else min(best, ms.value)
    return 2.0 * M * K * N / (best * 1e-3) / 1e12


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cfg = configs()[args.config]
    if args.config == "bert_b1":
        # bound the whole run to a few minutes: ~0.7 s of CPU work per encoder layer on one thread
        budget = 150.0
        per_layer = 0.7 / min(8, host_threads()) + 0.05
        sample = int(max(1, min(LAYERS, budget / (per_layer * (args.steps + args.warmup)))))
        from fluidml_b200 import models
        model, inputs, scale = models.build_bert(layers=sample), models.bert_inputs(), LAYERS / sample
        what = f"{sample} of {LAYERS} encoder layers (+ embeddings and pooler) per step, time scaled by {LAYERS}/{sample}"
    else:
        model, inputs, scale, what = cpu_sample(args.config, cfg, 150.0)
    from oracle import oracle as orc
    orc.set_threads(host_threads())
    for _ in range(args.warmup):
        orc.run_model(model, inputs, order=1)
    t = time.perf_counter()
    for _ in range(args.steps):
        orc.run_model(model, inputs, order=1)
    per_step = (time.perf_counter() - t) / args.steps * scale
    value = cfg["units"] / per_step
    desc = (f"{what}; oracle port of the reference's unfused execution, i-k-j matmul loops, matrix-product "
            f"rows over {host_threads()} host threads (the reference itself runs on one)")
    print(json.dumps({
        "impl": "reference", "metric": cfg["metric"], "value": value, "unit": cfg["unit"], "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["workload"]},
        "cpu_baseline": {"value": value, "unit": cfg["unit"], "cores": host_threads(), "kind": "port", "sample": desc,
                         "host_cores_available": os.cpu_count()},
        "e2e": {"value": value, "unit": cfg["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    ctx, rank, local = dist_setup(args.gpus)
    os.environ["FLUIDML_DEVICE"] = str(local)
    from fluidml_b200.executor import Executor, pinned_empty

    cfg = configs()[args.config]
    headline = args.config == "bert_b1"
    model = cfg["build"]()
    onnx_bytes = model.to_bytes()
    from fluidml_b200 import replicas
    # one input set per replica, dealt to the ranks as the replica path deals independent items
    seeds = cfg["inputs"](replicas.shard(list(range(1, args.gpus + 1)), rank, args.gpus)[0])

    # host buffers in pinned memory, as a serving front end would hold them
    host = {}
    for vi in (*model.inputs, *model.outputs):
        host[vi.name] = pinned_empty(vi.shape, NP_OF[vi.dtype])
    for k, v in seeds.items():
        host[k][...] = v
    h2d = sum(host[v.name].nbytes for v in model.inputs)
    d2h = sum(host[v.name].nbytes for v in model.outputs)

    ex_loop = Executor.make_dp_greedy(model.name, args.steps).compile(onnx_bytes)  # K replays per invoke
    ex_one = Executor.make_dp_greedy(model.name, 1).compile(onnx_bytes)
    stats = ex_one.stats()

    # warm-up
    for _ in range(args.warmup):
        ex_one.invoke(host)
    ex_loop.invoke(host)

    dist_barrier(ctx)
    sampler = ClockSampler(local) if rank == 0 else None
    # ---- device-timed: K graph replays between two events, inputs already in HBM; R repeats
    per_step = []
    for _ in range(args.repeats):
        per_step.append(ex_loop.invoke(host) * 1e-9)
    dev_s = dist_max(ctx, local, float(np.median(per_step)))
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
    units = cfg["units"]
    # every rank runs `units` per step; the job's rate is all of them over the slowest rank's time
    value = replicas.aggregate_throughput([units] * args.gpus, [dev_s] * args.gpus)
    e2e = replicas.aggregate_throughput([units] * args.gpus, [e2e_s] * args.gpus)

    # ---- where the pass goes, inside the graph (kernel-start stamps)
    peak, peak_kind = measured_peaks()
    try:
        trace = ex_one.trace({k: host[k] for k in seeds}, passes=9)
        kernels, pass_us, timing = trace["kernels"], trace["pass_us"], "kernel-start stamps inside the replayed graph (period = start to next start; periods add up to the pass)"
    except RuntimeError:
        prof = ex_one.profile({k: host[k] for k in seeds}, passes=3)
        kernels = {k: {"us": v["us"] / 3, "launches": v["launches"] // 3} for k, v in prof.items() if not k.startswith("(")}
        pass_us, timing = sum(v["us"] for v in kernels.values()), "event pair around every eager launch (this model's launch list does not stamp once per launch)"
    p_tc = tf32_peak_tflops() if args.gpus == 1 else None
    rows = model_work(model)
    flops = sum(f for _, f, _ in rows)
    nbytes = sum(b for _, _, b in rows)

    line = {
        "metric": cfg["metric"], "value": value, "unit": cfg["unit"], "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_s * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["workload"], "replicas": "one per GPU",
                   "executor": "make_dp_greedy", "gemm": "tcgen05 3xTF32",
                   "l2": ("342 MB of weights per pass exceed the 126 MB L2; no flush between iterations" if headline else
                          f"{stats.get('weight_bytes', 0) / 1e6:.0f} MB of weights and a {stats['peak_arena_bytes'] / 1e6:.1f} MB arena per pass; "
                          "no flush between iterations")},
        "ms_per_step_repeats": {"repeats": args.repeats, "median": float(np.median(per_step)) * 1e3,
                                "min": float(np.min(per_step)) * 1e3, "max": float(np.max(per_step)) * 1e3},
        "e2e": {"value": e2e, "unit": cfg["unit"], "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(stats["launches"]) * args.steps,
        "launches_per_step": int(stats["launches"]),
        "clocks": clocks,
        "peak_arena_bytes": stats["peak_arena_bytes"],
        "reference_arena_bytes_greedy": stats["reference_arena_bytes_greedy"],
        "kernel_time_us_per_pass": {k: v["us"] for k, v in kernels.items()},
        "kernel_launches_per_pass": {k: v["launches"] for k, v in kernels.items()},
        "kernel_timing": timing,
        "work_per_step": {"flops": flops, "compulsory_bytes": nbytes},
    }
    if p_tc is not None:
        line["tf32_peak"] = {"tflops": p_tc, "how": "fml_gemm with tuned tiles, single-pass TF32, M=8192 K=N=4096, best of 5 (CUDA events)"}

    if headline:
        # the dominant kernel: the tcgen05 GEMM (FusedGemmKernel launches: 48 tensor-core GEMMs per
        # pass + the pooler on the skinny kernel, ~1 % of the time)
        g = [v for k, v in kernels.items() if k in ("FusedGemmKernel", "MatMulKernel")]
        gemm_us = sum(v["us"] for v in g)
        gemm_launches = sum(v["launches"] for v in g)
        alg_bytes, alg_launches = gemm_algorithmic_bytes()
        achieved = alg_bytes / (gemm_us * 1e-6) / 1e9 if gemm_us else None
        ratio, ratio_src = captured_traffic_ratio()
        line["roofline"] = {
            "bound": "hbm", "kernel": "gemm_tc_kernel (FusedGemmKernel launches)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if achieved else None,
            "peak_source": peak_kind,
            "traffic": ratio * alg_bytes / alg_launches if ratio else None,
            "traffic_source": f"{ratio_src}: dram__bytes_read+write of the captured shape per algorithmic byte "
                              f"({ratio:.4f}), scaled to the average launch" if ratio else None,
            "algorithmic_bytes_per_launch": alg_bytes / alg_launches,
            "avg_launch_us": gemm_us / gemm_launches if gemm_launches else None,
            "launches_per_pass": gemm_launches,
            "share_of_pass": gemm_us / pass_us if pass_us else None,
            "timing": timing,
        }
        # whole-model roofline: every byte the fused plan must move / HBM peak (weights dominate)
        model_bytes = 513.9e6
        line["model_roofline"] = {"t_roof_us": model_bytes / (peak * 1e9) * 1e6, "t_measured_us": dev_s * 1e6,
                                  "frac": (model_bytes / (peak * 1e9)) / dev_s}
    else:
        # per-kernel formula: T_roof = sum max(F_k / P_tc, B_k / BW)
        p_use = p_tc or 500.0
        t_roof = roofline_time_us(rows, p_use, peak)
        top, top_t = max(kernels.items(), key=lambda kv: kv[1]["us"]) if kernels else (None, {"us": 0.0})
        # the operators the top kernel class runs, and which roof bounds them: the class's time on
        # the tensor pipe (flops / measured TF32 peak) against its time on HBM (compulsory bytes /
        # measured copy bandwidth); the larger one is the bound
        if top and top.startswith("Conv"):
            mine = [(f, b) for op, f, b in rows if op + "Kernel" == top]
        elif top and ("Gemm" in top or "MatMul" in top):
            mine = [(f, b) for op, f, b in rows if op in ("MatMul", "Gemm")]
        else:
            mine = []
        f_top, b_top = sum(f for f, _ in mine), sum(b for _, b in mine)
        t_tensor, t_hbm = f_top / (p_use * 1e12), b_top / (peak * 1e9)
        common = {"kernel": top, "traffic": None, "share_of_pass": top_t["us"] / pass_us if pass_us else None, "timing": timing,
                  "class_flops": f_top, "class_compulsory_bytes": b_top, "class_us_per_pass": top_t["us"],
                  "class_roof_us": {"tensor": t_tensor * 1e6, "hbm": t_hbm * 1e6}}
        if mine and top_t["us"] and t_tensor >= t_hbm:
            tf = f_top / (top_t["us"] * 1e-6) / 1e12
            line["roofline"] = {"bound": "tensor", "achieved": tf, "peak": p_use, "unit": "TFLOP/s", "frac": tf / p_use,
                                "peak_source": "tf32_peak (this run)" if p_tc else "assumed", **common,
                                "note": "flops of the operators this kernel class runs, counted once (not x3 for the TF32 split), "
                                        "over the class's in-graph time per pass"}
        elif mine and top_t["us"]:
            gbs = b_top / (top_t["us"] * 1e-6) / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                "peak_source": peak_kind, **common,
                                "note": "compulsory bytes of the operators this kernel class runs (inputs, weights and outputs "
                                        "once) over the class's in-graph time per pass"}
        else:
            gbs = nbytes / dev_s / 1e9
            line["roofline"] = {"bound": "hbm", "kernel": top, "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                "traffic": None, "peak_source": peak_kind, "timing": timing,
                                "note": "compulsory bytes of the whole pass over the pass time"}
        line["model_roofline"] = {"t_roof_us": t_roof, "t_measured_us": dev_s * 1e6, "frac": t_roof / (dev_s * 1e6),
                                  "formula": "sum over contraction and row-wise operators of max(flops / tf32_peak, bytes / hbm_peak)"}

    if args.gpus == 1:
        m, x, scale, what = cpu_sample(args.config, cfg, 20.0)
        secs = cpu_time(m, x, repeats=8 if headline else 1)
        line["cpu_baseline"] = {"value": units / (secs * scale), "unit": cfg["unit"], "cores": host_threads(), "kind": "port",
                                "host_cores_available": os.cpu_count(),
                                "sample": f"{what}, best of {8 if headline else 1} passes of {secs:.1f} s; oracle port of the reference's "
                                          "unfused execution, matrix-product rows over all host threads (the reference itself runs on one)"}
        if headline:
            line["concurrent_streams"] = concurrent_streams(onnx_bytes, model, seeds, args.steps)
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=25)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="bert_b1")
    args = ap.parse_args()
    if args.config not in ("bert_b1", "vgg16_b1", "vgg16_b32", "effnet_b1", "effnet_b64", "convbert_b8", "gptneox_b4s512"):
        ap.error("unknown --config")
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    args.repeats = max(1, args.repeats)
    if args.config != "bert_b1" and "--steps" not in sys.argv:
        args.steps = 20  # the larger configurations take milliseconds per pass
    # Rank 0 prints ONE JSON line and nothing else on stdout: libraries that log to file
    # descriptor 1 (NCCL prints its version there at the first collective) are sent to stderr for
    # the duration of the run, and the line goes to the descriptor stdout had at start.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    line_out = io.StringIO()
    try:
        with contextlib.redirect_stdout(line_out):
            if args.impl == "reference":
                run_reference(args)
            else:
                run_ours(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    sys.stdout.write(line_out.getvalue())
    sys.stdout.flush()


if __name__ == "__main__":
    main()
