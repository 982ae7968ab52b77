"""Measurement harness (not part of the library): runs one kernel of the library a few times
through the C ABI.  These are the small, self-contained commands to put under `ncu`; the
summaries under profiles/ name them.

    python profile_harness.py gemm --m 128 --k 3072 --n 768 --reps 3 [--precision 3xtf32]
    python profile_harness.py conv --batch 8 --ic 256 --oc 256 --hw 56 [--k 3] [--precision 3xtf32]
    python profile_harness.py attention --heads 12 --seq 128 --dim 64 [--batch 1]
    python profile_harness.py membound [--only layernorm]
    python profile_harness.py resident --layers 2 [--trace]

Each prints the average device time per launch (CUDA events, back-to-back launches) and the
arithmetic / algorithmic-byte rates that follow from it.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT


def _time(fn, reps):
    lib = cabi.lib()
    e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
    lib.fml_event_create(ctypes.byref(e0))
    lib.fml_event_create(ctypes.byref(e1))
    fn()  # warm-up
    cabi.sync()
    lib.fml_event_record(e0, None)
    for _ in range(reps):
        fn()
    lib.fml_event_record(e1, None)
    cabi.check_device()
    ms = ctypes.c_float()
    lib.fml_event_elapsed_ms(e0, e1, ctypes.byref(ms))
    return ms.value * 1e3 / reps


def resident(args, rng):
    """`--layers` BERT-base encoder layers (128 rows, random weights) as one resident program:
    device time per pass and, with --trace, the timeline of its steps."""
    H, F, nh = 768, 3072, 12
    rnd = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)
    x = DT.from_numpy(rnd(128, H))
    mask = DT.from_numpy(np.zeros((1, 1, 1, 128), np.float32))
    stages, cur = [], x
    for li in range(args.layers):
        p = {"wqkv": rnd(H, 3 * H, scale=0.03), "bqkv": rnd(3 * H, scale=0.1), "wo": rnd(H, H, scale=0.03), "bo": rnd(H, scale=0.1),
             "g1": np.ones(H, np.float32), "be1": np.zeros(H, np.float32), "w1": rnd(H, F, scale=0.03), "b1": rnd(F, scale=0.1),
             "w2": rnd(F, H, scale=0.03), "b2": rnd(H, scale=0.1), "g2": np.ones(H, np.float32), "be2": np.zeros(H, np.float32)}
        p = {k: DT.from_numpy(v) for k, v in p.items()}
        qkv, ctx, y1, mid, out = (DT((128, 3 * H), np.float32), DT((128, H), np.float32), DT((128, H), np.float32),
                                  DT((128, F), np.float32), DT((128, H), np.float32))
        q = qkv.view((1, nh, 128, 64), [0, 64, 3 * H, 1])
        kt = qkv.view((1, nh, 64, 128), [0, 64, 1, 3 * H], H)
        v = qkv.view((1, nh, 128, 64), [0, 64, 3 * H, 1], 2 * H)
        stages += [cabi.resident_gemm_stage(cur, p["wqkv"], qkv, bias=p["bqkv"]),
                   cabi.resident_attention_stage(q, kt, v, ctx.view((1, nh, 128, 64), [0, 64, H, 1]), mask=mask, divisor=8.0),
                   cabi.resident_gemm_stage(ctx, p["wo"], y1, bias=p["bo"], residual=cur, ln_scale=p["g1"], ln_bias=p["be1"], ln_eps=1e-12),
                   cabi.resident_gemm_stage(y1, p["w1"], mid, bias=p["b1"], act=cabi.ACT_GELU_ERF),
                   cabi.resident_gemm_stage(mid, p["w2"], out, bias=p["b2"], residual=y1, ln_scale=p["g2"], ln_bias=p["be2"], ln_eps=1e-12,
                                            out_external=li == args.layers - 1)]
        cur = out
    prog = cabi.ResidentProgram(stages)
    info = prog.info()
    print({f: getattr(info, f) for f, _ in info._fields_})
    us = _time(lambda: prog.launch(), args.reps)
    print(f"{us:.1f} us per pass of {args.layers} layers ({us / args.layers:.1f} us per layer)")
    if args.trace:
        prog.set_trace(True)
        prog.launch()
        prog.launch()
        cabi.check_device()
        tr = prog.read_trace().astype(np.int64)
        names = ["QKV unit", "QKV finish", "attention", "out-proj unit", "out-proj LN finish", "FFN1 unit", "FFN1 finish", "FFN2 unit",
                 "FFN2 LN finish"]
        t0 = tr[:96, 0, 0].min()
        print("step (median over CTAs 0-95): start, then microseconds after start of: inputs seen / staged / s3 / s4 / end")
        for st in range(min(tr.shape[1], 9 * min(args.layers, 2))):
            a = np.median(tr[:96, st, 0])
            cols = []
            for slot in (5, 2, 3, 4, 1):
                v = tr[:96, st, slot]
                cols.append("%6.2f" % ((np.median(v) - a) / 1e3) if (v > 0).all() else "     -")
            print("  layer %d %-20s %8.2f  %s" % (st // 9, names[st % 9], (a - t0) / 1e3, " ".join(cols)))


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="op", required=True)
    c = sub.add_parser("conv")
    c.add_argument("--batch", type=int, default=8)
    c.add_argument("--ic", type=int, default=256)
    c.add_argument("--oc", type=int, default=256)
    c.add_argument("--hw", type=int, default=56)
    c.add_argument("--k", type=int, default=3)
    c.add_argument("--precision", default="3xtf32", choices=["fp32", "3xtf32", "tf32"])
    c.add_argument("--reps", type=int, default=3)
    c.add_argument("--act", default="relu", choices=["none", "relu", "silu"])
    c.add_argument("--stride", type=int, default=1)
    c.add_argument("--depthwise", action="store_true", help="group = channels (oc is ignored)")
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=1)
    a.add_argument("--heads", type=int, default=12)
    a.add_argument("--seq", type=int, default=128)
    a.add_argument("--dim", type=int, default=64)
    a.add_argument("--reps", type=int, default=3)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=128)
    g.add_argument("--k", type=int, default=3072)
    g.add_argument("--n", type=int, default=768)
    g.add_argument("--batch", type=int, default=1)
    g.add_argument("--reps", type=int, default=3)
    g.add_argument("--precision", default="3xtf32", choices=["fp32", "3xtf32", "tf32"])
    g.add_argument("--tile-n", type=int, default=0)
    g.add_argument("--split-k", type=int, default=0)
    g.add_argument("--b-kmajor", action="store_true", help="B stored [n, k] (a Gemm with transB = 1: a classifier's weights)")
    r = sub.add_parser("resident")
    r.add_argument("--layers", type=int, default=2)
    r.add_argument("--reps", type=int, default=20)
    r.add_argument("--trace", action="store_true", help="print the per-step timeline of the first two layers (median over CTAs)")
    mb = sub.add_parser("membound")
    mb.add_argument("--rows", type=int, default=131072)
    mb.add_argument("--cols", type=int, default=768)
    mb.add_argument("--only", default="", help="run just one of: add, bias_gelu, layernorm, softmax, transpose")
    mb.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    rng = np.random.Generator(np.random.PCG64(0))

    if args.op == "gemm":
        prec = {"fp32": cabi.GEMM_FP32, "3xtf32": cabi.GEMM_3XTF32, "tf32": cabi.GEMM_TF32}[args.precision]
        lead = (args.batch,) if args.batch > 1 else ()
        a = DT.from_numpy(rng.standard_normal((*lead, args.m, args.k)).astype(np.float32))
        if args.b_kmajor:
            bt = DT.from_numpy(rng.standard_normal((*lead, args.n, args.k)).astype(np.float32))
            st = list(bt.strides)
            st[-1], st[-2] = st[-2], st[-1]
            b = bt.view((*lead, args.k, args.n), st, 0)
        else:
            b = DT.from_numpy(rng.standard_normal((*lead, args.k, args.n)).astype(np.float32))
        c = DT((*lead, args.m, args.n), np.float32)
        p = cabi.gemm_params(precision=prec, tile_n=args.tile_n, split_k=args.split_k)
        info = cabi.gemm_plan(a, b, c, p)
        print(f"plan: tensor_cores={info.uses_tensor_cores} tile_n={info.tile_n} split_k={info.split_k} "
              f"stages={info.stages} smem={info.shared_memory_bytes}")
        us = _time(lambda: cabi.gemm(a, b, c, params=p), args.reps)
        nbytes = (args.m * args.k + args.k * args.n + args.m * args.n) * 4 * args.batch
        print(f"{us:.2f} us per launch, {nbytes / us / 1e3:.1f} GB/s algorithmic, "
              f"{2.0 * args.m * args.n * args.k * args.batch / us / 1e6:.1f} TFLOP/s")
        return

    if args.op == "resident":
        resident(args, rng)
        return

    if args.op == "membound":
        # the HBM-bound kernels on tensors far larger than L2: achieved GB/s of algorithmic bytes
        R, C = args.rows, args.cols
        x = DT.from_numpy(rng.standard_normal((R, C)).astype(np.float32))
        y = DT.from_numpy(rng.standard_normal((R, C)).astype(np.float32))
        o = DT((R, C), np.float32)
        vec = DT.from_numpy(rng.standard_normal(C).astype(np.float32))
        ot = DT((C, R), np.float32)
        nb = R * C * 4.0
        cases = {
            "add": (lambda: cabi.elementwise(cabi.ADD, x, y, o), 3 * nb),
            "bias_gelu": (lambda: cabi.bias_gelu(x, vec, o, float(np.sqrt(2.0)), 1.0, 0.5), 2 * nb),
            "layernorm": (lambda: cabi.layernorm(x, y, vec, vec, o, 1, 1e-5), 3 * nb),
            "softmax": (lambda: cabi.softmax(x, None, 8.0, o, 1), 2 * nb),
            "transpose": (lambda: cabi.copy_strided(x.view((C, R), [1, C], 0), ot), 2 * nb),
        }
        for name, (fn, nbytes) in cases.items():
            if args.only and name != args.only:
                continue
            us = _time(fn, args.reps)
            print(f"{name:10s} [{R} x {C}] {us:9.1f} us  {nbytes / us / 1e3:8.1f} GB/s")
        return

    if args.op == "conv":
        prec = {"fp32": cabi.GEMM_FP32, "3xtf32": cabi.GEMM_3XTF32, "tf32": cabi.GEMM_TF32}[args.precision]
        pad = args.k // 2
        act = {"none": cabi.ACT_NONE, "relu": cabi.ACT_RELU, "silu": cabi.ACT_SILU}[args.act]
        oc, group, st = (args.ic, args.ic, args.stride) if args.depthwise else (args.oc, 1, args.stride)
        ohw = (args.hw + 2 * pad - args.k) // st + 1
        x = DT.from_numpy(rng.standard_normal((args.batch, args.ic, args.hw, args.hw)).astype(np.float32))
        wh = (rng.standard_normal((oc, args.ic // group, args.k, args.k)) * 0.05).astype(np.float32)
        # group 1: tap-major, output channel innermost -- what the Builder bakes for the tensor-core path
        w = DT.from_numpy(wh) if args.depthwise else DT.from_numpy(wh, [3, 2, 0, 1])
        b = DT.from_numpy(np.zeros(oc, np.float32))
        y = DT((args.batch, oc, ohw, ohw), np.float32)
        print("tensor cores:", (not args.depthwise) and cabi.conv_uses_tensor_cores(x, w, y, [pad, pad], prec))
        us = _time(lambda: cabi.conv(x, w, b, y, [pad, pad], [st, st], [1, 1], group, act=act, precision=prec), args.reps)
        flop = 2.0 * args.batch * oc * (args.ic // group) * args.k * args.k * ohw * ohw
        nbytes = 4.0 * (args.batch * (args.ic * args.hw * args.hw + oc * ohw * ohw) + wh.size)
        print(f"{us:.2f} us per launch, {flop / us / 1e6:.1f} TFLOP/s, {nbytes / us / 1e3:.1f} GB/s algorithmic")
    else:
        B, H, S, D = args.batch, args.heads, args.seq, args.dim
        qkv = DT.from_numpy(rng.standard_normal((B * S, 3 * H * D)).astype(np.float32))
        row = 3 * H * D
        q = qkv.view((B, H, S, D), [S * row, D, row, 1], 0)
        kt = qkv.view((B, H, D, S), [S * row, D, 1, row], H * D)
        v = qkv.view((B, H, S, D), [S * row, D, row, 1], 2 * H * D)
        mask = DT.from_numpy(np.zeros((B, 1, 1, S), np.float32))
        ctx = DT((B * S, H * D), np.float32)
        out = ctx.view((B, H, S, D), [S * H * D, D, H * D, 1], 0)
        us = _time(lambda: cabi.attention(q, kt, v, mask, float(np.sqrt(D)), out), args.reps)
        flop = 4.0 * B * H * S * S * D
        nbytes = 4.0 * (4 * B * H * S * D + B * S)
        print(f"{us:.2f} us per launch, {flop / us / 1e6:.2f} TFLOP/s, {nbytes / us / 1e3:.1f} GB/s algorithmic")


if __name__ == "__main__":
    main()
