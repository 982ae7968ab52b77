"""Runs one convolution or one attention block a few times through the C ABI: the small,
self-contained commands to put under `ncu` when profiling those kernels.

    python -m fluidml_b200.profile_ops conv --batch 8 --ic 256 --oc 256 --hw 56 [--k 3] [--precision 3xtf32]
    python -m fluidml_b200.profile_ops attention --heads 12 --seq 128 --dim 64 [--batch 1]

Prints the average device time per launch (CUDA events, back-to-back launches) and the
arithmetic / algorithmic-byte rates that follow from it.
"""
from __future__ import annotations

import argparse
import ctypes

import numpy as np

from . import cabi
from .cabi import DeviceTensor as DT


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
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=1)
    a.add_argument("--heads", type=int, default=12)
    a.add_argument("--seq", type=int, default=128)
    a.add_argument("--dim", type=int, default=64)
    a.add_argument("--reps", type=int, default=3)
    mb = sub.add_parser("membound")
    mb.add_argument("--rows", type=int, default=131072)
    mb.add_argument("--cols", type=int, default=768)
    mb.add_argument("--only", default="", help="run just one of: add, bias_gelu, layernorm, softmax, transpose")
    mb.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    rng = np.random.Generator(np.random.PCG64(0))

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
        x = DT.from_numpy(rng.standard_normal((args.batch, args.ic, args.hw, args.hw)).astype(np.float32))
        w = DT.from_numpy((rng.standard_normal((args.oc, args.ic, args.k, args.k)) * 0.05).astype(np.float32),
                          [3, 2, 0, 1])  # tap-major, output channel innermost: what the Builder bakes
        b = DT.from_numpy(np.zeros(args.oc, np.float32))
        y = DT((args.batch, args.oc, args.hw, args.hw), np.float32)
        print("tensor cores:", cabi.conv_uses_tensor_cores(x, w, y, [pad, pad], prec))
        us = _time(lambda: cabi.conv(x, w, b, y, [pad, pad], [1, 1], [1, 1], 1, act=cabi.ACT_RELU, precision=prec), args.reps)
        flop = 2.0 * args.batch * args.oc * args.ic * args.k * args.k * args.hw * args.hw
        nbytes = 4.0 * (args.batch * (args.ic + args.oc) * args.hw * args.hw + args.oc * args.ic * args.k * args.k)
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
