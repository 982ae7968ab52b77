"""Runs one GEMM shape a few times through the C ABI: the small, self-contained command to put
under `ncu` when profiling the tensor-core kernel (weights larger than nothing else on the
device, one kernel, a handful of launches).

    python -m fluidml_b200.profile_gemm --m 128 --k 3072 --n 768 --reps 3 [--precision 3xtf32]

Prints the chosen plan and the average device time per launch (CUDA events, back-to-back
launches, L2-warm after the first).
"""
from __future__ import annotations

import argparse
import ctypes

import numpy as np

from . import cabi
from .cabi import DeviceTensor as DT


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=128)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--n", type=int, default=768)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--precision", default="3xtf32", choices=["fp32", "3xtf32", "tf32"])
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    args = ap.parse_args()
    prec = {"fp32": cabi.GEMM_FP32, "3xtf32": cabi.GEMM_3XTF32, "tf32": cabi.GEMM_TF32}[args.precision]
    rng = np.random.Generator(np.random.PCG64(0))
    lead = (args.batch,) if args.batch > 1 else ()
    a = DT.from_numpy(rng.standard_normal((*lead, args.m, args.k)).astype(np.float32))
    b = DT.from_numpy(rng.standard_normal((*lead, args.k, args.n)).astype(np.float32))
    c = DT((*lead, args.m, args.n), np.float32)
    p = cabi.gemm_params(precision=prec, tile_n=args.tile_n, split_k=args.split_k)
    info = cabi.gemm_plan(a, b, c, p)
    print(f"plan: tensor_cores={info.uses_tensor_cores} tile_n={info.tile_n} split_k={info.split_k} "
          f"stages={info.stages} smem={info.shared_memory_bytes}")
    lib = cabi.lib()
    e0, e1 = ctypes.c_void_p(), ctypes.c_void_p()
    lib.fml_event_create(ctypes.byref(e0))
    lib.fml_event_create(ctypes.byref(e1))
    cabi.gemm(a, b, c, params=p)  # warm-up
    cabi.sync()
    lib.fml_event_record(e0, None)
    for _ in range(args.reps):
        cabi.gemm(a, b, c, params=p)
    lib.fml_event_record(e1, None)
    cabi.check_device()
    ms = ctypes.c_float()
    lib.fml_event_elapsed_ms(e0, e1, ctypes.byref(ms))
    nbytes = (args.m * args.k + args.k * args.n + args.m * args.n) * 4 * args.batch
    us = ms.value * 1e3 / args.reps
    print(f"{us:.2f} us per launch, {nbytes / us / 1e3:.1f} GB/s algorithmic, "
          f"{2.0 * args.m * args.n * args.k * args.batch / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    main()
