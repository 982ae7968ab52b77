"""ctypes front end of the CPU oracle and an unfused whole-graph interpreter over it.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
legs of the benchmark driver.  The shipped library never imports this package.

``run_model`` executes an ONNX graph node by node, one oracle kernel per node and one
freshly allocated buffer per tensor -- the unfused, single-thread execution the reference
produces (src/worker/builder.cpp:400-491 walks the sequence and emits one kernel per node;
src/worker/lower.cpp:39-46 adds no fusion, tiling or threading).  Operand-pattern rules
follow src/worker/converter.cpp (which inputs must be constants, defaults for axis/epsilon).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Dict, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libfml_oracle.so")
_SRC = os.path.join(_HERE, "fml_oracle.c")
MAX_RANK = 8


def build(force: bool = False) -> str:
    """Compile fml_oracle.c.  -ffp-contract=off keeps a*b+c as two rounded operations, as
    the reference's separate arith.mulf / arith.addf ops are."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(["gcc", "-O3", "-march=native", "-ffp-contract=off", "-fopenmp", "-fPIC",
                               "-shared", "-o", _SO, _SRC, "-lm"])
    return _SO


class _T(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_RANK), ("stride", ctypes.c_int64 * MAX_RANK)]


_CODE = {np.dtype(np.float32): 1, np.dtype(np.int32): 6, np.dtype(np.int64): 7,
         np.dtype(np.bool_): 9, np.dtype(np.uint8): 9}
_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_gen_all_orders.restype = ctypes.c_int64
    return _lib


def T(a: np.ndarray) -> _T:
    """Describe an ndarray (any strides, e.g. a transposed view) to the oracle."""
    t = _T()
    t.data = a.ctypes.data
    t.dtype = _CODE[a.dtype]
    t.rank = a.ndim
    for i in range(a.ndim):
        t.shape[i] = a.shape[i]
        assert a.strides[i] % a.itemsize == 0
        t.stride[i] = a.strides[i] // a.itemsize
    return t


def _p(t):
    return ctypes.byref(t) if t is not None else None


def _i64(v):
    return (ctypes.c_int64 * len(v))(*[int(x) for x in v])


BIN = {"Add": 0, "Mul": 1, "Div": 2, "Sub": 3, "Pow": 4, "Equal": 5}
UN = {"Erf": 0, "Tanh": 1, "Sqrt": 2, "Neg": 3, "Relu": 4, "Sigmoid": 5, "Clip": 6, "Not": 7,
      "Identity": 8, "Dropout": 8, "Exp": 9}


def binary(op: str, a, b, out):
    assert lib().orc_binary(BIN[op], _p(T(a)), _p(T(b)), _p(T(out))) == 0
    return out


def unary(op: str, x, out, p0=0.0, p1=0.0):
    assert lib().orc_unary(UN[op], _p(T(x)), _p(T(out)), ctypes.c_float(p0),
                           ctypes.c_float(p1)) == 0
    return out


def set_threads(n: int) -> None:
    """Host threads the matrix products may use (rows are independent: the bits do not change)."""
    lib().orc_set_threads(int(n))


def matmul(a, b, out, order=1, acc64=False):
    lib().orc_matmul(_p(T(a)), _p(T(b)), _p(T(out)), int(order), int(acc64))
    return out


def gemm(a, b, bias, out, alpha=1.0, beta=1.0, transA=0, transB=0, acc64=False):
    lib().orc_gemm(_p(T(a)), _p(T(b)), _p(T(bias)) if bias is not None else None, _p(T(out)),
                   ctypes.c_float(alpha), ctypes.c_float(beta), int(transA), int(transB),
                   int(acc64))
    return out


def softmax(x, out, axis=-1):
    lib().orc_softmax(_p(T(x)), _p(T(out)), int(axis))
    return out


def layernorm(x, scale, bias, out, axis=-1, eps=1e-5, acc64=False):
    lib().orc_layernorm(_p(T(x)), _p(T(scale)), _p(T(bias)), _p(T(out)), int(axis),
                        ctypes.c_float(eps), int(acc64))
    return out


def transpose(x, out, perm):
    lib().orc_transpose(_p(T(x)), _p(T(out)), _i64(perm))
    return out


def reshape(x, out):
    lib().orc_reshape(_p(T(x)), _p(T(out)))
    return out


def gather(data, ind, out, axis=0):
    lib().orc_gather(_p(T(data)), _p(T(np.asarray(ind, dtype=np.int64))), _p(T(out)), int(axis))
    return out


def where(cond, x, y, out):
    lib().orc_where(_p(T(cond)), _p(T(x)), _p(T(y)), _p(T(out)))
    return out


def slice_(x, out, starts):
    lib().orc_slice(_p(T(x)), _p(T(out)), _i64(starts))
    return out


def concat2(a, b, out, axis):
    lib().orc_concat2(_p(T(a)), _p(T(b)), _p(T(out)), int(axis))
    return out


def pad(x, out, pads_begin):
    lib().orc_pad(_p(T(x)), _p(T(out)), _i64(pads_begin))
    return out


def reduce_mean(x, out, axes):
    flags = (ctypes.c_int32 * x.ndim)(*[1 if i in axes else 0 for i in range(x.ndim)])
    lib().orc_reduce_mean(_p(T(x)), _p(T(out)), flags)
    return out


def cumsum(x, out, axis):
    lib().orc_cumsum(_p(T(x)), _p(T(out)), int(axis))
    return out


def cast(x, out):
    lib().orc_cast(_p(T(x)), _p(T(out)))
    return out


def conv(x, w, bias, out, pads, strides, dilations, group=1, acc64=False):
    lib().orc_conv(_p(T(x)), _p(T(w)), _p(T(bias)) if bias is not None else None, _p(T(out)),
                   _i64(pads), _i64(strides), _i64(dilations), ctypes.c_int64(group), int(acc64))
    return out


def pool2d(x, out, mode, kernel, strides):
    lib().orc_pool2d(_p(T(x)), _p(T(out)), int(mode), _i64(kernel), _i64(strides))
    return out


def gen_strides(shape, layout):
    out = (ctypes.c_int64 * len(shape))()
    lib().orc_gen_strides(_i64(shape), _i64(layout), len(shape), out)
    return list(out)


def gen_all_orders(n: int):
    import math
    cnt = math.factorial(n)
    out = (ctypes.c_int64 * max(1, cnt * n))()
    got = lib().orc_gen_all_orders(n, out)
    assert got == cnt
    return [list(out[i * n:(i + 1) * n]) for i in range(cnt)]


def broadcast_shape(a, b):
    out = (ctypes.c_int64 * MAX_RANK)()
    r = lib().orc_broadcast_shape(_i64(a), len(a), _i64(b), len(b), out)
    return None if r < 0 else list(out[:r])


def broadcast_matmul_shape(a, b):
    out = (ctypes.c_int64 * MAX_RANK)()
    r = lib().orc_broadcast_matmul_shape(_i64(a), len(a), _i64(b), len(b), out)
    return None if r < 0 else list(out[:r])


# ------------------------------------------------------------------------------ interpreter
def run_model(model, inputs: Dict[str, np.ndarray], acc64: bool = False, order: int = 1,
              keep: Optional[set] = None) -> Dict[str, np.ndarray]:
    """Execute ``model`` (fluidml_b200.onnx_lite.Model or any object with the same fields)
    node by node.  Returns every graph output (plus the tensors named in ``keep``)."""
    from fluidml_b200.onnx_lite import np_dtype  # message schema only, no compute

    env: Dict[str, np.ndarray] = {k: np.asarray(v).copy() for k, v in model.initializers.items()}
    for vi in model.inputs:
        a = np.ascontiguousarray(inputs[vi.name])
        assert a.shape == tuple(vi.shape) and a.dtype == np_dtype(vi.dtype), vi.name
        env[vi.name] = a
    info = {vi.name: vi for vi in (*model.value_info, *model.outputs)}

    def new(name):
        vi = info[name]
        return np.empty(vi.shape, dtype=np_dtype(vi.dtype))

    # last use of every tensor, to free memory as the reference's arena would reuse it
    last = {}
    for i, n in enumerate(model.nodes):
        for x in n.inputs:
            last[x] = i
    outs = {v.name for v in model.outputs} | (keep or set())

    for i, n in enumerate(model.nodes):
        op, a = n.op_type, n.attrs
        x = [env[k] if k else None for k in n.inputs]
        o = new(n.outputs[0])
        if op in BIN:
            binary(op, x[0], x[1], o)
        elif op in ("Erf", "Tanh", "Sqrt", "Neg", "Relu", "Sigmoid", "Not", "Identity",
                    "Dropout", "Exp"):
            unary(op, x[0], o)
        elif op == "Clip":
            lo = float(x[1]) if len(x) > 1 and x[1] is not None else float(a.get("min", -3.4e38))
            hi = float(x[2]) if len(x) > 2 and x[2] is not None else float(a.get("max", 3.4e38))
            unary("Clip", x[0], o, lo, hi)
        elif op == "MatMul":
            matmul(x[0], x[1], o, order, acc64)
        elif op == "Gemm":
            gemm(x[0], x[1], x[2] if len(x) > 2 else None, o, a.get("alpha", 1.0),
                 a.get("beta", 1.0), a.get("transA", 0), a.get("transB", 0), acc64)
        elif op == "Softmax":
            softmax(x[0], o, a.get("axis", -1))
        elif op == "LayerNormalization":
            layernorm(x[0], x[1], x[2], o, a.get("axis", -1), a.get("epsilon", 1e-5), acc64)
        elif op == "Transpose":
            perm = a.get("perm") or list(range(x[0].ndim))[::-1]
            transpose(x[0], o, perm)
        elif op in ("Reshape", "Unsqueeze", "Squeeze", "Flatten"):
            reshape(x[0], o)
        elif op == "Gather":
            gather(x[0], x[1], o, a.get("axis", 0))
        elif op == "Where":
            where(x[0], x[1], x[2], o)
        elif op == "Slice":
            starts = [0] * x[0].ndim
            axes = x[3] if len(x) > 3 and x[3] is not None else range(len(x[1]))
            for st, ax in zip(x[1], axes):
                starts[int(ax)] = int(st)
            slice_(x[0], o, starts)
        elif op == "Concat":
            concat2(x[0], x[1], o, a["axis"] % o.ndim)
        elif op == "Pad":
            pad(x[0], o, [int(v) for v in x[1][:x[0].ndim]])
        elif op == "ReduceMean":
            axes = x[1] if len(x) > 1 and x[1] is not None else a["axes"]
            reduce_mean(x[0], o, [int(v) % x[0].ndim for v in axes])
        elif op == "CumSum":
            cumsum(x[0], o, int(x[1]) % x[0].ndim)
        elif op == "Cast":
            cast(x[0], o)
        elif op == "Conv":
            nd = x[0].ndim - 2
            conv(x[0], x[1], x[2] if len(x) > 2 else None, o, a.get("pads", [0] * 2 * nd)[:nd],
                 a.get("strides", [1] * nd), a.get("dilations", [1] * nd), a.get("group", 1),
                 acc64)
        elif op in ("MaxPool", "AveragePool"):
            assert not any(a.get("pads", [0])), "pools take no padding (converter.cpp:581-592)"
            pool2d(x[0], o, int(op == "AveragePool"), a["kernel_shape"],
                   a.get("strides", [1, 1]))
        else:
            raise NotImplementedError(op)
        env[n.outputs[0]] = o
        for k in n.inputs:
            if k and last.get(k) == i and k not in outs and k not in model.initializers:
                env.pop(k, None)
    return {k: env[k] for k in outs}
