"""Python mirror of the reference's pybind11 module (src/python/pybind.cpp:66-87):

    Executor.make_plain_linear / make_plain_greedy / make_dp_greedy(name, epoch=1)
    executor.compile(input, mlir=None, llvm=None, json=None)
    executor.invoke({tensor name: numpy array}) -> nanoseconds per forward pass

Inputs and pre-allocated outputs are passed in one dict and outputs are written in place, as
in the reference (test/python/node/node_test.py:33-53).  The binding goes through the C ABI
of include/fluidml_executor.h; the native library is the only implementation and importing
this module fails when it has not been built.
"""
from __future__ import annotations

import ctypes
import json as _json
import os
from typing import Dict, Optional

import numpy as np

from . import cabi

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfluidml_b200.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(f"{_LIB_PATH} is missing: run `python -m fluidml_b200.build` "
                              "(there is no fallback implementation)")
        cabi.lib()  # the kernel library first, so the host library resolves against it
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.fml_executor_last_error.restype = ctypes.c_char_p
        _lib.fml_executor_stats_json.restype = ctypes.c_char_p
        _lib.fml_host_gen_all_orders.restype = ctypes.c_longlong
    return _lib


PLAIN_LINEAR, PLAIN_GREEDY, DP_GREEDY = 0, 1, 2


class Executor:
    def __init__(self, name: str, mode: int, epoch: int = 1):
        self._h = ctypes.c_void_p()
        st = lib().fml_executor_create(name.encode(), mode, ctypes.c_size_t(epoch), ctypes.byref(self._h))
        self._check(st)

    # -- factories (pybind.cpp:68-76)
    @staticmethod
    def make_plain_linear(name: str, epoch: int = 1) -> "Executor":
        return Executor(name, PLAIN_LINEAR, epoch)

    @staticmethod
    def make_plain_greedy(name: str, epoch: int = 1) -> "Executor":
        return Executor(name, PLAIN_GREEDY, epoch)

    @staticmethod
    def make_dp_greedy(name: str, epoch: int = 1) -> "Executor":
        return Executor(name, DP_GREEDY, epoch)

    def _check(self, st: int) -> None:
        if st == 0:
            return
        msg = lib().fml_executor_last_error(self._h).decode() if self._h else "executor was not created"
        if st == 2:
            raise KeyError(msg)  # std::out_of_range in the reference (src/worker/runner.cpp:70)
        raise RuntimeError(msg)

    def set_option(self, key: str, value) -> "Executor":
        self._check(lib().fml_executor_set_option(self._h, key.encode(), str(value).encode()))
        return self

    @staticmethod
    def _opt(p: Optional[str]):
        return p.encode() if p is not None else None

    def compile(self, input, mlir: Optional[str] = None, llvm: Optional[str] = None,
                json: Optional[str] = None) -> "Executor":
        """`input` is a path to an ONNX file, or the file's bytes."""
        if isinstance(input, (bytes, bytearray, memoryview)):
            buf = bytes(input)
            st = lib().fml_executor_compile_buffer(self._h, buf, ctypes.c_size_t(len(buf)), self._opt(mlir),
                                                   self._opt(llvm), self._opt(json))
        else:
            st = lib().fml_executor_compile_file(self._h, os.fspath(input).encode(), self._opt(mlir),
                                                 self._opt(llvm), self._opt(json))
        self._check(st)
        return self

    def plan(self, onnx_bytes: bytes, llvm: Optional[str] = None, json: Optional[str] = None) -> dict:
        """Everything compile() does before it touches the device; needs no GPU."""
        st = lib().fml_executor_plan_buffer(self._h, onnx_bytes, ctypes.c_size_t(len(onnx_bytes)),
                                            self._opt(llvm), self._opt(json))
        self._check(st)
        return self.stats()

    def invoke(self, args: Dict[str, np.ndarray]) -> int:
        names, ptrs = [], []
        for k, a in args.items():
            if not isinstance(a, np.ndarray) or not a.flags["C_CONTIGUOUS"]:
                raise TypeError(f"argument '{k}' must be a C-contiguous numpy array")
            names.append(k.encode())
            ptrs.append(a.ctypes.data)
        n = len(names)
        c_names = (ctypes.c_char_p * n)(*names)
        c_ptrs = (ctypes.c_void_p * n)(*ptrs)
        ns = ctypes.c_size_t()
        self._check(lib().fml_executor_invoke(self._h, c_names, c_ptrs, ctypes.c_size_t(n), ctypes.byref(ns)))
        return ns.value

    def profile(self, args: Dict[str, np.ndarray], passes: int = 1) -> dict:
        """Per-kernel device time of `passes` eager forward passes (event pair per launch)."""
        names = [k.encode() for k in args]
        ptrs = [a.ctypes.data for a in args.values()]
        n = len(names)
        out = ctypes.c_char_p()
        self._check(lib().fml_executor_profile(self._h, (ctypes.c_char_p * n)(*names), (ctypes.c_void_p * n)(*ptrs),
                                               ctypes.c_size_t(n), ctypes.c_size_t(passes), ctypes.byref(out)))
        return _json.loads(out.value.decode())

    def trace(self, args: Dict[str, np.ndarray], passes: int = 5) -> dict:
        """Per-kernel device time inside the replayed graph, from kernel-start stamps: the periods of a
        pass add up to the pass ({"pass_us": .., "kernels": {name: {"us": per pass, "launches": n}}})."""
        names = [k.encode() for k in args]
        ptrs = [a.ctypes.data for a in args.values()]
        n = len(names)
        out = ctypes.c_char_p()
        self._check(lib().fml_executor_trace(self._h, (ctypes.c_char_p * n)(*names), (ctypes.c_void_p * n)(*ptrs),
                                             ctypes.c_size_t(n), ctypes.c_size_t(passes), ctypes.byref(out)))
        return _json.loads(out.value.decode())

    def stats(self) -> dict:
        return _json.loads(lib().fml_executor_stats_json(self._h).decode())

    def __del__(self):
        try:
            if self._h:
                lib().fml_executor_destroy(self._h)
                self._h = None
        except Exception:
            pass


def _layout_arg(layout):
    return None if layout is None else (ctypes.c_longlong * len(layout))(*layout)


def model_gemm_cost_ns(m: int, k: int, n: int, a_layout=None, c_layout=None, precision: int = 0) -> float:
    """What the layout search charges for a MatMul [m,k] x constant [k,n] (fml_host_model_gemm_cost)."""
    ns = ctypes.c_double()
    st = lib().fml_host_model_gemm_cost(ctypes.c_longlong(m), ctypes.c_longlong(k), ctypes.c_longlong(n),
                                        _layout_arg(a_layout), _layout_arg(c_layout), int(precision), ctypes.byref(ns))
    if st:
        raise ValueError("fml_host_model_gemm_cost: bad arguments")
    return ns.value


def model_layernorm_cost_ns(rows: int, cols: int, in_layout=None, out_layout=None) -> float:
    """What the layout search charges for a LayerNormalization over the last axis of [rows, cols]."""
    ns = ctypes.c_double()
    st = lib().fml_host_model_layernorm_cost(ctypes.c_longlong(rows), ctypes.c_longlong(cols),
                                             _layout_arg(in_layout), _layout_arg(out_layout), ctypes.byref(ns))
    if st:
        raise ValueError("fml_host_model_layernorm_cost: bad arguments")
    return ns.value


_PINNED_OWNERS = []  # page-locked blocks live until the process exits


def pinned_empty(shape, dtype) -> np.ndarray:
    """A numpy array over page-locked host memory (cudaMallocHost)."""
    dtype = np.dtype(dtype)
    count = int(np.prod(shape))
    nbytes = max(count * dtype.itemsize, 1)
    p = ctypes.c_void_p()
    cabi.check(cabi.lib().fml_host_alloc_pinned(ctypes.byref(p), ctypes.c_size_t(nbytes)))
    buf = (ctypes.c_uint8 * nbytes).from_address(p.value)
    _PINNED_OWNERS.append(buf)
    return np.frombuffer(buf, dtype=dtype, count=count).reshape(shape)
