"""ctypes binding of the kernel library's C ABI (include/fluidml_cuda.h).

The CUDA library is the only implementation: importing this module raises if the shared
object has not been built, and every call raises on a non-zero status.  There is no CPU
path behind these functions.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import numpy as np

MAX_RANK = 8
_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib",
                         "libfluidml_b200_kernels.so")

F32, I32, I64, BOOL = 1, 6, 7, 9
_CODE = {np.dtype(np.float32): F32, np.dtype(np.int32): I32, np.dtype(np.int64): I64,
         np.dtype(np.bool_): BOOL}
_NP = {F32: np.float32, I32: np.int32, I64: np.int64, BOOL: np.bool_}

# fml_ew_op
ADD, MUL, DIV, SUB, POW, EQUAL = 0, 1, 2, 3, 4, 5
ADD_SCALAR, MUL_SCALAR, DIV_SCALAR, RSUB_SCALAR, POW_SCALAR, EQUAL_SCALAR, CLIP, \
    RSUB_MUL_SCALAR = 16, 17, 18, 19, 20, 21, 22, 23
ERF, TANH, SQRT, NEG, RELU, SIGMOID, NOT, COPY, CAST, EXP, SILU = range(32, 43)
# fml_gemm_act / precision
ACT_NONE, ACT_GELU_ERF, ACT_RELU, ACT_TANH, ACT_SIGMOID, ACT_SILU = range(6)
GEMM_AUTO, GEMM_FP32, GEMM_3XTF32, GEMM_TF32 = range(4)


class FmlError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"fml status {status}: {msg}")
        self.status = status


class Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("rank", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_RANK), ("stride", ctypes.c_int64 * MAX_RANK)]


class GemmParams(ctypes.Structure):
    _fields_ = [("precision", ctypes.c_int32), ("act", ctypes.c_int32),
                ("divisor", ctypes.c_float), ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
                ("act_param", ctypes.c_float * 3), ("split_k", ctypes.c_int32),
                ("tile_n", ctypes.c_int32), ("b_constant", ctypes.c_int32), ("l2_prefetch", ctypes.c_void_p),
                ("l2_prefetch_bytes", ctypes.c_uint64)]


class ConvParams(ctypes.Structure):
    _fields_ = [("pads_begin", ctypes.c_int64 * 2), ("strides", ctypes.c_int64 * 2),
                ("dilations", ctypes.c_int64 * 2), ("group", ctypes.c_int64),
                ("act", ctypes.c_int32), ("precision", ctypes.c_int32)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(f"{_LIB_PATH} is missing: run `python -m fluidml_b200.build` "
                              "(there is no fallback implementation)")
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.fml_last_error.restype = ctypes.c_char_p
    return _lib


def check(status: int) -> None:
    if status != 0:
        raise FmlError(status, lib().fml_last_error().decode())


def gen_strides(shape: Sequence[int], layout: Optional[Sequence[int]] = None):
    """Element strides of a tensor stored with `layout` (layout[i] = physical position of
    logical dim i), as utils::GenStrides does (src/utils/utils.cpp:64-102)."""
    r = len(shape)
    layout = list(range(r)) if layout is None else list(layout)
    phys = [0] * r
    for i in range(r):
        phys[layout[i]] = shape[i]
    ps = [1] * r
    for i in range(r - 1, 0, -1):
        ps[i - 1] = ps[i] * phys[i]
    return [ps[layout[i]] for i in range(r)]


class DeviceBuffer:
    """A device allocation owned by Python (freed on garbage collection)."""

    def __init__(self, nbytes: int):
        p = ctypes.c_void_p()
        check(lib().fml_malloc(ctypes.byref(p), ctypes.c_size_t(max(1, nbytes))))
        self.ptr, self.nbytes = p.value, nbytes

    def __del__(self):
        try:
            if self.ptr:
                lib().fml_free(ctypes.c_void_p(self.ptr))
        except Exception:
            pass

    def zero(self):
        check(lib().fml_memset(ctypes.c_void_p(self.ptr), 0, ctypes.c_size_t(self.nbytes), None))


class DeviceTensor:
    """Shape + strides over a DeviceBuffer; converts from/to numpy through any layout."""

    def __init__(self, shape, dtype, layout=None, buf: Optional[DeviceBuffer] = None,
                 offset_elems: int = 0, strides=None):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.layout = list(range(len(self.shape))) if layout is None else list(layout)
        self.strides = list(strides) if strides is not None else gen_strides(self.shape, self.layout)
        n = int(np.prod(self.shape)) if self.shape else 1
        self.buf = buf or DeviceBuffer(n * self.dtype.itemsize)
        self.offset = offset_elems

    @staticmethod
    def from_numpy(a: np.ndarray, layout=None) -> "DeviceTensor":
        a = np.asarray(a)
        t = DeviceTensor(a.shape, a.dtype, layout)
        order = list(np.argsort(t.layout)) if a.ndim else []
        phys = np.ascontiguousarray(a.transpose(order)) if a.ndim else np.array(a)
        check(lib().fml_memcpy_h2d(ctypes.c_void_p(t.buf.ptr), phys.ctypes.data_as(ctypes.c_void_p),
                                   ctypes.c_size_t(phys.nbytes), None))
        check(lib().fml_stream_sync(None))
        return t

    def numpy(self) -> np.ndarray:
        r = len(self.shape)
        phys_shape = [0] * r
        for i in range(r):
            phys_shape[self.layout[i]] = self.shape[i]
        phys = np.empty(phys_shape, dtype=self.dtype)
        check(lib().fml_stream_sync(None))
        check(lib().fml_memcpy_d2h(phys.ctypes.data_as(ctypes.c_void_p),
                                   ctypes.c_void_p(self.buf.ptr + self.offset * self.dtype.itemsize),
                                   ctypes.c_size_t(phys.nbytes), None))
        check(lib().fml_stream_sync(None))
        return np.ascontiguousarray(phys.transpose(self.layout)) if r else phys

    def view(self, shape, strides, offset_elems=0) -> "DeviceTensor":
        return DeviceTensor(shape, self.dtype, None, self.buf, self.offset + offset_elems, strides)

    def c(self) -> Tensor:
        t = Tensor()
        t.data = self.buf.ptr + self.offset * self.dtype.itemsize
        t.dtype = _CODE[self.dtype]
        t.rank = len(self.shape)
        for i, (s, st) in enumerate(zip(self.shape, self.strides)):
            t.shape[i], t.stride[i] = s, st
        return t


def _ref(t: Optional[DeviceTensor]):
    return ctypes.byref(t.c()) if t is not None else None


def _i64(v):
    return (ctypes.c_int64 * len(v))(*[int(x) for x in v])


# ------------------------------------------------------------------ thin call wrappers
def elementwise(op, a, b, out, p0=0.0, p1=0.0, stream=None):
    check(lib().fml_elementwise(int(op), _ref(a), _ref(b), _ref(out), ctypes.c_double(p0),
                                ctypes.c_double(p1), stream))


def mul_add(a, b, c, out, stream=None):
    check(lib().fml_mul_add(_ref(a), _ref(b), _ref(c), _ref(out), stream))


def squeeze_excite_gate(x, w1, b1, w2, b2, act1, act2, gate, stream=None):
    """ReduceMean over H, W -> 1x1 conv (+act1) -> 1x1 conv (+act2) in one launch; b1 / b2 may be None."""
    check(lib().fml_squeeze_excite_gate(_ref(x), _ref(w1), _ref(b1), _ref(w2), _ref(b2), int(act1), int(act2),
                                        _ref(gate), stream))


def sum_of_products(a_list, b_list, out, stream=None):
    """out = a0*b0 + a1*b1 + ... in the rounding order of the Mul / Add chain (up to 12 pairs)."""
    n = len(a_list)
    assert n == len(b_list)
    arr_a = (ctypes.POINTER(Tensor) * n)(*[ctypes.pointer(t.c()) for t in a_list])
    arr_b = (ctypes.POINTER(Tensor) * n)(*[ctypes.pointer(t.c()) for t in b_list])
    check(lib().fml_sum_of_products(n, arr_a, arr_b, _ref(out), stream))


def rotary(x, cosv, sinv, rot, out, stream=None):
    """Rotary position embedding over the first `rot` features (halves convention)."""
    check(lib().fml_rotary(_ref(x), _ref(cosv), _ref(sinv), ctypes.c_int64(int(rot)), _ref(out), stream))


def bias_gelu(x, bias, out, c0, c1, c2, stream=None):
    check(lib().fml_bias_gelu(_ref(x), _ref(bias), _ref(out), ctypes.c_float(c0),
                              ctypes.c_float(c1), ctypes.c_float(c2), stream))


def where(cond, x, y, y_scalar, out, stream=None):
    check(lib().fml_where(_ref(cond), _ref(x), _ref(y), ctypes.c_float(y_scalar), _ref(out), stream))


def copy_strided(src, out, stream=None):
    check(lib().fml_copy_strided(_ref(src), _ref(out), stream))


def concat2(lhs, rhs, out, axis, stream=None):
    check(lib().fml_concat2(_ref(lhs), _ref(rhs), _ref(out), int(axis), stream))


def reshape_copy(src, out, stream=None):
    check(lib().fml_reshape_copy(_ref(src), _ref(out), stream))


def gather(data, indices, out, axis, stream=None):
    check(lib().fml_gather(_ref(data), _ref(indices), _ref(out), int(axis), stream))


def embedding(table, ids, add0, add1, out, stream=None):
    check(lib().fml_embedding(_ref(table), _ref(ids), _ref(add0), _ref(add1), _ref(out), stream))


def pad(src, out, pads_begin, stream=None):
    check(lib().fml_pad(_ref(src), _ref(out), _i64(pads_begin), stream))


def softmax(x, mask, divisor, out, axis, stream=None):
    check(lib().fml_softmax(_ref(x), _ref(mask), ctypes.c_float(divisor), _ref(out), int(axis), stream))


def attention(q, kt, v, mask, divisor, out, stream=None):
    check(lib().fml_attention(_ref(q), _ref(kt), _ref(v), _ref(mask), ctypes.c_float(divisor), _ref(out), stream))


def attention_uses_tensor_cores(q, kt, v) -> bool:
    uses = ctypes.c_int()
    check(lib().fml_attention_uses_tensor_cores(_ref(q), _ref(kt), _ref(v), ctypes.byref(uses)))
    return bool(uses.value)


def attention_supported(s_q, s_k, d, d_v) -> bool:
    f = lib().fml_attention_supported
    f.argtypes = [ctypes.c_int64] * 4
    return bool(f(s_q, s_k, d, d_v))


def layernorm(x, residual, scale, bias, out, axis, eps, stream=None):
    check(lib().fml_layernorm(_ref(x), _ref(residual), _ref(scale), _ref(bias), _ref(out),
                              int(axis), ctypes.c_float(eps), stream))


def reduce_mean(x, out, axes, stream=None):
    flags = (ctypes.c_int32 * len(x.shape))(*[1 if i in axes else 0 for i in range(len(x.shape))])
    check(lib().fml_reduce_mean(_ref(x), _ref(out), flags, stream))


def cumsum(x, out, axis, stream=None):
    check(lib().fml_cumsum(_ref(x), _ref(out), int(axis), stream))


def gemm_params(precision=GEMM_AUTO, act=ACT_NONE, divisor=1.0, alpha=1.0, beta=1.0,
                split_k=0, tile_n=0, act_param=None) -> GemmParams:
    p = GemmParams()
    lib().fml_gemm_default_params(ctypes.byref(p))
    p.precision, p.act, p.divisor, p.alpha, p.beta = precision, act, divisor, alpha, beta
    p.split_k, p.tile_n = split_k, tile_n
    if act_param is not None:
        for i in range(3):
            p.act_param[i] = act_param[i]
    return p


class GemmPlanInfo(ctypes.Structure):
    _fields_ = [("uses_tensor_cores", ctypes.c_int32), ("tile_n", ctypes.c_int32), ("split_k", ctypes.c_int32),
                ("stages", ctypes.c_int32), ("b_mn_major", ctypes.c_int32), ("three_pass", ctypes.c_int32),
                ("shared_memory_bytes", ctypes.c_uint64)]


def gemm_plan(a, b, c, params) -> GemmPlanInfo:
    """Tile / split-K / pipeline depth the library picks for these operands (host only)."""
    info = GemmPlanInfo()
    check(lib().fml_gemm_plan(_ref(a), _ref(b), _ref(c), ctypes.byref(params), ctypes.byref(info)))
    return info


def gemm_autotune(a, b, c, params, bias=None, residual=None, stream=None) -> GemmParams:
    """fml_gemm_autotune: times the candidate tiles on the device and returns the parameters with the
    fastest tile_n / split_k filled in (C is overwritten with valid results)."""
    tuned = GemmParams()
    check(lib().fml_gemm_autotune(_ref(a), _ref(b), _ref(c), _ref(bias), _ref(residual), ctypes.byref(params),
                                  stream, ctypes.byref(tuned)))
    return tuned


def gemm_uses_tensor_cores(a, b, c, params) -> bool:
    u = ctypes.c_int()
    check(lib().fml_gemm_uses_tensor_cores(_ref(a), _ref(b), _ref(c), ctypes.byref(params),
                                           ctypes.byref(u)))
    return bool(u.value)


def gemm(a, b, c, bias=None, residual=None, params=None, stream=None):
    params = params or gemm_params()
    check(lib().fml_gemm(_ref(a), _ref(b), _ref(c), _ref(bias), _ref(residual), ctypes.byref(params), stream))


def gemm_skinny_noalloc(a, b, c, bias=None, residual=None, params=None, stream=None):
    """fml_gemm_skinny_noalloc: at most 32 rows, scratch inside the module, nothing allocated."""
    params = params or gemm_params()
    check(lib().fml_gemm_skinny_noalloc(_ref(a), _ref(b), _ref(c), _ref(bias), _ref(residual),
                                        ctypes.byref(params), stream))


def conv(x, w, bias, y, pads_begin, strides, dilations, group=1, act=ACT_NONE, stream=None, precision=None):
    p = ConvParams()
    nd = len(pads_begin)
    for i in range(2):
        p.pads_begin[i] = pads_begin[i] if i < nd else 0
        p.strides[i] = strides[i] if i < nd else 1
        p.dilations[i] = dilations[i] if i < nd else 1
    p.group, p.act, p.precision = group, act, GEMM_AUTO if precision is None else precision
    check(lib().fml_conv(_ref(x), _ref(w), _ref(bias), _ref(y), ctypes.byref(p), stream))


def conv_scaled(x, x_scale, w, bias, y, pads_begin, strides, dilations, act=ACT_NONE, stream=None, precision=None):
    """y = conv(x * x_scale, w) + bias with x_scale broadcastable to [N, IC, 1, 1] (group 1)."""
    p = ConvParams()
    nd = len(pads_begin)
    for i in range(2):
        p.pads_begin[i] = pads_begin[i] if i < nd else 0
        p.strides[i] = strides[i] if i < nd else 1
        p.dilations[i] = dilations[i] if i < nd else 1
    p.group, p.act, p.precision = 1, act, GEMM_AUTO if precision is None else precision
    check(lib().fml_conv_scaled(_ref(x), _ref(x_scale), _ref(w), _ref(bias), _ref(y), ctypes.byref(p), stream))


def conv_uses_tensor_cores(x, w, y, pads_begin, precision=None) -> bool:
    p = ConvParams()
    for i in range(2):
        p.pads_begin[i], p.strides[i], p.dilations[i] = pads_begin[i], 1, 1
    p.group, p.precision = 1, GEMM_AUTO if precision is None else precision
    uses = ctypes.c_int()
    check(lib().fml_conv_uses_tensor_cores(_ref(x), _ref(w), _ref(y), ctypes.byref(p), ctypes.byref(uses)))
    return bool(uses.value)


def pool2d(x, y, mode, kernel, strides, stream=None):
    check(lib().fml_pool2d(_ref(x), _ref(y), int(mode), _i64(kernel), _i64(strides), stream))


def sync(stream=None):
    check(lib().fml_stream_sync(stream))


def check_device(stream=None):
    check(lib().fml_check_device(stream))


def device_count() -> int:
    n = ctypes.c_int()
    check(lib().fml_device_count(ctypes.byref(n)))
    return n.value


# ------------------------------------------------------------------ resident stage program
RESIDENT_GEMM, RESIDENT_ATTENTION = 1, 2


class ResidentStage(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("out_external", ctypes.c_int32), ("out", Tensor),
                ("a", Tensor), ("w", Tensor), ("bias", Tensor), ("residual", Tensor),
                ("act", ctypes.c_int32), ("act_param", ctypes.c_float * 3),
                ("layernorm", ctypes.c_int32), ("ln_scale", Tensor), ("ln_bias", Tensor),
                ("ln_eps", ctypes.c_float), ("tile_n", ctypes.c_int32), ("split_k", ctypes.c_int32),
                ("q", Tensor), ("kt", Tensor), ("v", Tensor), ("mask", Tensor),
                ("divisor", ctypes.c_float)]


class ResidentInfo(ctypes.Structure):
    _fields_ = [("ctas", ctypes.c_int32), ("stages", ctypes.c_int32), ("steps", ctypes.c_int32),
                ("buffers", ctypes.c_int32), ("ring_slots", ctypes.c_int32), ("slot_bytes", ctypes.c_int32),
                ("packed_weight_bytes", ctypes.c_uint64), ("scratch_bytes", ctypes.c_uint64),
                ("shared_memory_bytes", ctypes.c_uint64)]


def _t(x) -> Tensor:
    """DeviceTensor, ctypes Tensor or None -> Tensor (a null data pointer means "absent")."""
    if x is None:
        return Tensor()
    return x if isinstance(x, Tensor) else x.c()


def resident_gemm_stage(a, w, out, bias=None, residual=None, act=ACT_NONE, act_param=(1.4142135381698608, 1.0, 0.5),
                        ln_scale=None, ln_bias=None, ln_eps=1e-5, out_external=False, tile_n=0,
                        split_k=0) -> ResidentStage:
    s = ResidentStage()
    s.kind, s.out_external, s.out = RESIDENT_GEMM, int(out_external), _t(out)
    s.a, s.w, s.bias, s.residual = _t(a), _t(w), _t(bias), _t(residual)
    s.act = act
    for i in range(3):
        s.act_param[i] = act_param[i]
    s.layernorm = int(ln_scale is not None)
    s.ln_scale, s.ln_bias, s.ln_eps = _t(ln_scale), _t(ln_bias), ln_eps
    s.tile_n, s.split_k = tile_n, split_k
    s._keep = (a, w, out, bias, residual, ln_scale, ln_bias)  # the struct holds raw pointers only
    return s


def resident_attention_stage(q, kt, v, out, mask=None, divisor=1.0, out_external=False) -> ResidentStage:
    s = ResidentStage()
    s.kind, s.out_external, s.out = RESIDENT_ATTENTION, int(out_external), _t(out)
    s.q, s.kt, s.v, s.mask, s.divisor = _t(q), _t(kt), _t(v), _t(mask), divisor
    s._keep = (q, kt, v, out, mask)
    return s


def resident_plan(stages, ctas: int = 0) -> ResidentInfo:
    """Plans and checks a program on the host; `ctas` > 0 needs no device."""
    arr = (ResidentStage * len(stages))(*stages)
    info = ResidentInfo()
    check(lib().fml_resident_plan(arr, len(stages), int(ctas), ctypes.byref(info)))
    return info


class ResidentProgram:
    """A created resident program (fml_resident_create); destroyed on garbage collection."""

    def __init__(self, stages):
        arr = (ResidentStage * len(stages))(*stages)
        self._stages = list(stages)  # keeps the operands' device buffers alive as long as the program
        self._h = ctypes.c_void_p()
        check(lib().fml_resident_create(arr, len(stages), ctypes.byref(self._h)))

    def launch(self, stream=None):
        check(lib().fml_resident_launch(self._h, stream))

    def info(self) -> ResidentInfo:
        info = ResidentInfo()
        check(lib().fml_resident_info_of(self._h, ctypes.byref(info)))
        return info

    def reset(self, stream=None):
        check(lib().fml_resident_reset(self._h, stream))

    def set_trace(self, on: bool):
        check(lib().fml_resident_set_trace(self._h, int(on)))

    def read_trace(self) -> np.ndarray:
        """[cta][step][8] uint64 nanosecond stamps of the last traced pass (fml_resident_set_trace)."""
        info = self.info()
        cap = info.ctas * 2048 * 8
        buf = np.zeros(cap, np.uint64)
        ctas, steps = ctypes.c_int32(), ctypes.c_int32()
        check(lib().fml_resident_read_trace(self._h, buf.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(cap),
                                            ctypes.byref(ctas), ctypes.byref(steps)))
        return buf[:ctas.value * steps.value * 8].reshape(ctas.value, steps.value, 8)

    def __del__(self):
        try:
            if self._h:
                lib().fml_resident_destroy(self._h)
                self._h = None
        except Exception:
            pass
