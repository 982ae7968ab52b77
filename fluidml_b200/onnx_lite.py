"""Minimal ONNX (protobuf wire format) writer and reader.

FluidML consumes static-shape ONNX files whose every intermediate tensor carries a
``value_info`` entry and whose scalars are rank-0 initialisers
(reference: src/worker/parser.cpp:193-332).  The ``onnx`` Python package and ``protoc``
are not available where this library is built, so this module encodes and decodes exactly
the message fields that parser touches, with field numbers from the public ONNX
specification (onnx.proto3):

    ModelProto      ir_version=1 producer_name=2 graph=7 opset_import=8
    OperatorSetId   domain=1 version=2
    GraphProto      node=1 name=2 initializer=5 input=11 output=12 value_info=13
    NodeProto       input=1 output=2 name=3 op_type=4 attribute=5
    AttributeProto  name=1 f=2 i=3 s=4 t=5 floats=7 ints=8 type=20
    TensorProto     dims=1 data_type=2 float_data=4 int32_data=5 int64_data=7 name=8
                    raw_data=9 double_data=10
    ValueInfoProto  name=1 type=2
    TypeProto       tensor_type=1 ;  Tensor: elem_type=1 shape=2
    TensorShape     dim=1 ; Dimension: dim_value=1 dim_param=2

The same fields are decoded by the C++ front end (csrc/host/onnx_reader.cpp); the two are
tested against each other.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

# ONNX TensorProto.DataType codes the reference understands (src/utils/type.cpp:8-23).
FLOAT, INT32, INT64, BOOL, FLOAT16 = 1, 6, 7, 9, 10
_NP_OF = {FLOAT: np.float32, INT32: np.int32, INT64: np.int64, BOOL: np.bool_,
          FLOAT16: np.float16, 11: np.float64}
_CODE_OF = {np.dtype(np.float32): FLOAT, np.dtype(np.int32): INT32,
            np.dtype(np.int64): INT64, np.dtype(np.bool_): BOOL,
            np.dtype(np.float16): FLOAT16, np.dtype(np.float64): 11}

# AttributeProto.AttributeType
A_FLOAT, A_INT, A_STRING, A_TENSOR, A_FLOATS, A_INTS = 1, 2, 3, 4, 6, 7


def dtype_code(dt) -> int:
    return _CODE_OF[np.dtype(dt)]


def np_dtype(code: int):
    return _NP_OF[code]


# ----------------------------------------------------------------------------- wire
def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(fieldno: int, wt: int) -> bytes:
    return _varint((fieldno << 3) | wt)


def _f_varint(fieldno: int, v: int) -> bytes:
    return _key(fieldno, 0) + _varint(int(v))


def _f_bytes(fieldno: int, b: bytes) -> bytes:
    return _key(fieldno, 2) + _varint(len(b)) + b


def _f_str(fieldno: int, s: str) -> bytes:
    return _f_bytes(fieldno, s.encode("utf-8"))


def _f_float(fieldno: int, v: float) -> bytes:
    return _key(fieldno, 5) + struct.pack("<f", v)


def _packed_varints(fieldno: int, vals: Sequence[int]) -> bytes:
    return _f_bytes(fieldno, b"".join(_varint(int(v)) for v in vals))


def _read_varint(buf: memoryview, pos: int) -> Tuple[int, int]:
    shift = 0
    val = 0
    while True:
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            break
        shift += 7
    return val, pos


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _fields(buf):
    """Yield (field number, wire type, value) for every field of one message."""
    buf = memoryview(buf)
    pos, n = 0, len(buf)
    while pos < n:
        k, pos = _read_varint(buf, pos)
        fno, wt = k >> 3, k & 7
        if wt == 0:
            v, pos = _read_varint(buf, pos)
            yield fno, wt, v
        elif wt == 1:
            yield fno, wt, bytes(buf[pos:pos + 8])
            pos += 8
        elif wt == 2:
            ln, pos = _read_varint(buf, pos)
            yield fno, wt, buf[pos:pos + ln]
            pos += ln
        elif wt == 5:
            yield fno, wt, bytes(buf[pos:pos + 4])
            pos += 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")


def _unpack_varints(v, wt) -> List[int]:
    if wt == 0:
        return [_signed(v)]
    out, pos, mv = [], 0, memoryview(v)
    while pos < len(mv):
        x, pos = _read_varint(mv, pos)
        out.append(_signed(x))
    return out


# ----------------------------------------------------------------------------- model
@dataclass
class ValueInfo:
    name: str
    dtype: int
    shape: Tuple[int, ...]


@dataclass
class Node:
    op_type: str
    inputs: List[str]
    outputs: List[str]
    name: str = ""
    attrs: Dict[str, Union[int, float, List[int], List[float], np.ndarray, str]] = field(
        default_factory=dict)


@dataclass
class Model:
    """An ONNX graph: what ``Parser`` reads (src/worker/parser.cpp:199-249)."""
    name: str = "graph"
    nodes: List[Node] = field(default_factory=list)
    initializers: Dict[str, np.ndarray] = field(default_factory=dict)
    inputs: List[ValueInfo] = field(default_factory=list)
    outputs: List[ValueInfo] = field(default_factory=list)
    value_info: List[ValueInfo] = field(default_factory=list)
    opset: int = 18

    def info(self, name: str) -> Optional[ValueInfo]:
        for vi in (*self.inputs, *self.outputs, *self.value_info):
            if vi.name == name:
                return vi
        if name in self.initializers:
            a = self.initializers[name]
            return ValueInfo(name, dtype_code(a.dtype), tuple(a.shape))
        return None

    # ------------------------------------------------------------------ encode
    def to_bytes(self) -> bytes:
        g = bytearray()
        for n in self.nodes:
            g += _f_bytes(1, _enc_node(n))
        g += _f_str(2, self.name)
        for name, arr in self.initializers.items():
            g += _f_bytes(5, _enc_tensor(name, arr))
        for vi in self.inputs:
            g += _f_bytes(11, _enc_value_info(vi))
        for vi in self.outputs:
            g += _f_bytes(12, _enc_value_info(vi))
        for vi in self.value_info:
            g += _f_bytes(13, _enc_value_info(vi))
        m = bytearray()
        m += _f_varint(1, 8)                      # ir_version
        m += _f_str(2, "fluidml_b200")            # producer_name
        m += _f_bytes(7, bytes(g))
        m += _f_bytes(8, _f_str(1, "") + _f_varint(2, self.opset))
        return bytes(m)

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.to_bytes())

    # ------------------------------------------------------------------ decode
    @staticmethod
    def from_bytes(data: bytes) -> "Model":
        m = Model()
        for fno, wt, v in _fields(data):
            if fno == 7:
                _dec_graph(v, m)
            elif fno == 8:
                for f2, _, v2 in _fields(v):
                    if f2 == 2:
                        m.opset = v2
        return m

    @staticmethod
    def load(path: str) -> "Model":
        with open(path, "rb") as f:
            return Model.from_bytes(f.read())


def _enc_tensor(name: str, arr: np.ndarray) -> bytes:
    arr = np.asarray(arr)
    code = dtype_code(arr.dtype)
    t = bytearray()
    if arr.ndim:
        t += _packed_varints(1, arr.shape)
    t += _f_varint(2, code)
    t += _f_str(8, name)
    t += _f_bytes(9, np.ascontiguousarray(arr).tobytes())
    return bytes(t)


def _dec_tensor(buf) -> Tuple[str, np.ndarray]:
    dims: List[int] = []
    code, name, raw = FLOAT, "", None
    floats: List[float] = []
    ints: List[int] = []
    doubles: List[float] = []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            dims += _unpack_varints(v, wt)
        elif fno == 2:
            code = v
        elif fno == 8:
            name = bytes(v).decode()
        elif fno == 9:
            raw = bytes(v)
        elif fno == 4:
            floats += list(np.frombuffer(bytes(v), "<f4")) if wt == 2 else \
                [struct.unpack("<f", v)[0]]
        elif fno in (5, 7):
            ints += _unpack_varints(v, wt)
        elif fno == 10:
            doubles += list(np.frombuffer(bytes(v), "<f8")) if wt == 2 else \
                [struct.unpack("<d", v)[0]]
    dt = np_dtype(code)
    if raw is not None:
        arr = np.frombuffer(raw, dtype=dt).copy()
    elif floats:
        arr = np.asarray(floats, dtype=dt)
    elif doubles:
        arr = np.asarray(doubles, dtype=dt)
    else:
        arr = np.asarray(ints, dtype=dt)
    return name, arr.reshape(dims)


def _enc_value_info(vi: ValueInfo) -> bytes:
    shape = b"".join(_f_bytes(1, _f_varint(1, d)) for d in vi.shape)
    tensor = _f_varint(1, vi.dtype) + _f_bytes(2, shape)
    return _f_str(1, vi.name) + _f_bytes(2, _f_bytes(1, tensor))


def _dec_value_info(buf) -> ValueInfo:
    name, code, shape = "", FLOAT, []
    for fno, _, v in _fields(buf):
        if fno == 1:
            name = bytes(v).decode()
        elif fno == 2:
            for f2, _, v2 in _fields(v):
                if f2 != 1:
                    continue
                for f3, _, v3 in _fields(v2):
                    if f3 == 1:
                        code = v3
                    elif f3 == 2:
                        for f4, _, v4 in _fields(v3):
                            if f4 == 1:
                                dv = 0
                                for f5, _, v5 in _fields(v4):
                                    if f5 == 1:
                                        dv = _signed(v5)
                                shape.append(dv)
    return ValueInfo(name, code, tuple(shape))


def _enc_attr(name: str, val) -> bytes:
    a = bytearray(_f_str(1, name))
    if isinstance(val, (bool, int, np.integer)):
        a += _f_varint(3, int(val)) + _f_varint(20, A_INT)
    elif isinstance(val, (float, np.floating)):
        a += _f_float(2, float(val)) + _f_varint(20, A_FLOAT)
    elif isinstance(val, str):
        a += _f_bytes(4, val.encode()) + _f_varint(20, A_STRING)
    elif isinstance(val, np.ndarray):
        a += _f_bytes(5, _enc_tensor("", val)) + _f_varint(20, A_TENSOR)
    elif isinstance(val, (list, tuple)):
        if val and isinstance(val[0], float):
            a += _f_bytes(7, b"".join(struct.pack("<f", x) for x in val))
            a += _f_varint(20, A_FLOATS)
        else:
            a += _packed_varints(8, val) + _f_varint(20, A_INTS)
    else:
        raise TypeError(f"attribute {name}: unsupported value {type(val)}")
    return bytes(a)


def _dec_attr(buf):
    name, typ = "", 0
    f = i = s = t = None
    floats: List[float] = []
    ints: List[int] = []
    for fno, wt, v in _fields(buf):
        if fno == 1:
            name = bytes(v).decode()
        elif fno == 2:
            f = struct.unpack("<f", v)[0]
        elif fno == 3:
            i = _signed(v)
        elif fno == 4:
            s = bytes(v).decode()
        elif fno == 5:
            t = _dec_tensor(v)[1]
        elif fno == 7:
            floats += list(np.frombuffer(bytes(v), "<f4")) if wt == 2 else \
                [struct.unpack("<f", v)[0]]
        elif fno == 8:
            ints += _unpack_varints(v, wt)
        elif fno == 20:
            typ = v
    val = {A_FLOAT: f, A_INT: i, A_STRING: s, A_TENSOR: t, A_FLOATS: [float(x) for x in floats],
           A_INTS: ints}.get(typ)
    if typ == 0:  # writers that omit `type`
        val = next((x for x in (i, f, s, t) if x is not None), ints or floats)
    return name, val


def _enc_node(n: Node) -> bytes:
    b = bytearray()
    for x in n.inputs:
        b += _f_str(1, x)
    for x in n.outputs:
        b += _f_str(2, x)
    b += _f_str(3, n.name)
    b += _f_str(4, n.op_type)
    for k, v in n.attrs.items():
        b += _f_bytes(5, _enc_attr(k, v))
    return bytes(b)


def _dec_node(buf) -> Node:
    n = Node("", [], [])
    for fno, _, v in _fields(buf):
        if fno == 1:
            n.inputs.append(bytes(v).decode())
        elif fno == 2:
            n.outputs.append(bytes(v).decode())
        elif fno == 3:
            n.name = bytes(v).decode()
        elif fno == 4:
            n.op_type = bytes(v).decode()
        elif fno == 5:
            k, val = _dec_attr(v)
            n.attrs[k] = val
    return n


def _dec_graph(buf, m: Model) -> None:
    for fno, _, v in _fields(buf):
        if fno == 1:
            m.nodes.append(_dec_node(v))
        elif fno == 2:
            m.name = bytes(v).decode()
        elif fno == 5:
            name, arr = _dec_tensor(v)
            m.initializers[name] = arr
        elif fno == 11:
            m.inputs.append(_dec_value_info(v))
        elif fno == 12:
            m.outputs.append(_dec_value_info(v))
        elif fno == 13:
            m.value_info.append(_dec_value_info(v))
