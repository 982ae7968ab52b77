"""Seeded, static-shape ONNX model builders.

The reference benchmarks download ONNX-model-zoo files (cmake/models.cmake:13-88,
benchmark/bert.cpp:21-29) that are not redistributable here; these builders construct
graphs with the same operator sequences, shapes and dtypes from a seed, in the form the
reference parser requires: every intermediate has a ``value_info`` entry
(src/worker/parser.cpp:246-248) and scalars are rank-0 initialisers (:226-237).

Weights are drawn from ``numpy.random.Generator(PCG64(seed))`` in a fixed order documented
per builder, so any process can regenerate bit-identical models.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .onnx_lite import BOOL, FLOAT, INT64, Model, Node, ValueInfo, dtype_code

F32_LOWEST = float(np.finfo(np.float32).min)


def _bshape(a: Sequence[int], b: Sequence[int]) -> Tuple[int, ...]:
    return tuple(np.broadcast_shapes(tuple(a), tuple(b)))


class GraphBuilder:
    """Emits nodes while tracking static shapes (what onnx shape inference would give)."""

    def __init__(self, name: str):
        self.m = Model(name=name)
        self.shapes: Dict[str, Tuple[int, ...]] = {}
        self.dtypes: Dict[str, int] = {}
        self._n = 0
        self._outputs: List[str] = []

    # -------------------------------------------------------------- declarations
    def input(self, name: str, dtype: int, shape: Sequence[int]) -> str:
        self.m.inputs.append(ValueInfo(name, dtype, tuple(shape)))
        self.shapes[name], self.dtypes[name] = tuple(shape), dtype
        return name

    def const(self, name: str, arr: np.ndarray) -> str:
        arr = np.asarray(arr)
        self.m.initializers[name] = arr
        self.shapes[name], self.dtypes[name] = tuple(arr.shape), dtype_code(arr.dtype)
        return name

    def scalar(self, value, dtype=np.float32) -> str:
        self._n += 1
        return self.const(f"c{self._n}", np.asarray(value, dtype=dtype))

    def output(self, name: str) -> None:
        self._outputs.append(name)

    def finish(self) -> Model:
        outs = set(self._outputs)
        ins = {v.name for v in self.m.inputs}
        self.m.outputs = [ValueInfo(o, self.dtypes[o], self.shapes[o]) for o in self._outputs]
        self.m.value_info = [ValueInfo(n, self.dtypes[n], self.shapes[n])
                             for n in self.shapes
                             if n not in outs and n not in ins and n not in self.m.initializers]
        return self.m

    # -------------------------------------------------------------- node helper
    def _emit(self, op: str, ins: List[str], shape, dtype=None, out: Optional[str] = None,
              **attrs) -> str:
        self._n += 1
        out = out or f"{op.lower()}_{self._n}"
        # ONNX float attributes are fp32: keep the in-memory graph equal to the saved one.
        attrs = {k: float(np.float32(v)) if isinstance(v, float) else v
                 for k, v in attrs.items()}
        self.m.nodes.append(Node(op, list(ins), [out], name=f"{op}_{self._n}", attrs=attrs))
        self.shapes[out] = tuple(int(s) for s in shape)
        self.dtypes[out] = dtype if dtype is not None else self.dtypes[ins[0]]
        return out

    # -------------------------------------------------------------- operators
    def binary(self, op: str, a: str, b: str, out=None) -> str:
        dt = self.dtypes[a] if self.shapes[a] != () or self.shapes[b] == () else self.dtypes[b]
        return self._emit(op, [a, b], _bshape(self.shapes[a], self.shapes[b]), dt, out)

    def add(self, a, b, out=None): return self.binary("Add", a, b, out)
    def sub(self, a, b, out=None): return self.binary("Sub", a, b, out)
    def mul(self, a, b, out=None): return self.binary("Mul", a, b, out)
    def div(self, a, b, out=None): return self.binary("Div", a, b, out)
    def pow(self, a, b, out=None): return self.binary("Pow", a, b, out)

    def unary(self, op: str, a: str, out=None, **attrs) -> str:
        return self._emit(op, [a], self.shapes[a], None, out, **attrs)

    def erf(self, a, out=None): return self.unary("Erf", a, out)
    def tanh(self, a, out=None): return self.unary("Tanh", a, out)
    def relu(self, a, out=None): return self.unary("Relu", a, out)
    def sigmoid(self, a, out=None): return self.unary("Sigmoid", a, out)
    def sqrt(self, a, out=None): return self.unary("Sqrt", a, out)
    def neg(self, a, out=None): return self.unary("Neg", a, out)

    def softmax(self, a, axis=-1, out=None):
        return self.unary("Softmax", a, out, axis=axis)

    def layernorm(self, x, scale, bias, axis=-1, eps=1e-5, out=None):
        return self._emit("LayerNormalization", [x, scale, bias], self.shapes[x], None, out,
                          axis=axis, epsilon=float(eps))

    def matmul(self, a, b, out=None):
        sa, sb = self.shapes[a], self.shapes[b]
        batch = _bshape(sa[:-2], sb[:-2])
        assert sa[-1] == sb[-2], (sa, sb)
        return self._emit("MatMul", [a, b], (*batch, sa[-2], sb[-1]), None, out)

    def gemm(self, a, b, c, transA=0, transB=0, alpha=1.0, beta=1.0, out=None):
        sa, sb = self.shapes[a], self.shapes[b]
        m = sa[1] if transA else sa[0]
        n = sb[0] if transB else sb[1]
        return self._emit("Gemm", [a, b, c], (m, n), None, out, alpha=float(alpha),
                          beta=float(beta), transA=int(transA), transB=int(transB))

    def gather(self, data, indices, axis=0, out=None):
        sd, si = self.shapes[data], self.shapes[indices]
        shape = (*sd[:axis], *si, *sd[axis + 1:])
        return self._emit("Gather", [data, indices], shape, self.dtypes[data], out, axis=axis)

    def reshape(self, a, shape: Sequence[int], out=None):
        self._n += 1
        sh = self.const(f"shape{self._n}", np.asarray(shape, dtype=np.int64))
        shape = list(shape)
        if -1 in shape:
            known = -int(np.prod(shape))
            shape[shape.index(-1)] = int(np.prod(self.shapes[a])) // known
        return self._emit("Reshape", [a, sh], shape, None, out)

    def transpose(self, a, perm: Sequence[int], out=None):
        s = self.shapes[a]
        return self._emit("Transpose", [a], [s[p] for p in perm], None, out, perm=list(perm))

    def unsqueeze(self, a, axes: Sequence[int], out=None):
        self._n += 1
        ax = self.const(f"axes{self._n}", np.asarray(axes, dtype=np.int64))
        s = list(self.shapes[a])
        for x in sorted(axes):
            s.insert(x, 1)
        return self._emit("Unsqueeze", [a, ax], s, None, out)

    def squeeze(self, a, axes: Sequence[int], out=None):
        self._n += 1
        ax = self.const(f"axes{self._n}", np.asarray(axes, dtype=np.int64))
        s = [d for i, d in enumerate(self.shapes[a]) if i not in axes]
        return self._emit("Squeeze", [a, ax], s, None, out)

    def flatten(self, a, axis=1, out=None):
        s = self.shapes[a]
        return self._emit("Flatten", [a], (int(np.prod(s[:axis])), int(np.prod(s[axis:]))),
                          None, out, axis=axis)

    def conv(self, x, w, b=None, pads=None, strides=None, dilations=None, group=1, out=None):
        sx, sw = self.shapes[x], self.shapes[w]
        nd = len(sx) - 2
        pads = list(pads) if pads is not None else [0] * (2 * nd)
        strides = list(strides) if strides is not None else [1] * nd
        dilations = list(dilations) if dilations is not None else [1] * nd
        sp = [(sx[2 + i] + pads[i] + pads[nd + i] - dilations[i] * (sw[2 + i] - 1) - 1)
              // strides[i] + 1 for i in range(nd)]
        ins = [x, w] + ([b] if b is not None else [])
        return self._emit("Conv", ins, (sx[0], sw[0], *sp), None, out, dilations=dilations,
                          group=int(group), kernel_shape=list(sw[2:]), pads=pads,
                          strides=strides)

    def _pool(self, op, x, kernel, strides, out=None):
        sx = self.shapes[x]
        sp = [(sx[2 + i] - kernel[i]) // strides[i] + 1 for i in range(len(kernel))]
        return self._emit(op, [x], (sx[0], sx[1], *sp), None, out, kernel_shape=list(kernel),
                          pads=[0] * (2 * len(kernel)), strides=list(strides))

    def maxpool(self, x, kernel, strides, out=None):
        return self._pool("MaxPool", x, kernel, strides, out)

    def avgpool(self, x, kernel, strides=None, out=None):
        return self._pool("AveragePool", x, kernel, strides or [1] * len(kernel), out)

    def reduce_mean(self, x, axes: Sequence[int], out=None):
        self._n += 1
        ax = self.const(f"axes{self._n}", np.asarray(axes, dtype=np.int64))
        s = [1 if i in axes else d for i, d in enumerate(self.shapes[x])]
        return self._emit("ReduceMean", [x, ax], s, None, out, keepdims=1)

    def slice(self, x, starts, ends, axes, out=None):
        self._n += 1
        n = self._n
        s = list(self.shapes[x])
        for st, en, ax in zip(starts, ends, axes):
            s[ax] = min(en, s[ax]) - st
        ins = [x, self.const(f"starts{n}", np.asarray(starts, dtype=np.int64)),
               self.const(f"ends{n}", np.asarray(ends, dtype=np.int64)),
               self.const(f"saxes{n}", np.asarray(axes, dtype=np.int64)),
               self.const(f"steps{n}", np.ones(len(axes), dtype=np.int64))]
        return self._emit("Slice", ins, s, None, out)

    def pad(self, x, pads: Sequence[int], out=None):
        """Constant (zero) padding; `pads` = begins of every dim then ends, as in ONNX."""
        self._n += 1
        pc = self.const(f"pads{self._n}", np.asarray(pads, dtype=np.int64))
        r = len(self.shapes[x])
        s = [d + pads[i] + pads[r + i] for i, d in enumerate(self.shapes[x])]
        return self._emit("Pad", [x, pc], s, None, out)

    def concat(self, a, b, axis, out=None):
        s = list(self.shapes[a])
        s[axis] += self.shapes[b][axis]
        return self._emit("Concat", [a, b], s, None, out, axis=axis)

    def where(self, cond, x, y, out=None):
        shape = _bshape(_bshape(self.shapes[cond], self.shapes[x]), self.shapes[y])
        return self._emit("Where", [cond, x, y], shape, self.dtypes[x], out)

    def clip(self, x, lo, hi, out=None):
        return self._emit("Clip", [x, self.scalar(lo), self.scalar(hi)], self.shapes[x], None, out)


# ------------------------------------------------------------------------------ BERT
def build_bert(seed: int = 0, layers: int = 12, hidden: int = 768, heads: int = 12,
               ffn: int = 3072, vocab: int = 30522, max_pos: int = 512, type_vocab: int = 2,
               batch: int = 1, seq: int = 128, eps: float = 1e-12,
               name: str = "bert") -> Model:
    """BERT encoder + pooler, post-LN, erf-GELU, in the op sequence a transformers→ONNX
    opset-18 export produces after constant folding.

    Draw order (all fp32, N(0, 0.02)): word, position, token-type embeddings; then per layer
    the weights q,k,v,o,ffn1,ffn2 followed by the biases q,k,v,o,ffn1,ffn2; then the pooler
    weight and bias.  LayerNorm gamma = 1, beta = 0.  ``token_type_ids`` are all zero, so
    the token-type embedding is folded to its row 0; position ids are 0..seq-1.
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    nrm = lambda *s: rng.normal(0.0, 0.02, size=s).astype(np.float32)
    hd = hidden // heads
    g = GraphBuilder(name)
    ids = g.input("input_ids", INT64, (batch, seq))
    am = g.input("attention_mask", FLOAT, (batch, seq))

    word = g.const("embeddings.word", nrm(vocab, hidden))
    pos_full = nrm(max_pos, hidden)
    typ_full = nrm(type_vocab, hidden)
    pos = g.const("embeddings.position", pos_full[:seq].reshape(1, seq, hidden).copy())
    typ = g.const("embeddings.token_type", typ_full[0].copy())
    ones = np.ones(hidden, np.float32)
    zeros = np.zeros(hidden, np.float32)

    x = g.gather(word, ids, axis=0)
    x = g.add(x, pos)
    x = g.add(x, typ)
    x = g.layernorm(x, g.const("embeddings.ln.g", ones), g.const("embeddings.ln.b", zeros),
                    axis=-1, eps=eps)

    m = g.unsqueeze(am, [1])
    m = g.unsqueeze(m, [2])
    m = g.sub(g.scalar(1.0), m)
    mask = g.mul(m, g.scalar(F32_LOWEST))

    for l in range(layers):
        p = f"layer{l}."
        w = {k: nrm(*s) for k, s in (("q", (hidden, hidden)), ("k", (hidden, hidden)),
                                     ("v", (hidden, hidden)), ("o", (hidden, hidden)),
                                     ("f1", (hidden, ffn)), ("f2", (ffn, hidden)))}
        b = {k: nrm(s) for k, s in (("q", hidden), ("k", hidden), ("v", hidden),
                                    ("o", hidden), ("f1", ffn), ("f2", hidden))}
        for k in w:
            g.const(p + k + ".w", w[k])
            g.const(p + k + ".b", b[k])

        def proj(t, k):
            return g.add(p + k + ".b", g.matmul(t, p + k + ".w"))

        q = g.transpose(g.reshape(proj(x, "q"), (batch, seq, heads, hd)), (0, 2, 1, 3))
        kt = g.transpose(g.reshape(proj(x, "k"), (batch, seq, heads, hd)), (0, 2, 3, 1))
        v = g.transpose(g.reshape(proj(x, "v"), (batch, seq, heads, hd)), (0, 2, 1, 3))
        s = g.matmul(q, kt)
        s = g.div(s, g.scalar(math.sqrt(hd)))
        s = g.add(s, mask)
        s = g.softmax(s, axis=-1)
        c = g.matmul(s, v)
        c = g.reshape(g.transpose(c, (0, 2, 1, 3)), (batch, seq, hidden))
        a = g.add(proj(c, "o"), x)
        x = g.layernorm(a, g.const(p + "ln1.g", ones), g.const(p + "ln1.b", zeros),
                        axis=-1, eps=eps)
        h = proj(x, "f1")
        e = g.erf(g.div(h, g.scalar(math.sqrt(2.0))))
        h = g.mul(g.mul(h, g.add(e, g.scalar(1.0))), g.scalar(0.5))
        a = g.add(proj(h, "f2"), x)
        last = l == layers - 1
        x = g.layernorm(a, g.const(p + "ln2.g", ones), g.const(p + "ln2.b", zeros),
                        axis=-1, eps=eps, out="last_hidden_state" if last else None)

    cls = g.gather(x, g.scalar(0, np.int64), axis=1)
    pw = g.const("pooler.w", nrm(hidden, hidden))
    pb = g.const("pooler.b", nrm(hidden))
    pooled = g.gemm(cls, pw, pb, transB=1, alpha=1.0, beta=1.0)
    g.tanh(pooled, out="pooler_output")
    g.output("last_hidden_state")
    g.output("pooler_output")
    return g.finish()


def bert_inputs(seed: int = 1, batch: int = 1, seq: int = 128, vocab: int = 30522):
    """input_ids uniform in [0, vocab), attention_mask all ones."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return {"input_ids": rng.integers(0, vocab, size=(batch, seq), dtype=np.int64),
            "attention_mask": np.ones((batch, seq), np.float32)}


# ------------------------------------------------------------------------------ VGG-16
def build_vgg16(seed: int = 0, batch: int = 1, image: int = 224, classes: int = 1000,
                widths=(64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M",
                        512, 512, 512, "M"),
                fc: int = 4096, name: str = "vgg16") -> Model:
    """13 conv3x3 (pad 1, stride 1) + ReLU, 2x2 max-pools, Flatten, 3 Gemm (transB).

    He-normal weights in layer order, zero biases; input NCHW ``input`` ~ N(0,1).
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    g = GraphBuilder(name)
    x = g.input("input", FLOAT, (batch, 3, image, image))
    cin, hw, i = 3, image, 0
    for wd in widths:
        if wd == "M":
            x = g.maxpool(x, [2, 2], [2, 2])
            hw //= 2
            continue
        std = math.sqrt(2.0 / (cin * 9))
        w = g.const(f"conv{i}.w", rng.normal(0, std, (wd, cin, 3, 3)).astype(np.float32))
        b = g.const(f"conv{i}.b", np.zeros(wd, np.float32))
        x = g.relu(g.conv(x, w, b, pads=[1, 1, 1, 1], strides=[1, 1], dilations=[1, 1]))
        cin, i = wd, i + 1
    x = g.flatten(x, 1)
    dims = [cin * hw * hw, fc, fc, classes]
    for j in range(3):
        std = math.sqrt(2.0 / dims[j])
        w = g.const(f"fc{j}.w", rng.normal(0, std, (dims[j + 1], dims[j])).astype(np.float32))
        b = g.const(f"fc{j}.b", np.zeros(dims[j + 1], np.float32))
        x = g.gemm(x, w, b, transB=1, out="output" if j == 2 else None)
        if j < 2:
            x = g.relu(x)
    g.output("output")
    return g.finish()


def vgg_inputs(seed: int = 1, batch: int = 1, image: int = 224):
    rng = np.random.Generator(np.random.PCG64(seed))
    return {"input": rng.normal(0, 1, (batch, 3, image, image)).astype(np.float32)}


# ------------------------------------------------------------------------------ ConvBERT
def build_convbert(seed: int = 0, layers: int = 12, hidden: int = 768, heads: int = 12, head_ratio: int = 2,
                   conv_kernel: int = 9, ffn: int = 3072, vocab: int = 30522, max_pos: int = 512,
                   batch: int = 8, seq: int = 128, eps: float = 1e-12, name: str = "convbert") -> Model:
    """ConvBERT encoder: per layer `heads / head_ratio` self-attention heads plus a span-based
    dynamic convolution branch of the same width, concatenated before the output projection;
    then the BERT feed-forward block.  The dynamic convolution is written with the operators
    the reference converts: a depthwise Conv (1-D, kernel 9) + pointwise Conv over the
    transposed hidden states make the span-aware key, key x query goes through a Linear to
    `conv_kernel` logits per head and a Softmax, and the "unfold + matmul" over the value
    projection is a zero Pad along the sequence followed by `conv_kernel` (Slice, Slice, Mul,
    Add) steps.  Weights N(0, 0.02) from PCG64(seed) in graph order, LayerNorm gamma 1 beta 0."""
    rng = np.random.Generator(np.random.PCG64(seed))
    nrm = lambda *s: rng.normal(0.0, 0.02, size=s).astype(np.float32)
    nh = heads // head_ratio
    hd = hidden // heads
    width = nh * hd  # of each branch
    half = conv_kernel // 2
    g = GraphBuilder(name)
    ids = g.input("input_ids", INT64, (batch, seq))
    am = g.input("attention_mask", FLOAT, (batch, seq))
    word = g.const("embeddings.word", nrm(vocab, hidden))
    pos = g.const("embeddings.position", nrm(max_pos, hidden)[:seq].reshape(1, seq, hidden).copy())
    typ = g.const("embeddings.token_type", nrm(2, hidden)[0].copy())
    ones, zeros = np.ones(hidden, np.float32), np.zeros(hidden, np.float32)
    x = g.add(g.add(g.gather(word, ids, axis=0), pos), typ)
    x = g.layernorm(x, g.const("embeddings.ln.g", ones), g.const("embeddings.ln.b", zeros), axis=-1, eps=eps)
    m = g.unsqueeze(g.unsqueeze(am, [1]), [2])
    mask = g.mul(g.sub(g.scalar(1.0), m), g.scalar(F32_LOWEST))

    for l in range(layers):
        p = f"layer{l}."

        def linear(t, key, n_in, n_out):
            w = g.const(p + key + ".w", nrm(n_in, n_out))
            b = g.const(p + key + ".b", nrm(n_out))
            return g.add(b, g.matmul(t, w))

        q = linear(x, "q", hidden, width)
        k = linear(x, "k", hidden, width)
        v = linear(x, "v", hidden, width)
        # span-aware key: depthwise conv over the sequence, then a pointwise conv (+ bias)
        xt = g.transpose(x, (0, 2, 1))
        dw = g.conv(xt, g.const(p + "kconv.dw", nrm(hidden, 1, conv_kernel)), None, pads=[half, half], strides=[1],
                    dilations=[1], group=hidden)
        pw = g.conv(dw, g.const(p + "kconv.pw", nrm(width, hidden, 1)), g.const(p + "kconv.b", nrm(width)),
                    pads=[0, 0], strides=[1], dilations=[1])
        kc = g.transpose(pw, (0, 2, 1))
        ck = linear(g.mul(kc, q), "ck", width, nh * conv_kernel)
        ck = g.softmax(g.reshape(ck, (batch, seq, nh, conv_kernel)), axis=-1)
        co = g.reshape(linear(x, "co", hidden, width), (batch, seq, nh, hd))
        co = g.pad(co, [0, half, 0, 0, 0, half, 0, 0])
        acc = None
        for j in range(conv_kernel):
            term = g.mul(g.slice(co, [j], [j + seq], [1]), g.slice(ck, [j], [j + 1], [3]))
            acc = term if acc is None else g.add(acc, term)
        conv_out = g.reshape(acc, (batch, seq, width))
        # self-attention over the other half of the heads
        qh = g.transpose(g.reshape(q, (batch, seq, nh, hd)), (0, 2, 1, 3))
        kt = g.transpose(g.reshape(k, (batch, seq, nh, hd)), (0, 2, 3, 1))
        vh = g.transpose(g.reshape(v, (batch, seq, nh, hd)), (0, 2, 1, 3))
        s = g.softmax(g.add(g.div(g.matmul(qh, kt), g.scalar(math.sqrt(hd))), mask), axis=-1)
        ctx = g.reshape(g.transpose(g.matmul(s, vh), (0, 2, 1, 3)), (batch, seq, width))
        cat = g.concat(ctx, conv_out, axis=2)
        a = g.add(linear(cat, "o", hidden, hidden), x)
        x = g.layernorm(a, g.const(p + "ln1.g", ones), g.const(p + "ln1.b", zeros), axis=-1, eps=eps)
        h = linear(x, "f1", hidden, ffn)
        e = g.erf(g.div(h, g.scalar(math.sqrt(2.0))))
        h = g.mul(g.mul(h, g.add(e, g.scalar(1.0))), g.scalar(0.5))
        a = g.add(linear(h, "f2", ffn, hidden), x)
        x = g.layernorm(a, g.const(p + "ln2.g", ones), g.const(p + "ln2.b", zeros), axis=-1, eps=eps,
                        out="last_hidden_state" if l == layers - 1 else None)
    g.output("last_hidden_state")
    return g.finish()


def convbert_inputs(seed: int = 1, batch: int = 8, seq: int = 128, vocab: int = 30522):
    return bert_inputs(seed, batch, seq, vocab)


# ------------------------------------------------------------------------------ EfficientNet-B0
# (expand ratio, depthwise kernel, stride, output channels, repeats) of the seven stages
_EFFNET_B0_STAGES = ((1, 3, 1, 16, 1), (6, 3, 2, 24, 2), (6, 5, 2, 40, 2), (6, 3, 2, 80, 3),
                     (6, 5, 1, 112, 3), (6, 5, 2, 192, 4), (6, 3, 1, 320, 1))


def build_efficientnet_b0(seed: int = 0, batch: int = 1, image: int = 224, classes: int = 1000,
                          width: float = 1.0, stages=_EFFNET_B0_STAGES, std: float = 0.02) -> Model:
    """EfficientNet-B0 with batch norm folded into the convolutions (every conv carries a bias):
    stem conv3x3 stride 2 (32 channels), 16 MBConv blocks (1x1 expansion, depthwise 3x3 / 5x5,
    squeeze-and-excite with ratio 0.25 of the block input, 1x1 projection, residual when the
    shape is kept), head conv1x1 (1280), global average pool, FC.  SiLU is written Sigmoid x Mul,
    the SE gate Sigmoid.  Weights N(0, std) (0.02 as configured; tests widen it so that the
    logits are not all bias), biases N(0, 0.02), from PCG64(seed), drawn in graph order.
    `width` scales the channel counts (tests use a narrow copy); `image` must make the final
    feature map square with an integral size (multiples of 32)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    g = GraphBuilder("efficientnet_b0")
    ch = lambda c: max(8, int(round(c * width / 8)) * 8)
    counter = [0]

    def conv(x, cout, k, stride=1, group=1, act=None):
        counter[0] += 1
        cin = g.shapes[x][1]
        w = g.const(f"conv{counter[0]}.w", (rng.standard_normal((cout, cin // group, k, k)) * std).astype(np.float32))
        b = g.const(f"conv{counter[0]}.b", (rng.standard_normal(cout) * 0.02).astype(np.float32))
        y = g.conv(x, w, b, pads=[k // 2] * 4, strides=[stride, stride], dilations=[1, 1], group=group)
        if act == "silu":
            y = g.mul(y, g.sigmoid(y))
        elif act == "sigmoid":
            y = g.sigmoid(y)
        return y

    x = g.input("input", 1, (batch, 3, image, image))
    y = conv(x, ch(32), 3, stride=2, act="silu")
    for expand, k, stride, cout, repeats in stages:
        for r in range(repeats):
            cin = g.shapes[y][1]
            s = stride if r == 0 else 1
            t = y
            if expand != 1:
                t = conv(t, cin * expand, 1, act="silu")
            mid = g.shapes[t][1]
            t = conv(t, mid, k, stride=s, group=mid, act="silu")
            gate = g.reduce_mean(t, [2, 3])
            gate = conv(gate, max(1, cin // 4), 1, act="silu")
            gate = conv(gate, mid, 1, act="sigmoid")
            t = g.mul(t, gate)
            t = conv(t, ch(cout), 1)
            y = g.add(y, t) if s == 1 and cin == ch(cout) else t
    y = conv(y, ch(1280), 1, act="silu")
    hw = g.shapes[y][2]
    y = g.avgpool(y, [hw, hw])
    y = g.flatten(y, 1)
    fc_w = g.const("fc.w", (rng.standard_normal((classes, g.shapes[y][1])) * 0.02).astype(np.float32))
    fc_b = g.const("fc.b", (rng.standard_normal(classes) * 0.02).astype(np.float32))
    g.output(g.gemm(y, fc_w, fc_b, transB=1, out="logits"))
    return g.finish()


def efficientnet_inputs(seed: int = 1, batch: int = 1, image: int = 224):
    rng = np.random.Generator(np.random.PCG64(seed))
    return {"input": rng.standard_normal((batch, 3, image, image)).astype(np.float32)}


# ------------------------------------------------------------------------------ GPT-NeoX
def build_gpt_neox(seed: int = 0, layers: int = 24, hidden: int = 1024, heads: int = 16,
                   ffn: int = 4096, vocab: int = 50304, batch: int = 4, seq: int = 512,
                   rotary_pct: float = 0.25, base: float = 10000.0, eps: float = 1e-5,
                   name: str = "gpt_neox") -> Model:
    """GPT-NeoX decoder (Pythia shape): parallel residual, rotary on the first
    ``rotary_pct`` of each head, causal mask through Where with a constant condition.

    Draw order: token embedding; per layer qkv (as three [hidden,hidden] weights q,k,v), o,
    ffn1, ffn2 weights, then their biases; final LN gamma=1 beta=0; no LM head (the output is
    the final hidden state, as in the zoo model the reference benchmarks).
    """
    rng = np.random.Generator(np.random.PCG64(seed))
    nrm = lambda *s: rng.normal(0.0, 0.02, size=s).astype(np.float32)
    hd = hidden // heads
    rot = int(hd * rotary_pct)
    g = GraphBuilder(name)
    ids = g.input("input_ids", INT64, (batch, seq))
    emb = g.const("embed_in", nrm(vocab, hidden))
    x = g.gather(emb, ids, axis=0)
    inv = 1.0 / (base ** (np.arange(0, rot, 2, dtype=np.float64) / rot))
    ang = np.outer(np.arange(seq, dtype=np.float64), inv)
    ang = np.concatenate([ang, ang], axis=-1)
    cos = g.const("rotary.cos", np.cos(ang).astype(np.float32).reshape(1, 1, seq, rot))
    sin = g.const("rotary.sin", np.sin(ang).astype(np.float32).reshape(1, 1, seq, rot))
    causal = g.const("causal", np.tril(np.ones((seq, seq), np.bool_)).reshape(1, 1, seq, seq))
    ones, zeros = np.ones(hidden, np.float32), np.zeros(hidden, np.float32)

    def rope(t):
        tr = g.slice(t, [0], [rot], [3])
        tp = g.slice(t, [rot], [hd], [3])
        t1 = g.slice(tr, [0], [rot // 2], [3])
        t2 = g.slice(tr, [rot // 2], [rot], [3])
        rh = g.concat(g.neg(t2), t1, 3)
        tr = g.add(g.mul(tr, cos), g.mul(rh, sin))
        return g.concat(tr, tp, 3)

    for l in range(layers):
        p = f"layer{l}."
        w = {k: nrm(*s) for k, s in (("q", (hidden, hidden)), ("k", (hidden, hidden)),
                                     ("v", (hidden, hidden)), ("o", (hidden, hidden)),
                                     ("f1", (hidden, ffn)), ("f2", (ffn, hidden)))}
        b = {k: nrm(s) for k, s in (("q", hidden), ("k", hidden), ("v", hidden),
                                    ("o", hidden), ("f1", ffn), ("f2", hidden))}
        for k in w:
            g.const(p + k + ".w", w[k])
            g.const(p + k + ".b", b[k])

        def proj(t, k):
            return g.add(p + k + ".b", g.matmul(t, p + k + ".w"))

        h1 = g.layernorm(x, g.const(p + "ln1.g", ones), g.const(p + "ln1.b", zeros), -1, eps)
        h2 = g.layernorm(x, g.const(p + "ln2.g", ones), g.const(p + "ln2.b", zeros), -1, eps)
        q = g.transpose(g.reshape(proj(h1, "q"), (batch, seq, heads, hd)), (0, 2, 1, 3))
        k_ = g.transpose(g.reshape(proj(h1, "k"), (batch, seq, heads, hd)), (0, 2, 1, 3))
        v = g.transpose(g.reshape(proj(h1, "v"), (batch, seq, heads, hd)), (0, 2, 1, 3))
        q, k_ = rope(q), rope(k_)
        s = g.matmul(q, g.transpose(k_, (0, 1, 3, 2)))
        s = g.div(s, g.scalar(math.sqrt(hd)))
        s = g.where(causal, s, g.scalar(F32_LOWEST))
        s = g.softmax(s, axis=-1)
        c = g.reshape(g.transpose(g.matmul(s, v), (0, 2, 1, 3)), (batch, seq, hidden))
        attn = proj(c, "o")
        f = proj(h2, "f1")
        e = g.erf(g.div(f, g.scalar(math.sqrt(2.0))))
        f = g.mul(g.mul(f, g.add(e, g.scalar(1.0))), g.scalar(0.5))
        f = proj(f, "f2")
        x = g.add(g.add(attn, f), x)
    g.layernorm(x, g.const("final_ln.g", ones), g.const("final_ln.b", zeros), -1, eps,
                out="last_hidden_state")
    g.output("last_hidden_state")
    return g.finish()


def gpt_neox_inputs(seed: int = 1, batch: int = 4, seq: int = 512, vocab: int = 50304):
    rng = np.random.Generator(np.random.PCG64(seed))
    return {"input_ids": rng.integers(0, vocab, size=(batch, seq), dtype=np.int64)}
