"""Generates tests/golden/ops_golden.npz: seeded inputs and torch-CPU (fp64 where it matters)
outputs for the operators on the hot path.

The reference's own operator tests compare against onnxruntime on unseeded inputs and store
nothing (test/python/node/node_test.py); onnxruntime is not available offline, so torch CPU
stands in as the independent implementation of the same ONNX operator semantics.  Shapes are
scaled-down versions of the shapes those tests use.  Run from the repository root:

    python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

torch.manual_seed(0)
rng = np.random.Generator(np.random.PCG64(2024))
out = {}


def rnd(*s):
    return rng.standard_normal(s).astype(np.float32)


def put(name, **kw):
    for k, v in kw.items():
        out[f"{name}.{k}"] = np.asarray(v)


T = lambda a: torch.from_numpy(np.asarray(a))
D = lambda a: T(a).double()

# MatMul (node_test.py:788-789, :825 shapes, scaled) and Gemm (gemm.py)
a, b = rnd(1, 4, 32, 16), rnd(1, 4, 16, 32)
put("matmul_batched", a=a, b=b, y=(D(a) @ D(b)).numpy())
a, b = rnd(1, 32, 96), rnd(96, 48)
put("matmul_bcast", a=a, b=b, y=(D(a) @ D(b)).numpy())
a, b, c = rnd(1, 96), rnd(64, 96), rnd(64)
put("gemm_transb", a=a, b=b, c=c, y=(D(a) @ D(b).T + D(c)).numpy())
a, b, c = rnd(8, 12), rnd(12, 6), rnd(8, 6)
put("gemm_alpha_beta", a=a, b=b, c=c, y=(0.5 * (D(a) @ D(b)) + 2.0 * D(c)).numpy())

# elementwise + broadcast
a, b = rnd(1, 1, 3), rnd(2, 3)
put("add_bcast", a=a, b=b, y=(T(a) + T(b)).numpy())
a, b = rnd(2, 5, 7), rnd(5, 1) + 3
put("div_bcast", a=a, b=b, y=(T(a) / T(b)).numpy())
x = rnd(4, 33)
put("erf", x=x, y=torch.erf(D(x)).numpy())
put("tanh", x=x, y=torch.tanh(D(x)).numpy())
put("sigmoid", x=x, y=torch.sigmoid(D(x)).numpy())
put("sqrt", x=np.abs(x), y=torch.sqrt(D(np.abs(x))).numpy())
put("pow3", x=np.abs(x), y=(D(np.abs(x)) ** 3).numpy())
put("gelu", x=x, y=torch.nn.functional.gelu(D(x)).numpy())

# Softmax (node_test.py:1236) and LayerNormalization (layer_normalization.py, eps 1e-12)
x = rnd(1, 4, 16, 96) * 3
put("softmax", x=x, y=torch.softmax(D(x), -1).numpy())
put("softmax_axis1", x=x, y=torch.softmax(D(x), 1).numpy())
x, g, bb = rnd(1, 16, 96) * 2 + 0.3, rnd(96) + 1, rnd(96)
put("layernorm", x=x, g=g, b=bb,
    y=torch.nn.functional.layer_norm(D(x), (96,), D(g), D(bb), float(np.float32(1e-12))).numpy())

# Conv (conv0.py depthwise 1-D k=9 pad 4; conv2.py 3x3 pad 1), strided / dilated for ONNX semantics
x, w, b = rnd(1, 8, 14, 14), rnd(6, 8, 3, 3) * 0.2, rnd(6)
put("conv3x3_pad1", x=x, w=w, b=b, y=torch.nn.functional.conv2d(D(x), D(w), D(b), padding=1).numpy())
put("conv3x3_s2", x=x, w=w, b=b, y=torch.nn.functional.conv2d(D(x), D(w), D(b), stride=2, padding=1).numpy())
put("conv3x3_d2", x=x, w=w, b=b, y=torch.nn.functional.conv2d(D(x), D(w), D(b), dilation=2, padding=2).numpy())
x, w = rnd(2, 12, 40), rnd(12, 1, 9) * 0.3
put("conv1d_depthwise", x=x, w=w, y=torch.nn.functional.conv1d(D(x), D(w), None, padding=4, groups=12).numpy())
x = rnd(1, 4, 8, 8)
put("maxpool2", x=x, y=torch.nn.functional.max_pool2d(T(x), 2, 2).numpy())
x = rnd(1, 16, 7, 7)
put("avgpool7", x=x, y=torch.nn.functional.avg_pool2d(D(x), 7).numpy())

# data movement (bit-exact)
x = rng.integers(0, 2 ** 31 - 1, (2, 3, 4, 5)).astype(np.float32)
put("transpose_0213", x=x, y=x.transpose(0, 2, 1, 3))
put("reshape", x=x, y=x.reshape(6, 20))
tab, ids = rnd(50, 8), rng.integers(0, 50, (2, 7)).astype(np.int64)
put("gather_rows", t=tab, i=ids, y=tab[ids])
x = rnd(2, 5, 4)
put("gather_axis1_scalar", x=x, y=x[:, 3, :])
idx = np.array([[1, 0], [4, 4]], np.int64)
put("gather_axis1_tensor", x=x, i=idx, y=np.take(x, idx, axis=1))
cond = np.tril(np.ones((6, 6), np.bool_)).reshape(1, 1, 6, 6)
x = rnd(2, 3, 6, 6)
put("where_scalar", c=cond, x=x, y=np.where(cond, x, np.float32(-3.0)))
x = rnd(3, 4)
put("pad", x=x, y=np.pad(x, ((1, 0), (2, 1))))
x = rng.integers(0, 5, (3, 9)).astype(np.int64)
put("cumsum", x=x, y=np.cumsum(x, 1))
x = rnd(2, 6, 5, 5)
put("reduce_mean", x=x, y=D(x).mean((2, 3), keepdim=True).numpy())

path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ops_golden.npz")
np.savez_compressed(path, **out)
print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")
