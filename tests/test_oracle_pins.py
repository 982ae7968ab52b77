"""Pins of the CPU oracle (no GPU needed).

1. The reference's own known-answer tests for this path: the gtest vectors for the
   addressing helpers (test/utils/gen_test.cpp:5-51, test/tensor/meta_test.cpp:6-26,
   test/tensor/tensor_test.cpp:6-20).
2. Golden vectors produced by an independent implementation of the same ONNX operator
   semantics (torch CPU; tests/golden/make_golden.py), standing in for the onnxruntime
   comparison of test/python/node/node_test.py.
"""
import math
import os

import numpy as np
import pytest

from oracle import oracle as orc

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ops_golden.npz"))


def g(name):
    return {k.split(".", 1)[1]: G[k] for k in G.files if k.startswith(name + ".")}


def close(got, ref, tol):
    ref = np.asarray(ref, np.float64)
    return np.abs(np.asarray(got, np.float64) - ref).max() <= tol * max(1.0, np.abs(ref).max())


# ------------------------------------------------------------------ reference gtest vectors
def test_gen_all_orders_gtest():
    orders = orc.gen_all_orders(8)  # GenTest.OrderTest: 8! distinct permutations of 0..7
    assert len(orders) == math.factorial(8)
    assert len({tuple(o) for o in orders}) == math.factorial(8)
    assert all(sorted(o) == list(range(8)) for o in orders)
    # enumeration order of the reference: the fully reversed permutation comes first
    assert orc.gen_all_orders(3)[0] == [2, 1, 0]
    assert orc.gen_all_orders(3) == [[2, 1, 0], [1, 2, 0], [1, 0, 2], [2, 0, 1], [0, 2, 1], [0, 1, 2]]


def test_gen_strides_gtest():
    assert orc.gen_strides([2, 3, 4], [0, 1, 2]) == [12, 4, 1]  # GenTest.StrideTest
    # layout[i] = physical position of logical dim i (utils.cpp:64-102)
    assert orc.gen_strides([2, 3, 4], [2, 0, 1]) == [1, 8, 2]
    assert orc.gen_strides([5], [0]) == [1]


def test_index_order_gtest():
    # GenTest.IndexTest: row-major enumeration of {2,3,4} has linear index i0*12 + i1*4 + i2
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    out = np.empty(24, np.float32)
    orc.reshape(x, out)
    assert np.array_equal(out, np.arange(24, dtype=np.float32))


def test_broadcast_shapes_gtest():
    assert orc.broadcast_shape([1, 1, 3], [2, 3]) == [1, 2, 3]           # MetaTest.BroadcastTest
    assert orc.broadcast_matmul_shape([2, 1, 3], [3, 2]) == [2, 1, 2]    # MetaTest.BroadcastMatMulTest
    assert orc.broadcast_shape([2, 3], [4, 3]) is None
    assert orc.broadcast_matmul_shape([2, 3], [4, 2]) is None


def test_tensor_get_row_major_gtest():
    # TensorTest.BasicTest: Tensor{1,2,3} element {0,1,2} is the last of six row-major values
    x = np.arange(6, dtype=np.float32).reshape(1, 2, 3)
    out = np.empty((1, 3), np.float32)
    orc.gather(x, np.asarray(1, np.int64), out, 1)
    assert out[0, 2] == 5.0


# ------------------------------------------------------------------ golden operator vectors
@pytest.mark.parametrize("name", ["matmul_batched", "matmul_bcast"])
@pytest.mark.parametrize("acc64", [False, True])
def test_matmul_golden(name, acc64):
    d = g(name)
    for order in (0, 1):
        got = orc.matmul(d["a"], d["b"], np.empty(d["y"].shape, np.float32), order, acc64)
        assert close(got, d["y"], 2e-6)
    # the two loop orders accumulate each output in the same k order: identical bits
    y0 = orc.matmul(d["a"], d["b"], np.empty(d["y"].shape, np.float32), 0, False)
    y1 = orc.matmul(d["a"], d["b"], np.empty(d["y"].shape, np.float32), 1, False)
    assert np.array_equal(y0, y1)


def test_gemm_golden():
    d = g("gemm_transb")
    assert close(orc.gemm(d["a"], d["b"], d["c"], np.empty(d["y"].shape, np.float32), 1, 1, 0, 1), d["y"], 2e-6)
    d = g("gemm_alpha_beta")  # ONNX: alpha scales the product, beta the bias
    assert close(orc.gemm(d["a"], d["b"], d["c"], np.empty(d["y"].shape, np.float32), 0.5, 2.0), d["y"], 2e-6)


def test_elementwise_golden():
    d = g("add_bcast")
    assert np.array_equal(orc.binary("Add", d["a"], d["b"], np.empty(d["y"].shape, np.float32)), d["y"])
    d = g("div_bcast")
    assert np.array_equal(orc.binary("Div", d["a"], d["b"], np.empty(d["y"].shape, np.float32)), d["y"])
    for name, op in (("erf", "Erf"), ("tanh", "Tanh"), ("sigmoid", "Sigmoid"), ("sqrt", "Sqrt")):
        d = g(name)
        assert close(orc.unary(op, d["x"], np.empty_like(d["x"])), d["y"], 3e-7), name
    d = g("pow3")
    assert close(orc.binary("Pow", d["x"], np.asarray(3.0, np.float32), np.empty_like(d["x"])), d["y"], 1e-6)
    d = g("gelu")  # the exporter's chain: x * (erf(x / sqrt2) + 1) * 0.5
    x = d["x"]
    t = orc.unary("Erf", orc.binary("Div", x, np.asarray(math.sqrt(2), np.float32), np.empty_like(x)), np.empty_like(x))
    assert close(x * (t + 1) * np.float32(0.5), d["y"], 1e-6)


def test_softmax_layernorm_golden():
    d = g("softmax")
    assert close(orc.softmax(d["x"], np.empty_like(d["x"]), -1), d["y"], 1e-6)
    d = g("softmax_axis1")
    assert close(orc.softmax(d["x"], np.empty_like(d["x"]), 1), d["y"], 1e-6)
    d = g("layernorm")
    for acc64 in (False, True):
        got = orc.layernorm(d["x"], d["g"], d["b"], np.empty_like(d["x"]), -1, np.float32(1e-12), acc64)
        assert close(got, d["y"], 3e-6)


def test_conv_pool_golden():
    for name, pads, strides, dil, group in (("conv3x3_pad1", (1, 1), (1, 1), (1, 1), 1), ("conv3x3_s2", (1, 1), (2, 2), (1, 1), 1),
                                            ("conv3x3_d2", (2, 2), (1, 1), (2, 2), 1), ("conv1d_depthwise", (4,), (1,), (1,), 12)):
        d = g(name)
        got = orc.conv(d["x"], d["w"], d.get("b"), np.empty(d["y"].shape, np.float32), pads, strides, dil, group, True)
        assert close(got, d["y"], 2e-6), name
    d = g("maxpool2")
    assert np.array_equal(orc.pool2d(d["x"], np.empty(d["y"].shape, np.float32), 0, (2, 2), (2, 2)), d["y"])
    d = g("avgpool7")
    assert close(orc.pool2d(d["x"], np.empty(d["y"].shape, np.float32), 1, (7, 7), (1, 1)), d["y"], 1e-6)


def test_data_movement_golden_bit_exact():
    d = g("transpose_0213")
    assert np.array_equal(orc.transpose(d["x"], np.empty(d["y"].shape, np.float32), (0, 2, 1, 3)), d["y"])
    d = g("reshape")
    assert np.array_equal(orc.reshape(d["x"], np.empty(d["y"].shape, np.float32)), d["y"])
    # a reshape keeps the logical order whatever the layouts are: feed a transposed view
    xt = np.ascontiguousarray(d["x"].transpose(3, 1, 0, 2)).transpose(2, 1, 3, 0)
    assert np.array_equal(orc.reshape(xt, np.empty(d["y"].shape, np.float32)), d["y"])
    d = g("gather_rows")
    assert np.array_equal(orc.gather(d["t"], d["i"], np.empty(d["y"].shape, np.float32), 0), d["y"])
    d = g("gather_axis1_scalar")
    assert np.array_equal(orc.gather(d["x"], np.asarray(3, np.int64), np.empty(d["y"].shape, np.float32), 1), d["y"])
    d = g("gather_axis1_tensor")
    assert np.array_equal(orc.gather(d["x"], d["i"], np.empty(d["y"].shape, np.float32), 1), d["y"])
    d = g("where_scalar")
    assert np.array_equal(orc.where(d["c"], d["x"], np.asarray(-3.0, np.float32), np.empty_like(d["x"])), d["y"])
    d = g("pad")
    assert np.array_equal(orc.pad(d["x"], np.empty(d["y"].shape, np.float32), [1, 2]), d["y"])
    d = g("cumsum")
    assert np.array_equal(orc.cumsum(d["x"], np.empty_like(d["x"]), 1), d["y"])
    d = g("reduce_mean")
    assert close(orc.reduce_mean(d["x"], np.empty(d["y"].shape, np.float32), [2, 3]), d["y"], 1e-6)


def test_whole_model_against_torch():
    """The unfused interpreter on a small BERT equals a direct torch fp64 forward pass."""
    import torch
    from fluidml_b200 import models
    L, H, heads = 2, 64, 4
    m = models.build_bert(layers=L, hidden=H, heads=heads, ffn=128, vocab=500, seq=16)
    x = models.bert_inputs(seq=16, vocab=500)
    x["attention_mask"][0, 12:] = 0
    W = {k: torch.from_numpy(v).double() if v.dtype == np.float32 else torch.from_numpy(v) for k, v in m.initializers.items()}
    ids, am = torch.from_numpy(x["input_ids"]), torch.from_numpy(x["attention_mask"]).double()
    ln = lambda t: torch.nn.functional.layer_norm(t, (H,), eps=float(np.float32(1e-12)))
    h = ln(W["embeddings.word"][ids] + W["embeddings.position"] + W["embeddings.token_type"])
    mask = (1 - am[:, None, None, :]) * torch.finfo(torch.float32).min
    for l in range(L):
        p = f"layer{l}."
        sp = lambda t: t.view(1, 16, heads, H // heads).transpose(1, 2)
        q, k, v = (sp(h @ W[p + n + ".w"] + W[p + n + ".b"]) for n in "qkv")
        s = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(H // heads) + mask, -1)
        c = (s @ v).transpose(1, 2).reshape(1, 16, H)
        h = ln(c @ W[p + "o.w"] + W[p + "o.b"] + h)
        f = h @ W[p + "f1.w"] + W[p + "f1.b"]
        f = f * 0.5 * (1 + torch.erf(f / math.sqrt(2.0)))
        h = ln(f @ W[p + "f2.w"] + W[p + "f2.b"] + h)
    pooled = torch.tanh(h[:, 0] @ W["pooler.w"].T + W["pooler.b"])
    for acc64 in (False, True):
        got = orc.run_model(m, x, acc64=acc64)
        assert close(got["last_hidden_state"], h.numpy(), 5e-6)
        assert close(got["pooler_output"], pooled.numpy(), 5e-6)
