"""GPU parity of the memory-bound kernels against the CPU oracle, through the C ABI.

Bit-exact for data movement (Transpose / Reshape / Gather / Slice / Concat / Where / Pad);
fp32 elementwise and reductions within the tolerance written beside each case.
"""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT
from oracle import oracle as orc

RNG = np.random.Generator(np.random.PCG64(1234))


def rnd(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def relerr(got, ref):
    ref = ref.astype(np.float64)
    return float(np.abs(got.astype(np.float64) - ref).max() / max(1e-30, np.abs(ref).max()))


# ------------------------------------------------------------------ elementwise
BIN_CASES = [
    ((1, 128, 768), (768,)),            # bias add
    ((1, 128, 768), (1, 128, 768)),     # residual
    ((1, 12, 128, 128), (1, 1, 1, 128)),  # attention mask
    ((3, 5, 7), (5, 1)),                # ragged broadcast, odd sizes
    ((2, 1, 3), (1, 4, 3)),             # both sides broadcast
    ((0, 4), (4,)),                     # empty
    ((6, 10, 8, 12), (6, 10, 1, 1)),    # per-plane scale (squeeze-and-excite gate): 16-byte path, scalar rhs
    ((5, 7, 3, 64), (5, 7, 3, 1)),      # per-row scale with odd outer extents
    ((6, 10, 1, 1), (6, 10, 8, 12)),    # the same with the operands swapped
]


@pytest.mark.parametrize("op,name", [(cabi.ADD, "Add"), (cabi.MUL, "Mul"), (cabi.SUB, "Sub"),
                                     (cabi.DIV, "Div")])
@pytest.mark.parametrize("sa,sb", BIN_CASES)
def test_binary_broadcast(op, name, sa, sb):
    a, b = rnd(*sa), rnd(*sb) + 3.0
    so = np.broadcast_shapes(sa, sb)
    ref = orc.binary(name, a, b, np.empty(so, np.float32))
    out = DT(so, np.float32)
    cabi.elementwise(op, DT.from_numpy(a), DT.from_numpy(b), out)
    assert np.array_equal(out.numpy(), ref)  # one IEEE operation per element: bit-exact


@pytest.mark.parametrize("sa,sb,sc", [
    ((8, 128, 6, 64), (8, 128, 6, 1), (8, 128, 6, 64)),   # ConvBERT's span convolution step: per-row weight
    ((4, 16, 512, 32), (1, 1, 512, 32), (4, 16, 512, 32)),  # rotary embedding: table broadcast over batch and heads
    ((3, 5, 7), (5, 1), (7,)),                             # ragged: the element-wise path
    ((2, 6, 8), (2, 6, 8), (1,)),                          # scalar addend
    ((0, 4), (4,), (4,)),
])
def test_mul_add_is_mul_then_add(sa, sb, sc):
    """fml_mul_add rounds twice, like MulCommon followed by AddCommon: bit-exact against the oracle's
    two kernels."""
    a, b, c = rnd(*sa), rnd(*sb), rnd(*sc)
    sp = np.broadcast_shapes(sa, sb)
    so = np.broadcast_shapes(sp, sc)
    prod = orc.binary("Mul", a, b, np.empty(sp, np.float32))
    ref = orc.binary("Add", prod, c, np.empty(so, np.float32))
    out = DT(so, np.float32)
    cabi.mul_add(DT.from_numpy(a), DT.from_numpy(b), DT.from_numpy(c), out)
    assert np.array_equal(out.numpy(), ref)


def _oracle_act(v, act):
    v = v.astype(np.float32)
    if act == 2:
        return np.maximum(v, np.float32(0))
    if act == 4:
        return orc.unary("Sigmoid", v, np.empty_like(v))
    if act == 5:
        return orc.binary("Mul", v, orc.unary("Sigmoid", v, np.empty_like(v)), np.empty_like(v))
    return v


@pytest.mark.parametrize("n,c,h,w,cr,act1,act2,bias,layout", [
    (1, 32, 112, 112, 8, 5, 4, True, None),      # EfficientNet's first block: large planes, CTA per plane
    (1, 144, 56, 56, 6, 5, 4, True, None),
    (2, 240, 28, 28, 10, 5, 4, True, None),      # warp per plane
    (1, 1152, 7, 7, 48, 5, 4, True, None),       # last stage: odd plane size
    (3, 20, 5, 3, 7, 2, 0, False, None),         # ragged everything, relu / none, no biases
    (2, 5, 4, 4, 3, 0, 4, True, None),           # fewer channels than a full cluster
    (2, 24, 6, 10, 4, 5, 4, True, (0, 2, 3, 1)), # channel-innermost x: strided planes
    (0, 8, 4, 4, 2, 5, 4, True, None),           # empty batch
])
def test_squeeze_excite_gate_matches_the_three_kernels(n, c, h, w, cr, act1, act2, bias, layout):
    """fml_squeeze_excite_gate against the oracle's ReduceMean -> Conv -> Conv (activations applied
    with the oracle's own kernels).  fp32 sums in another order: 2e-6 of the largest gate value
    plus 1e-6 absolute."""
    x = rnd(n, c, h, w)
    w1, w2 = rnd(cr, c, 1, 1) * np.float32(0.3), rnd(c, cr, 1, 1) * np.float32(0.5)
    b1 = rnd(cr) if bias else None
    b2 = rnd(c) if bias else None
    gate = DT((n, c, 1, 1), np.float32)
    cabi.squeeze_excite_gate(DT.from_numpy(x, layout), DT.from_numpy(w1), DT.from_numpy(b1) if bias else None,
                             DT.from_numpy(w2), DT.from_numpy(b2) if bias else None, act1, act2, gate)
    got = gate.numpy()
    if n == 0:
        assert got.shape == (0, c, 1, 1)
        return
    mean = orc.reduce_mean(x, np.empty((n, c, 1, 1), np.float32), (2, 3))
    hid = orc.conv(mean, w1, b1, np.empty((n, cr, 1, 1), np.float32), [0, 0, 0, 0], [1, 1], [1, 1])
    hid = _oracle_act(hid, act1)
    ref = orc.conv(hid, w2, b2, np.empty((n, c, 1, 1), np.float32), [0, 0, 0, 0], [1, 1], [1, 1])
    ref = _oracle_act(ref, act2)
    tol = 2e-6 * float(np.abs(ref).max()) + 1e-6
    assert float(np.abs(got - ref).max()) <= tol


def test_squeeze_excite_gate_rejects_what_it_cannot_take():
    x = DT.from_numpy(rnd(1, 8, 4, 4))
    gate = DT((1, 8, 1, 1), np.float32)
    with pytest.raises(cabi.FmlError):   # hidden width of w2 does not match w1
        cabi.squeeze_excite_gate(x, DT.from_numpy(rnd(2, 8, 1, 1)), None, DT.from_numpy(rnd(8, 3, 1, 1)), None, 5, 4, gate)
    with pytest.raises(cabi.FmlError):   # exact GELU is not one of the gate activations
        cabi.squeeze_excite_gate(x, DT.from_numpy(rnd(2, 8, 1, 1)), None, DT.from_numpy(rnd(8, 2, 1, 1)), None, 1, 4, gate)


@pytest.mark.parametrize("shape,rot,cs_shape,strided", [
    ((4, 16, 512, 64), 16, (512, 16), True),    # GPT-NeoX: a quarter of each head rotated, x a transposed view of [B, S, H, D]
    ((2, 3, 10, 64), 64, (1, 1, 10, 64), False),  # the whole head rotated
    ((2, 5, 6), 4, (5, 4), False),               # rot not a multiple of 8: element path
    ((3, 7, 10), 10, (7, 10), False),            # odd everything
])
def test_rotary_equals_the_exported_chain(shape, rot, cs_shape, strided):
    """fml_rotary against the oracle's kernels run as the exported graph runs them (Slice, Neg,
    Concat, Mul, Mul, Add, Concat): bit-exact."""
    x = rnd(*shape)
    cosv, sinv = rnd(*cs_shape), rnd(*cs_shape)
    half = rot // 2
    xr = np.ascontiguousarray(x[..., :rot])
    rh = np.concatenate([orc.unary("Neg", np.ascontiguousarray(xr[..., half:]), np.empty(xr[..., half:].shape, np.float32)),
                         xr[..., :half]], axis=-1)
    p_sin = orc.binary("Mul", np.ascontiguousarray(rh), sinv, np.empty(xr.shape, np.float32))
    p_cos = orc.binary("Mul", xr, cosv, np.empty(xr.shape, np.float32))
    ref = np.concatenate([orc.binary("Add", p_cos, p_sin, np.empty(xr.shape, np.float32)), x[..., rot:]], axis=-1)
    if strided:  # stored [B, S, H, D], seen as [B, H, S, D]
        base = DT.from_numpy(np.ascontiguousarray(x.transpose(0, 2, 1, 3)))
        st = list(base.strides)
        st[1], st[2] = st[2], st[1]
        dx = base.view(shape, st, 0)
    else:
        dx = DT.from_numpy(x)
    out = DT(shape, np.float32)
    cabi.rotary(dx, DT.from_numpy(cosv), DT.from_numpy(sinv), rot, out)
    assert np.array_equal(out.numpy(), ref)


@pytest.mark.parametrize("shape,bshape,n,windows", [
    ((8, 128, 6, 64), (8, 128, 6, 1), 9, True),    # ConvBERT's span convolution: sliding windows of one padded tensor x softmax columns
    ((2, 5, 7, 3), (2, 5, 7, 3), 3, False),       # odd sizes: element path
    ((4, 32, 16), (1, 32, 1), 12, False),          # the maximum number of pairs, broadcast along two dims
    ((3, 40), (3, 40), 1, False),                  # a single product
])
def test_sum_of_products_equals_the_mul_add_chain(shape, bshape, n, windows):
    """fml_sum_of_products rounds every product and every partial sum like the chain MulCommon ->
    (MulCommon, AddCommon) x (n - 1) it replaces: bit-exact against the oracle's kernels run in
    that order, also when the operands are overlapping strided views of one buffer."""
    if windows:  # a_i = padded[:, i : i + L] (views), b_i = columns of one [..., n] tensor (views)
        B, L, H, D = shape
        padded = rnd(B, L + n - 1, H, D)
        taps = rnd(B, L, H, n)
        dp, dt = DT.from_numpy(padded), DT.from_numpy(taps)
        a_h = [padded[:, i:i + L] for i in range(n)]
        b_h = [taps[..., i:i + 1] for i in range(n)]
        a_d = [dp.view(shape, dp.strides, i * dp.strides[1]) for i in range(n)]
        b_d = [dt.view(bshape, dt.strides, i) for i in range(n)]
    else:
        a_h = [rnd(*shape) for _ in range(n)]
        b_h = [rnd(*bshape) for _ in range(n)]
        a_d = [DT.from_numpy(t) for t in a_h]
        b_d = [DT.from_numpy(t) for t in b_h]
    acc = orc.binary("Mul", np.ascontiguousarray(a_h[0]), np.ascontiguousarray(b_h[0]), np.empty(shape, np.float32))
    for i in range(1, n):
        prod = orc.binary("Mul", np.ascontiguousarray(a_h[i]), np.ascontiguousarray(b_h[i]), np.empty(shape, np.float32))
        acc = orc.binary("Add", prod, acc, np.empty(shape, np.float32))
    out = DT(shape, np.float32)
    cabi.sum_of_products(a_d, b_d, out)
    assert np.array_equal(out.numpy(), acc)


@pytest.mark.parametrize("sa,sb,axis,dtype", [
    ((4, 16, 64, 16), (4, 16, 64, 16), 3, np.float32),   # rotary halves: 16-byte groups, split inside the innermost dim
    ((2, 8, 12, 32), (2, 4, 12, 32), 1, np.float32),     # 16-byte groups, split along an outer dim
    ((2, 3, 5), (2, 4, 5), 1, np.float32),               # ragged rows: element path
    ((3, 7), (3, 2), 1, np.float32),
    ((2, 5), (3, 5), 0, np.int64),
    ((0, 4), (2, 4), 0, np.float32),
])
def test_concat2_in_one_launch(sa, sb, axis, dtype):
    a = (RNG.standard_normal(sa) * 100).astype(dtype)
    b = (RNG.standard_normal(sb) * 100).astype(dtype)
    ref = np.concatenate([a, b], axis=axis)
    out = DT(ref.shape, dtype)
    cabi.concat2(DT.from_numpy(a), DT.from_numpy(b), out, axis)
    assert np.array_equal(out.numpy(), ref)
    if len(sa) == 3:  # operands and output in permuted layouts
        out = DT(ref.shape, dtype, [1, 2, 0])
        cabi.concat2(DT.from_numpy(a, [2, 0, 1]), DT.from_numpy(b, [0, 2, 1]), out, axis)
        assert np.array_equal(out.numpy(), ref)


@pytest.mark.parametrize("layouts", [((0, 1, 2), (2, 0, 1), (1, 2, 0)), ((2, 1, 0), (0, 1, 2), (0, 2, 1))])
def test_binary_any_layout(layouts):
    la, lb, lo = layouts
    a, b = rnd(4, 6, 8), rnd(4, 6, 8)
    out = DT((4, 6, 8), np.float32, lo)
    cabi.elementwise(cabi.ADD, DT.from_numpy(a, la), DT.from_numpy(b, lb), out)
    assert np.array_equal(out.numpy(), a + b)


@pytest.mark.parametrize("op,name,p0,p1,tol", [
    (cabi.ERF, "Erf", 0, 0, 2e-6), (cabi.TANH, "Tanh", 0, 0, 2e-6), (cabi.SQRT, "Sqrt", 0, 0, 0),
    (cabi.NEG, "Neg", 0, 0, 0), (cabi.RELU, "Relu", 0, 0, 0), (cabi.SIGMOID, "Sigmoid", 0, 0, 2e-6),
    (cabi.CLIP, "Clip", -0.5, 0.75, 0)])
def test_unary(op, name, p0, p1, tol):
    x = np.abs(rnd(1, 128, 3072)) if name == "Sqrt" else rnd(1, 128, 3072)
    ref = orc.unary(name, x, np.empty_like(x), p0, p1)
    out = DT(x.shape, np.float32)
    cabi.elementwise(op, DT.from_numpy(x), None, out, p0, p1)
    got = out.numpy()
    if tol == 0:
        assert np.array_equal(got, ref)
    else:  # libm vs CUDA math library: a few ulp
        assert np.abs(got - ref).max() <= tol


def test_scalar_variants():
    x = rnd(1, 12, 128, 128)
    for op, ref in ((cabi.ADD_SCALAR, x + np.float32(1.0)), (cabi.MUL_SCALAR, x * np.float32(0.5)),
                    (cabi.DIV_SCALAR, x / np.float32(8.0)), (cabi.RSUB_SCALAR, np.float32(1.0) - x)):
        p0 = {cabi.ADD_SCALAR: 1.0, cabi.MUL_SCALAR: 0.5, cabi.DIV_SCALAR: 8.0, cabi.RSUB_SCALAR: 1.0}[op]
        out = DT(x.shape, np.float32)
        cabi.elementwise(op, DT.from_numpy(x), None, out, p0)
        assert np.array_equal(out.numpy(), ref)
    p = np.float32(3.0)
    out = DT(x.shape, np.float32)
    cabi.elementwise(cabi.POW_SCALAR, DT.from_numpy(np.abs(x)), None, out, 3.0)
    assert relerr(out.numpy(), np.abs(x).astype(np.float64) ** 3) < 1e-6
    # mask preprocessing (1 - m) * lowest, fused
    m = (RNG.random((2, 1, 1, 128)) > 0.3).astype(np.float32)
    out = DT(m.shape, np.float32)
    lowest = float(np.finfo(np.float32).min)
    cabi.elementwise(cabi.RSUB_MUL_SCALAR, DT.from_numpy(m), None, out, 1.0, lowest)
    assert np.array_equal(out.numpy(), (np.float32(1.0) - m) * np.float32(lowest))


def test_int64_and_bool_ops():
    a = RNG.integers(-50, 50, (3, 17)).astype(np.int64)
    b = RNG.integers(-50, 50, (17,)).astype(np.int64)
    for op, ref in ((cabi.ADD, a + b), (cabi.MUL, a * b), (cabi.SUB, a - b)):
        out = DT(a.shape, np.int64)
        cabi.elementwise(op, DT.from_numpy(a), DT.from_numpy(b), out)
        assert np.array_equal(out.numpy(), ref)
    out = DT(a.shape, np.bool_)
    cabi.elementwise(cabi.EQUAL_SCALAR, DT.from_numpy(a), None, out, 3)
    assert np.array_equal(out.numpy(), a == 3)
    nb = DT(a.shape, np.bool_)
    cabi.elementwise(cabi.NOT, out, None, nb)
    assert np.array_equal(nb.numpy(), a != 3)
    f = DT(a.shape, np.float32)
    cabi.elementwise(cabi.CAST, DT.from_numpy(a), None, f)
    assert np.array_equal(f.numpy(), a.astype(np.float32))


def test_bias_gelu_matches_unfused_chain():
    x, b = rnd(1, 128, 3072), rnd(3072)
    c0, c1, c2 = np.float32(np.sqrt(2.0)), np.float32(1.0), np.float32(0.5)
    t = orc.binary("Add", x, b, np.empty_like(x))
    e = orc.unary("Erf", orc.binary("Div", t, np.asarray(c0), np.empty_like(x)), np.empty_like(x))
    ref = (t * (e + c1)) * c2
    out = DT(x.shape, np.float32)
    cabi.bias_gelu(DT.from_numpy(x), DT.from_numpy(b), out, c0, c1, c2)
    assert np.abs(out.numpy() - ref).max() <= 4e-6


def test_where():
    cond = np.tril(np.ones((64, 64), np.bool_)).reshape(1, 1, 64, 64)
    x = rnd(2, 4, 64, 64)
    lowest = float(np.finfo(np.float32).min)
    out = DT(x.shape, np.float32)
    cabi.where(DT.from_numpy(cond), DT.from_numpy(x), None, lowest, out)
    ref = orc.where(cond, x, np.asarray(lowest, np.float32), np.empty_like(x))
    assert np.array_equal(out.numpy(), ref)
    y = rnd(64)
    cabi.where(DT.from_numpy(cond), DT.from_numpy(x), DT.from_numpy(y), 0.0, out)
    assert np.array_equal(out.numpy(), np.where(cond, x, y))


@pytest.mark.parametrize("shape,cshape,yshape", [((3, 5, 7), (5, 7), (7,)),       # odd inner extent: scalar kernel
                                                 ((2, 6, 16), (2, 6, 1), (16,)),   # condition broadcast along rows
                                                 ((4, 8, 32), (8, 32), (4, 8, 1))])  # y broadcast along rows
def test_where_broadcast_forms(shape, cshape, yshape):
    rng = np.random.default_rng(7)
    cond = rng.random(cshape) < 0.5
    x, y = rnd(*shape), rnd(*yshape)
    out = DT(shape, np.float32)
    cabi.where(DT.from_numpy(cond), DT.from_numpy(x), DT.from_numpy(y), 0.0, out)
    assert np.array_equal(out.numpy(), np.where(cond, x, y))


@pytest.mark.parametrize("xshape,bshape", [((5, 33), (33,)), ((6, 64), (6, 1)), ((2, 8, 64), (8, 64))])
def test_bias_gelu_broadcast_forms(xshape, bshape):
    x, b = rnd(*xshape), rnd(*bshape)
    c0, c1, c2 = np.float32(np.sqrt(2.0)), np.float32(1.0), np.float32(0.5)
    t = x + b
    e = orc.unary("Erf", (t / c0).astype(np.float32), np.empty_like(t))
    out = DT(xshape, np.float32)
    cabi.bias_gelu(DT.from_numpy(x), DT.from_numpy(b), out, c0, c1, c2)
    assert np.abs(out.numpy() - (t * (e + c1)) * c2).max() <= 4e-6


# ------------------------------------------------------------------ data movement (bit-exact)
@pytest.mark.parametrize("shape,perm", [((1, 128, 12, 64), (0, 2, 1, 3)), ((1, 128, 12, 64), (0, 2, 3, 1)),
                                        ((1, 12, 128, 64), (0, 2, 1, 3)), ((5, 7, 3), (2, 0, 1)),
                                        ((33, 65), (1, 0)), ((2, 3, 4, 5), (3, 2, 1, 0)),
                                        ((260, 196), (1, 0)), ((2, 128, 3, 68), (0, 2, 3, 1))])
@pytest.mark.parametrize("dtype", [np.float32, np.int64, np.bool_])
def test_transpose_bit_exact(shape, perm, dtype):
    x = (RNG.integers(0, 2**31 - 1, shape)).astype(dtype)
    oshape = tuple(shape[p] for p in perm)
    ref = orc.transpose(x, np.empty(oshape, dtype), perm)
    assert np.array_equal(ref, x.transpose(perm))
    src = DT.from_numpy(x)
    out = DT(oshape, dtype)
    view = src.view(oshape, [src.strides[p] for p in perm])  # Transpose = permuted-stride view
    cabi.copy_strided(view, out)
    assert np.array_equal(out.numpy(), ref)


@pytest.mark.parametrize("li,lo", [((0, 1, 2), (0, 1, 2, 3)), ((2, 0, 1), (0, 1, 2, 3)),
                                   ((0, 1, 2), (3, 1, 0, 2)), ((1, 2, 0), (2, 3, 1, 0))])
def test_reshape_logical_order_any_layout(li, lo):
    x = rnd(2, 16, 24)
    ref = orc.reshape(x, np.empty((2, 16, 4, 6), np.float32))
    assert np.array_equal(ref, x.reshape(2, 16, 4, 6))
    out = DT((2, 16, 4, 6), np.float32, lo)
    cabi.reshape_copy(DT.from_numpy(x, li), out)
    assert np.array_equal(out.numpy(), ref)


def test_gather_variants():
    table = rnd(30522, 768)
    ids = RNG.integers(0, 30522, (1, 128)).astype(np.int64)
    ref = orc.gather(table, ids, np.empty((1, 128, 768), np.float32), 0)
    out = DT((1, 128, 768), np.float32)
    cabi.gather(DT.from_numpy(table), DT.from_numpy(ids), out, 0)
    assert np.array_equal(out.numpy(), ref)
    cabi.check_device()
    x = rnd(2, 128, 768)
    out = DT((2, 768), np.float32)
    cabi.gather(DT.from_numpy(x), DT.from_numpy(np.asarray(0, np.int64)), out, 1)
    assert np.array_equal(out.numpy(), x[:, 0, :])
    idx = np.array([[3, 0], [5, 5]], np.int64)
    x = rnd(4, 6, 5)
    out = DT((4, 2, 2, 5), np.float32)
    cabi.gather(DT.from_numpy(x, (2, 0, 1)), DT.from_numpy(idx), out, 1)
    assert np.array_equal(out.numpy(), np.take(x, idx, axis=1))


def test_gather_out_of_range_is_reported_not_faulted():
    table = rnd(10, 8)
    ids = np.array([1, 12, -3], np.int64)
    out = DT((3, 8), np.float32)
    cabi.gather(DT.from_numpy(table), DT.from_numpy(ids), out, 0)
    with pytest.raises(cabi.FmlError) as e:
        cabi.check_device()
    assert e.value.status == 7
    got = out.numpy()
    assert np.array_equal(got[0], table[1]) and np.array_equal(got[1], table[9]) and np.array_equal(got[2], table[0])
    cabi.check_device()  # cleared


def test_embedding_fused():
    table, pos, typ = rnd(1000, 768), rnd(1, 128, 768), rnd(768)
    ids = RNG.integers(0, 1000, (2, 128)).astype(np.int64)
    out = DT((2, 128, 768), np.float32)
    cabi.embedding(DT.from_numpy(table), DT.from_numpy(ids), DT.from_numpy(pos), DT.from_numpy(typ), out)
    assert np.array_equal(out.numpy(), (table[ids] + pos) + typ)


def test_slice_concat_pad_through_views():
    x = rnd(2, 4, 16, 64)
    src = DT.from_numpy(x)
    # Slice [.., 16:48] on the last axis
    out = DT((2, 4, 16, 32), np.float32)
    cabi.copy_strided(src.view((2, 4, 16, 32), src.strides, 16), out)
    assert np.array_equal(out.numpy(), x[..., 16:48])
    # Concat(-x2, x1) as in rotary
    cat = DT((2, 4, 16, 64), np.float32)
    cabi.copy_strided(src.view((2, 4, 16, 32), src.strides, 32), cat.view((2, 4, 16, 32), cat.strides, 0))
    cabi.copy_strided(src.view((2, 4, 16, 32), src.strides, 0), cat.view((2, 4, 16, 32), cat.strides, 32))
    assert np.array_equal(cat.numpy(), np.concatenate([x[..., 32:], x[..., :32]], -1))
    p = DT((2, 4, 18, 67), np.float32)
    cabi.pad(src, p, [0, 0, 1, 2])
    ref = orc.pad(x, np.empty((2, 4, 18, 67), np.float32), [0, 0, 1, 2])
    assert np.array_equal(p.numpy(), ref)


# ------------------------------------------------------------------ reductions
@pytest.mark.parametrize("shape,axis", [((1, 12, 128, 128), -1), ((1, 12, 128, 768), 3), ((4, 7, 33), -1),
                                        ((3, 50, 6), 1), ((2, 5000), 1)])
def test_softmax(shape, axis):
    x = rnd(*shape) * 3
    ref = orc.softmax(x, np.empty_like(x), axis)
    out = DT(shape, np.float32)
    cabi.softmax(DT.from_numpy(x), None, 1.0, out, axis)
    got = out.numpy()
    # expf ulp differences and a different summation order: 2e-5 relative
    assert np.allclose(got, ref, rtol=2e-5, atol=1e-9)
    assert np.abs(got.sum(axis) - 1).max() < 1e-5


def test_softmax_fused_scale_mask_matches_chain():
    s = rnd(2, 12, 128, 128) * 4
    m = (RNG.random((2, 1, 1, 128)) > 0.2).astype(np.float32)
    mask = (np.float32(1.0) - m) * np.float32(np.finfo(np.float32).min)
    chain = orc.binary("Add", orc.binary("Div", s, np.asarray(8.0, np.float32), np.empty_like(s)), mask,
                       np.empty_like(s))
    ref = orc.softmax(chain, np.empty_like(s), -1)
    out = DT(s.shape, np.float32)
    cabi.softmax(DT.from_numpy(s), DT.from_numpy(mask), 8.0, out, -1)
    assert np.allclose(out.numpy(), ref, rtol=2e-5, atol=1e-9)


@pytest.mark.parametrize("shape,eps", [((1, 128, 768), 1e-12), ((4, 512, 1024), 1e-5), ((3, 10, 50), 1e-5)])
@pytest.mark.parametrize("residual", [False, True])
def test_layernorm(shape, eps, residual):
    x, r = rnd(*shape) * 2 + 0.5, rnd(*shape)
    g, b = rnd(shape[-1]) + 1, rnd(shape[-1])
    xin = x + r if residual else x
    ref = orc.layernorm(xin, g, b, np.empty_like(x), -1, np.float32(eps), acc64=True)
    out = DT(shape, np.float32)
    cabi.layernorm(DT.from_numpy(x), DT.from_numpy(r) if residual else None, DT.from_numpy(g),
                   DT.from_numpy(b), out, -1, eps)
    # fp32 sums in a different order than the oracle's fp64: 1e-5 of the output scale
    assert relerr(out.numpy(), ref) <= 1e-5


def test_layernorm_strided_axis():
    x = rnd(6, 40, 9)
    g, b = rnd(40) + 1, rnd(40)
    ref = orc.layernorm(x, g, b, np.empty_like(x), 1, np.float32(1e-5), acc64=True)
    out = DT(x.shape, np.float32, (1, 2, 0))
    cabi.layernorm(DT.from_numpy(x, (2, 0, 1)), None, DT.from_numpy(g), DT.from_numpy(b), out, 1, 1e-5)
    assert relerr(out.numpy(), ref) <= 1e-5


def test_reduce_mean_cumsum():
    x = rnd(2, 32, 7, 7)
    out = DT((2, 32, 1, 1), np.float32)
    cabi.reduce_mean(DT.from_numpy(x), out, [2, 3])
    ref = orc.reduce_mean(x, np.empty((2, 32, 1, 1), np.float32), [2, 3])
    assert relerr(out.numpy(), ref) <= 1e-6
    v = RNG.integers(0, 5, (3, 40)).astype(np.int64)
    o = DT(v.shape, np.int64)
    cabi.cumsum(DT.from_numpy(v), o, 1)
    assert np.array_equal(o.numpy(), np.cumsum(v, 1))


# ------------------------------------------------------------------ conv / pool
@pytest.mark.parametrize("cfg", [
    dict(x=(1, 3, 32, 32), w=(16, 3, 3, 3), pads=(1, 1), strides=(1, 1), dil=(1, 1), group=1),
    dict(x=(2, 8, 14, 14), w=(12, 8, 3, 3), pads=(1, 1), strides=(2, 2), dil=(1, 1), group=1),
    dict(x=(1, 16, 9, 9), w=(8, 16, 1, 1), pads=(0, 0), strides=(1, 1), dil=(1, 1), group=1),
    dict(x=(1, 12, 20, 20), w=(12, 1, 5, 5), pads=(2, 2), strides=(2, 2), dil=(1, 1), group=12),
    dict(x=(2, 24, 64), w=(24, 1, 9), pads=(4,), strides=(1,), dil=(1,), group=24),
    dict(x=(1, 4, 12, 12), w=(6, 4, 3, 3), pads=(2, 2), strides=(1, 1), dil=(2, 2), group=1),
    # short reductions (IC * KH * KW <= 64): the direct kernel, strided / dilated / 1-D / ragged channel block
    dict(x=(2, 3, 33, 37), w=(32, 3, 3, 3), pads=(1, 1), strides=(2, 2), dil=(1, 1), group=1),
    dict(x=(1, 2, 16, 16), w=(40, 2, 5, 5), pads=(2, 2), strides=(1, 1), dil=(1, 1), group=1),
    dict(x=(2, 4, 50), w=(5, 4, 7), pads=(3,), strides=(3,), dil=(2,), group=1),
    # pointwise over a small map, one or two images: the weight-streaming product with 33-64 rows
    dict(x=(1, 96, 7, 7), w=(40, 96, 1, 1), pads=(0, 0), strides=(1, 1), dil=(1, 1), group=1),
    dict(x=(2, 640, 8, 8), w=(24, 640, 1, 1), pads=(0, 0), strides=(1, 1), dil=(1, 1), group=1),
])
def test_conv(cfg):
    x, w = rnd(*cfg["x"]), rnd(*cfg["w"]) * 0.2
    b = rnd(cfg["w"][0])
    nd = len(cfg["x"]) - 2
    osp = [(cfg["x"][2 + i] + 2 * cfg["pads"][i] - cfg["dil"][i] * (cfg["w"][2 + i] - 1) - 1) // cfg["strides"][i] + 1
           for i in range(nd)]
    oshape = (cfg["x"][0], cfg["w"][0], *osp)
    ref = orc.conv(x, w, b, np.empty(oshape, np.float32), cfg["pads"], cfg["strides"], cfg["dil"], cfg["group"],
                   acc64=True)
    out = DT(oshape, np.float32)
    cabi.conv(DT.from_numpy(x), DT.from_numpy(w), DT.from_numpy(b), out, cfg["pads"], cfg["strides"], cfg["dil"],
              cfg["group"])
    assert relerr(out.numpy(), ref) <= 1e-5


@pytest.mark.parametrize("shape,k,stride,pad,act", [
    ((2, 32, 112, 112), 3, 1, 1, 0),   # row-tiled plane, float4 stores
    ((2, 24, 112, 112), 3, 2, 1, 5),   # stride 2, SiLU
    ((3, 40, 56, 56), 5, 2, 2, 0),
    ((2, 48, 28, 28), 5, 1, 2, 5),     # one whole plane per CTA
    ((3, 37, 14, 14), 5, 1, 2, 0),     # planes batched four to a CTA, 14-wide rows (scalar stores), ragged plane count
    ((5, 21, 7, 7), 3, 1, 1, 0),       # eighteen planes to a CTA, width 7
    ((2, 19, 7, 7), 5, 1, 2, 5),
    ((1, 8, 33, 45), 3, 2, 1, 0),      # odd sizes: ragged strips and row tiles
    ((1, 6, 61, 130), 7, 1, 3, 0),     # 7x7 window
    ((1, 5, 30, 30), 3, 1, 0, 0),      # no padding
    # the pipelined kernels: several tiles per persistent CTA (both buffers reused, parities wrap)
    ((16, 144, 56, 56), 3, 1, 1, 5),   # tensor-map copies, one plane per tile
    ((8, 40, 112, 112), 3, 2, 1, 5),   # ... two bands per plane, stride 2
    ((64, 48, 28, 28), 5, 1, 2, 0),    # ... five planes per tile, the last tile ragged
    ((64, 672, 14, 14), 5, 1, 2, 5),   # bulk copies of whole planes, sixteen per tile
    ((2, 50, 14, 14), 5, 2, 2, 0),     # ... stride 2, a ragged last tile
    ((4, 33, 7, 7), 3, 1, 1, 0),       # ... width 7
    ((64, 1152, 7, 7), 5, 1, 2, 5),
])
def test_depthwise_conv_tiled(shape, k, stride, pad, act):
    """The tiled depthwise kernel (every window / stride variant, every plane-batching mode) against
    the oracle's convolution, bias and activation included."""
    n, c, h, w_ = shape
    x, w, b = rnd(*shape), rnd(c, 1, k, k) * 0.3, rnd(c)
    oh, ow = (h + 2 * pad - k) // stride + 1, (w_ + 2 * pad - k) // stride + 1
    ref = orc.conv(x, w, b, np.empty((n, c, oh, ow), np.float32), (pad, pad), (stride, stride), (1, 1), c, acc64=True)
    if act == cabi.ACT_SILU:
        ref = ref / (1.0 + np.exp(-ref.astype(np.float64)))
    out = DT((n, c, oh, ow), np.float32)
    cabi.conv(DT.from_numpy(x), DT.from_numpy(w), DT.from_numpy(b), out, (pad, pad), (stride, stride), (1, 1), c, act=act)
    assert relerr(out.numpy(), ref) <= 1e-5


def test_depthwise_conv_1d_window_9():
    """ConvBERT's span convolution: 1-D depthwise, window 9, rows of 128."""
    x, w, b = rnd(8, 96, 128), rnd(96, 1, 9) * 0.3, rnd(96)
    ref = orc.conv(x, w, b, np.empty((8, 96, 128), np.float32), (4,), (1,), (1,), 96, acc64=True)
    out = DT((8, 96, 128), np.float32)
    cabi.conv(DT.from_numpy(x), DT.from_numpy(w), DT.from_numpy(b), out, (4,), (1,), (1,), 96)
    assert relerr(out.numpy(), ref) <= 1e-5


@pytest.mark.parametrize("shape,k,stride,pad,act", [((8, 96, 128), 9, 1, 4, 0), ((2, 37, 50), 3, 2, 1, 5),
                                                    ((2, 16, 9, 11), 3, 1, 1, 0)])
def test_depthwise_conv_channel_innermost(shape, k, stride, pad, act):
    """Depthwise convolution whose operands are transposed views of channel-last buffers (how ConvBERT's
    span convolution reads a [batch, length, channels] activation)."""
    nd = len(shape) - 2
    c = shape[1]
    x, w, b = rnd(*shape), rnd(c, 1, *([k] * nd)) * 0.3, rnd(c)
    osp = [(d + 2 * pad - k) // stride + 1 for d in shape[2:]]
    oshape = (shape[0], c, *osp)
    ref = orc.conv(x, w, b, np.empty(oshape, np.float32), (pad,) * nd, (stride,) * nd, (1,) * nd, c, acc64=True)
    if act == cabi.ACT_SILU:
        ref = ref / (1.0 + np.exp(-ref.astype(np.float64)))
    cl = [0, nd + 1] + list(range(1, nd + 1))  # channel dim physically innermost
    xd, out = DT.from_numpy(x, cl), DT(oshape, np.float32, cl)
    assert xd.strides[1] == 1 and out.strides[1] == 1
    cabi.conv(xd, DT.from_numpy(w), DT.from_numpy(b), out, (pad,) * nd, (stride,) * nd, (1,) * nd, c, act=act)
    assert relerr(out.numpy(), ref) <= 1e-5


def test_pointwise_conv_on_a_small_map_with_baked_weight_layout():
    """1152 -> 192 on a 7 x 7 map, one image, weights stored tap-major with the output channel
    innermost (what the Builder bakes), SiLU: the N-major path of the wide weight-streaming kernel."""
    x, w, b = rnd(1, 1152, 7, 7), rnd(192, 1152, 1, 1) * 0.05, rnd(192)
    ref = orc.conv(x, w, b, np.empty((1, 192, 7, 7), np.float32), (0, 0), (1, 1), (1, 1), 1, acc64=True)
    ref = ref / (1.0 + np.exp(-ref.astype(np.float64)))
    out = DT((1, 192, 7, 7), np.float32)
    cabi.conv(DT.from_numpy(x), DT.from_numpy(w, [3, 2, 0, 1]), DT.from_numpy(b), out, (0, 0), (1, 1), (1, 1), 1,
              act=cabi.ACT_SILU)
    assert relerr(out.numpy(), ref) <= 1e-5


@pytest.mark.parametrize("shape,k,pad,dil", [((8, 96, 128), 9, 4, 1), ((3, 45, 70), 5, 4, 2), ((1, 7, 33), 3, 0, 1)])
def test_depthwise_conv_1d_channel_innermost_input_only(shape, k, pad, dil):
    """The mixed case: the input is a transposed view of a channel-last buffer, the output is in the
    default layout (the tile goes through shared memory)."""
    c = shape[1]
    x, w, b = rnd(*shape), rnd(c, 1, k) * 0.3, rnd(c)
    ol = shape[2] + 2 * pad - dil * (k - 1)
    ref = orc.conv(x, w, b, np.empty((shape[0], c, ol), np.float32), (pad,), (1,), (dil,), c, acc64=True)
    xd, out = DT.from_numpy(x, [0, 2, 1]), DT((shape[0], c, ol), np.float32)
    assert xd.strides[1] == 1 and out.strides[2] == 1
    cabi.conv(xd, DT.from_numpy(w), DT.from_numpy(b), out, (pad,), (1,), (dil,), c)
    assert relerr(out.numpy(), ref) <= 1e-5


@pytest.mark.parametrize("mode,shape,k,s", [(0, (1, 64, 32, 32), (2, 2), (2, 2)), (1, (2, 1280, 7, 7), (7, 7), (1, 1)),
                                            (0, (1, 3, 9, 11), (3, 2), (2, 3)), (1, (2, 8, 16, 20), (2, 2), (2, 2)),
                                            (0, (3, 5, 6, 8), (2, 2), (2, 2))])
def test_pool(mode, shape, k, s):
    x = rnd(*shape)
    oshape = (shape[0], shape[1], (shape[2] - k[0]) // s[0] + 1, (shape[3] - k[1]) // s[1] + 1)
    ref = orc.pool2d(x, np.empty(oshape, np.float32), mode, k, s)
    out = DT(oshape, np.float32)
    cabi.pool2d(DT.from_numpy(x), out, mode, k, s)
    if mode == 0:
        assert np.array_equal(out.numpy(), ref)
    else:
        assert relerr(out.numpy(), ref) <= 1e-6


def test_bad_arguments_are_reported():
    a, b = DT.from_numpy(rnd(4, 5)), DT.from_numpy(rnd(4, 6))
    out = DT((4, 5), np.float32)
    with pytest.raises(cabi.FmlError) as e:
        cabi.elementwise(cabi.ADD, a, b, out)
    assert e.value.status == 1
    with pytest.raises(cabi.FmlError):
        cabi.softmax(a, None, 1.0, out, 5)
    with pytest.raises(cabi.FmlError):
        cabi.copy_strided(a, DT((5, 4), np.float32))
