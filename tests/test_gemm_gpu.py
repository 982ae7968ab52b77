"""GPU parity of the GEMM paths (fp32 FMA, tcgen05 TF32 and 3xTF32) against the oracle's
fp64-accumulated product, through the C ABI.

Tolerances, as max|gpu - ref| / max|ref| over the output:
  fp32 FMA   1e-5   (fp32 accumulation order differs from the oracle's)
  3xTF32     2e-5   (products carry ~2^-21 relative error)
  TF32       2e-3   (products carry ~2^-11 relative error; operands truncated by the MMA)
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT
from oracle import oracle as orc

RNG = np.random.Generator(np.random.PCG64(99))
TOL = {cabi.GEMM_FP32: 1e-5, cabi.GEMM_3XTF32: 2e-5, cabi.GEMM_TF32: 2e-3}


def rnd(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def relerr(got, ref):
    ref = ref.astype(np.float64)
    return float(np.abs(got.astype(np.float64) - ref).max() / max(1e-30, np.abs(ref).max()))


def ref_matmul(a, b):
    sh = (*np.broadcast_shapes(a.shape[:-2], b.shape[:-2]), a.shape[-2], b.shape[-1])
    return orc.matmul(a, b, np.empty(sh, np.float32), acc64=True)


SHAPES = [  # (A shape, B shape)
    ((128, 768), (768, 768)), ((1, 128, 768), (768, 3072)), ((1, 128, 3072), (3072, 768)),
    ((1, 12, 128, 64), (1, 12, 64, 128)), ((1, 12, 128, 128), (1, 12, 128, 64)),
    ((200, 96), (96, 80)), ((2, 3, 130, 40), (40, 48)), ((512, 256), (256, 512)),
]


@pytest.mark.parametrize("prec", [cabi.GEMM_FP32, cabi.GEMM_3XTF32, cabi.GEMM_TF32])
@pytest.mark.parametrize("sa,sb", SHAPES)
@pytest.mark.parametrize("b_kmajor", [False, True])
def test_gemm_precisions(prec, sa, sb, b_kmajor):
    a, b = rnd(*sa), rnd(*sb)
    ref = ref_matmul(a, b)
    rb = len(sb)
    # K-major B: store B with k innermost (the layout a pre-transposed weight has)
    lb = list(range(rb))
    if b_kmajor:
        lb[rb - 2], lb[rb - 1] = rb - 1, rb - 2
    da, db = DT.from_numpy(a), DT.from_numpy(b, lb)
    out = DT(ref.shape, np.float32)
    p = cabi.gemm_params(precision=prec)
    if prec != cabi.GEMM_FP32:
        assert cabi.gemm_uses_tensor_cores(da, db, out, p)
    cabi.gemm(da, db, out, params=p)
    cabi.check_device()
    assert relerr(out.numpy(), ref) <= TOL[prec]


@pytest.mark.parametrize("split_k,tile_n", [(1, 64), (2, 64), (4, 32), (8, 64), (2, 128), (8, 16), (4, 256), (8, 48), (1, 192)])
def test_gemm_split_k_and_tiles(split_k, tile_n):
    a, b = rnd(128, 768), rnd(768, 768)
    ref = ref_matmul(a, b)
    p = cabi.gemm_params(precision=cabi.GEMM_3XTF32, split_k=split_k, tile_n=tile_n)
    for kmajor in (False, True):
        da, db = DT.from_numpy(a), DT.from_numpy(b, [1, 0] if kmajor else None)
        out = DT(ref.shape, np.float32)
        info = cabi.gemm_plan(da, db, out, p)
        assert info.uses_tensor_cores and info.split_k == split_k
        cabi.gemm(da, db, out, params=p)
        first = out.numpy()
        assert relerr(first, ref) <= TOL[cabi.GEMM_3XTF32]
        # the cluster reduction adds the partial tiles in rank order: a second launch agrees bit for bit
        out2 = DT(ref.shape, np.float32)
        cabi.gemm(da, db, out2, params=p)
        cabi.check_device()
        assert np.array_equal(out2.numpy(), first)


def test_gemm_auto_plan_fills_the_machine():
    """The planner's own choice for the benchmark shapes uses split-K clusters of at most 8."""
    for (m, k, n) in ((128, 768, 768), (128, 768, 3072), (128, 3072, 768)):
        a, b, c = DT((m, k), np.float32), DT((k, n), np.float32), DT((m, n), np.float32)
        info = cabi.gemm_plan(a, b, c, cabi.gemm_params(precision=cabi.GEMM_3XTF32))
        ctas = -(-n // info.tile_n) * info.split_k
        assert info.uses_tensor_cores and 1 <= info.split_k <= 8 and 64 <= ctas <= 148, (m, k, n, info.tile_n, info.split_k)


def test_gemm_epilogues():
    x, w, bias, res = rnd(128, 768), rnd(768, 3072) * 0.05, rnd(3072), rnd(128, 3072)
    mm = ref_matmul(x, w).astype(np.float64)
    c0, c1, c2 = np.float32(np.sqrt(2.0)), 1.0, 0.5
    import math
    erf = np.vectorize(math.erf)
    t = mm + bias
    cases = {
        "bias": (dict(), t, bias, None),
        "bias_gelu": (dict(act=cabi.ACT_GELU_ERF), t * (erf(t / c0) + c1) * c2, bias, None),
        "bias_res": (dict(), t + res, bias, res),
        "div_relu": (dict(act=cabi.ACT_RELU, divisor=8.0), np.maximum(mm / 8.0, 0), None, None),
        "tanh": (dict(act=cabi.ACT_TANH), np.tanh(t), bias, None),
    }
    for prec in (cabi.GEMM_FP32, cabi.GEMM_3XTF32):
        for name, (kw, ref, bb, rr) in cases.items():
            out = DT((128, 3072), np.float32)
            cabi.gemm(DT.from_numpy(x), DT.from_numpy(w), out, DT.from_numpy(bb) if bb is not None else None,
                      DT.from_numpy(rr) if rr is not None else None, cabi.gemm_params(precision=prec, **kw))
            assert relerr(out.numpy(), ref) <= 3e-5, (prec, name)


def test_gemm_attention_views_and_strided_output():
    """Q/K/V are head-strided views of [S, 3H]; the context is written straight into [S, H]."""
    S, H, nh, hd = 128, 768, 12, 64
    qkv = rnd(S, 3 * H)
    src = DT.from_numpy(qkv)
    q = src.view((nh, S, hd), [hd, 3 * H, 1], 0)
    k_t = src.view((nh, hd, S), [hd, 1, 3 * H], H)       # K^T: k-major B without a transpose
    v = src.view((nh, S, hd), [hd, 3 * H, 1], 2 * H)     # V: n-major B
    qn = qkv[:, :H].reshape(S, nh, hd).transpose(1, 0, 2)
    kn = qkv[:, H:2 * H].reshape(S, nh, hd).transpose(1, 0, 2)
    vn = qkv[:, 2 * H:].reshape(S, nh, hd).transpose(1, 0, 2)
    scores = DT((nh, S, S), np.float32)
    p = cabi.gemm_params(precision=cabi.GEMM_3XTF32, divisor=8.0)
    assert cabi.gemm_uses_tensor_cores(q, k_t, scores, p)
    cabi.gemm(q, k_t, scores, params=p)
    ref_s = ref_matmul(np.ascontiguousarray(qn), np.ascontiguousarray(kn.transpose(0, 2, 1))) / np.float32(8)
    assert relerr(scores.numpy(), ref_s) <= 2e-5
    ctx = DT((S, H), np.float32)
    ctx_view = ctx.view((nh, S, hd), [hd, H, 1], 0)
    p2 = cabi.gemm_params(precision=cabi.GEMM_3XTF32)
    assert cabi.gemm_uses_tensor_cores(scores, v, ctx_view, p2)
    cabi.gemm(scores, v, ctx_view, params=p2)
    cabi.check_device()
    ref_c = ref_matmul(ref_s, np.ascontiguousarray(vn)).transpose(1, 0, 2).reshape(S, H)
    assert relerr(ctx.numpy(), ref_c) <= 3e-5


def test_gemm_linearity_full_size():
    """Size-independent property at the FFN shape: (A1 + A2) B == A1 B + A2 B."""
    a1, a2, b = rnd(128, 3072), rnd(128, 3072), rnd(3072, 768)
    outs = []
    for a in (a1, a2, a1 + a2):
        o = DT((128, 768), np.float32)
        cabi.gemm(DT.from_numpy(a), DT.from_numpy(b), o, params=cabi.gemm_params(precision=cabi.GEMM_3XTF32))
        outs.append(o.numpy().astype(np.float64))
    cabi.check_device()
    assert np.abs(outs[2] - (outs[0] + outs[1])).max() / np.abs(outs[2]).max() <= 2e-5


def test_gemm_small_and_odd_shapes_fall_back():
    for sa, sb in (((1, 768), (768, 768)), ((3, 5), (5, 7)), ((17, 33), (33, 9))):
        a, b = rnd(*sa), rnd(*sb)
        out = DT((sa[0], sb[1]), np.float32)
        p = cabi.gemm_params()
        assert not cabi.gemm_uses_tensor_cores(DT.from_numpy(a), DT.from_numpy(b), out, p)
        cabi.gemm(DT.from_numpy(a), DT.from_numpy(b), out, params=p)
        assert relerr(out.numpy(), ref_matmul(a, b)) <= 1e-5
    with pytest.raises(cabi.FmlError) as e:  # forcing tensor cores on unaligned operands is refused
        a, b = rnd(17, 33), rnd(33, 9)
        cabi.gemm(DT.from_numpy(a), DT.from_numpy(b), DT((17, 9), np.float32),
                  params=cabi.gemm_params(precision=cabi.GEMM_TF32))
    assert e.value.status == 3


SKINNY = [  # (M, K, N): pooler, VGG classifier heads at batch 1, ragged edges, several rows
    (1, 768, 768), (1, 25088, 4096), (1, 4096, 1000), (4, 1000, 130), (32, 515, 97), (7, 64, 33), (2, 3, 5),
]


@pytest.mark.parametrize("m,k,n", SKINNY)
@pytest.mark.parametrize("b_kmajor", [False, True])
def test_gemm_skinny_rows_stream_the_weights(m, k, n, b_kmajor):
    """Products with at most 32 rows run on the weight-streaming kernel (split-K partials in
    library scratch).  Two launches in a row agree bit for bit: the partials are added in split
    order and the tile counters reset themselves."""
    a, b, bias = rnd(m, k), rnd(k, n), rnd(n)
    ref = ref_matmul(a, b).astype(np.float64) + bias
    da, db = DT.from_numpy(a), DT.from_numpy(b, [1, 0] if b_kmajor else None)
    p = cabi.gemm_params(precision=cabi.GEMM_FP32)
    outs = []
    for _ in range(2):
        out = DT((m, n), np.float32)
        cabi.gemm(da, db, out, DT.from_numpy(bias), None, p)
        outs.append(out.numpy())
    cabi.check_device()
    assert relerr(outs[0], ref) <= 1e-5
    assert np.array_equal(outs[0], outs[1])


def test_gemm_skinny_batched_and_tanh():
    a, b, bias = rnd(3, 2, 300), rnd(3, 300, 70), rnd(70)
    ref = np.tanh(ref_matmul(a, b).astype(np.float64) + bias)
    out = DT((3, 2, 70), np.float32)
    cabi.gemm(DT.from_numpy(a), DT.from_numpy(b), out, DT.from_numpy(bias), None,
              cabi.gemm_params(act=cabi.ACT_TANH))
    cabi.check_device()
    assert relerr(out.numpy(), ref) <= 1e-5


@pytest.mark.parametrize("m,k,n,prec", [(128, 256, 192, cabi.GEMM_3XTF32), (128, 256, 192, cabi.GEMM_FP32),
                                        (4, 300, 130, cabi.GEMM_FP32), (40, 96, 80, cabi.GEMM_FP32)])
@pytest.mark.parametrize("bias_rank", [1, 2])
def test_gemm_alpha_beta_with_bias_of_rank_one_and_two(m, k, n, prec, bias_rank):
    """Gemm with alpha = 0.5, beta = 2 on the tcgen05, skinny and fp32-FMA paths against the
    oracle's Gemm.  The library and the oracle compute the ONNX form alpha * (A B) + beta * C;
    the reference's kernel swaps the two factors (gemm.cpp:166-181), which only agrees for
    alpha = beta = 1, so this is the case where the two definitions part."""
    alpha, beta = 0.5, 2.0
    a, b = rnd(m, k), rnd(k, n)
    bias = rnd(n) if bias_rank == 1 else rnd(m, n)
    ref = orc.gemm(a, b, bias, np.empty((m, n), np.float32), alpha=alpha, beta=beta, acc64=True)
    swapped = alpha * bias.astype(np.float64) + beta * ref_matmul(a, b).astype(np.float64)  # what the reference would give
    assert relerr(swapped, ref) > 1e-2
    da, db, out = DT.from_numpy(a), DT.from_numpy(b), DT((m, n), np.float32)
    p = cabi.gemm_params(precision=prec, alpha=alpha, beta=beta)
    assert cabi.gemm_uses_tensor_cores(da, db, out, p) == (prec == cabi.GEMM_3XTF32)
    cabi.gemm(da, db, out, DT.from_numpy(bias), None, p)
    cabi.check_device()
    assert relerr(out.numpy(), ref) <= TOL[prec]
