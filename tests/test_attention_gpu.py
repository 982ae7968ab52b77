"""GPU parity of the fused attention core (`fml_attention`) against the oracle's unfused
MatMul -> Div -> Add -> Softmax -> MatMul chain, through the C ABI.

Tolerance: max|gpu - ref| / max|ref| <= 2e-5 (fp32 FMA on both sides; the summation order
differs and the softmax goes through expf).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT
from oracle import oracle as orc

RNG = np.random.Generator(np.random.PCG64(314))
TOL = 2e-5


def rnd(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def oracle_attention(q, kt, v, mask, divisor):
    sh = (*q.shape[:-1], kt.shape[-1])
    s = orc.matmul(q, kt, np.empty(sh, np.float32))
    s = (s / np.float32(divisor)).astype(np.float32)
    if mask is not None:
        s = (s + mask).astype(np.float32)
    p = orc.softmax(np.ascontiguousarray(s), np.empty(sh, np.float32), axis=-1)
    return orc.matmul(p, v, np.empty((*q.shape[:-1], v.shape[-1]), np.float32))


def relerr(got, ref):
    return float(np.abs(got.astype(np.float64) - ref).max() / max(1e-30, np.abs(ref).max()))


@pytest.mark.parametrize("shape", [  # (batch dims, S_q, S_k, D, D_v)
    ((1, 12), 128, 128, 64, 64), ((2, 3), 37, 50, 8, 12), ((4,), 16, 160, 32, 128), ((), 5, 7, 4, 4),
    ((1, 2), 130, 129, 128, 64),
    # more keys than fit in shared memory at once: chunks of 128 keys, running-maximum softmax
    ((2, 4), 512, 512, 64, 64), ((3,), 40, 700, 32, 128), ((1,), 16, 129, 128, 64), ((2,), 100, 1000, 8, 4),
])
@pytest.mark.parametrize("with_mask", [False, True])
def test_attention_contiguous(shape, with_mask):
    lead, sq, sk, d, dv = shape
    q, kt, v = rnd(*lead, sq, d), rnd(*lead, d, sk), rnd(*lead, sk, dv)
    mask = None
    if with_mask:  # additive key mask, broadcast over heads and query rows
        mask = np.where(RNG.random((*([1] * len(lead)), 1, sk)) < 0.2, -10000.0, 0.0).astype(np.float32)
    assert cabi.attention_supported(sq, sk, d, dv)
    out = DT((*lead, sq, dv), np.float32)
    cabi.attention(DT.from_numpy(q), DT.from_numpy(kt), DT.from_numpy(v),
                   DT.from_numpy(mask) if mask is not None else None, float(np.sqrt(d)), out)
    cabi.check_device()
    assert relerr(out.numpy(), oracle_attention(q, kt, v, mask, np.sqrt(d))) <= TOL


def test_attention_on_head_strided_views():
    """Q, K^T, V as views of the merged [S, 3H] projection; the context written head-interleaved
    into [S, H], as the executor calls it for BERT."""
    S, H, nh, hd = 128, 768, 12, 64
    qkv = rnd(S, 3 * H)
    src = DT.from_numpy(qkv)
    q = src.view((1, nh, S, hd), [0, hd, 3 * H, 1], 0)
    k_t = src.view((1, nh, hd, S), [0, hd, 1, 3 * H], H)
    v = src.view((1, nh, S, hd), [0, hd, 3 * H, 1], 2 * H)
    mask = np.where(RNG.random((1, 1, 1, S)) < 0.1, -10000.0, 0.0).astype(np.float32)
    ctx = DT((S, H), np.float32)
    cabi.attention(q, k_t, v, DT.from_numpy(mask), 8.0, ctx.view((1, nh, S, hd), [0, hd, H, 1], 0))
    cabi.check_device()
    qn = qkv[:, :H].reshape(S, nh, hd).transpose(1, 0, 2)[None]
    kn = qkv[:, H:2 * H].reshape(S, nh, hd).transpose(1, 2, 0)[None]
    vn = qkv[:, 2 * H:].reshape(S, nh, hd).transpose(1, 0, 2)[None]
    ref = oracle_attention(*(np.ascontiguousarray(x) for x in (qn, kn, vn)), mask, 8.0)
    assert relerr(ctx.numpy(), ref[0].transpose(1, 0, 2).reshape(S, H)) <= TOL


def test_attention_generic_strides_and_limits():
    # every operand stored with a permuted layout: no unit-stride fast path applies to Q and V
    q, kt, v = rnd(2, 20, 16), rnd(2, 16, 24), rnd(2, 24, 8)
    out = DT((2, 20, 8), np.float32, [2, 0, 1])
    cabi.attention(DT.from_numpy(q, [1, 0, 2]), DT.from_numpy(kt, [2, 1, 0]), DT.from_numpy(v, [1, 0, 2]), None, 4.0, out)
    cabi.check_device()
    assert relerr(out.numpy(), oracle_attention(q, kt, v, None, 4.0)) <= TOL
    assert not cabi.attention_supported(128, 128, 66, 64)      # head size not a multiple of 4
    assert not cabi.attention_supported(128, 128, 256, 64)     # head size above 128
    assert cabi.attention_supported(128, 4096, 64, 64)         # long key sequences stream in chunks
    with pytest.raises(cabi.FmlError) as e:
        cabi.attention(DT.from_numpy(rnd(8, 6)), DT.from_numpy(rnd(6, 8)), DT.from_numpy(rnd(8, 4)), None, 1.0,
                       DT((8, 4), np.float32))
    assert e.value.status == 2


@pytest.mark.parametrize("s", [64, 512])
def test_attention_causal_mask(s):
    """A causal additive mask [1, 1, S, S] (0 on and below the diagonal, the float lowest above):
    per-row mask values, in the kernel that stages K and V whole (S = 64) and in the streaming
    one (S = 512)."""
    q, kt, v = rnd(2, 3, s, 64), rnd(2, 3, 64, s), rnd(2, 3, s, 64)
    mask = np.where(np.tril(np.ones((s, s), bool)), 0.0, np.finfo(np.float32).min).astype(np.float32)[None, None]
    out = DT((2, 3, s, 64), np.float32)
    cabi.attention(DT.from_numpy(q), DT.from_numpy(kt), DT.from_numpy(v), DT.from_numpy(mask), 8.0, out)
    cabi.check_device()
    assert relerr(out.numpy(), oracle_attention(q, kt, v, mask, 8.0)) <= TOL


# ------------------------------------------------------------------ tensor-core kernel
def _as_kt(k):
    """K [.., S_k, D] on the device, handed over as the K^T view [.., D, S_k] (D stride 1)."""
    t = DT.from_numpy(k)
    shape = (*k.shape[:-2], k.shape[-1], k.shape[-2])
    strides = list(t.strides)
    strides[-1], strides[-2] = strides[-2], strides[-1]
    return t.view(shape, strides, 0)


@pytest.mark.parametrize("cfg", [  # batch, heads, S_q, S_k, D, D_v, mask kind
    (4, 8, 512, 512, 64, 64, "causal"), (4, 8, 300, 333, 64, 64, "key"), (6, 8, 256, 384, 32, 64, None),
    (6, 16, 128, 640, 64, 32, "key"), (1, 16, 1024, 130, 64, 64, "causal"),
])  # each at least 96 tiles of 128 query rows and 200 Mflop: what fml_attention sends to this kernel
def test_attention_on_tensor_cores(cfg):
    """The tcgen05 kernel (3xTF32, scores in tensor memory, streaming softmax over blocks of 128
    keys) against the oracle's unfused chain: ragged sizes, key and causal masks, both head sizes."""
    B, H, sq, sk, d, dv, kind = cfg
    q, k, v = rnd(B, H, sq, d), rnd(B, H, sk, d), rnd(B, H, sk, dv)
    mask = None
    if kind == "key":
        mask = np.where(RNG.random((B, 1, 1, sk)) < 0.2, -10000.0, 0.0).astype(np.float32)
    elif kind == "causal":  # what the folded Where leaves: 0 where allowed, the lowest float elsewhere
        mask = np.where(np.tril(np.ones((sq, sk), np.bool_), k=sk - sq), 0.0, np.finfo(np.float32).min)
        mask = mask.astype(np.float32).reshape(1, 1, sq, sk)
    qd, ktd, vd = DT.from_numpy(q), _as_kt(k), DT.from_numpy(v)
    assert cabi.attention_uses_tensor_cores(qd, ktd, vd)
    out = DT((B, H, sq, dv), np.float32)
    cabi.attention(qd, ktd, vd, DT.from_numpy(mask) if mask is not None else None, float(np.sqrt(d)), out)
    cabi.check_device()
    ref = oracle_attention(q, np.ascontiguousarray(np.swapaxes(k, -1, -2)), v, mask, np.sqrt(d))
    assert relerr(out.numpy(), ref) <= TOL


def test_attention_on_tensor_cores_from_merged_projection_views():
    """Batch 8 of BERT-base: Q, K^T, V as views of the merged [B*S, 3H] projection, context written
    head-interleaved into [B*S, H] -- the call the executor makes."""
    B, S, H, nh, hd = 8, 128, 768, 12, 64
    qkv = rnd(B * S, 3 * H)
    src = DT.from_numpy(qkv)
    q = src.view((B, nh, S, hd), [S * 3 * H, hd, 3 * H, 1], 0)
    k_t = src.view((B, nh, hd, S), [S * 3 * H, hd, 1, 3 * H], H)
    v = src.view((B, nh, S, hd), [S * 3 * H, hd, 3 * H, 1], 2 * H)
    assert cabi.attention_uses_tensor_cores(q, k_t, v)
    mask = np.where(RNG.random((B, 1, 1, S)) < 0.1, -10000.0, 0.0).astype(np.float32)
    ctx = DT((B * S, H), np.float32)
    cabi.attention(q, k_t, v, DT.from_numpy(mask), 8.0, ctx.view((B, nh, S, hd), [S * H, hd, H, 1], 0))
    cabi.check_device()
    x = qkv.reshape(B, S, 3, nh, hd)
    qn, kn, vn = (np.ascontiguousarray(x[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
    ref = oracle_attention(qn, np.ascontiguousarray(kn.transpose(0, 1, 3, 2)), vn, mask, 8.0)
    assert relerr(ctx.numpy(), ref.transpose(0, 2, 1, 3).reshape(B * S, H)) <= TOL
