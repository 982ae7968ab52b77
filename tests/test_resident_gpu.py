"""GPU parity of the resident stage program (one persistent kernel for a chain of GEMM /
attention / LayerNorm stages over 128 rows) against the oracle, through the C ABI.

Tolerance: 3xTF32 products carry ~2^-21 relative error, the oracle accumulates in fp64;
per-stage results must agree within 2e-5 of max|ref| and a chain of stages (an encoder layer:
ten products deep) within 1e-4, far inside the 1e-3 bar on final outputs.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT
from oracle import oracle as orc

RNG = np.random.Generator(np.random.PCG64(2024))
GELU = (1.4142135381698608, 1.0, 0.5)


def rnd(*shape, scale=1.0):
    return (RNG.standard_normal(shape) * scale).astype(np.float32)


def relerr(got, ref):
    ref = ref.astype(np.float64)
    return float(np.abs(got.astype(np.float64) - ref).max() / max(1e-30, np.abs(ref).max()))


def ref_gemm(a, w, bias=None, act=None, residual=None, ln=None):
    """act(a @ w + bias) + residual, then LayerNorm, through the oracle (fp64 accumulation)."""
    y = orc.matmul(a, w, np.empty((*a.shape[:-1], w.shape[1]), np.float32), acc64=True).astype(np.float64)
    if bias is not None:
        y = y + bias
    y = y.astype(np.float32)
    if act == "gelu":
        t = np.empty_like(y)
        orc.unary("Erf", (y / np.float32(GELU[0])).astype(np.float32), t)
        y = (y * (t + np.float32(GELU[1])) * np.float32(GELU[2])).astype(np.float32)
    if residual is not None:
        y = (y + residual).astype(np.float32)
    if ln is not None:
        y = orc.layernorm(y, ln[0], ln[1], np.empty_like(y), axis=-1, eps=ln[2], acc64=True)
    return y


def run(stages):
    prog = cabi.ResidentProgram(stages)
    prog.launch()
    cabi.check_device()
    return prog


@pytest.mark.parametrize("K,N,tile_n,split_k", [(768, 768, 0, 0), (768, 2304, 64, 4), (768, 2304, 128, 8),
                                                 (768, 2304, 192, 12), (3072, 768, 64, 12), (256, 512, 32, 2),
                                                 (768, 3072, 128, 6), (64, 48, 16, 1)])
def test_single_gemm_stage_with_bias_and_gelu(K, N, tile_n, split_k):
    a, w, b = rnd(128, K), rnd(K, N, scale=0.05), rnd(N)
    da, dw, db = DT.from_numpy(a), DT.from_numpy(w), DT.from_numpy(b)
    out = DT((128, N), np.float32)
    run([cabi.resident_gemm_stage(da, dw, out, bias=db, act=cabi.ACT_GELU_ERF, out_external=True,
                                  tile_n=tile_n, split_k=split_k)])
    assert relerr(out.numpy(), ref_gemm(a, w, b, "gelu")) <= 2e-5


@pytest.mark.parametrize("w_kmajor", [False, True])
def test_gemm_residual_layernorm_and_weight_layouts(w_kmajor):
    K, N = 768, 768
    a, w, b, r = rnd(1, 128, K), rnd(K, N, scale=0.05), rnd(N), rnd(1, 128, N)
    g, be = rnd(N), rnd(N)
    da, dw = DT.from_numpy(a), DT.from_numpy(w, [1, 0] if w_kmajor else None)
    out = DT((1, 128, N), np.float32)
    run([cabi.resident_gemm_stage(da, dw, out, bias=DT.from_numpy(b), residual=DT.from_numpy(r),
                                  ln_scale=DT.from_numpy(g), ln_bias=DT.from_numpy(be), ln_eps=1e-12,
                                  out_external=True)])
    assert relerr(out.numpy(), ref_gemm(a, w, b, None, r, (g, be, 1e-12))) <= 2e-5


def test_two_gemms_chained_through_the_tiled_order_twice_in_a_row():
    """FFN: GELU(x W1 + b1) W2 + b2 + x, LayerNorm.  The intermediate never leaves the program's tiled
    order; a second launch of the same program must give the same bits (counters are re-armed)."""
    H, F = 768, 3072
    x, w1, b1, w2, b2 = rnd(128, H), rnd(H, F, scale=0.03), rnd(F, scale=0.1), rnd(F, H, scale=0.03), rnd(H, scale=0.1)
    g, be = rnd(H), rnd(H)
    dx = DT.from_numpy(x)
    mid, out = DT((128, F), np.float32), DT((128, H), np.float32)
    prog = run([cabi.resident_gemm_stage(dx, DT.from_numpy(w1), mid, bias=DT.from_numpy(b1), act=cabi.ACT_GELU_ERF),
                cabi.resident_gemm_stage(mid, DT.from_numpy(w2), out, bias=DT.from_numpy(b2), residual=dx,
                                         ln_scale=DT.from_numpy(g), ln_bias=DT.from_numpy(be), ln_eps=1e-12,
                                         out_external=True)])
    first = out.numpy()
    ref = ref_gemm(ref_gemm(x, w1, b1, "gelu"), w2, b2, None, x, (g, be, 1e-12))
    assert relerr(first, ref) <= 5e-5
    prog.launch()
    cabi.check_device()
    assert np.array_equal(first, out.numpy())


def encoder_layer_stages(x_dev, p, bufs, mask_dev, last):
    H, nh = 768, 12
    qkv, ctx, y1, mid, out = bufs
    q = qkv.view((1, nh, 128, 64), [0, 64, 3 * H, 1])
    kt = qkv.view((1, nh, 64, 128), [0, 64, 1, 3 * H], H)
    v = qkv.view((1, nh, 128, 64), [0, 64, 3 * H, 1], 2 * H)
    ctx_heads = ctx.view((1, nh, 128, 64), [0, 64, H, 1])
    return [
        cabi.resident_gemm_stage(x_dev, p["wqkv"], qkv, bias=p["bqkv"]),
        cabi.resident_attention_stage(q, kt, v, ctx_heads, mask=mask_dev, divisor=8.0),
        cabi.resident_gemm_stage(ctx, p["wo"], y1, bias=p["bo"], residual=x_dev, ln_scale=p["g1"], ln_bias=p["be1"],
                                 ln_eps=1e-12),
        cabi.resident_gemm_stage(y1, p["w1"], mid, bias=p["b1"], act=cabi.ACT_GELU_ERF),
        cabi.resident_gemm_stage(mid, p["w2"], out, bias=p["b2"], residual=y1, ln_scale=p["g2"], ln_bias=p["be2"],
                                 ln_eps=1e-12, out_external=last),
    ]


def ref_encoder_layer(x, p, mask):
    H, nh = 768, 12
    qkv = ref_gemm(x, p["wqkv"], p["bqkv"])
    q, k, v = (qkv[:, i * H:(i + 1) * H].reshape(128, nh, 64).transpose(1, 0, 2) for i in range(3))
    s = orc.matmul(np.ascontiguousarray(q), np.ascontiguousarray(k.transpose(0, 2, 1)), np.empty((nh, 128, 128), np.float32), acc64=True)
    s = (s / np.float32(8.0) + mask).astype(np.float32)
    pr = orc.softmax(s, np.empty_like(s), axis=-1)
    c = orc.matmul(pr, np.ascontiguousarray(v), np.empty((nh, 128, 64), np.float32), acc64=True)
    ctx = np.ascontiguousarray(c.transpose(1, 0, 2)).reshape(128, H)
    y1 = ref_gemm(ctx, p["wo"], p["bo"], None, x, (p["g1"], p["be1"], 1e-12))
    mid = ref_gemm(y1, p["w1"], p["b1"], "gelu")
    return ref_gemm(mid, p["w2"], p["b2"], None, y1, (p["g2"], p["be2"], 1e-12))


def layer_params():
    H, F = 768, 3072
    return {"wqkv": rnd(H, 3 * H, scale=0.03), "bqkv": rnd(3 * H, scale=0.1), "wo": rnd(H, H, scale=0.03),
            "bo": rnd(H, scale=0.1), "g1": (1 + rnd(H, scale=0.1)).astype(np.float32), "be1": rnd(H, scale=0.1),
            "w1": rnd(H, F, scale=0.03), "b1": rnd(F, scale=0.1), "w2": rnd(F, H, scale=0.03), "b2": rnd(H, scale=0.1),
            "g2": (1 + rnd(H, scale=0.1)).astype(np.float32), "be2": rnd(H, scale=0.1)}


def test_two_encoder_layers_in_one_launch():
    H, F = 768, 3072
    x = rnd(128, H)
    mask = np.zeros((1, 1, 1, 128), np.float32)
    mask[..., 100:] = -10000.0  # the last 28 keys are padding
    params = [layer_params() for _ in range(2)]
    dx, dmask = DT.from_numpy(x), DT.from_numpy(mask)
    stages, keep, cur = [], [], dx
    for li, p in enumerate(params):
        dp = {k: DT.from_numpy(v) for k, v in p.items()}
        bufs = (DT((128, 3 * H), np.float32), DT((128, H), np.float32), DT((128, H), np.float32),
                DT((128, F), np.float32), DT((128, H), np.float32))
        keep.append((dp, bufs))
        stages += encoder_layer_stages(cur, dp, bufs, dmask, last=li == 1)
        cur = bufs[4]
    prog = run(stages)
    got = cur.numpy()
    ref = x
    for p in params:
        ref = ref_encoder_layer(ref, p, mask[0, 0])
    assert relerr(got, ref) <= 1e-4
    info = prog.info()
    assert info.stages == 10 and info.ctas >= 128
    prog.launch()
    cabi.check_device()
    assert np.array_equal(got, cur.numpy())


def test_unsupported_shapes_are_refused_not_run():
    a, w = DT.from_numpy(rnd(64, 64)), DT.from_numpy(rnd(64, 64))
    with pytest.raises(cabi.FmlError) as e:
        cabi.ResidentProgram([cabi.resident_gemm_stage(a, w, DT((64, 64), np.float32), out_external=True)])
    assert e.value.status == 2  # FML_UNSUPPORTED: the caller launches the operators one by one instead
