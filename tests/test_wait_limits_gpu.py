"""The failure path of the bounded waits, exercised without faulting or hanging anything: a test
hook shortens the iteration limit of every mbarrier wait in the tensor-core kernels and makes their
producers issue no loads, so that each wait of a launch runs out.  The kernel must then report the
timeout through the status word (`fml_check_device` -> FML_DEVICE_TIMEOUT), return, and leave the
context usable: the same call with the hook off gives the right result."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT

RNG = np.random.Generator(np.random.PCG64(99))
DEVICE_TIMEOUT = 5


def rnd(*shape):
    return RNG.standard_normal(shape).astype(np.float32)


def expect_timeout_then_recover(launch, verify):
    lib = cabi.lib()
    cabi.check_device()  # start from a clean status word
    try:
        cabi.check(lib.fml_debug_wait_test(2000, 1))
        launch()
        with pytest.raises(cabi.FmlError) as e:
            cabi.check_device()
        assert e.value.status == DEVICE_TIMEOUT
    finally:
        cabi.check(lib.fml_debug_wait_test(0, 0))
    cabi.check_device()  # the status word was cleared by the read
    launch()
    cabi.check_device()
    verify()


def test_gemm_waits_run_out_and_the_context_survives():
    a, b = rnd(128, 768), rnd(768, 768) * 0.05
    da, db, dc = DT.from_numpy(a), DT.from_numpy(b), DT((128, 768), np.float32)
    p = cabi.gemm_params(tile_n=64, split_k=8)  # the clustered split-K path: every rank times out and still meets the barriers
    assert cabi.gemm_uses_tensor_cores(da, db, dc, p)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    expect_timeout_then_recover(lambda: cabi.gemm(da, db, dc, params=p),
                                lambda: np.testing.assert_allclose(dc.numpy(), ref, atol=1e-4 * np.abs(ref).max()))


def test_conv_waits_run_out_and_the_context_survives():
    x, w, b = rnd(1, 64, 14, 14), rnd(128, 64, 3, 3) * 0.05, rnd(128)
    dx, dw, db, dy = DT.from_numpy(x), DT.from_numpy(w, [3, 2, 0, 1]), DT.from_numpy(b), DT((1, 128, 14, 14), np.float32)
    assert cabi.conv_uses_tensor_cores(dx, dw, dy, (1, 1))
    from oracle import oracle as orc
    ref = orc.conv(x, w, b, np.empty((1, 128, 14, 14), np.float32), (1, 1), (1, 1), (1, 1), 1, acc64=True)
    expect_timeout_then_recover(lambda: cabi.conv(dx, dw, db, dy, (1, 1), (1, 1), (1, 1), 1),
                                lambda: np.testing.assert_allclose(dy.numpy(), ref, atol=1e-4 * np.abs(ref).max()))


def test_attention_waits_run_out_and_the_context_survives():
    B, H, S, D = 8, 12, 128, 64
    q, k, v = rnd(B, H, S, D), rnd(B, H, S, D), rnd(B, H, S, D)
    dq, dk, dv, out = DT.from_numpy(q), DT.from_numpy(k), DT.from_numpy(v), DT((B, H, S, D), np.float32)
    st = list(dk.strides)
    st[-1], st[-2] = st[-2], st[-1]
    kt = dk.view((B, H, D, S), st, 0)
    assert cabi.attention_uses_tensor_cores(dq, kt, dv)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / 8.0
    p = np.exp(s - s.max(-1, keepdims=True))
    ref = np.einsum("bhqk,bhkd->bhqd", p / p.sum(-1, keepdims=True), v.astype(np.float64))
    expect_timeout_then_recover(lambda: cabi.attention(dq, kt, dv, None, 8.0, out),
                                lambda: np.testing.assert_allclose(out.numpy(), ref, atol=2e-5 * np.abs(ref).max()))


def test_depthwise_waits_run_out_and_the_context_survives():
    """The pipelined depthwise kernel (one tensor-map copy per tile, two buffers): with the copies
    dropped both buffers' waits run out, every CTA leaves through the uniform outcome, and the next
    launch is correct."""
    x, w, b = rnd(2, 24, 28, 28), rnd(24, 1, 3, 3), rnd(24)
    dx, dw, db, dy = DT.from_numpy(x), DT.from_numpy(w), DT.from_numpy(b), DT((2, 24, 28, 28), np.float32)
    from oracle import oracle as orc
    ref = orc.conv(x, w, b, np.empty((2, 24, 28, 28), np.float32), (1, 1, 1, 1), (1, 1), (1, 1), 24)
    expect_timeout_then_recover(lambda: cabi.conv(dx, dw, db, dy, (1, 1), (1, 1), (1, 1), 24),
                                lambda: np.testing.assert_allclose(dy.numpy(), ref, atol=1e-5 * np.abs(ref).max()))
