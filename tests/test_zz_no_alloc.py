"""The skinny GEMM entry point that allocates nothing (`fml_gemm_skinny_noalloc`), through the
C ABI, against `fml_gemm` on the same operands.  Both run the same kernel and add the split-K
partial sums in split order, so the results must agree bit for bit, on a first call (which
does the per-device set-up) and on a second one (which finds the counters reset).

Named to be collected last: the check is that the entry point works after everything else
has used the device, and alone.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi
from fluidml_b200.cabi import DeviceTensor as DT


def _operands(m, k, n, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return (rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32),
            rng.standard_normal(n).astype(np.float32))


@pytest.mark.parametrize("b_kmajor", [False, True])
def test_noalloc_matches_fml_gemm_twice_in_a_row(b_kmajor):
    p = cabi.gemm_params(precision=cabi.GEMM_FP32, act=cabi.ACT_TANH)
    for call, (m, k, n) in enumerate(((1, 4096, 1000), (4, 2048, 520))):  # both split K
        a, b, bias = _operands(m, k, n, 7 + call)
        b *= np.float32(0.02)
        da, db, dbias = DT.from_numpy(a), DT.from_numpy(b, [1, 0] if b_kmajor else None), DT.from_numpy(bias)
        want, got = DT((m, n), np.float32), DT((m, n), np.float32)
        cabi.gemm(da, db, want, dbias, None, p)
        cabi.gemm_skinny_noalloc(da, db, got, dbias, None, p)
        cabi.check_device()
        ref = np.tanh(a.astype(np.float64) @ b.astype(np.float64) + bias)
        assert np.abs(want.numpy() - ref).max() <= 1e-5
        assert np.array_equal(got.numpy(), want.numpy()), (call, m, k, n)


def test_noalloc_refuses_what_does_not_fit():
    a, b, _ = _operands(40, 64, 64, 1)
    with pytest.raises(cabi.FmlError) as e:  # more than 32 rows
        cabi.gemm_skinny_noalloc(DT.from_numpy(a), DT.from_numpy(b), DT((40, 64), np.float32))
    assert e.value.status == 2
    # 32 rows x 9000 columns x 2 splits of partial sums exceed the 960 KiB built in
    a, b, _ = _operands(32, 512, 9000, 2)
    with pytest.raises(cabi.FmlError) as e:
        cabi.gemm_skinny_noalloc(DT.from_numpy(a), DT.from_numpy(b), DT((32, 9000), np.float32))
    assert e.value.status == 6 and "scratch" in str(e.value)
    cabi.check_device()


def test_noalloc_leaves_free_device_memory_unchanged():
    """The property in the name: after the per-device set-up has happened, a call changes the
    device's free memory by nothing (cudaMemGetInfo before and after, operands allocated first)."""
    import ctypes
    a, b, bias = _operands(4, 2048, 520, 11)
    da, db, dbias, out = DT.from_numpy(a), DT.from_numpy(b), DT.from_numpy(bias), DT((4, 520), np.float32)
    cabi.gemm_skinny_noalloc(da, db, out, dbias)  # set-up, if this is the first call of the process
    cabi.sync()

    def free_bytes():
        f, t = ctypes.c_size_t(), ctypes.c_size_t()
        cabi.check(cabi.lib().fml_mem_info(ctypes.byref(f), ctypes.byref(t)))
        return f.value

    before = free_bytes()
    for _ in range(3):
        cabi.gemm_skinny_noalloc(da, db, out, dbias)
    cabi.sync()
    assert free_bytes() == before
