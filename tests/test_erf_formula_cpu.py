"""The erf approximation of the tensor-core GEMM's GELU epilogue (Abramowitz & Stegun 7.1.26,
`erf_fast` in csrc/kernels/gemm_tc.cu), restated in float32 numpy with the same constants and the
same operation order: its error against the exact function is what the kernel's comment states (about 6e-7), and the GELU built on it stays two orders below the GEMM's own tolerance."""
import numpy as np
from scipy.special import erf

F = np.float32


def erf_fast(x):
    x = x.astype(F)
    ax = np.abs(x)
    t = F(1.0) / (F(0.3275911) * ax + F(1.0))
    p = F(1.061405429) * t + F(-1.453152027)
    p = p * t + F(1.421413741)
    p = p * t + F(-0.284496736)
    p = p * t + F(0.254829592)
    r = F(1.0) - (p * t) * np.exp(-(ax * ax)).astype(F)
    return np.copysign(r, x).astype(F)


def test_formula_error_is_below_the_stated_bound():
    x = np.linspace(-6.0, 6.0, 2_000_001).astype(F)
    err = np.abs(erf_fast(x).astype(np.float64) - erf(x.astype(np.float64)))
    assert float(err.max()) < 7e-7          # the kernel adds the fast exponential's rounding: below 1e-6 stated
    assert erf_fast(np.array([0.0], F))[0] == 0.0 or abs(float(erf_fast(np.array([0.0], F))[0])) < 1e-7


def test_gelu_built_on_it_is_far_inside_the_gemm_tolerance():
    v = np.linspace(-12.0, 12.0, 1_000_001).astype(F)
    ours = v * (erf_fast(v * F(1.0 / 1.4142135381698608)) + F(1.0)) * F(0.5)
    exact = v.astype(np.float64) * (erf(v.astype(np.float64) / np.sqrt(2.0)) + 1.0) * 0.5
    # 3xTF32 products are held to 2e-5 of max|C|; the activation's error relative to the largest value
    assert float(np.abs(ours - exact).max() / np.abs(exact).max()) < 5e-7
