"""The layout search plans with a cost model where the reference measures kernels
(src/evaluation/eval.cpp:64-100, :261-302).  These tests hold the model to the device: for a
GEMM 128x3072x768 and a LayerNormalization 128x768, each with its activation in the default and
in the transposed layout, the model must rank the variants in the order the kernels measure, and
the per-kernel comparison a Compile leaves in the stats must cover every kernel of the pass."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import cabi, executor, models
from fluidml_b200.cabi import DeviceTensor as DT

IDENT, TRANS = [0, 1], [1, 0]


def device_us(fn, reps=20, rounds=7):
    """Device time per launch of `fn(stream)`: `reps` launches captured in one CUDA graph (the way
    kernels run in a compiled model, and free of the interpreter's launch cost), median over
    `rounds` replays."""
    lib = cabi.lib()
    s, g, e0, e1 = (ctypes.c_void_p() for _ in range(4))
    cabi.check(lib.fml_stream_create(ctypes.byref(s)))
    for _ in range(3):
        fn(s)
    cabi.check(lib.fml_stream_sync(s))
    cabi.check(lib.fml_graph_begin_capture(s))
    for _ in range(reps):
        fn(s)
    cabi.check(lib.fml_graph_end_capture(s, ctypes.byref(g)))
    lib.fml_event_create(ctypes.byref(e0))
    lib.fml_event_create(ctypes.byref(e1))
    cabi.check(lib.fml_graph_launch(g, s))
    cabi.check(lib.fml_stream_sync(s))
    out = []
    for _ in range(rounds):
        lib.fml_event_record(e0, s)
        cabi.check(lib.fml_graph_launch(g, s))
        lib.fml_event_record(e1, s)
        cabi.check(lib.fml_stream_sync(s))
        ms = ctypes.c_float()
        lib.fml_event_elapsed_ms(e0, e1, ctypes.byref(ms))
        out.append(ms.value * 1e3 / reps)
    cabi.check_device()
    lib.fml_graph_destroy(g)
    lib.fml_event_destroy(e0)
    lib.fml_event_destroy(e1)
    lib.fml_stream_destroy(s)
    return float(np.median(out))


WITHIN = 2.0  # modelled and measured time agree within this factor


def test_model_ranks_gemm_layouts_as_measured():
    rng = np.random.default_rng(0)
    m, k, n = 128, 3072, 768
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = DT.from_numpy((rng.standard_normal((k, n)) * 0.03).astype(np.float32))
    c = DT((m, n), np.float32)
    ref = a.astype(np.float64) @ b.numpy().astype(np.float64)
    measured, modelled = {}, {}
    for name, layout in (("identity", IDENT), ("transposed", TRANS)):
        at = DT.from_numpy(a, layout)
        cabi.gemm(at, b, c)
        assert np.abs(c.numpy() - ref).max() <= 1e-3 * np.abs(ref).max()
        measured[name] = device_us(lambda st: cabi.gemm(at, b, c, stream=st))
        modelled[name] = executor.model_gemm_cost_ns(m, k, n, layout, IDENT) * 1e-3
    print("gemm 128x3072x768 us  measured", measured, " modelled", modelled)
    assert (measured["transposed"] > measured["identity"]) == (modelled["transposed"] > modelled["identity"])
    for name in measured:
        assert modelled[name] / WITHIN <= measured[name] <= modelled[name] * WITHIN, (name, measured, modelled)


def test_model_ranks_layernorm_layouts_as_measured():
    rng = np.random.default_rng(1)
    rows, cols = 128, 768
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    g = DT.from_numpy(np.ones(cols, np.float32))
    be = DT.from_numpy(np.zeros(cols, np.float32))
    mu = x.mean(-1, keepdims=True)
    ref = (x - mu) / np.sqrt(x.var(-1, keepdims=True) + 1e-5)
    measured, modelled = {}, {}
    for name, layout in (("identity", IDENT), ("transposed", TRANS)):
        xt, out = DT.from_numpy(x, layout), DT((rows, cols), np.float32, layout)
        cabi.layernorm(xt, None, g, be, out, 1, 1e-5)
        assert np.abs(out.numpy() - ref).max() <= 1e-4
        measured[name] = device_us(lambda st: cabi.layernorm(xt, None, g, be, out, 1, 1e-5, stream=st))
        modelled[name] = executor.model_layernorm_cost_ns(rows, cols, layout, layout) * 1e-3
    print("layernorm 128x768 us  measured", measured, " modelled", modelled)
    assert (measured["transposed"] > measured["identity"]) == (modelled["transposed"] > modelled["identity"])
    for name in measured:
        assert modelled[name] / WITHIN <= measured[name] <= modelled[name] * WITHIN, (name, measured, modelled)


def test_compile_reports_measured_beside_modelled_cost():
    model = models.build_bert(layers=2)
    ex = executor.Executor.make_dp_greedy("bert2").compile(model.to_bytes())
    report = ex.stats()["cost_model"]
    assert isinstance(report, dict), report
    launches = 0
    for kernel, entry in report.items():
        assert entry["measured_us"] > 0 and entry["launches"] >= 1, kernel
        assert entry["modelled_us"] > 0, kernel
        launches += entry["launches"]
    assert launches == ex.stats()["launches"]
    assert any("Gemm" in k for k in report)
    for k, e in report.items():  # every kernel class of the pass is modelled within the factor
        assert e["modelled_us"] / WITHIN <= e["measured_us"] <= e["modelled_us"] * WITHIN, (k, report)
    print("cost_model", report)
