"""End-to-end parity of the Executor (the drop-in boundary) against the CPU oracle.

Final fp32 outputs must agree within 1e-3 (the tolerance the hot-path specification states),
both as max|gpu - ref| / max|ref| and element by element with an absolute floor (see relerr);
the indexing operators underneath are covered bit-exactly in test_kernels_gpu.py.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import models
from fluidml_b200.executor import Executor
from oracle import oracle as orc

TOL = 1e-3


def relerr(got, ref):
    """The larger of two measures, both of which must stay within the tolerance:
    the largest absolute error over the largest reference magnitude, and the largest
    element-wise relative error |gpu - ref| / max(|ref|, floor) with floor = 5e-2 max|ref|
    (an element-wise check that small-magnitude outputs cannot hide behind, while elements that
    are numerically zero next to the tensor's scale are measured against the floor)."""
    ref = ref.astype(np.float64)
    err = np.abs(got.astype(np.float64) - ref)
    scale = max(1e-30, float(np.abs(ref).max()))
    return float(max(err.max() / scale, (err / np.maximum(np.abs(ref), 5e-2 * scale)).max()))


def run(model, inputs, factory, **options):
    ex = factory(model.name)
    for k, v in options.items():
        ex.set_option(k, v)
    ex.compile(model.to_bytes())
    outs = {o.name: np.zeros(o.shape, np.float32) for o in model.outputs}
    ns = ex.invoke({**inputs, **outs})
    assert ns > 0
    return outs, ex


@pytest.fixture(scope="module")
def bert2():
    m = models.build_bert(layers=2)
    x = models.bert_inputs()
    return m, x, orc.run_model(m, x, acc64=True)


@pytest.mark.parametrize("factory", [Executor.make_plain_linear, Executor.make_plain_greedy, Executor.make_dp_greedy])
@pytest.mark.parametrize("fusion", [0, 1])
def test_bert_two_layers_all_modes(bert2, factory, fusion):
    m, x, ref = bert2
    outs, ex = run(m, x, factory, fusion=fusion)
    for k in ref:
        assert relerr(outs[k], ref[k]) <= TOL, k
    st = ex.stats()
    if fusion:
        assert st["flow_nodes"] < st["graph_nodes"]


def test_fused_mul_add_chain_equals_the_unfused_plan_bit_for_bit():
    """FusedMulAdd / FusedMulAddChain round like the Mul and Add kernels they replace: both plans
    agree exactly."""
    from test_host_cpu import _mul_add_chain
    m = _mul_add_chain()
    rng = np.random.Generator(np.random.PCG64(5))
    x = {vi.name: rng.standard_normal(vi.shape).astype(np.float32) for vi in m.inputs}
    a, _ = run(m, x, Executor.make_dp_greedy, fusion=0)
    b, ex = run(m, x, Executor.make_dp_greedy, fusion=1)
    assert np.array_equal(a["y"], b["y"])
    ref = orc.run_model(m, x)["y"]
    assert np.array_equal(b["y"], ref)
    assert ex.stats()["launches"] == 5  # one sum of three products, the shared product, the Relu, two Adds


# single-pass TF32 is an option, not the default: it misses the 1e-3 bar (element-wise up to ~2e-2)
@pytest.mark.parametrize("precision,tol", [("fp32", 1e-4), ("3xtf32", 1e-4), ("tf32", 4e-2)])
def test_bert_gemm_precisions(bert2, precision, tol):
    m, x, ref = bert2
    outs, _ = run(m, x, Executor.make_dp_greedy, gemm_precision=precision)
    for k in ref:
        assert relerr(outs[k], ref[k]) <= tol, (precision, k)


def test_bert_masked_batch():
    """Padding mask with zeros and batch 2: the mask path actually changes the result."""
    m = models.build_bert(layers=1, batch=2, seq=64, vocab=2000)
    x = models.bert_inputs(batch=2, seq=64, vocab=2000)
    x["attention_mask"][0, 40:] = 0.0
    x["attention_mask"][1, 10:] = 0.0
    ref = orc.run_model(m, x, acc64=True)
    for factory in (Executor.make_plain_greedy, Executor.make_dp_greedy):
        outs, _ = run(m, x, factory)
        for k in ref:
            assert relerr(outs[k], ref[k]) <= TOL, k


def test_bert_base_full_size():
    """The benchmark configuration: 12 layers, hidden 768, seq 128, batch 1."""
    m = models.build_bert()
    x = models.bert_inputs()
    ref = orc.run_model(m, x, acc64=True)
    outs, ex = run(m, x, Executor.make_dp_greedy)
    for k in ref:
        assert relerr(outs[k], ref[k]) <= TOL, k
    # run-to-run bit stability (split-K partials are reduced in a fixed order)
    outs2 = {o.name: np.zeros(o.shape, np.float32) for o in m.outputs}
    ex.invoke({**x, **outs2})
    for k in ref:
        assert np.array_equal(outs[k], outs2[k])
    # idempotence under epochs: replaying the graph several times leaves the same outputs
    ex3 = Executor.make_dp_greedy("bert", 5).compile(m.to_bytes())
    outs3 = {o.name: np.zeros(o.shape, np.float32) for o in m.outputs}
    ex3.invoke({**x, **outs3})
    for k in ref:
        assert np.array_equal(outs[k], outs3[k])


def test_bert_base_as_one_resident_program():
    """Option resident=1: the twelve encoder layers run as one persistent kernel (a resident stage
    program) behind the same Executor calls.  Same tolerance, same bits on every pass, and the pass
    is a handful of launches."""
    m = models.build_bert()
    x = models.bert_inputs()
    ref = orc.run_model(m, x, acc64=True)
    outs, ex = run(m, x, Executor.make_dp_greedy, resident=1)
    for k in ref:
        assert relerr(outs[k], ref[k]) <= TOL, k
    st = ex.stats()
    assert st["resident_programs"] == 1 and st["resident_stages"] == 60 and st["launches"] <= 14
    assert st["kernels"].get("ResidentProgramKernel") == 1
    for _ in range(3):
        again = {o.name: np.zeros(o.shape, np.float32) for o in m.outputs}
        ex.invoke({**x, **again})
        for k in ref:
            assert np.array_equal(outs[k], again[k])
    ex5 = Executor.make_dp_greedy("bert", 5)
    ex5.set_option("resident", 1)
    ex5.compile(m.to_bytes())
    outs5 = {o.name: np.zeros(o.shape, np.float32) for o in m.outputs}
    ex5.invoke({**x, **outs5})
    for k in ref:
        assert np.array_equal(outs[k], outs5[k])


def test_invoke_argument_errors(bert2):
    m, x, _ = bert2
    ex = Executor.make_plain_greedy("bert").compile(m.to_bytes())
    with pytest.raises(KeyError):  # std::out_of_range in the reference (runner.cpp:70)
        ex.invoke(dict(x))
    with pytest.raises(RuntimeError):
        Executor.make_plain_greedy("x").invoke({})
    with pytest.raises(RuntimeError):
        Executor.make_plain_greedy("x").compile(b"not an onnx file")


def test_out_of_range_token_id_is_reported(bert2):
    m, x, _ = bert2
    ex = Executor.make_plain_greedy("bert").compile(m.to_bytes())
    bad = {k: v.copy() for k, v in x.items()}
    bad["input_ids"][0, 3] = 10 ** 6
    outs = {o.name: np.zeros(o.shape, np.float32) for o in m.outputs}
    with pytest.raises(RuntimeError, match="gather index"):
        ex.invoke({**bad, **outs})
    ex.invoke({**x, **outs})  # the executor stays usable


def test_vgg_small_and_gpt_neox_small():
    v = models.build_vgg16(image=32, fc=128, classes=10)
    xv = models.vgg_inputs(image=32)
    ref = orc.run_model(v, xv, acc64=True)
    for factory in (Executor.make_plain_greedy, Executor.make_dp_greedy):
        outs, _ = run(v, xv, factory)
        assert relerr(outs["output"], ref["output"]) <= TOL
    g = models.build_gpt_neox(layers=2, hidden=256, heads=4, ffn=1024, vocab=1000, batch=2, seq=64)
    xg = models.gpt_neox_inputs(batch=2, seq=64, vocab=1000)
    ref = orc.run_model(g, xg, acc64=True)
    for factory in (Executor.make_plain_greedy, Executor.make_dp_greedy):
        outs, _ = run(g, xg, factory)
        assert relerr(outs["last_hidden_state"], ref["last_hidden_state"]) <= TOL


def test_plan_cache_and_cli_run(tmp_path):
    """A second Compile of the same bytes with the same options takes layouts and GEMM tiles from
    the plan cache and produces the same outputs; the CLI compiles and runs a model."""
    import subprocess
    import fluidml_b200.build as b
    m = models.build_bert(layers=2, vocab=500)
    x = models.bert_inputs(vocab=500)
    outs, states = [], []
    for _ in range(2):
        ex = Executor.make_dp_greedy("bert", 1)
        ex.set_option("plan_cache", str(tmp_path))
        ex.compile(m.to_bytes())
        states.append(ex.stats()["plan_cache"])
        host = {vi.name: np.zeros(vi.shape, {1: np.float32, 7: np.int64}[vi.dtype]) for vi in (*m.inputs, *m.outputs)}
        for k, v in x.items():
            host[k][...] = v
        ex.invoke(host)
        outs.append({k: host[k].copy() for k in ("last_hidden_state", "pooler_output")})
    assert states == ["miss", "hit"]
    assert len(list(tmp_path.glob("*.plan"))) == 1
    for k in outs[0]:
        assert np.array_equal(outs[0][k], outs[1][k])
    path = tmp_path / "m.onnx"
    path.write_bytes(m.to_bytes())
    exe = os.path.join(os.path.dirname(b.HOST_SO), "..", "bin", "fluidml-compiler")
    r = subprocess.run([exe, "-n", "bert", "-i", str(path), "-m", "dp_greedy", "-e", "3", "--run",
                        "--mlir", str(tmp_path / "launches.txt")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "ns per pass" in r.stdout
    assert "FusedGemmKernel" in (tmp_path / "launches.txt").read_text()


def test_efficientnet_b0_and_full_size_vgg():
    """EfficientNet-B0 (strided and depthwise convolutions, SiLU, squeeze-and-excite: operators
    the reference cannot run) against the oracle on a narrow low-resolution copy whose weights
    are wide enough for the logits not to be all bias; then the full-size models run and repeat
    bit for bit (the oracle needs minutes for those)."""
    e = models.build_efficientnet_b0(image=64, width=0.5, std=0.25, classes=100)
    xe = models.efficientnet_inputs(image=64)
    ref = orc.run_model(e, xe, acc64=True)
    assert float(np.abs(ref["logits"]).max()) > 0.2
    for factory in (Executor.make_plain_greedy, Executor.make_dp_greedy):
        outs, ex = run(e, xe, factory)
        assert relerr(outs["logits"], ref["logits"]) <= TOL
        assert "SiluKernel" not in ex.stats()["kernels"]  # every SiLU rides in a convolution epilogue
        # each block's ReduceMean -> Conv -> Conv gate is one launch
        assert ex.stats()["kernels"].get("SqueezeExciteGateKernel") == 16 and "ReduceMeanKernel" not in ex.stats()["kernels"]
        assert "MulCommonKernel" not in ex.stats()["kernels"]  # ... and the gate is applied inside the projection convolution
    # the same model with every fusion off (separate ReduceMean and gate convolutions) agrees too
    outs, ex = run(e, xe, Executor.make_dp_greedy, fusion=0)
    assert relerr(outs["logits"], ref["logits"]) <= TOL and ex.stats()["kernels"].get("ReduceMeanKernel") == 16
    # full-size EfficientNet-B0 (224 x 224: every map size from 112 down to 7 and 1) against the
    # oracle, again with weights wide enough for the logits to carry signal
    full = models.build_efficientnet_b0(std=0.16)
    xf = models.efficientnet_inputs()
    ref = orc.run_model(full, xf, acc64=True)
    outs, _ = run(full, xf, Executor.make_dp_greedy)
    assert float(np.abs(ref["logits"]).max()) > 0.2 and relerr(outs["logits"], ref["logits"]) <= TOL
    for model, x, out in ((models.build_efficientnet_b0(), models.efficientnet_inputs(), "logits"),
                          (models.build_vgg16(), models.vgg_inputs(), "output")):
        a, _ = run(model, x, Executor.make_dp_greedy)
        b, _ = run(model, x, Executor.make_dp_greedy)
        assert np.isfinite(a[out]).all() and np.array_equal(a[out], b[out])


def test_convbert_small():
    """ConvBERT: the span-based dynamic convolution branch (1-D depthwise + pointwise Conv over
    the transposed hidden states, Softmax over the 9 kernel taps, Pad + sliding Slices) beside
    the attention heads, Concat of the two; the Slices must stay views."""
    m = models.build_convbert(layers=2, hidden=256, heads=8, ffn=512, vocab=400, batch=3, seq=48)
    x = models.convbert_inputs(batch=3, seq=48, vocab=400)
    ref = orc.run_model(m, x, acc64=True)
    for factory in (Executor.make_plain_greedy, Executor.make_dp_greedy):
        outs, ex = run(m, x, factory)
        assert relerr(outs["last_hidden_state"], ref["last_hidden_state"]) <= TOL
        assert "SliceKernel" not in ex.stats()["kernels"]
