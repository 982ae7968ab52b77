"""Full-size parity of the benchmark configurations other than BERT-base batch 1 against the CPU
oracle, through the Executor (the drop-in boundary).

Every configuration runs on the GPU at the size BASELINE.json names.  The oracle interprets the
same graph; where a whole batch would take it tens of minutes (VGG-16 batch 32, EfficientNet-B0
batch 64, GPT-NeoX batch 4) it runs the batch-1 model of the same seed -- the same weights -- on
single entries of the batch: no operator of these models mixes batch entries, so entry i of the
batched output must equal the batch-1 output on input i.  Tolerance 1e-3 on the final fp32
outputs, as max|gpu - ref| / max|ref| and element-wise with a floor (relerr).
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from fluidml_b200 import models
from fluidml_b200.executor import Executor
from oracle import oracle as orc

TOL = 1e-3
THREADS = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def relerr(got, ref):
    ref = ref.astype(np.float64)
    err = np.abs(got.astype(np.float64) - ref)
    scale = max(1e-30, float(np.abs(ref).max()))
    return float(max(err.max() / scale, (err / np.maximum(np.abs(ref), 5e-2 * scale)).max()))


def run_gpu(model, inputs):
    ex = Executor.make_dp_greedy(model.name).compile(model.to_bytes())
    outs = {o.name: np.zeros(o.shape, np.float32) for o in model.outputs}
    assert ex.invoke({**inputs, **outs}) > 0
    return outs


def check_entries(batched_out, single_model, batched_inputs, entries, out_name):
    """Entries of the batched GPU output against the oracle's batch-1 result on the same input rows."""
    orc.set_threads(THREADS)
    for i in entries:
        one = {k: np.ascontiguousarray(v[i:i + 1]) for k, v in batched_inputs.items()}
        ref = orc.run_model(single_model, one, acc64=True)[out_name]
        assert float(np.abs(ref).max()) > 0
        assert relerr(batched_out[out_name][i:i + 1], ref) <= TOL, (out_name, i)


def test_vgg16_batch_1_and_32_full_size():
    single = models.build_vgg16(batch=1)
    x1 = models.vgg_inputs(batch=1)
    orc.set_threads(THREADS)
    ref = orc.run_model(single, x1, acc64=True)["output"]
    assert relerr(run_gpu(single, x1)["output"], ref) <= TOL
    x32 = models.vgg_inputs(batch=32)
    out32 = run_gpu(models.build_vgg16(batch=32), x32)
    assert np.isfinite(out32["output"]).all()
    check_entries(out32, single, x32, (0, 31), "output")


def test_efficientnet_b0_batch_64_full_size():
    # weights wide enough (std 0.16) for the logits to carry signal rather than bias alone
    single = models.build_efficientnet_b0(batch=1, std=0.16)
    x64 = models.efficientnet_inputs(batch=64)
    out64 = run_gpu(models.build_efficientnet_b0(batch=64, std=0.16), x64)
    assert np.isfinite(out64["logits"]).all()
    check_entries(out64, single, x64, (0, 21, 63), "logits")


def test_convbert_base_batch_8_seq_128_full_size():
    m = models.build_convbert(batch=8, seq=128)
    x = models.convbert_inputs(batch=8, seq=128)
    orc.set_threads(THREADS)
    ref = orc.run_model(m, x, acc64=True)
    out = run_gpu(m, x)
    for k in ref:
        assert relerr(out[k], ref[k]) <= TOL, k


def test_gpt_neox_prefill_batch_4_seq_512_full_size():
    single = models.build_gpt_neox(batch=1, seq=512)
    x4 = models.gpt_neox_inputs(batch=4, seq=512)
    out4 = run_gpu(models.build_gpt_neox(batch=4, seq=512), x4)
    assert np.isfinite(out4["last_hidden_state"]).all()
    check_entries(out4, single, x4, (0, 3), "last_hidden_state")
