"""The benchmark's output contract, checked where no GPU is needed: the reference arm (the oracle
port on the host cores) prints exactly one line on stdout, that line is JSON, and it carries the
keys the driver reads."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout[:500]
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "bert_base_s128_sequences_per_sec"
    assert line["unit"] == "sequences/s" and line["higher_is_better"] is True and line["n_gpus"] == 1
    assert line["value"] > 0 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "BERT-base" in line["config"]["workload"]
