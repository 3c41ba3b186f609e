"""The reference arm of bench.py runs without a GPU (it times the reference's C++ operator on the
host cores): its JSON line must carry the contract's keys, and the ours arm must refuse to run
without a CUDA device instead of falling back."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=600):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, cwd=ROOT, capture_output=True,
                          text=True, timeout=timeout)


def test_reference_arm_line():
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "converse2d_ref.so")):
        pytest.skip("oracle/_ref not built")
    r = _run(["--impl", "reference", "--steps", "1", "--warmup", "1", "--models", "none"])
    assert r.returncode == 0, r.stderr[-800:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "converse2d_fwd_throughput"
    assert line["unit"] == "Mpix/s" and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["steps"] == 1 and line["warmup"] == 1 and line["value"] > 0
    assert "cfg2" in line["config"]["workload"]
    cb = line["cpu_baseline"]
    assert cb["kind"] == "reference" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "Mpix/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without CUDA")
def test_ours_arm_needs_a_gpu():
    r = _run(["--steps", "1", "--warmup", "1"], timeout=300)
    assert r.returncode != 0
    assert "CUDA" in (r.stderr + r.stdout)


def test_both_arms_share_metric_and_config():
    import argparse
    import bench
    a = argparse.Namespace(gpus=1, steps=3, warmup=1)
    ours, ref = bench.base_line(a), bench.base_line(a, "reference")
    assert ref["impl"] == "reference" and "impl" not in ours
    for key in ("metric", "unit", "higher_is_better", "config", "scaling", "dtype", "data"):
        assert ours[key] == ref[key]
    assert set(bench.BENCH_MODELS) <= set(bench.MODEL_CFG)
