"""Dry run of the benchmark harness on CPU with a toy-sized model: every arm prints one JSON line with the
keys the contract names (the real numbers come from the GPU runs)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
        "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "impl", "first_loss", "final_loss"}


def _run(*extra):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--tiny", "--steps", "2", "--warmup", "2",
                          *extra], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout
    return json.loads(lines[0])


@pytest.mark.parametrize("impl", ["ours", "baseline"])
def test_bench_line_has_contract_keys(impl):
    d = _run("--impl", impl)
    assert KEYS <= set(d), KEYS - set(d)
    assert d["impl"] == impl and d["value"] > 0 and d["e2e"]["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] == 2 * 32 * 8 and d["e2e"]["d2h_bytes_per_step"] == 4
    assert d["first_loss"] == d["first_loss"] and d["final_loss"] < 7.0   # ln(512) = 6.24


def test_reference_arm_runs_or_says_unavailable():
    d = _run("--impl", "reference")
    assert d["impl"] == "reference"
    if "unavailable" not in d:
        assert KEYS <= set(d) and d["final_loss"] < 7.0
