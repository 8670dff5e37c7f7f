"""The benchmark's command-line contract that needs no GPU: the reference arm (the oracle's CPU
restatement, timed on the host cores) prints one JSON line with the agreed keys, and the native
arm refuses to run without a CUDA device instead of falling back to the CPU."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def _run(*args: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_the_contract_line():
    done = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "decode_gemv_hbm_gbs" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["steps"] == 1
    assert line["gpu_launches"] == 0 and line["vs_baseline"] is None
    assert line["config"]["workload"]
    baseline = line["cpu_baseline"]
    assert baseline["kind"] == "port" and baseline["cores"] >= 1 and baseline["sample"]
    assert baseline["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a host without a GPU")
def test_native_arm_has_no_cpu_path():
    done = _run("--steps", "1", "--warmup", "1")
    assert done.returncode != 0
    assert not [line for line in done.stdout.splitlines() if line.startswith("{")]


def test_watchdog_ends_a_stalled_multi_gpu_run_with_a_diagnostic_line():
    """The watchdog of multi-GPU runs (a host-side stall must not hold a node without a word): it
    prints which stage the rank was in, rank 0 prints a JSON line with an error, exit code 5; a
    single-GPU run gets no timer."""
    stalled = "import bench, time; w = bench.Watchdog(1, 0, 2); w.stage = 'tp_check'; time.sleep(20)"
    done = subprocess.run([sys.executable, "-c", stalled], cwd=ROOT, capture_output=True, text=True, timeout=60)
    assert done.returncode == 5
    line = json.loads(done.stdout.strip())
    assert line["n_gpus"] == 2 and "tp_check" in line["error"] and "tp_check" in done.stderr
    single = "import bench, time; w = bench.Watchdog(1, 0, 1); time.sleep(2); w.cancel(); print('done')"
    done = subprocess.run([sys.executable, "-c", single], cwd=ROOT, capture_output=True, text=True, timeout=60)
    assert done.returncode == 0 and done.stdout.strip() == "done"

