"""Parts of the benchmark's command-line contract that need no GPU: the reference arm answers with
one JSON line and exit code 0 when the reference cannot run, for any GPU count it is asked about."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("gpus", [1, 8])
def test_reference_arm_reports_unavailable_in_one_json_line(gpus):
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", str(gpus), "--steps", "2", "--warmup", "3"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-500:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and "\n" not in record["unavailable"]


def test_bench_help_lists_the_driver_flags():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert proc.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--config"):
        assert flag in proc.stdout
