"""bench.py contract pieces that need no GPU: the reference arm's line and the argument surface."""
import json
import subprocess
import sys


def test_reference_arm_reports_unavailable_and_exits_zero():
    out = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--gpus", "1", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-1000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_bench_help_lists_the_driver_flags():
    out = subprocess.run([sys.executable, "bench.py", "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--zero-stage"):
        assert flag in out.stdout
