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


def test_wall_limit_rule():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    stop = bench.stop_for_wall_limit
    assert not stop(3, 10_000.0, 30.0, 830.0)          # never before the minimum number of timed steps
    assert not stop(10, 400.0, 30.0, 0.0)              # no limit
    assert not stop(19, 760.0, 30.5, 830.0)            # the 20th step still fits (ends near 792 s)
    assert stop(18, 800.0, 32.7, 830.0)                # the next one would not
    assert "--wall-limit-s" in subprocess.run([sys.executable, "bench.py", "--help"], capture_output=True, text=True,
                                              timeout=120).stdout
