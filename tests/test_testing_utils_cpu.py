"""The test-support helpers themselves (arctic_platform_b200/testing_utils.py)."""
import logging
import sys
import unittest
from types import SimpleNamespace

import pytest

from arctic_platform_b200 import testing_utils as tu


def test_env_flags(monkeypatch):
    monkeypatch.delenv("APB_T_FLAG", raising=False)
    assert tu.parse_flag_from_env("APB_T_FLAG") is False and tu.parse_flag_from_env("APB_T_FLAG", True) is True
    for raw, want in (("yes", True), ("TRUE", True), ("1", True), ("off", False), ("No", False)):
        monkeypatch.setenv("APB_T_FLAG", raw)
        assert tu.parse_flag_from_env("APB_T_FLAG") is want
    monkeypatch.setenv("APB_T_FLAG", "maybe")
    with pytest.raises(ValueError):
        tu.parse_flag_from_env("APB_T_FLAG")
    monkeypatch.setenv("APB_T_INT", "12")
    assert tu.parse_int_from_env("APB_T_INT") == 12 and tu.parse_int_from_env("APB_T_MISSING", 3) == 3
    monkeypatch.setenv("APB_T_INT", "x")
    with pytest.raises(ValueError):
        tu.parse_int_from_env("APB_T_INT")
    monkeypatch.setenv("PYTEST_XDIST_WORKER", "gw7")
    monkeypatch.setenv("PYTEST_XDIST_WORKER_COUNT", "8")
    assert tu.get_xdist_worker_id() == 7 and tu.get_xdist_worker_count() == 8


def test_decorators_skip_by_capability():
    class T(unittest.TestCase):
        @tu.require_torch_no_gpus
        def test_cpu_only(self):
            pass

        @tu.require_torch_multi_gpu
        def test_multi(self):
            pass

        @tu.require_torch
        @tu.require_torch_up_to_2_gpus
        @tu.require_torch_non_multi_gpu
        def test_small(self):
            pass

        @tu.require_module("no_such_module_anywhere")
        def test_needs_module(self):
            pass

    res = unittest.TestResult()
    unittest.defaultTestLoader.loadTestsFromTestCase(T).run(res)
    skipped = {t.id().rsplit(".", 1)[-1] for t, _ in res.skipped}
    n = tu.get_gpu_count()
    assert "test_needs_module" in skipped and ("test_multi" in skipped) == (n < 2) and ("test_cpu_only" in skipped) == (n > 0)
    assert not res.failures and not res.errors
    assert tu.is_torch_available() and isinstance(tu.is_deepspeed_available(), bool)


def test_files_paths_and_logger(tmp_path):
    f = tmp_path / "a" / "b.json"
    tu.write_file(f, '{"x": 1, "y": "one one"}')
    assert tu.read_json_file(f) == {"x": 1, "y": "one one"}
    assert tu.replace_str_in_file(f, "one", "two") == 2 and tu.read_json_file(f)["y"] == "two two"
    assert tu.replace_str_in_file(f, "absent", "z") == 0
    assert tu.get_tests_dir().endswith("tests") and tu.get_tests_dir("fake_service.py").endswith("tests/fake_service.py")
    with tu.ExtendSysPath(tmp_path):
        assert sys.path[0] == str(tmp_path)
    assert str(tmp_path) not in sys.path
    log = logging.getLogger("apb.test.capture")
    log.setLevel(logging.INFO)
    with tu.CaptureLogger(log) as cl:
        log.info("hello %s", "there")
    assert cl.out == "hello there\n" and "hello there" in repr(cl)
    log.info("not captured")
    assert cl.out == "hello there\n"


def test_report_files(tmp_path):
    rep = lambda nodeid, dur, text="": SimpleNamespace(nodeid=nodeid, duration=dur, when="call", longreprtext=text, longrepr=("f", 1, "Skipped: no gpu"))
    tr = SimpleNamespace(stats={"passed": [rep("t::a", 0.5), rep("t::b", 2.0)], "failed": [rep("t::c", 0.1, "Traceback\nAssertionError: boom")],
                                "skipped": [rep("t::d", 0.0)]})
    files = tu.pytest_terminal_summary_main(tr, "run1", root=str(tmp_path))
    assert set(files) == {"durations", "failures_line", "failures_long", "passes", "skipped", "stats"}
    assert open(files["durations"]).read().splitlines()[0].endswith("t::b")
    assert open(files["failures_line"]).read() == "t::c: AssertionError: boom\n"
    assert "Traceback" in open(files["failures_long"]).read() and open(files["passes"]).read() == "t::a\nt::b\n"
    assert "Skipped: no gpu" in open(files["skipped"]).read() and "failed: 1" in open(files["stats"]).read()

    class P:
        def __init__(self):
            self.opts = []

        def addoption(self, *a, **kw):
            if a in self.opts:
                raise ValueError("dup")
            self.opts.append(a)

    p = P()
    tu.pytest_addoption_shared(p)
    tu.pytest_addoption_shared(p)                       # a second conftest asking for the same option is fine
    assert p.opts == [("--make-reports",)]


def test_gpu_partitioning_for_xdist_workers(monkeypatch):
    ids = list(range(8))
    assert [tu.gpu_slice_for_worker(w, 4, ids) for w in range(4)] == [["0", "1"], ["2", "3"], ["4", "5"], ["6", "7"]]
    assert [tu.gpu_slice_for_worker(w, 3, ids) for w in range(3)] == [["0", "1"], ["2", "3"], ["4", "5"]]     # equal slices
    assert [tu.gpu_slice_for_worker(w, 4, [0, 1]) for w in range(4)] == [["0"], ["1"], ["0"], ["1"]]            # sharing
    assert tu.gpu_slice_for_worker(0, 1, ids) == [str(i) for i in ids] and tu.gpu_slice_for_worker(2, 4, []) == []
    for k in ("PYTEST_XDIST_WORKER", "PYTEST_XDIST_WORKER_COUNT", "ARL_GPU_PARTITIONED", "CUDA_VISIBLE_DEVICES"):
        monkeypatch.delenv(k, raising=False)
    assert tu.partition_gpus_for_xdist() is None                                   # not under xdist
    monkeypatch.setenv("PYTEST_XDIST_WORKER", "gw1")
    monkeypatch.setenv("PYTEST_XDIST_WORKER_COUNT", "2")
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "4,5,6,7")
    assert tu.visible_gpu_ids() == ["4", "5", "6", "7"]
    assert tu.partition_gpus_for_xdist() == "6,7" and tu.partition_gpus_for_xdist() is None    # once per process
    monkeypatch.delenv("ARL_GPU_PARTITIONED")
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    assert tu.partition_gpus_for_xdist() is None                                   # a CPU-only run stays CPU-only
