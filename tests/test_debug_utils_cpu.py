"""Debug helpers that need no GPU: rank / device accessors, rank-filtered printing, the step-loop timers."""
import time

from arctic_platform_b200.utils import debug


def test_accessors_and_rank_printing(monkeypatch, capsys):
    monkeypatch.setenv("RANK", "3")
    assert debug.get_rank() == 3
    monkeypatch.delenv("RANK")
    assert debug.get_rank() == 0 and debug.get_device_id() == 0
    assert isinstance(debug.get_nvml_mem(), dict)
    debug.gc_empty_accelerator_cache()
    debug.print_rank("only rank one", ranks=(1,))
    debug.print_rank0("from", "rank zero")
    debug.print_rank("everybody")
    out = capsys.readouterr().out
    assert "only rank one" not in out and "[0] from rank zero" in out and "[0] everybody" in out


def test_step_loop_timers(capsys):
    t = debug.SynchronizedWallClockTimerSimple()
    for _ in range(3):
        t("fwd").start()
        time.sleep(0.002)
        t("fwd").stop()
    t("bwd").start()
    t("bwd").stop()
    means = t.means(["fwd"], reset=False)
    assert 1.0 < means["fwd"] < 500.0 and t.counts["fwd"] == 3
    line = t.log(["fwd", "bwd", "absent"])
    assert line.startswith("fwd: ") and " | bwd: " in line and "time (ms) | fwd" in capsys.readouterr().out
    assert t.means() == {} and t("fwd").elapsed() == 0.0                      # log() reset what it reported
    d = debug.SynchronizedWallClockTimerSimpleDummy()
    assert d("x").start().stop() == 0.0 and d.log() == "" and d.means() == {} and d("x").elapsed() == 0.0


def test_memory_history_is_inert_without_a_gpu(tmp_path):
    import torch
    with debug.MemoryHistory(True, str(tmp_path), "r0") as mh:
        x = torch.zeros(4)
    if not torch.cuda.is_available():
        assert mh.path is None and not mh.enabled and list(tmp_path.iterdir()) == []
    with debug.MemoryHistory(False, str(tmp_path)) as off:
        pass
    assert off.path is None and x.sum() == 0
