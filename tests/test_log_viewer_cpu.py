"""Log viewer: cache names and files, resume from the saved cursor without re-fetching, follow with back-off,
filters and wrapping, the command-line entry."""
import io
import json
import pytest

from cortex_client.dss_client.tui import format as fmt
from cortex_client.dss_client.tui.__main__ import main as tui_main
from cortex_client.dss_client.tui.log_cache import LogCache, cache_root, cached_pages, safe_source_name, unsafe_source_name
from cortex_client.dss_client.tui.viewer import LogViewer


def test_cache_root_and_source_names(monkeypatch, tmp_path):
    monkeypatch.setenv("NEUTRINO_TUI_CACHE_DIR", str(tmp_path / "x"))
    assert cache_root() == tmp_path / "x"
    monkeypatch.delenv("NEUTRINO_TUI_CACHE_DIR")
    monkeypatch.setenv("XDG_CACHE_HOME", str(tmp_path / "xdg"))
    assert cache_root() == tmp_path / "xdg" / "neutrino-tui"
    for sid in ("worker-0", "a/b:c%d", "ünï", "..", "."):
        name = safe_source_name(sid)
        assert "/" not in name and name not in (".", "..") and unsafe_source_name(name) == sid
    long = "x/" * 300
    n = safe_source_name(long)
    assert len(n) <= 200 and n != safe_source_name(long + "y")


def test_cache_files_cursor_and_rotation(tmp_path):
    c = LogCache("job/1", tmp_path, max_bytes=400)
    assert c.get_cursor("s") is None and c.load_entries("s") == [] and c.cached_sources() == []
    assert c.append_entries("s", [{"message": f"m{i}"} for i in range(3)]) == 3
    c.set_cursor("s", "3")
    c.set_cursor("t:2", "9")
    assert c.get_cursor("s") == "3" and c.cached_sources() == ["s", "t:2"]
    assert [e["message"] for e in c.load_entries("s", limit=2)] == ["m1", "m2"]
    with open(c._jsonl("s"), "a") as f:
        f.write('{"message": "cut off')                          # a crash in the middle of a line
    assert len(c.load_entries("s")) == 3
    c.append_entries("s", [{"message": "y" * 50} for _ in range(20)])       # past max_bytes: newest half stays
    kept = c.load_entries("s")
    assert 0 < len(kept) < 23 and kept[-1]["message"] == "y" * 50 and c.get_cursor("s") == "3"
    c.set_cursor("s", None)
    assert c.get_cursor("s") is None
    c.clear()
    assert not c.dir.exists()


class _Service:
    def __init__(self, n):
        self.logs = [{"ts": f"t{i}", "level": "ERROR" if i % 4 == 0 else "INFO", "message": f"line {i}"} for i in range(n)]
        self.requests = []

    def fetch_execution_logs(self, job_id, cursor=0):
        self.requests.append(cursor)
        return self.logs[cursor:cursor + 4]

    def list_jobs(self, status=None):
        return [{"job_id": "a", "status": "DONE", "created_at": "2026-01-01T00:00:00Z", "name": "old"},
                {"job_id": "b", "status": "RUNNING", "created_at": "2025-01-01T00:00:00Z", "name": "live",
                 "sub_jobs": [{"type": "training", "config": {"model_name": "qwen3-4b", "num_gpus": 8}}]}]


def test_viewer_resumes_from_cache_and_follows(tmp_path):
    svc = _Service(10)
    out = io.StringIO()
    v = LogViewer(svc, out=out, cache_root=tmp_path, width=200, color=False, sleep=lambda s: None)
    assert v.show("j1") == 10
    assert svc.requests == [0, 4, 8, 10]                          # pages of four, then the empty page that ends it
    first = out.getvalue().splitlines()
    assert first[0] == "t0 [ERROR] line 0" and len(first) == 10
    # a second session repaints from disk and asks the service only for what is new
    svc.requests.clear()
    svc.logs += [{"ts": "t10", "level": "INFO", "message": "line 10"}]
    out2 = io.StringIO()
    v2 = LogViewer(svc, out=out2, cache_root=tmp_path, width=200, color=False, sleep=lambda s: None)
    assert v2.show("j1") == 11 and svc.requests == [10, 11]
    assert out2.getvalue().splitlines()[-1] == "t10 [INFO] line 10"
    # filters and tail
    out3 = io.StringIO()
    v3 = LogViewer(svc, out=out3, cache_root=tmp_path, width=200, color=False, sleep=lambda s: None)
    assert v3.show("j1", min_level="error") == 3 and v3.show("j1", query="line 1") == 2 and v3.show("j1", tail=2) == 2
    # follow: empty polls back off, new lines are picked up, max_polls ends the loop
    sleeps = []
    svc2 = _Service(2)
    v4 = LogViewer(svc2, out=io.StringIO(), cache_root=tmp_path / "f", width=200, color=False, sleep=sleeps.append)
    assert v4.show("j2", follow=True, max_polls=5) == 2
    assert sleeps == pytest.approx([1.0, 1.25, 1.5625])           # the fifth poll ends the loop before sleeping
    # colours only when asked; long lines wrap without losing characters
    col = io.StringIO()
    LogViewer(svc, out=col, cache_root=tmp_path, width=200, color=True, sleep=lambda s: None).show("j1", min_level="ERROR")
    assert all(ln.startswith("\x1b[31m") and ln.endswith("\x1b[0m") for ln in col.getvalue().splitlines())
    assert "".join(ln.strip() for ln in fmt.wrap_log_line("abcdefghijklmnopqrstuvwxyz", 10)) == "abcdefghijklmnopqrstuvwxyz"


def test_cached_pages_survives_an_unwritable_cache(tmp_path):
    class Broken(LogCache):
        def append_entries(self, *a, **k):
            raise OSError("disk full")
    pages = list(cached_pages(lambda cur: {"entries": [1, 2] if cur is None else [], "next_cursor": "2", "eof": cur is not None},
                              Broken("j", tmp_path), "s"))
    assert pages == [[1, 2]]


def test_format_helpers_and_cli(tmp_path, monkeypatch):
    assert fmt.format_log_entry({"ts": "T", "level": "warn", "source": "rank3", "message": "m"}) == "T [WARN] (rank3) m"
    assert fmt.format_log_entry("raw text") == "raw text"
    assert fmt.entry_at_level({"level": "DEBUG"}, "INFO") is False and fmt.entry_at_level({"level": "ERROR"}, 30)
    assert fmt.is_active_status("running") and not fmt.is_active_status("DONE")
    assert fmt.job_status_color("FAILED") == "red" and fmt.job_status_color("weird") == "dim"
    jobs = fmt.sort_jobs(_Service(0).list_jobs())
    assert [j["job_id"] for j in jobs] == ["b", "a"]               # the running job first although it is older
    assert "training:qwen3-4b:8g" in fmt.format_job_row(jobs[0]) and fmt.format_created_at(None) == "-"
    assert fmt.job_matches(jobs[0], "QWEN") and not fmt.job_matches(jobs[1], "qwen")
    assert fmt.colorize("x", "red", True) == "\x1b[31mx\x1b[0m" and fmt.colorize("x", "red", False) == "x"
    monkeypatch.setenv("NEUTRINO_TUI_CACHE_DIR", str(tmp_path))
    out = io.StringIO()
    assert tui_main(["--no-color", "jobs", "--filter", "live"], client=_Service(0), out=out) == 0
    assert out.getvalue().count("\n") == 1 and "RUNNING" in out.getvalue()
    out = io.StringIO()
    assert tui_main(["--no-color", "logs", "j9", "--level", "ERROR"], client=_Service(6), out=out) == 0
    assert out.getvalue().splitlines() == ["t0 [ERROR] line 0", "t4 [ERROR] line 4"]
    assert json.loads((tmp_path / "j9" / "cursors.json").read_text()) == {"execution": "6"}
