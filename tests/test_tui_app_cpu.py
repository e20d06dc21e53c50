"""The full-screen viewer's loop driven by a scripted terminal against the in-memory service."""
from pathlib import Path

import pytest

from cortex_client.dss_client import NeutrinoClient, SubJobConfig
from cortex_client.dss_client.tui.app import App, JobsModel, LogModel, draw_jobs, draw_log
from tests.fake_service import FakeServiceSession


class ScriptedTerminal:
    def __init__(self, keys, width=100, height=12):
        self.keys = list(keys)
        self.w, self.h = width, height
        self.frames = []

    def size(self):
        return self.w, self.h

    def read_key(self, timeout):
        return self.keys.pop(0) if self.keys else None

    def draw(self, lines):
        assert len(lines) == self.h and all(len(ln) == self.w for ln in lines), [len(ln) for ln in lines]
        self.frames.append(lines)


class Clock:
    """Every look at the clock advances it, so each tick of the loop is also a poll."""

    def __init__(self):
        self.t = 0.0

    def __call__(self):
        self.t += 1.0
        return self.t


def _client():
    s = FakeServiceSession(ready_after=0)
    c = NeutrinoClient("http://svc", session=s, max_retries=0, sleep=lambda _t: None, poll_interval=0.0)
    return c, s


def _app(c, keys, tmp_path, **kw):
    term = ScriptedTerminal(keys, **kw)
    return App(c, term, cache_root=tmp_path / "cache", poll_interval=0.5, save_dir=tmp_path / "saved", color=False,
               clock=Clock()), term


def test_browse_filter_open_and_follow(tmp_path):
    c, s = _client()
    a = c.create_job([SubJobConfig.training_job("alpha-model", num_gpus=2)], name="alpha")["job_id"]
    b = c.create_job([SubJobConfig.sampling_job("beta-model", num_gpus=2)], name="beta")["job_id"]
    s.jobs[a]["status"], s.jobs[b]["status"] = "COMPLETED", "RUNNING"
    app, term = _app(c, ["/", "b", "e", "t", "enter", "enter", None, "q", "q"], tmp_path)
    assert app.run(max_ticks=20) == 0
    first = term.frames[0]
    assert first[0].startswith("jobs: 2 of 2") and first[1].startswith("> ") and b in first[1]   # the active job leads
    typing = term.frames[3]
    assert typing[-1].startswith("/be_") and typing[0].startswith("jobs: 1 of 2   filter: be")
    log_frame = next(f for f in term.frames if "[execution]" in f[0])
    assert b in log_frame[0] and any("line 4" in ln for ln in log_frame) and "following" in log_frame[-1]
    assert term.frames[-1][0].startswith("jobs: 1 of 2")                 # q on the log screen goes back, the filter stays


def test_log_screen_levels_filter_pause_scroll_save_and_sources(tmp_path):
    c, s = _client()
    jid = c.create_job([SubJobConfig.training_job("m", num_gpus=1)], name="x")["job_id"]
    s.jobs[jid]["sub_jobs"] = [{"sub_job_id": f"{jid}:training:0", "sub_job_type": "training"}]
    s.logs = [{"ts": f"t{i:02d}", "level": "ERROR" if i % 10 == 0 else "INFO", "message": f"line {i}"} for i in range(40)]
    keys = ["enter", "l", "l", "l", "l", None, "/", "3", "0", "enter", "s", "esc"]
    app, term = _app(c, keys, tmp_path)
    app.run(max_ticks=len(keys) + 1)
    m_frames = [f for f in term.frames if "[execution]" in f[0]]
    assert "level>=ERROR" in m_frames[5][-1]
    body = [ln.strip() for ln in m_frames[5][1:-1] if ln.strip()]
    assert body == [f"t{i:02d} [ERROR] line {i}" for i in (0, 10, 20, 30)]
    saved = list((tmp_path / "saved").glob(f"{jid}-execution-*.log"))
    assert len(saved) == 1 and saved[0].read_text() == "t30 [ERROR] line 30\n"
    assert app.log is None
    # scrolling up pauses the view and stops polling; G resumes at the end; tab walks the sources
    app.jobs.refresh()
    app._jobs_key("enter")
    m = app.log
    assert [lab for _sid, lab in m.sources] == ["execution", "training 0", "events"]
    w, h = term.size()
    app._log_key("pgup", w, h)
    assert m.paused and m.top == 40 - 10 - 10
    s.logs.append({"ts": "t40", "level": "INFO", "message": "line 40"})
    assert m.poll() == 0 and len(m.entries["execution"]) == 40
    shown = draw_log(m, w, h, None)
    assert "paused" in shown[-1] and "line 20" in shown[1] and "line 29" in shown[10]
    app._log_key("g", w, h)
    assert m.top == 0
    app._log_key("G", w, h)
    assert not m.paused and m.top is None and m.poll() == 1
    assert "line 40" in draw_log(m, w, h, None)[10]
    app._log_key("tab", w, h)
    assert m.source == f"sub:{jid}:training:0" and len(m.entries[m.source]) == 2           # one page of the sub-job log
    app._log_key("tab", w, h)
    assert m.source == "events" and "SCHEDULED" in "".join(draw_log(m, w, h, None))
    app._log_key("tab", w, h)
    assert m.source == "execution"
    app._log_key(" ", w, h)
    assert m.paused
    assert app._log_key("ctrl-c", w, h) is False


def test_reopening_a_job_replays_the_cache_and_continues(tmp_path):
    c, s = _client()
    jid = c.create_job([SubJobConfig.training_job("m", num_gpus=1)])["job_id"]
    m = LogModel(c, {"job_id": jid}, tmp_path)
    assert m.poll() == 5 and m.poll() == 0
    s.logs.append({"ts": "t5", "level": "WARN", "message": "late"})
    n_calls = len(s.calls)
    again = LogModel(c, {"job_id": jid}, tmp_path)
    assert again.poll() == 1 and len(again.entries["execution"]) == 6                      # 5 from disk + 1 fetched
    assert s.calls[n_calls][2] == {"cursor": 5}
    s.fail_next = [400]
    assert again.poll() == 0 and again.status.startswith("fetch failed")
    assert again.poll() == 0 and again.status == ""


def test_jobs_model_survives_a_failing_service_and_long_lists(tmp_path):
    c, s = _client()
    for i in range(30):
        c.create_job([SubJobConfig.training_job("m", num_gpus=1)], name=f"n{i}")
    m = JobsModel(c)
    m.refresh()
    m.move(25)
    lines = draw_jobs(m, 80, 10, None)
    assert sum(ln.startswith("> ") for ln in lines) == 1 and lines[8].startswith("> ")       # the cursor stays on screen
    m.move(100)
    assert m.cursor == 29
    s.fail_next = [400]
    m.refresh()
    assert m.error.startswith("refresh failed") and len(m.jobs) == 30
    assert "refresh failed" in draw_jobs(m, 80, 10, None)[-1]
    m.set_query("no such job")
    assert m.selected() is None and draw_jobs(m, 80, 10, None)[0].startswith("jobs: 0 of 30")


def test_terminal_reads_keys_from_a_pseudo_terminal():
    import io
    import os
    import pty

    from cortex_client.dss_client.tui.app import Terminal
    master, slave = pty.openpty()
    out = io.StringIO()
    with os.fdopen(slave, "rb", buffering=0) as tty_in:
        with Terminal(stdin=tty_in, stdout=out) as term:
            assert term.read_key(0.05) is None                                   # nothing typed
            os.write(master, b"j")
            assert term.read_key(1.0) == "j"
            os.write(master, b"\x1b[A")
            assert term.read_key(1.0) == "up"
            os.write(master, b"\x1b[6~")
            assert term.read_key(1.0) == "pgdn"
            os.write(master, b"\r")
            assert term.read_key(1.0) == "enter"
            os.write(master, b"\x1b")
            assert term.read_key(1.0) == "esc"                                   # a lone escape, after the short wait
            os.write(master, b"\x7f")
            assert term.read_key(1.0) == "backspace"
            term.draw(["ab", "cd"])
            w, h = term.size()
            assert w > 0 and h > 0
        text = out.getvalue()
        assert text.startswith("\x1b[?1049h\x1b[?25l") and "\x1b[Hab\r\ncd" in text and text.endswith("\x1b[?25h\x1b[?1049l")
    os.close(master)
