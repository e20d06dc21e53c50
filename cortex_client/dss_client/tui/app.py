"""Full-screen job browser and log viewer on a plain terminal (ANSI escapes + raw keyboard; no UI toolkit).

    python -m cortex_client.dss_client.tui app [--url ... | --config ...]

Two screens.  **Jobs**: active jobs first, newest first; ``j``/``k`` or arrows move, ``Enter`` opens the job's log,
``/`` filters as you type (``Enter`` keeps the filter, ``Esc`` drops it), ``r`` refreshes, ``q`` quits.  **Log**: the
entries of one source of the job (its execution log, each sub-job's log, the scheduling events), read through the
on-disk cache so reopening a job continues where the last session stopped; ``Tab`` switches source, ``l`` cycles the
minimum level, ``/`` filters, ``p`` or space pauses following, arrows / ``PgUp`` / ``PgDn`` / ``g`` / ``G`` scroll
(scrolling up pauses, ``G`` resumes), ``s`` saves what the filters show to a file, ``Esc`` or ``q`` goes back.

The program is a loop of *read a key or time out -> update a model -> draw the model*.  Models and drawing are pure
(``JobsModel``, ``LogModel``, ``draw_*`` return lists of lines), the terminal sits behind ``Terminal`` -- tests drive
the same loop with a scripted terminal.  Counterpart of cortex-client/dss_client/tui/app.py in the reference (a
Textual application there).
"""
from __future__ import annotations

import os
import sys
import time
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

from .format import (colorize, entry_at_level, entry_matches, format_event, format_job_row, format_job_summary,
                     format_log_entry, job_matches, job_status_color, sort_jobs, wrap_log_line)
from .log_cache import LogCache

LEVEL_CYCLE = (None, "DEBUG", "INFO", "WARN", "ERROR")
LEVEL_COLOR = {"ERROR": "red", "FATAL": "red", "CRITICAL": "red", "WARN": "yellow", "WARNING": "yellow", "DEBUG": "dim"}
MAX_ENTRIES = 50_000            # per source, in memory; the cache on disk keeps more
KEYS = {"\x1b[A": "up", "\x1b[B": "down", "\x1b[5~": "pgup", "\x1b[6~": "pgdn", "\x1b[H": "home", "\x1b[F": "end",
        "\x1bOA": "up", "\x1bOB": "down", "\r": "enter", "\n": "enter", "\x7f": "backspace", "\x08": "backspace",
        "\t": "tab", "\x1b": "esc", "\x03": "ctrl-c"}


# ------------------------------------------------------------------------------------------------- models
class JobsModel:
    def __init__(self, client):
        self.client = client
        self.jobs: List[dict] = []
        self.query = ""
        self.cursor = 0
        self.error = ""

    def refresh(self) -> None:
        try:
            self.jobs = sort_jobs(self.client.list_jobs())
            self.error = ""
        except Exception as exc:                       # the screen stays usable; the status line says what happened
            self.error = f"refresh failed: {exc}"
        self.cursor = min(self.cursor, max(0, len(self.visible()) - 1))

    def visible(self) -> List[dict]:
        return [j for j in self.jobs if job_matches(j, self.query)]

    def move(self, delta: int) -> None:
        n = len(self.visible())
        self.cursor = 0 if n == 0 else max(0, min(n - 1, self.cursor + delta))

    def set_query(self, q: str) -> None:
        self.query, self.cursor = q, 0

    def selected(self) -> Optional[dict]:
        vis = self.visible()
        return vis[self.cursor] if vis else None


class LogModel:
    """Entries of one job, per source.  ``poll()`` fetches at most one page of the current source."""

    def __init__(self, client, job: dict, cache_root: Optional[Path] = None):
        self.client = client
        self.job = job
        self.job_id = str(job.get("job_id") or job.get("id"))
        self.cache = LogCache(self.job_id, cache_root)
        self.sources = self._sources(job)
        self.source_idx = 0
        self.entries: Dict[str, List[Any]] = {}
        self.cursors: Dict[str, Optional[str]] = {}
        self.level_idx = 0
        self.query = ""
        self.paused = False
        self.top: Optional[int] = None           # first visible wrapped line; None = stick to the end
        self.status = ""

    @staticmethod
    def _sources(job: dict) -> List[Tuple[str, str]]:
        """(id, label): the execution log, one log per sub-job, the scheduling events."""
        out = [("execution", "execution")]
        for sj in job.get("sub_jobs") or []:
            sid = sj.get("sub_job_id") if isinstance(sj, dict) else None
            if sid:
                kind = sj.get("sub_job_type") or sj.get("job_type") or "sub-job"
                out.append((f"sub:{sid}", f"{kind} {str(sid).rsplit(':', 1)[-1]}"))
        out.append(("events", "events"))
        return out

    @property
    def source(self) -> str:
        return self.sources[self.source_idx][0]

    @property
    def min_level(self) -> Optional[str]:
        return LEVEL_CYCLE[self.level_idx]

    def next_source(self) -> None:
        self.source_idx = (self.source_idx + 1) % len(self.sources)
        self.top = None

    def cycle_level(self) -> None:
        self.level_idx = (self.level_idx + 1) % len(LEVEL_CYCLE)

    def _fetch(self, source: str, cursor: Optional[str]) -> Dict[str, Any]:
        if source == "execution":
            start = int(cursor or 0)
            got = self.client.fetch_execution_logs(self.job_id, start)
            return {"entries": got, "next_cursor": str(start + len(got))}
        if source == "events":
            page = self.client.tail_events(self.job_id, cursor=cursor)
            return {"entries": page.get("events") or [], "next_cursor": page.get("next_cursor", cursor)}
        page = self.client.tail_logs(self.job_id, cursor=cursor, sub_job_id=source[4:])
        return {"entries": page.get("entries") or [], "next_cursor": page.get("next_cursor", cursor)}

    def poll(self) -> int:
        """One fetch for the current source (none while paused).  The first poll of a source replays its cache."""
        src = self.source
        if src not in self.entries:
            self.entries[src] = self.cache.load_entries(src, MAX_ENTRIES)
            self.cursors[src] = self.cache.get_cursor(src)
        if self.paused:
            return 0
        try:
            page = self._fetch(src, self.cursors[src])
        except Exception as exc:
            self.status = f"fetch failed: {exc}"
            return 0
        self.status = ""
        new, nxt = list(page.get("entries") or []), page.get("next_cursor")
        try:
            self.cache.append_entries(src, new)
            if nxt is not None and nxt != self.cursors[src]:
                self.cache.set_cursor(src, nxt)
        except OSError:
            pass                                  # an unwritable cache costs the resume point, not the session
        if nxt is not None:
            self.cursors[src] = nxt
        buf = self.entries[src]
        buf.extend(new)
        if len(buf) > MAX_ENTRIES:
            del buf[:len(buf) - MAX_ENTRIES]
        return len(new)

    def _text(self, entry: Any) -> str:
        return format_event(entry) if self.source == "events" else format_log_entry(entry)

    def filtered(self) -> List[Any]:
        if self.source == "events":                # events carry no level; the text filter applies to what is shown
            q = self.query.strip().lower()
            return [e for e in self.entries.get("events", []) if not q or q in format_event(e).lower()]
        return [e for e in self.entries.get(self.source, [])
                if entry_at_level(e, self.min_level) and entry_matches(e, self.query)]

    def lines(self, width: int) -> List[Tuple[str, str]]:
        """(text, colour) per screen line after filtering and wrapping."""
        out: List[Tuple[str, str]] = []
        for e in self.filtered():
            level = str(e.get("level", "INFO")).upper() if isinstance(e, dict) else "INFO"
            for ln in wrap_log_line(self._text(e), width):
                out.append((ln, LEVEL_COLOR.get(level, "")))
        return out

    def scroll(self, delta: int, total: int, height: int) -> None:
        last_top = max(0, total - height)
        cur = last_top if self.top is None else self.top
        cur = max(0, min(last_top, cur + delta))
        self.top = None if cur >= last_top and delta > 0 else cur
        if delta < 0:
            self.paused = True                    # reading older lines: stop the view from running away

    def to_end(self) -> None:
        self.top, self.paused = None, False

    def save(self, directory: Optional[Path] = None) -> Path:
        directory = Path(directory) if directory else Path.cwd()
        directory.mkdir(parents=True, exist_ok=True)
        safe = self.source.replace(":", "_").replace("/", "_")
        path = directory / f"{self.job_id}-{safe}-{time.strftime('%Y%m%d-%H%M%S')}.log"
        path.write_text("".join(self._text(e) + "\n" for e in self.filtered()), encoding="utf-8")
        self.status = f"saved {path}"
        return path


# ------------------------------------------------------------------------------------------------- drawing
def _fit(text: str, width: int) -> str:
    return text[:width].ljust(width) if width > 0 else ""


def draw_jobs(m: JobsModel, width: int, height: int, editing: Optional[str], color: bool = False) -> List[str]:
    vis = m.visible()
    body_h = max(1, height - 2)
    first = max(0, min(m.cursor - body_h + 1, len(vis) - body_h)) if m.cursor >= body_h else 0
    lines = [_fit(f"jobs: {len(vis)} of {len(m.jobs)}" + (f"   filter: {m.query}" if m.query else ""), width)]
    for i in range(first, min(len(vis), first + body_h)):
        row = _fit(("> " if i == m.cursor else "  ") + format_job_row(vis[i]), width)
        lines.append(colorize(row, job_status_color(vis[i].get("status")), color))
    lines += [" " * width] * (height - 1 - len(lines))
    foot = f"/{editing}_" if editing is not None else (m.error or "enter open  / filter  r refresh  q quit")
    lines.append(_fit(foot, width))
    return lines


def draw_log(m: LogModel, width: int, height: int, editing: Optional[str], color: bool = False) -> List[str]:
    body_h = max(1, height - 2)
    all_lines = m.lines(width)
    top = max(0, len(all_lines) - body_h) if m.top is None else min(m.top, max(0, len(all_lines) - body_h))
    tabs = "  ".join(f"[{lab}]" if i == m.source_idx else lab for i, (_sid, lab) in enumerate(m.sources))
    head = f"{format_job_summary(m.job)}   {tabs}"
    lines = [_fit(head, width)]
    for text, col in all_lines[top:top + body_h]:
        lines.append(colorize(_fit(text, width), col, color))
    lines += [" " * width] * (height - 1 - len(lines))
    state = "paused" if m.paused else "following"
    foot = f"/{editing}_" if editing is not None else (
        m.status or f"{state}  level>={m.min_level or 'all'}" + (f"  filter: {m.query}" if m.query else "") +
        f"  {len(all_lines)} lines   tab source  l level  / filter  p pause  s save  esc back")
    lines.append(_fit(foot, width))
    return lines


# ------------------------------------------------------------------------------------------------- terminal
class Terminal:
    """Raw-mode terminal: ``read_key(timeout)`` returns a key name ('a', 'up', 'enter', ...) or None."""

    def __init__(self, stdin=None, stdout=None):
        self.stdin = stdin or sys.stdin
        self.stdout = stdout or sys.stdout
        self._saved = None

    def __enter__(self):
        import termios
        import tty
        fd = self.stdin.fileno()
        self._saved = termios.tcgetattr(fd)
        tty.setcbreak(fd)
        self.stdout.write("\x1b[?1049h\x1b[?25l")              # alternate screen, no cursor
        return self

    def __exit__(self, *exc):
        import termios
        self.stdout.write("\x1b[?25h\x1b[?1049l")
        self.stdout.flush()
        if self._saved is not None:
            termios.tcsetattr(self.stdin.fileno(), termios.TCSADRAIN, self._saved)

    def size(self) -> Tuple[int, int]:
        import shutil
        s = shutil.get_terminal_size((120, 40))
        return s.columns, s.lines

    def read_key(self, timeout: float) -> Optional[str]:
        import select
        fd = self.stdin.fileno()
        if not select.select([fd], [], [], timeout)[0]:
            return None
        data = os.read(fd, 1).decode(errors="ignore")
        if data == "\x1b":                                      # an escape sequence arrives in one burst
            while select.select([fd], [], [], 0.01)[0] and len(data) < 8:
                data += os.read(fd, 1).decode(errors="ignore")
                if data[-1].isalpha() or data[-1] == "~":
                    break
        return KEYS.get(data, data)

    def draw(self, lines: List[str]) -> None:
        self.stdout.write("\x1b[H" + "\r\n".join(lines))
        self.stdout.flush()


# ------------------------------------------------------------------------------------------------- the loop
class App:
    def __init__(self, client, terminal, cache_root: Optional[Path] = None, poll_interval: float = 1.0,
                 save_dir: Optional[Path] = None, color: bool = True, clock: Callable[[], float] = time.monotonic):
        self.client = client
        self.term = terminal
        self.cache_root = cache_root
        self.poll_interval = poll_interval
        self.save_dir = save_dir
        self.color = color
        self.clock = clock
        self.jobs = JobsModel(client)
        self.log: Optional[LogModel] = None
        self.editing: Optional[str] = None          # text of the filter being typed, None when not typing

    # -- filter line shared by both screens
    def _edit(self, key: str) -> None:
        target = self.log if self.log is not None else self.jobs
        setq = (lambda q: setattr(target, "query", q)) if self.log is not None else self.jobs.set_query
        if key == "enter":
            self.editing = None
        elif key == "esc":
            self.editing = None
            setq("")
        elif key == "backspace":
            self.editing = self.editing[:-1]
            setq(self.editing)
        elif len(key) == 1 and key.isprintable():
            self.editing += key
            setq(self.editing)

    def _jobs_key(self, key: str) -> bool:
        m = self.jobs
        if key in ("q", "ctrl-c"):
            return False
        if key in ("down", "j"):
            m.move(1)
        elif key in ("up", "k"):
            m.move(-1)
        elif key == "pgdn":
            m.move(10)
        elif key == "pgup":
            m.move(-10)
        elif key == "r":
            m.refresh()
        elif key == "/":
            self.editing = m.query
        elif key == "esc":
            m.set_query("")
        elif key == "enter" and m.selected() is not None:
            job = m.selected()
            try:
                job = self.client.get_job(str(job.get("job_id") or job.get("id")))   # sub-job ids for the source tabs
            except Exception:
                pass
            self.log = LogModel(self.client, job, self.cache_root)
            self.log.poll()
        return True

    def _log_key(self, key: str, width: int, height: int) -> bool:
        m = self.log
        body_h = max(1, height - 2)
        total = len(m.lines(width))
        if key == "ctrl-c":
            return False
        if key in ("esc", "q"):
            self.log = None
        elif key == "tab":
            m.next_source()
            m.poll()
        elif key == "l":
            m.cycle_level()
        elif key in ("p", " "):
            m.paused = not m.paused
        elif key == "/":
            self.editing = m.query
        elif key in ("up", "k"):
            m.scroll(-1, total, body_h)
        elif key in ("down", "j"):
            m.scroll(1, total, body_h)
        elif key == "pgup":
            m.scroll(-body_h, total, body_h)
        elif key == "pgdn":
            m.scroll(body_h, total, body_h)
        elif key in ("g", "home"):
            m.scroll(-total, total, body_h)
        elif key in ("G", "end"):
            m.to_end()
        elif key == "s":
            try:
                m.save(self.save_dir)
            except OSError as exc:
                m.status = f"save failed: {exc}"
        return True

    def frame(self) -> List[str]:
        w, h = self.term.size()
        if self.log is not None:
            return draw_log(self.log, w, h, self.editing, self.color)
        return draw_jobs(self.jobs, w, h, self.editing, self.color)

    def run(self, max_ticks: Optional[int] = None) -> int:
        self.jobs.refresh()
        next_poll = self.clock() + self.poll_interval
        ticks = 0
        while max_ticks is None or ticks < max_ticks:
            ticks += 1
            self.term.draw(self.frame())
            key = self.term.read_key(max(0.0, min(0.25, next_poll - self.clock())))
            if key is not None:
                if self.editing is not None:
                    self._edit(key)
                else:
                    w, h = self.term.size()
                    alive = self._log_key(key, w, h) if self.log is not None else self._jobs_key(key)
                    if not alive:
                        return 0
            if self.clock() >= next_poll:
                if self.log is not None:
                    self.log.poll()
                next_poll = self.clock() + self.poll_interval
        return 0


def main(client, cache_root: Optional[Path] = None) -> int:
    if not (sys.stdin.isatty() and sys.stdout.isatty()):
        sys.stderr.write("the full-screen viewer needs a terminal; use `tui jobs` / `tui logs JOB` for plain output\n")
        return 2
    with Terminal() as term:
        return App(client, term, cache_root).run()
