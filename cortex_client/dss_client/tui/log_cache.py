"""Persistent client-side cache for the log viewer.

Reopening a job must not fetch again what was fetched before: the service is stateless on purpose and every log
request costs it a query.  The transport is cursor based (``fetch(cursor) -> {entries, next_cursor, eof}``), so per
``(job, source)`` the client keeps

* the cursor returned last -- the next session resumes with a delta-only request, and
* the entries themselves as append-only JSON lines -- the next session repaints at once.

Standard library only, so the cache is testable without a terminal
(cortex-client/dss_client/tui/log_cache.py:1-400 in the reference)."""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
import time
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional

OVERRIDE_ENV = "NEUTRINO_TUI_CACHE_DIR"
_NAMESPACE = "neutrino-tui"
_SAFE = frozenset("ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789-_.")
_MAX_NAME = 200
POLL_BACKOFF = 1.25
POLL_MAX_INTERVAL = 6.0


def cache_root() -> Path:
    """``$NEUTRINO_TUI_CACHE_DIR``, else ``$XDG_CACHE_HOME/neutrino-tui``, else ``~/.cache/neutrino-tui``; created
    lazily by the writers."""
    override = os.environ.get(OVERRIDE_ENV)
    if override:
        return Path(override).expanduser()
    xdg = os.environ.get("XDG_CACHE_HOME")
    return (Path(xdg).expanduser() if xdg else Path.home() / ".cache") / _NAMESPACE


def safe_source_name(source_id: str) -> str:
    """One path component for an arbitrary source id: bytes outside ``[A-Za-z0-9-_.]`` become ``%XX``.  Reversible
    below 200 characters; longer ids are cut and get a digest (the id -> cursor map keeps the exact id)."""
    name = "".join(chr(b) if chr(b) in _SAFE else "%%%02X" % b for b in source_id.encode("utf-8"))
    if name in (".", ".."):
        name = name.replace(".", "%2E")
    if len(name) > _MAX_NAME:
        name = name[:_MAX_NAME - 13] + "-" + hashlib.sha1(source_id.encode("utf-8")).hexdigest()[:12]
    return name or "%00"


def unsafe_source_name(name: str) -> str:
    out = bytearray()
    i = 0
    while i < len(name):
        if name[i] == "%" and len(name) - i >= 3:
            out.append(int(name[i + 1:i + 3], 16))
            i += 3
        else:
            out += name[i].encode("utf-8")
            i += 1
    return out.decode("utf-8", "replace")


def _atomic_write_text(path: Path, text: str) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=str(path.parent), prefix=path.name + ".")
    try:
        with os.fdopen(fd, "w", encoding="utf-8") as f:
            f.write(text)
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise


class LogCache:
    """Cache of one job: ``<root>/<job>/cursors.json`` and ``<root>/<job>/logs/<source>.jsonl``.  A source file
    larger than ``max_bytes`` is rewritten with its newest half (the cursor is kept: old lines are simply no longer
    repainted)."""

    def __init__(self, job_id: str, root: Optional[Path] = None, max_bytes: int = 64 << 20):
        self.job_id = str(job_id)
        self.dir = (Path(root) if root is not None else cache_root()) / safe_source_name(self.job_id)
        self.max_bytes = int(max_bytes)

    def _jsonl(self, source_id: str) -> Path:
        return self.dir / "logs" / (safe_source_name(source_id) + ".jsonl")

    def _cursors_path(self) -> Path:
        return self.dir / "cursors.json"

    def _read_cursors(self) -> Dict[str, Any]:
        try:
            data = json.loads(self._cursors_path().read_text(encoding="utf-8"))
            return data if isinstance(data, dict) else {}
        except (OSError, ValueError):
            return {}

    def get_cursor(self, source_id: str) -> Optional[str]:
        return self._read_cursors().get(source_id)

    def set_cursor(self, source_id: str, cursor: Optional[str]) -> None:
        cur = self._read_cursors()
        if cursor is None:
            cur.pop(source_id, None)
        else:
            cur[source_id] = cursor
        _atomic_write_text(self._cursors_path(), json.dumps(cur, sort_keys=True))

    def append_entries(self, source_id: str, entries: Iterable[Any]) -> int:
        entries = list(entries)
        if not entries:
            return 0
        path = self._jsonl(source_id)
        path.parent.mkdir(parents=True, exist_ok=True)
        with open(path, "a", encoding="utf-8") as f:
            for e in entries:
                f.write(json.dumps(e, separators=(",", ":"), default=str) + "\n")
        self._rotate_if_needed(path)
        return len(entries)

    def load_entries(self, source_id: str, limit: Optional[int] = None) -> List[Any]:
        try:
            lines = self._jsonl(source_id).read_text(encoding="utf-8").splitlines()
        except OSError:
            return []
        if limit is not None:
            lines = lines[-limit:]
        out = []
        for ln in lines:
            try:
                out.append(json.loads(ln))
            except ValueError:
                continue                       # a line cut off by a crash: skip it, keep the rest
        return out

    def cached_sources(self) -> List[str]:
        known = set(self._read_cursors())
        logs = self.dir / "logs"
        if logs.is_dir():
            known.update(unsafe_source_name(p.stem) for p in logs.glob("*.jsonl"))
        return sorted(known)

    def clear(self) -> None:
        import shutil
        if self.dir.exists():
            shutil.rmtree(self.dir)

    def _rotate_if_needed(self, path: Path) -> None:
        try:
            if path.stat().st_size <= self.max_bytes:
                return
            lines = path.read_text(encoding="utf-8").splitlines(keepends=True)
            _atomic_write_text(path, "".join(lines[len(lines) // 2:]))
        except OSError:
            pass


def cached_pages(fetch: Callable[[Optional[str]], Dict[str, Any]], cache: LogCache, source_id: str, follow: bool = False,
                 sleep: Callable[[float], None] = time.sleep, poll_interval: float = 1.0,
                 max_polls: Optional[int] = None, replay_limit: Optional[int] = None) -> Iterator[List[Any]]:
    """Pages of log entries: first what the cache holds, then what ``fetch(cursor)`` returns from the saved cursor
    on.  ``fetch`` answers ``{"entries": [...], "next_cursor": str | None, "eof": bool}``.  Every page is appended
    to the cache and the cursor saved BEFORE the page is handed out, so an interrupted session loses nothing and
    repeats nothing.  Without ``follow`` the generator ends at ``eof`` (or at an empty page); with it, empty polls
    back off geometrically up to six seconds.  A cache that cannot be written only costs the resume point."""
    replay = cache.load_entries(source_id, replay_limit)
    if replay:
        yield replay
    cursor = cache.get_cursor(source_id)
    wait, polls = poll_interval, 0
    while True:
        page = fetch(cursor) or {}
        entries = list(page.get("entries") or [])
        nxt = page.get("next_cursor", cursor)
        try:
            cache.append_entries(source_id, entries)
            if nxt is not None and nxt != cursor:
                cache.set_cursor(source_id, nxt)
        except OSError:
            pass
        cursor = nxt if nxt is not None else cursor
        polls += 1
        if entries:
            wait = poll_interval
            yield entries
        if max_polls is not None and polls >= max_polls:
            return
        if not follow and (page.get("eof", not entries) or not entries):
            return
        if not entries:
            sleep(wait)
            wait = min(wait * POLL_BACKOFF, POLL_MAX_INTERVAL)


def cached_log_pages(cache: LogCache, client: Any, job_id: str, sub_job_id: str, *, follow: bool = False,
                     poll_interval: float = 1.0, replay_limit: Optional[int] = 2000, tail_lines: Optional[int] = 2000,
                     sleep: Callable[[float], None] = time.sleep, max_polls: Optional[int] = None) -> Iterator[List[Any]]:
    """``cached_pages`` over ``client.tail_logs`` for one sub-job (the cache is keyed by ``sub_job_id``).  The very
    first request of a sub-job (no saved cursor) asks only for the last ``tail_lines`` lines: a job that has run for
    hours is not read from its first line.  Later requests continue from the saved cursor and send no line limit."""
    def fetch(cursor: Optional[str]) -> Dict[str, Any]:
        kw: Dict[str, Any] = {"cursor": cursor, "sub_job_id": sub_job_id}
        if cursor is None and tail_lines:
            kw["max_lines"] = int(tail_lines)
        return client.tail_logs(job_id, **kw)

    return cached_pages(fetch, cache, sub_job_id, follow=follow, sleep=sleep, poll_interval=poll_interval,
                        max_polls=max_polls, replay_limit=replay_limit)
