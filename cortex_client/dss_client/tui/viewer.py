"""Terminal log viewer: replays a job's cached log lines, then follows the service from the saved cursor.  Output
is plain lines (ANSI colours on a terminal), so it works over ssh, in a pager and in CI logs."""
from __future__ import annotations

import shutil
import sys
import time
from typing import Any, Callable, Dict, List, Optional

from .format import (colorize, entry_at_level, entry_matches, format_job_row, format_log_entry, job_matches,
                     job_status_color, sort_jobs, wrap_log_line)
from .log_cache import LogCache, cached_pages

_LEVEL_COLOR = {"ERROR": "red", "FATAL": "red", "CRITICAL": "red", "WARN": "yellow", "WARNING": "yellow", "DEBUG": "dim"}


class LogViewer:
    def __init__(self, client, out=None, cache_root=None, width: Optional[int] = None, color: Optional[bool] = None,
                 sleep: Callable[[float], None] = time.sleep):
        self.client = client
        self.out = out if out is not None else sys.stdout
        self.cache_root = cache_root
        self.width = width or shutil.get_terminal_size((120, 40)).columns
        self.color = color if color is not None else bool(getattr(self.out, "isatty", lambda: False)())
        self.sleep = sleep

    # ------------------------------------------------------------------ jobs
    def list_jobs(self, query: str = "", status: Optional[str] = None) -> List[Dict[str, Any]]:
        jobs = [j for j in sort_jobs(self.client.list_jobs(status)) if job_matches(j, query)]
        for j in jobs:
            self.out.write(colorize(format_job_row(j), job_status_color(j.get("status")), self.color) + "\n")
        return jobs

    # ------------------------------------------------------------------ logs
    def _fetch(self, job_id: str) -> Callable[[Optional[str]], Dict[str, Any]]:
        """Adapts the client's integer-offset log call to the cursor protocol of the cache."""
        def fetch(cursor: Optional[str]) -> Dict[str, Any]:
            start = int(cursor or 0)
            entries = self.client.fetch_execution_logs(job_id, start)
            return {"entries": entries, "next_cursor": str(start + len(entries)), "eof": not entries}
        return fetch

    def show(self, job_id: str, follow: bool = False, min_level: Optional[str] = None, query: str = "",
             source: str = "execution", max_polls: Optional[int] = None, tail: Optional[int] = None) -> int:
        """Prints the job's log.  Returns the number of entries printed (after filters)."""
        cache = LogCache(job_id, self.cache_root)
        shown = 0
        for page in cached_pages(self._fetch(job_id), cache, source, follow=follow, sleep=self.sleep,
                                 max_polls=max_polls, replay_limit=tail):
            for e in page:
                if not (entry_at_level(e, min_level) and entry_matches(e, query)):
                    continue
                level = str(e.get("level", "INFO")).upper() if isinstance(e, dict) else "INFO"
                for ln in wrap_log_line(format_log_entry(e), self.width):
                    self.out.write(colorize(ln, _LEVEL_COLOR.get(level, ""), self.color) + "\n")
                shown += 1
            if hasattr(self.out, "flush"):
                self.out.flush()
        return shown
