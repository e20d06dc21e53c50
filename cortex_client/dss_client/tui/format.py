"""Lines for the log viewer: log entries, job rows, filters.  Pure functions over the service's JSON records
(cortex-client/dss_client/tui/format.py:18-356 in the reference)."""
from __future__ import annotations

import textwrap
from datetime import datetime, timezone
from typing import Any, List

LEVELS = {"TRACE": 5, "DEBUG": 10, "INFO": 20, "WARN": 30, "WARNING": 30, "ERROR": 40, "FATAL": 50, "CRITICAL": 50}
ACTIVE = {"PENDING", "QUEUED", "STARTING", "RUNNING", "CANCELLING"}
COLORS = {"RUNNING": "green", "PENDING": "yellow", "QUEUED": "yellow", "STARTING": "yellow", "FAILED": "red",
          "CANCELLED": "magenta", "CANCELLING": "magenta", "DONE": "blue", "SUCCEEDED": "blue", "COMPLETED": "blue"}
ANSI = {"red": "\x1b[31m", "green": "\x1b[32m", "yellow": "\x1b[33m", "blue": "\x1b[34m", "magenta": "\x1b[35m",
        "dim": "\x1b[2m", "reset": "\x1b[0m"}


def _level(entry: Any) -> str:
    if isinstance(entry, dict):
        return str(entry.get("level") or entry.get("severity") or "INFO").upper()
    return "INFO"


def format_log_entry(entry: Any) -> str:
    """``<timestamp> [LEVEL] (source) message`` from a dict entry; anything else is printed as text."""
    if not isinstance(entry, dict):
        return str(entry)
    ts = entry.get("ts") or entry.get("timestamp") or entry.get("time") or ""
    msg = entry.get("message", entry.get("msg", ""))
    src = entry.get("source") or entry.get("rank")
    head = f"{ts} " if ts else ""
    where = f"({src}) " if src not in (None, "") else ""
    return f"{head}[{_level(entry)}] {where}{msg}".rstrip()


def format_event(ev: Any) -> str:
    """``<timestamp> KIND [sub-job] detail`` for a scheduling event (placement, zone ready, restarts, ...)."""
    if not isinstance(ev, dict):
        return str(ev)
    ts = ev.get("ts") or ev.get("timestamp") or ev.get("time") or ""
    kind = ev.get("kind") or ev.get("type") or ev.get("event") or "EVENT"
    where = ev.get("sub_job_id") or ev.get("source") or ""
    detail = ev.get("message") or ev.get("reason") or ev.get("detail") or ""
    if isinstance(detail, (dict, list)):
        import json
        detail = json.dumps(detail, sort_keys=True)
    return " ".join(str(x) for x in (ts, kind, f"[{where}]" if where else "", detail) if x not in ("", None))


def source_label(source: Any) -> str:
    """Side-panel label of a log source (a sub-job: its id string or ``{"sub_job_id", "job_type"}``):
    ``"<type> #<index>"``, the type taken from ``job_type`` or else from the middle of ``<uuid>:<type>:<index>``."""
    if isinstance(source, dict):
        sid = str(source.get("sub_job_id") or source.get("id") or source.get("source_id") or "")
        kind = source.get("job_type") or source.get("type")
    else:
        sid, kind = str(source), None
    parts = sid.split(":")
    if kind is None and len(parts) >= 3:
        kind = parts[-2]
    index = parts[-1] if len(parts) >= 2 and parts[-1].isdigit() else None
    if kind and index is not None:
        return f"{kind} #{index}"
    return str(kind or sid or "?")


def wrap_log_line(text: Any, width: int) -> List[str]:
    """Hard wrap at ``width`` columns keeping every character (log lines hold stack traces and JSON: nothing is
    dropped, continuation lines are indented by two spaces)."""
    text = str(text)
    if width <= 4 or len(text) <= width:
        return text.split("\n") if "\n" in text else [text]
    out: List[str] = []
    for raw in text.split("\n"):
        first = True
        while raw:
            room = width if first else width - 2
            out.append(("" if first else "  ") + raw[:room])
            raw, first = raw[room:], False
        if first:
            out.append("")
    return out


def is_active_status(status: Any) -> bool:
    return str(status or "").upper() in ACTIVE


def job_status_color(status: Any) -> str:
    return COLORS.get(str(status or "").upper(), "dim")


def _created_epoch(raw: Any) -> float:
    if raw in (None, ""):
        return 0.0
    if isinstance(raw, (int, float)):
        return float(raw) / (1000.0 if raw > 1e11 else 1.0)
    try:
        return datetime.fromisoformat(str(raw).replace("Z", "+00:00")).timestamp()
    except ValueError:
        return 0.0


def format_created_at(raw: Any) -> str:
    t = _created_epoch(raw)
    return datetime.fromtimestamp(t, tz=timezone.utc).strftime("%Y-%m-%d %H:%M") if t else "-"


def sort_jobs(jobs: Any) -> list:
    """Active jobs first, newest first inside each class."""
    return sorted(list(jobs or []), key=lambda j: (not is_active_status(j.get("status")), -_created_epoch(j.get("created_at"))))


def _submitted(job: Any) -> dict:
    """The body the job was created with, when the service echoes it inside the record."""
    body = job.get("body") if isinstance(job, dict) else None
    return body if isinstance(body, dict) else {}


def format_job_config(job: Any) -> str:
    parts = []
    subs = job.get("sub_jobs") or _submitted(job).get("sub_jobs") or _submitted(job).get("sub_job_configs") or []
    for sj in subs:
        if not isinstance(sj, dict):
            continue
        cfg = sj.get("config") or sj
        bits = [str(sj.get("type") or sj.get("sub_job_type") or sj.get("job_type") or "?")]
        if cfg.get("model_name"):
            bits.append(str(cfg["model_name"]))
        gpus = next((cfg[k] for k in ("num_gpus", "gpus", "num_devices", "n_gpus") if cfg.get(k)), None)
        if gpus:
            bits.append(f"{gpus}g")
        parts.append(":".join(bits))
    return " + ".join(parts)


def format_job_row(job: Any) -> str:
    name = job.get("name") or _submitted(job).get("name") or ""
    return (f"{str(job.get('job_id') or job.get('id') or '?'):<14} {str(job.get('status') or '?'):<10} "
            f"{format_created_at(job.get('created_at')):<16} {name} {format_job_config(job)}").rstrip()


def format_job_summary(job: Any) -> str:
    return textwrap.shorten(f"{job.get('job_id') or job.get('id')} [{job.get('status')}] {format_job_config(job)}", 120)


def job_matches(job: Any, query: str) -> bool:
    q = (query or "").strip().lower()
    return not q or q in format_job_row(job).lower()


def entry_matches(entry: Any, query: str) -> bool:
    q = (query or "").strip().lower()
    return not q or q in format_log_entry(entry).lower()


def entry_at_level(entry: Any, min_level: Any) -> bool:
    if min_level in (None, ""):
        return True
    need = LEVELS.get(str(min_level).upper(), 0) if not isinstance(min_level, int) else min_level
    return LEVELS.get(_level(entry), 20) >= need


def colorize(text: str, color: str, enabled: bool) -> str:
    return f"{ANSI[color]}{text}{ANSI['reset']}" if enabled and color in ANSI else text
