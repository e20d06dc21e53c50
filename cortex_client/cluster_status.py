"""``python -m cortex_client.cluster_status``: which jobs hold how many GPUs, refreshed in place.

    python -m cortex_client.cluster_status --url http://host:port            # watch, every 10 s
    python -m cortex_client.cluster_status --config conn.json --once
    dss-neutrino list --compact | python -m cortex_client.cluster_status --jobs-json - --once

One table per watched state (running, then placing / pending) with the job id, its name, GPUs and a one-line
breakdown of its sub-jobs (``training x8 + sampling x8 (tp 2)``), a GPU total per state and the service's free
capacity when it reports one.  Connection flags are those of ``dss-neutrino``.  Counterpart of
cortex-client/cluster-status.py in the reference (which shells out to the command line; this one calls the client).
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import Any, Dict, Iterable, List, Optional, Tuple

WATCHED = ("RUNNING", "PLACING", "PENDING")
GPU_KEYS = ("n_gpus", "num_devices", "num_gpus")
CONFIG_HOLDERS = ("training_config", "inference_config", "sampling_config", "vllm_config")


def normalize_status(status: Any) -> str:
    word = str(status or "").strip().upper()
    return word[len("JOB_STATE_"):] if word.startswith("JOB_STATE_") else word


def _number(v: Any) -> Optional[float]:
    if isinstance(v, bool) or v is None:
        return None
    if isinstance(v, (int, float)):
        return float(v)
    try:
        return float(v)
    except (TypeError, ValueError):
        return None


def sub_job_gpus(sub: Dict[str, Any]) -> float:
    """GPUs of one sub-job: a count on the sub-job itself, else inside one of its config blocks, else 0."""
    for holder in (sub, *(sub.get(k) for k in CONFIG_HOLDERS)):
        if isinstance(holder, dict):
            for key in GPU_KEYS:
                n = _number(holder.get(key))
                if n is not None:
                    return n
    return 0.0


def _sub_jobs(job: Dict[str, Any]) -> List[dict]:
    body = job.get("body") if isinstance(job.get("body"), dict) else job
    for key in ("sub_jobs", "sub_job_configs"):
        subs = body.get(key)
        if isinstance(subs, list):
            return [s for s in subs if isinstance(s, dict)]
    return []


def job_gpus(job: Dict[str, Any]) -> float:
    subs = _sub_jobs(job)
    if subs:
        return sum(sub_job_gpus(s) for s in subs)
    return _number(job.get("n_gpus")) or 0.0


def _fmt(n: float) -> str:
    return str(int(n)) if float(n).is_integer() else f"{n:g}"


def sub_job_summary(job: Dict[str, Any]) -> str:
    parts = []
    for s in _sub_jobs(job):
        kind = str(s.get("sub_job_type") or s.get("job_type") or "?")
        tp = None
        for holder in (s.get("vllm_config"), s.get("inference_config")):
            if isinstance(holder, dict) and _number(holder.get("tensor_parallel_size")):
                tp = _number(holder["tensor_parallel_size"])
        parts.append(f"{kind} x{_fmt(sub_job_gpus(s))}" + (f" (tp {_fmt(tp)})" if tp and tp > 1 else ""))
    return " + ".join(parts) or "-"


def load_jobs(raw: str) -> List[dict]:
    """Accepts what ``dss-neutrino list`` / ``jobs list`` print: ``{"jobs": [...]}`` or a bare list."""
    obj = json.loads(raw)
    if isinstance(obj, dict):
        obj = obj.get("jobs", [])
    if not isinstance(obj, list):
        raise ValueError("expected a list of jobs or {\"jobs\": [...]}")
    return [j for j in obj if isinstance(j, dict)]


def render(jobs: Iterable[dict], capacity: Optional[dict] = None, now: Optional[str] = None) -> str:
    jobs = list(jobs)
    lines = [f"cluster status {now or time.strftime('%Y-%m-%d %H:%M:%S')}"]
    for state in WATCHED:
        rows: List[Tuple[str, str, str, str]] = []
        total = 0.0
        for j in jobs:
            if normalize_status(j.get("status")) != state:
                continue
            n = job_gpus(j)
            total += n
            name = str(j.get("name") or (j.get("body") or {}).get("name") or "")
            rows.append((str(j.get("job_id", "?")), name, _fmt(n), sub_job_summary(j)))
        if not rows and state != "RUNNING":
            continue
        lines.append("")
        lines.append(f"{state}: {len(rows)} job(s), {_fmt(total)} GPU(s)")
        if rows:
            w = [max(len(r[i]) for r in rows + [("job", "name", "gpus", "")]) for i in range(3)]
            lines.append(f"  {'job'.ljust(w[0])}  {'name'.ljust(w[1])}  {'gpus'.rjust(w[2])}  sub-jobs")
            for r in rows:
                lines.append(f"  {r[0].ljust(w[0])}  {r[1].ljust(w[1])}  {r[2].rjust(w[2])}  {r[3]}")
    if capacity:
        free = next((capacity[k] for k in ("free_gpus", "available_gpus") if k in capacity), None)
        total_cap = next((capacity[k] for k in ("total_gpus", "capacity_gpus") if k in capacity), None)
        if free is not None:
            lines += ["", f"free: {free} GPU(s)" + (f" of {total_cap}" if total_cap is not None else "")]
    return "\n".join(lines) + "\n"


def main(argv: Optional[List[str]] = None, session=None, out=sys.stdout, stdin=sys.stdin, sleep=time.sleep,
         max_refreshes: Optional[int] = None) -> int:
    ap = argparse.ArgumentParser(prog="cluster-status", description=__doc__.splitlines()[0])
    ap.add_argument("--url")
    ap.add_argument("--config")
    ap.add_argument("--jobs-json", help="read the job list from this file ('-' = stdin) instead of the service")
    ap.add_argument("--interval", type=float, default=10.0)
    ap.add_argument("--once", action="store_true")
    args = ap.parse_args(argv)
    client = None
    if not args.jobs_json:
        from .dss_client.dss_neutrino_cli import _client
        client = _client(args, session)
    n = 0
    while True:
        if client is None:
            raw = stdin.read() if args.jobs_json == "-" else open(args.jobs_json, encoding="utf-8").read()
            jobs, cap = load_jobs(raw), None
        else:
            jobs = client.list_jobs()
            try:
                cap = client.get_capacity()
            except Exception:
                cap = None                              # an optional endpoint: the tables are still worth showing
        text = render(jobs, cap)
        n += 1
        if args.once or client is None:
            out.write(text)
            return 0
        out.write("\x1b[2J\x1b[H" + text if getattr(out, "isatty", lambda: False)() else text)
        out.flush()
        if max_refreshes is not None and n >= max_refreshes:
            return 0
        sleep(args.interval)


if __name__ == "__main__":
    raise SystemExit(main())
