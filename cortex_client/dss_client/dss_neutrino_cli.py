"""``dss-neutrino``: command line over :class:`NeutrinoClient`.

    dss-neutrino --url http://host:port jobs list [--status RUNNING]
    dss-neutrino jobs get|cancel|wait JOB
    dss-neutrino jobs create --model qwen3-4b --training-gpus 8 --sampling-gpus 8
    dss-neutrino logs JOB [--follow]            # plain-text tail with an on-disk cursor cache
    dss-neutrino tui jobs | tui logs JOB [-f]   # the log viewer (cached entries + cursor, filters)
    dss-neutrino login | logout | whoami        # connection settings kept in a 0600 file
    dss-neutrino step JOB [--lr 1e-6] | save JOB [--path P] | sync JOB | capacity

Connection comes from ``--url`` or ``DSS_URL``; PAT auth from ``DSS_HOST`` / ``DSS_DATABASE`` / ``DSS_SCHEMA`` /
``DSS_PAT``.  Counterpart of cortex-client/dss_client/dss_neutrino_cli.py and its TUI log viewer (a terminal UI
toolkit is not a dependency here; ``logs --follow`` prints new lines as they arrive)."""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import List, Optional

from .neutrino_client import NeutrinoClient, SubJobConfig


def login_state_path() -> Path:
    """``$DSS_CONFIG_DIR/login.json``, else ``$XDG_CONFIG_HOME/dss-neutrino/login.json``, else under ``~/.config``."""
    root = os.environ.get("DSS_CONFIG_DIR")
    if root:
        return Path(root) / "login.json"
    xdg = os.environ.get("XDG_CONFIG_HOME")
    return (Path(xdg) if xdg else Path.home() / ".config") / "dss-neutrino" / "login.json"


def save_login(state: dict) -> Path:
    """Stores the connection settings for later invocations; the file is readable by its owner only."""
    p = login_state_path()
    p.parent.mkdir(parents=True, exist_ok=True)
    fd = os.open(p, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
    with os.fdopen(fd, "w") as f:
        json.dump(state, f)
    os.chmod(p, 0o600)
    return p


def load_login() -> dict:
    try:
        return json.loads(login_state_path().read_text())
    except (OSError, ValueError):
        return {}


def _client(args, session=None) -> NeutrinoClient:
    """Connection settings, first match wins: ``--url``, ``$DSS_URL``, the four ``DSS_*`` variables, the stored
    login."""
    url = getattr(args, "url", None) or os.environ.get("DSS_URL")
    if url:
        return NeutrinoClient(url, session=session)
    need = {k: os.environ.get(k) for k in ("DSS_HOST", "DSS_DATABASE", "DSS_SCHEMA", "DSS_PAT")}
    if all(need.values()):
        return NeutrinoClient.from_pat(need["DSS_HOST"], need["DSS_DATABASE"], need["DSS_SCHEMA"], need["DSS_PAT"], session=session)
    st = load_login()
    if st.get("url"):
        return NeutrinoClient(st["url"], session=session)
    if all(st.get(k) for k in ("host", "database", "schema", "pat")):
        return NeutrinoClient.from_pat(st["host"], st["database"], st["schema"], st["pat"], session=session)
    raise SystemExit("set --url / DSS_URL, or DSS_HOST + DSS_DATABASE + DSS_SCHEMA + DSS_PAT, or run `dss-neutrino login`")


def _log_cache(job_id: str) -> Path:
    root = Path(os.environ.get("DSS_CACHE_DIR", Path.home() / ".cache" / "dss-neutrino"))
    root.mkdir(parents=True, exist_ok=True)
    return root / f"{job_id}.cursor"


def tail_logs(client: NeutrinoClient, job_id: str, follow: bool, out=sys.stdout, sleep=time.sleep, max_polls: Optional[int] = None) -> int:
    cache = _log_cache(job_id)
    cursor = int(cache.read_text()) if cache.exists() else 0
    polls = 0
    while True:
        logs = client.fetch_execution_logs(job_id, cursor)
        for rec in logs:
            out.write(f"{rec.get('ts', '')} [{rec.get('level', 'INFO')}] {rec.get('message', '')}\n")
        cursor += len(logs)
        cache.write_text(str(cursor))
        polls += 1
        if not follow or (max_polls is not None and polls >= max_polls):
            return cursor
        if not logs:
            sleep(2.0)


def main(argv: Optional[List[str]] = None, session=None, out=sys.stdout) -> int:
    ap = argparse.ArgumentParser(prog="dss-neutrino")
    ap.add_argument("--url")
    sub = ap.add_subparsers(dest="cmd", required=True)
    jobs = sub.add_parser("jobs").add_subparsers(dest="jcmd", required=True)
    jl = jobs.add_parser("list")
    jl.add_argument("--status")
    for name in ("get", "cancel", "wait"):
        jobs.add_parser(name).add_argument("job")
    jc = jobs.add_parser("create")
    jc.add_argument("--model", required=True)
    jc.add_argument("--training-gpus", type=int, default=0)
    jc.add_argument("--sampling-gpus", type=int, default=0)
    jc.add_argument("--tp", type=int, default=1)
    jc.add_argument("--name")
    lg = sub.add_parser("logs")
    lg.add_argument("job")
    lg.add_argument("--follow", action="store_true")
    st = sub.add_parser("step")
    st.add_argument("job")
    st.add_argument("--lr", type=float)
    sv = sub.add_parser("save")
    sv.add_argument("job")
    sv.add_argument("--path")
    sub.add_parser("sync").add_argument("job")
    sub.add_parser("capacity")
    li = sub.add_parser("login")
    for name in ("--host", "--database", "--schema", "--pat", "--service-url"):
        li.add_argument(name)
    sub.add_parser("logout")
    sub.add_parser("whoami")
    tu = sub.add_parser("tui")
    tu.add_argument("rest", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    if args.cmd == "login":
        state = {"url": args.service_url} if args.service_url else \
            {"host": args.host, "database": args.database, "schema": args.schema, "pat": args.pat or os.environ.get("DSS_PAT")}
        if not (state.get("url") or all(state.values())):
            raise SystemExit("login needs --service-url, or --host --database --schema and a token (--pat or $DSS_PAT)")
        out.write(f"saved {save_login(state)}\n")
        return 0
    if args.cmd == "logout":
        p = login_state_path()
        if p.exists():
            p.unlink()
        out.write("logged out\n")
        return 0
    if args.cmd == "whoami":
        st = load_login()
        out.write(json.dumps({k: ("***" if k == "pat" and v else v) for k, v in st.items()} or {"login": None}) + "\n")
        return 0
    c = _client(args, session)
    if args.cmd == "tui":
        from .tui.__main__ import main as tui_main
        return tui_main(["--no-color", *args.rest] if not getattr(out, "isatty", lambda: False)() else list(args.rest),
                        client=c, out=out)
    show = lambda obj: out.write(json.dumps(obj, indent=1, default=str) + "\n")
    if args.cmd == "jobs":
        if args.jcmd == "list":
            show(c.list_jobs(args.status))
        elif args.jcmd == "get":
            show(c.get_job(args.job))
        elif args.jcmd == "cancel":
            c.cancel_job(args.job)
            show({"cancelled": args.job})
        elif args.jcmd == "wait":
            show(c.wait_for_job(args.job))
        else:
            subs = []
            if args.training_gpus:
                subs.append(SubJobConfig.training_job(args.model, num_gpus=args.training_gpus))
            if args.sampling_gpus:
                subs.append(SubJobConfig.sampling_job(args.model, num_gpus=args.sampling_gpus, tensor_parallel_size=args.tp))
            show(c.create_job(subs, name=args.name))
    elif args.cmd == "logs":
        tail_logs(c, args.job, args.follow, out)
    elif args.cmd == "step":
        show(c.step(args.job, args.lr))
    elif args.cmd == "save":
        show(c.save(args.job, args.path))
    elif args.cmd == "sync":
        show(c.weight_sync(args.job))
    elif args.cmd == "capacity":
        show(c.get_capacity())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
