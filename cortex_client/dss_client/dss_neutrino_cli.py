"""``dss-neutrino``: command line over :class:`NeutrinoClient`.

    dss-neutrino --url http://host:port jobs list [--status RUNNING]
    dss-neutrino jobs get|cancel|wait JOB
    dss-neutrino jobs create --model qwen3-4b --training-gpus 8 --sampling-gpus 8
    dss-neutrino logs JOB [--follow]            # plain-text tail with an on-disk cursor cache
    dss-neutrino tui jobs | tui logs JOB [-f]   # the log viewer (cached entries + cursor, filters)
    dss-neutrino tui app                        # full-screen job browser and log viewer
    dss-neutrino login | logout | whoami        # connection settings kept in a 0600 file
    dss-neutrino step JOB [--lr 1e-6] | save JOB [--path P] | sync JOB | capacity
    dss-neutrino submit job.json|- [--job-id ID] [--dry-run] [--wait]      # a whole create-job body
    dss-neutrino list [--status S]                                         # oldest first, newest at the prompt
    dss-neutrino checkpoints JOB [--export ID | --delete ID]
    dss-neutrino --job JOB fwd-bwd batch.json | generate request.json      # JSON descriptions, see batch_spec.py
    dss-neutrino --job JOB load CKPT [--source-job-id J] [--target-sub-job-id S] [--no-poll]
    dss-neutrino --job JOB weight-sync [--source-sub-job-id S] [--target-sub-job-id T ...] [--weight-format F]
    dss-neutrino download-log JOB [-o DIR]                                 # one file per sub-job log
    dss-neutrino --config conn.json ... | login --config conn.json         # connection settings from a JSON file

Failures of a command (bad JSON, a refused request, an unreadable file) print ``error: ...`` on stderr and return 1.

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


CONFIG_KEYS = {"url", "host", "pat", "database", "schema", "endpoint", "poll_interval", "request_timeout", "verify_ssl"}
CONFIG_ALIASES = {"base_url": "url", "db": "database", "poll_timeout": "request_timeout"}


def load_connection_config(path: str) -> dict:
    """A JSON object (optionally under ``"connection"``) with ``url`` *or* ``host`` + ``pat`` + ``database``
    (+ ``schema``, default ``PUBLIC``), and optionally ``endpoint``, ``poll_interval``, ``request_timeout``,
    ``verify_ssl`` / ``no_verify_ssl``.  ``base_url``, ``db`` and ``poll_timeout`` are accepted spellings; any other
    key is an error (a typo must not silently fall back to a default)."""
    try:
        raw = json.loads(Path(path).expanduser().read_text(encoding="utf-8"))
    except ValueError as exc:
        raise ValueError(f"invalid JSON in config {path}: {exc}") from exc
    if isinstance(raw, dict) and isinstance(raw.get("connection"), dict):
        raw = raw["connection"]
    if not isinstance(raw, dict):
        raise ValueError(f"config {path} must be a JSON object")
    out, unknown = {}, []
    for k, v in raw.items():
        if k == "no_verify_ssl":
            k, v = "verify_ssl", (not v if isinstance(v, bool) else v)
        k = CONFIG_ALIASES.get(k, k)
        if k not in CONFIG_KEYS:
            unknown.append(k)
        else:
            out[k] = v
    if unknown:
        raise ValueError(f"unknown config key(s): {', '.join(sorted(unknown))}")
    for k in ("url", "host", "pat", "database", "schema", "endpoint"):
        if out.get(k) is not None and not isinstance(out[k], str):
            raise ValueError(f"config {k} must be a string")
    for k in ("poll_interval", "request_timeout"):
        if out.get(k) is not None and (isinstance(out[k], bool) or not isinstance(out[k], (int, float))):
            raise ValueError(f"config {k} must be a number")
    if out.get("verify_ssl") is not None and not isinstance(out["verify_ssl"], bool):
        raise ValueError("config verify_ssl must be true or false")
    if not (out.get("url") or (out.get("host") and out.get("pat") and out.get("database"))):
        raise ValueError(f"config {path} needs url, or host + pat + database")
    return out


def _client_from_config(cfg: dict, session=None) -> NeutrinoClient:
    kw = {k: float(cfg[k]) for k in ("poll_interval", "request_timeout") if cfg.get(k) is not None}
    if cfg.get("url"):
        c = NeutrinoClient(cfg["url"], session=session, **kw)
    else:
        host = cfg["host"].split("://", 1)[-1].rstrip("/")
        c = NeutrinoClient.from_pat(host, cfg["database"], cfg.get("schema") or "PUBLIC", cfg["pat"],
                                    endpoint=cfg.get("endpoint") or "cortex-training", session=session, **kw)
    if cfg.get("verify_ssl") is False and hasattr(c.session, "verify"):
        c.session.verify = False
    return c


def _client(args, session=None) -> NeutrinoClient:
    """Connection settings, first match wins: ``--config``, ``--url``, ``$DSS_URL``, the four ``DSS_*`` variables, the
    stored login (which may itself point at a config file)."""
    cfg_path = getattr(args, "config", None) or os.environ.get("DSS_CONFIG")
    if cfg_path:
        return _client_from_config(load_connection_config(cfg_path), session)
    url = getattr(args, "url", None) or os.environ.get("DSS_URL")
    if url:
        return NeutrinoClient(url, session=session)
    need = {k: os.environ.get(k) for k in ("DSS_HOST", "DSS_DATABASE", "DSS_SCHEMA", "DSS_PAT")}
    if all(need.values()):
        return NeutrinoClient.from_pat(need["DSS_HOST"], need["DSS_DATABASE"], need["DSS_SCHEMA"], need["DSS_PAT"], session=session)
    st = load_login()
    if st.get("config_path"):
        return _client_from_config(load_connection_config(st["config_path"]), session)
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


def read_json_object(path: str, stdin=sys.stdin) -> dict:
    raw = stdin.read() if path == "-" else Path(path).expanduser().read_text(encoding="utf-8")
    try:
        obj = json.loads(raw)
    except ValueError as exc:
        raise ValueError(f"invalid JSON in {path}: {exc}") from exc
    if not isinstance(obj, dict):
        raise ValueError(f"{path}: expected a JSON object")
    return obj


def jobs_oldest_first(jobs: List[dict]) -> List[dict]:
    """Sorted by ``created_at`` (ISO 8601, ``Z`` accepted) so the newest job is the last line printed; jobs without
    a readable timestamp keep their relative order at the end.  Without any timestamp the service's newest-first
    order is simply reversed."""
    from datetime import datetime, timezone

    def stamp(job) -> Optional[float]:
        raw = str(job.get("created_at") or "").strip() if isinstance(job, dict) else ""
        if not raw:
            return None
        try:
            t = datetime.fromisoformat(raw[:-1] + "+00:00" if raw.endswith("Z") else raw)
        except ValueError:
            return None
        return (t if t.tzinfo else t.replace(tzinfo=timezone.utc)).timestamp()

    stamps = [stamp(j) for j in jobs]
    if not any(s is not None for s in stamps):
        return list(reversed(jobs))
    order = sorted(range(len(jobs)), key=lambda i: (stamps[i] is None, stamps[i] or 0.0, i))
    return [jobs[i] for i in order]


def _need_job(args, what: str) -> str:
    if not getattr(args, "job", None):
        raise ValueError(f"{what} needs --job JOB_ID")
    return args.job


def _cmd_submit(args, client_of, show, stdin) -> None:
    body = read_json_object(args.json_file, stdin)
    subs = body.get("sub_jobs", body.get("sub_job_configs"))
    if not isinstance(subs, list) or not subs:
        raise ValueError("the job JSON needs a non-empty sub_jobs list")
    if args.job_id is not None:
        body = {**body, "job_id": args.job_id}
    if args.dry_run:
        show(body)
        return
    c = client_of()
    resp = c.create_job_from_body(body)
    if args.wait:
        jid = (resp.get("job_id") if isinstance(resp, dict) else None) or body.get("job_id")
        if not jid:
            raise ValueError("submit --wait: the service's reply carries no job_id")
        resp = c.wait_for_job(str(jid))
    show(resp)


def _poll_flag(spec: dict, what: str) -> bool:
    poll = spec.get("poll", True)
    if not isinstance(poll, bool):
        raise ValueError(f"{what}: poll must be true or false")
    return poll


def _cmd_fwd_bwd(args, c, show, stdin) -> None:
    from .batch_spec import build_forward_backward_kwargs
    job = _need_job(args, "fwd-bwd")
    spec = read_json_object(args.json_file, stdin)
    poll = _poll_flag(spec, "fwd-bwd")
    body = spec.get("payload", spec)
    if not isinstance(body, dict):
        raise ValueError("fwd-bwd: payload must be an object")
    batch = build_forward_backward_kwargs(body)
    res = c.forward_backward(job, batch, body.get("meta"), body.get("processing"), wait=poll)
    n_bytes = sum(v.numel() * v.element_size() for v in batch.values() if hasattr(v, "numel"))
    show({"job_id": job, "tensor_bytes": n_bytes, **({"result": res} if poll else {"request_id": res})})


def _cmd_generate(args, c, show, stdin) -> None:
    job = _need_job(args, "generate")
    spec = read_json_object(args.json_file, stdin)
    poll = _poll_flag(spec, "generate")
    body = spec.get("payload", spec)
    if not isinstance(body, dict):
        raise ValueError("generate: payload must be an object")
    prompts = body.get("prompts")
    if not isinstance(prompts, list) or not prompts or not all(isinstance(p, list) for p in prompts):
        raise ValueError("generate: prompts must be a non-empty list of token-id lists")
    sp = body.get("sampling_params")
    if sp is not None and not isinstance(sp, dict):
        raise ValueError("generate: sampling_params must be an object")
    strict = body.get("strict")
    if strict is not None and not isinstance(strict, bool):
        raise ValueError("generate: strict must be true or false")
    res = c.generate(job, prompts, sp, routing_key=body.get("routing_key"), strict=strict, wait=poll,
                     validate_lengths=True)
    show({"job_id": job, "prompt_count": len(prompts), **({"result": res} if poll else {"request_id": res})})


def _cmd_download_log(args, c, show) -> None:
    root = Path(args.output_dir).expanduser() if args.output_dir else Path.cwd()
    saved = []
    for i, rec in enumerate(c.fetch_execution_logs(args.job_id)):
        sub = str(rec.get("sub_job_id") or "unknown").replace("/", "_").replace(":", "_")
        name = os.path.basename(str(rec.get("filename") or f"log-{i}.txt")) or f"log-{i}.txt"
        text = rec.get("content")
        if text is None:                                       # line records instead of whole files
            text = f"{rec.get('ts', '')} [{rec.get('level', 'INFO')}] {rec.get('message', '')}\n"
            name = "execution.log"
        dest = root / sub / name
        dest.parent.mkdir(parents=True, exist_ok=True)
        with open(dest, "a" if rec.get("content") is None else "w", encoding="utf-8") as f:
            f.write(text)
        if not saved or saved[-1]["saved_path"] != str(dest):
            saved.append({"sub_job_id": rec.get("sub_job_id"), "filename": name, "saved_path": str(dest)})
    show({"job_id": args.job_id, "logs": saved})


def main(argv: Optional[List[str]] = None, session=None, out=sys.stdout, err=sys.stderr, stdin=sys.stdin) -> int:
    from .neutrino_client import NeutrinoError
    try:
        return _main(argv, session, out, stdin)
    except (ValueError, OSError, NeutrinoError) as exc:
        err.write(f"error: {exc}\n")
        return 1


def _main(argv, session, out, stdin) -> int:
    ap = argparse.ArgumentParser(prog="dss-neutrino")
    ap.add_argument("--url")
    ap.add_argument("--config", help="connection settings as a JSON file (also $DSS_CONFIG)")
    ap.add_argument("--compact", action="store_true", help="one-line JSON output")
    ap.add_argument("--job", "--job-id", dest="job", help="job id for fwd-bwd / generate / load / weight-sync")
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
    li.add_argument("--config", dest="login_config", help="remember this connection file instead of the settings")
    sm = sub.add_parser("submit")
    sm.add_argument("json_file")
    sm.add_argument("--job-id")
    sm.add_argument("--dry-run", action="store_true")
    sm.add_argument("--wait", action="store_true")
    sub.add_parser("list").add_argument("--status")
    ck = sub.add_parser("checkpoints")
    ck.add_argument("job_id")
    ck.add_argument("--export")
    ck.add_argument("--delete")
    sub.add_parser("fwd-bwd").add_argument("json_file")
    sub.add_parser("generate").add_argument("json_file")
    ld = sub.add_parser("load")
    ld.add_argument("checkpoint_id")
    ld.add_argument("--source-job-id")
    ld.add_argument("--target-sub-job-id")
    ld.add_argument("--no-poll", action="store_true")
    ws = sub.add_parser("weight-sync")
    ws.add_argument("--source-sub-job-id")
    ws.add_argument("--target-sub-job-id", dest="target_sub_job_ids", action="append")
    ws.add_argument("--weight-format")
    ws.add_argument("--no-poll", action="store_true")
    dl = sub.add_parser("download-log")
    dl.add_argument("job_id")
    dl.add_argument("-o", "--output-dir")
    sub.add_parser("logout")
    sub.add_parser("whoami")
    tu = sub.add_parser("tui")
    tu.add_argument("rest", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    show = lambda obj: out.write((json.dumps(obj, separators=(",", ":"), sort_keys=True, default=str) if args.compact
                                  else json.dumps(obj, indent=1, default=str)) + "\n")
    if args.cmd == "login" and args.login_config:
        load_connection_config(args.login_config)                       # refuse to remember a file that does not load
        saved = str(Path(args.login_config).expanduser().resolve())
        save_login({"config_path": saved})
        show({"config_path": saved, "logged_in": True})
        return 0
    if args.cmd == "submit" and args.dry_run:
        _cmd_submit(args, None, show, stdin)
        return 0
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
    if args.cmd == "submit":
        _cmd_submit(args, lambda: c, show, stdin)
    elif args.cmd == "list":
        show({"jobs": jobs_oldest_first(c.list_jobs(args.status))})
    elif args.cmd == "checkpoints":
        if args.export:
            show(c.export_checkpoint(args.job_id, args.export))
        elif args.delete:
            c.delete_checkpoint(args.job_id, args.delete)
            show({"deleted": args.delete, "job_id": args.job_id})
        else:
            show({"checkpoints": c.list_checkpoints(args.job_id)})
    elif args.cmd == "fwd-bwd":
        _cmd_fwd_bwd(args, c, show, stdin)
    elif args.cmd == "generate":
        _cmd_generate(args, c, show, stdin)
    elif args.cmd == "load":
        job = _need_job(args, "load")
        res = c.load(job, checkpoint_id=args.checkpoint_id, source_job_id=args.source_job_id,
                     target_sub_job_id=args.target_sub_job_id, wait=not args.no_poll)
        reply = {"job_id": job, "checkpoint_id": args.checkpoint_id}
        for k in ("source_job_id", "target_sub_job_id"):
            if getattr(args, k) is not None:
                reply[k] = getattr(args, k)
        show({**reply, **({"request_id": res} if args.no_poll else {"result": res})})
    elif args.cmd == "weight-sync":
        job = _need_job(args, "weight-sync")
        src = args.source_sub_job_id or f"{job}:training:0"
        dst = args.target_sub_job_ids or [f"{job}:sampling:0"]
        res = c.weight_sync(job, src, dst, args.weight_format, wait=not args.no_poll)
        reply = {"job_id": job, "source_sub_job_id": src, "target_sub_job_ids": dst}
        if args.weight_format:
            reply["weight_format"] = args.weight_format
        show({**reply, **({"request_id": res} if args.no_poll else {"result": res})})
    elif args.cmd == "download-log":
        _cmd_download_log(args, c, show)
    elif args.cmd == "jobs":
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
