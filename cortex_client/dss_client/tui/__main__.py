"""``python -m dss_client.tui [app | jobs | logs JOB]``: the full-screen browser, or plain output: list jobs, view /
follow one job's log through the cache."""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional

from .viewer import LogViewer


def main(argv: Optional[List[str]] = None, client=None, out=None) -> int:
    ap = argparse.ArgumentParser(prog="neutrino-tui")
    ap.add_argument("--url")
    ap.add_argument("--config")
    ap.add_argument("--no-color", action="store_true")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("app")
    j = sub.add_parser("jobs")
    j.add_argument("--filter", default="")
    j.add_argument("--status")
    lg = sub.add_parser("logs")
    lg.add_argument("job")
    lg.add_argument("--follow", "-f", action="store_true")
    lg.add_argument("--level")
    lg.add_argument("--grep", default="")
    lg.add_argument("--tail", type=int)
    lg.add_argument("--clear-cache", action="store_true")
    args = ap.parse_args(argv)
    if client is None:
        from ..dss_neutrino_cli import _client
        client = _client(args)
    if args.cmd == "app":
        from .app import main as app_main
        return app_main(client)
    viewer = LogViewer(client, out=out, color=False if args.no_color else None)
    if args.cmd == "jobs":
        viewer.list_jobs(args.filter, args.status)
        return 0
    if args.clear_cache:
        from .log_cache import LogCache
        LogCache(args.job).clear()
    viewer.show(args.job, follow=args.follow, min_level=args.level, query=args.grep, tail=args.tail)
    return 0


if __name__ == "__main__":
    sys.exit(main())
