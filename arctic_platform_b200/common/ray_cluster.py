"""Ray cluster bring-up for the Ray protocol (arctic_platform/common/ray_cluster.py:88-270 in the reference).

``init_ray_cluster(auto_attach)`` attaches to a running Ray cluster only if it has GPUs; otherwise it starts a
head node on free ports with a private temp dir, fans ``ray start --address`` out to the peers listed in
``/job/hostfile`` (via ``pdsh`` when present) and registers an ``atexit`` hook that stops only the cluster it
started.  Ray is optional in this build: without it the function reports ``{"ray": False}`` and the clients
fall back to in-process / spawned actors.
"""
from __future__ import annotations

import atexit
import os
import shutil
import socket
import subprocess
import tempfile
import uuid
from typing import Dict, List, Optional

from ..rl.config import primary_ip  # noqa: F401  (re-exported for callers of the reference API)

_started: Dict[str, Optional[str]] = {"temp_dir": None}


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def read_hostfile(path: str = "/job/hostfile") -> List[str]:
    if not os.path.exists(path):
        return []
    hosts = []
    for line in open(path):
        line = line.strip()
        if line and not line.startswith("#"):
            hosts.append(line.split()[0])
    return hosts


def ray_available() -> bool:
    try:
        import ray  # noqa: F401
        return True
    except Exception:
        return False


def init_ray_cluster(auto_attach: bool = True) -> Dict[str, object]:
    if not ray_available():
        return {"ray": False, "reason": "ray is not installed; using local actors"}
    import ray
    if ray.is_initialized():
        return {"ray": True, "attached": True}
    if auto_attach:
        try:
            ray.init(address="auto", ignore_reinit_error=True)
            if ray.cluster_resources().get("GPU", 0) > 0:
                return {"ray": True, "attached": True}
            ray.shutdown()                       # a CPU-only cluster is not ours to use
        except Exception:
            pass
    temp_dir = os.environ.get("ARL_RAY_TEMP_DIR") or os.path.join(tempfile.gettempdir(), f"arl-ray-{uuid.uuid4().hex[:8]}")
    port = int(os.environ.get("RAY_PORT", 0)) or free_port()
    dash = int(os.environ.get("RAY_DASHBOARD_PORT", 0)) or free_port()
    cmd = head_start_command(port, dash, temp_dir)
    subprocess.run(cmd, check=True, capture_output=True)
    _started["temp_dir"] = temp_dir
    atexit.register(shutdown_own_cluster)
    head = f"{primary_ip()}:{port}"
    peers = [h for h in read_hostfile() if h not in (socket.gethostname(), primary_ip())]
    if peers and shutil.which("pdsh"):
        subprocess.run(["pdsh", "-w", ",".join(peers), f"ray start --address={head}"], check=False, capture_output=True)
    ray.init(address=head, ignore_reinit_error=True)
    return {"ray": True, "attached": False, "address": head, "temp_dir": temp_dir, "peers": peers}


def _worker_port_range() -> List[str]:
    lo, hi = os.environ.get("ARL_RAY_MIN_WORKER_PORT"), os.environ.get("ARL_RAY_MAX_WORKER_PORT")
    return [f"--min-worker-port={lo}", f"--max-worker-port={hi}"] if lo and hi else []


def head_start_command(port: int, dashboard_port: Optional[int] = None, temp_dir: Optional[str] = None,
                       num_gpus: Optional[int] = None) -> List[str]:
    """``ray start --head ...`` with this platform's conventions: a private temp dir (which is also how the cluster's
    processes are found again, see ``own_cluster_pids``) and the worker port range of ``ARL_RAY_MIN/MAX_WORKER_PORT``."""
    cmd = ["ray", "start", "--head", f"--port={port}"]
    if dashboard_port:
        cmd.append(f"--dashboard-port={dashboard_port}")
    if temp_dir:
        cmd.append(f"--temp-dir={temp_dir}")
    if num_gpus is not None:
        cmd.append(f"--num-gpus={num_gpus}")
    return cmd + _worker_port_range()


def worker_start_command(head_address: str, temp_dir: Optional[str] = None, num_gpus: Optional[int] = None) -> List[str]:
    cmd = ["ray", "start", f"--address={head_address}"]
    if temp_dir:
        cmd.append(f"--temp-dir={temp_dir}")
    if num_gpus is not None:
        cmd.append(f"--num-gpus={num_gpus}")
    return cmd + _worker_port_range()


def stop_cluster_by_temp_dir(temp_dir: str, grace_s: float = 5.0) -> int:
    """Ends the Ray processes that were started with ``--temp-dir=temp_dir`` on THIS machine (exact PIDs, terminate
    then kill) and nothing else.  Returns how many processes were found."""
    import psutil
    procs = []
    for pid in own_cluster_pids(temp_dir):
        try:
            p = psutil.Process(pid)
            p.terminate()
            procs.append(p)
        except psutil.Error:
            pass
    _gone, alive = psutil.wait_procs(procs, timeout=grace_s)
    for p in alive:
        try:
            p.kill()
        except psutil.Error:
            pass
    return len(procs)


def main(argv=None) -> int:
    """``python -m arctic_platform_b200.common.ray_cluster head|worker|stop``: print the start command of a node, or
    stop this node's part of the cluster named by ``--temp-dir`` (default ``$ARL_RAY_TEMP_DIR``)."""
    import argparse
    import shlex
    ap = argparse.ArgumentParser()
    ap.add_argument("role", choices=["head", "worker", "stop"])
    ap.add_argument("--port", type=int, default=6379)
    ap.add_argument("--head-address", default=None)
    ap.add_argument("--temp-dir", default=os.environ.get("ARL_RAY_TEMP_DIR"))
    ap.add_argument("--num-gpus", type=int, default=None)
    args = ap.parse_args(argv)
    if args.role == "stop":
        if not args.temp_dir:
            print("stop needs --temp-dir (or ARL_RAY_TEMP_DIR): only a cluster with a known temp dir is ours to stop")
            return 2
        print(stop_cluster_by_temp_dir(args.temp_dir))
        return 0
    if args.role == "worker" and not args.head_address:
        print("worker needs --head-address host:port")
        return 2
    cmd = head_start_command(args.port, None, args.temp_dir, args.num_gpus) if args.role == "head" else \
        worker_start_command(args.head_address, args.temp_dir, args.num_gpus)
    print(" ".join(shlex.quote(c) for c in cmd))
    return 0


def own_cluster_pids(temp_dir: str) -> List[int]:
    """Processes of the Ray cluster started with ``--temp-dir=temp_dir``: every Ray daemon carries that path on its
    command line, and the directory name is unique to this process, so nothing of another cluster matches."""
    import psutil
    key = os.path.basename(os.path.normpath(temp_dir))
    me = os.getpid()
    pids = []
    for proc in psutil.process_iter(["pid", "cmdline"]):
        try:
            cmd = " ".join(proc.info.get("cmdline") or [])
        except (psutil.NoSuchProcess, psutil.AccessDenied):
            continue
        if key and key in cmd and proc.info["pid"] != me:
            pids.append(int(proc.info["pid"]))
    return pids


def shutdown_own_cluster() -> None:
    """Stops the Ray cluster this process started -- identified by its private temp dir -- and nothing else: a
    machine-wide ``ray stop`` would take other users' clusters down with it."""
    temp_dir = _started.get("temp_dir")
    if not temp_dir:
        return
    try:
        import ray
        if ray.is_initialized():
            ray.shutdown()
    except Exception:
        pass
    try:
        import psutil
        procs = []
        for pid in own_cluster_pids(temp_dir):
            try:
                p = psutil.Process(pid)
                p.terminate()
                procs.append(p)
            except psutil.Error:
                pass
        _gone, alive = psutil.wait_procs(procs, timeout=5)
        for p in alive:
            try:
                p.kill()
            except psutil.Error:
                pass
    except ImportError:
        pass
    _started["temp_dir"] = None


if __name__ == "__main__":
    raise SystemExit(main())
