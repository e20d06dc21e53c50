"""Ray bring-up against a fake ``ray`` module and recorded subprocess calls: attach only to clusters with GPUs, start
a private head otherwise, fan out to the hostfile's peers, and stop nothing but the cluster this process started."""
import sys
import types

import pytest

from arctic_platform_b200.common import ray_cluster as rc


class FakeRay(types.ModuleType):
    def __init__(self, gpus_on_auto):
        super().__init__("ray")
        self.gpus_on_auto, self.inited, self.calls = gpus_on_auto, None, []

    def is_initialized(self):
        return self.inited is not None

    def init(self, address=None, ignore_reinit_error=False):
        if address == "auto" and self.gpus_on_auto is None:
            raise ConnectionError("no cluster")
        self.inited = address
        self.calls.append(("init", address))

    def shutdown(self):
        self.calls.append(("shutdown", self.inited))
        self.inited = None

    def cluster_resources(self):
        return {"GPU": self.gpus_on_auto or 0, "CPU": 8}


@pytest.fixture
def recorded(monkeypatch):
    runs = []

    def run(cmd, **kw):
        runs.append((list(cmd) if not isinstance(cmd, str) else cmd, kw))
        return types.SimpleNamespace(returncode=0, stdout=b"", stderr=b"")
    monkeypatch.setattr(rc.subprocess, "run", run)
    monkeypatch.setattr(rc.atexit, "register", lambda fn: runs.append(("atexit", fn.__name__)))
    monkeypatch.setattr(rc, "primary_ip", lambda: "10.0.0.1")
    rc._started["temp_dir"] = None
    yield runs
    rc._started["temp_dir"] = None


def test_without_ray_the_platform_falls_back(monkeypatch):
    monkeypatch.setitem(sys.modules, "ray", None)                   # import ray -> ImportError
    assert rc.ray_available() is False
    assert rc.init_ray_cluster() == {"ray": False, "reason": "ray is not installed; using local actors"}


def test_attaches_only_to_a_cluster_with_gpus(monkeypatch, recorded):
    ray = FakeRay(gpus_on_auto=8)
    monkeypatch.setitem(sys.modules, "ray", ray)
    assert rc.init_ray_cluster() == {"ray": True, "attached": True}
    assert not [c for c in recorded if isinstance(c[0], list)] and ray.inited == "auto"
    assert rc.init_ray_cluster() == {"ray": True, "attached": True}         # already initialised: nothing to do


def test_starts_a_private_head_and_fans_out(monkeypatch, recorded, tmp_path):
    ray = FakeRay(gpus_on_auto=0)                                             # a CPU-only cluster is around: not ours
    monkeypatch.setitem(sys.modules, "ray", ray)
    hostfile = tmp_path / "hostfile"
    hostfile.write_text("# nodes\nnode-a slots=8\n10.0.0.1 slots=8\n\nnode-b slots=8\n")
    real_read = rc.read_hostfile
    monkeypatch.setattr(rc, "read_hostfile", lambda path=str(hostfile): real_read(path))
    monkeypatch.setattr(rc.shutil, "which", lambda name: "/usr/bin/pdsh" if name == "pdsh" else None)
    monkeypatch.setenv("ARL_RAY_TEMP_DIR", str(tmp_path / "ray-tmp"))
    monkeypatch.setenv("RAY_PORT", "6400")
    monkeypatch.setenv("ARL_RAY_MIN_WORKER_PORT", "20000")
    monkeypatch.setenv("ARL_RAY_MAX_WORKER_PORT", "20100")
    out = rc.init_ray_cluster()
    assert out["attached"] is False and out["address"] == "10.0.0.1:6400" and out["peers"] == ["node-a", "node-b"]
    head = [c[0] for c in recorded if isinstance(c[0], list)][0]
    assert head[:3] == ["ray", "start", "--head"] and "--port=6400" in head and f"--temp-dir={tmp_path / 'ray-tmp'}" in head
    assert "--min-worker-port=20000" in head and "--max-worker-port=20100" in head
    assert ("atexit", "shutdown_own_cluster") in recorded
    pdsh = [c for c in recorded if isinstance(c[0], list) and c[0][0] == "pdsh"][0][0]
    assert pdsh == ["pdsh", "-w", "node-a,node-b", "ray start --address=10.0.0.1:6400"]
    assert ("shutdown", "auto") in ray.calls and ray.inited == "10.0.0.1:6400"
    assert rc._started["temp_dir"] == str(tmp_path / "ray-tmp")
    assert rc.read_hostfile(str(tmp_path / "missing")) == []


def test_shutdown_stops_only_the_own_cluster(monkeypatch, recorded):
    import psutil
    ended = []

    class P:
        def __init__(self, pid, cmd):
            self.info = {"pid": pid, "cmdline": cmd}
            self.pid = pid

        def terminate(self):
            ended.append(("term", self.pid))

        def kill(self):
            ended.append(("kill", self.pid))
    procs = {11: P(11, ["raylet", "--temp-dir=/tmp/arl-ray-abc123/session"]),
             12: P(12, ["gcs_server", "--log-dir=/tmp/arl-ray-abc123/logs"]),
             13: P(13, ["raylet", "--temp-dir=/tmp/arl-ray-other/session"]),          # somebody else's cluster
             14: P(14, ["python", "train.py"])}
    monkeypatch.setattr(psutil, "process_iter", lambda attrs=None: list(procs.values()))
    monkeypatch.setattr(psutil, "Process", lambda pid: procs[pid])
    monkeypatch.setattr(psutil, "wait_procs", lambda ps, timeout=None: ([p for p in ps if p.pid == 11], [p for p in ps if p.pid == 12]))
    monkeypatch.setitem(sys.modules, "ray", FakeRay(gpus_on_auto=None))
    assert rc.own_cluster_pids("/tmp/arl-ray-abc123") == [11, 12]
    rc.shutdown_own_cluster()                                            # nothing was started by this process
    assert ended == []
    rc._started["temp_dir"] = "/tmp/arl-ray-abc123"
    rc.shutdown_own_cluster()
    assert ended == [("term", 11), ("term", 12), ("kill", 12)] and rc._started["temp_dir"] is None
    assert not [c for c in recorded if isinstance(c[0], list) and c[0][:2] == ["ray", "stop"]]     # no machine-wide stop
