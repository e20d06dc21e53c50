"""Host-side failure handling: all-or-nothing initialisation, heartbeats, spawned actors that die or raise,
placement arithmetic.  No GPU involved; failures are injected with fake workers."""
import os
import time

import pytest

from arctic_platform_b200.common.local_actors import ActorDied, ActorError, SpawnedActor
from arctic_platform_b200.common.server import ArcticRLServerCore, JobError
from arctic_platform_b200.common.utils.ray_pg import (ColocatePlacement, gpu_fraction, pg_scheduling_options,
                                                      plan_colocate_placement)


class FakeWorker:
    created = []

    def __init__(self, fail_init=False):
        self.fail_init = fail_init
        self.killed = False
        self.calls = []
        FakeWorker.created.append(self)

    def call(self, method, *args, **kwargs):
        self.calls.append(method)
        if method == "initialize" and self.fail_init:
            raise RuntimeError("boom")
        if method == "step":
            return {"metrics": {"last_lr": 1e-5, "grad_norm": 1.0}, "batch": {}}
        return True

    def kill(self):
        self.killed = True


def test_initialize_is_all_or_nothing():
    FakeWorker.created = []
    core = ArcticRLServerCore(worker_factory=lambda cfg, r, n: FakeWorker(fail_init=(r == 2)))
    with pytest.raises(JobError) as e:
        core.initialize({"model_name": "m", "job_type": "training", "num_devices": 4})
    assert e.value.status == 500 and len(FakeWorker.created) == 4
    assert all(w.killed for w in FakeWorker.created)            # nothing of the failed job survives
    assert core.status()["jobs"] == []
    # a second attempt is not blocked by the failed one
    core2 = ArcticRLServerCore(worker_factory=lambda cfg, r, n: FakeWorker())
    info = core2.initialize({"model_name": "m", "job_type": "training", "num_devices": 2})
    assert info["status"] == "RUNNING" and info["num_devices"] == 2
    with pytest.raises(JobError) as e2:
        core2.initialize({"model_name": "m", "job_type": "training"})
    assert e2.value.status == 409
    with pytest.raises(JobError) as e3:
        core2.step(999)
    assert e3.value.status == 404
    with pytest.raises(JobError) as e4:
        core2.generate(info["job_id"], [[1]])
    assert e4.value.status == 400
    assert core2.step(info["job_id"])["metrics"]["grad_norm"] == 1.0
    core2.destroy(info["job_id"])
    assert all(w.killed for w in FakeWorker.created[-2:])


def test_missed_heartbeat_fails_the_job():
    core = ArcticRLServerCore(worker_factory=lambda cfg, r, n: FakeWorker(), heartbeat_timeout=0.05)
    info = core.initialize({"model_name": "m", "job_type": "training"})
    core.heartbeat(info["job_id"])
    assert core.step(info["job_id"])["job_id"] == info["job_id"]
    time.sleep(0.1)
    with pytest.raises(JobError) as e:
        core.step(info["job_id"])
    assert e.value.status == 409 and core.get_job_status(info["job_id"])["status"] == "FAILED"


class _Echo:
    def ping(self, x):
        return x + 1

    def pid(self):
        return os.getpid()

    def fail(self):
        raise ValueError("bad input")

    def die(self):
        os._exit(3)

    def env(self, k):
        return os.environ.get(k)


def _bad_factory():
    raise RuntimeError("cannot build")


def test_spawned_actor_rpc_errors_and_death():
    a = SpawnedActor(_Echo, env={"APB_TEST_VAR": "7"})
    try:
        assert a.call("ping", 41) == 42 and a.call("pid") != os.getpid() and a.call("env", "APB_TEST_VAR") == "7"
        assert a.heartbeat()
        with pytest.raises(ActorError, match="bad input"):
            a.call("fail")
        assert a.call("ping", 1) == 2                      # an exception does not kill the actor
        with pytest.raises(ActorDied):
            a.call("die", timeout=10)
        assert not a.heartbeat()
        with pytest.raises(ActorDied):
            a.call("ping", 1)
    finally:
        a.kill()
    with pytest.raises(ActorError, match="cannot build"):
        SpawnedActor(_bad_factory)


def test_placement_arithmetic():
    plan = plan_colocate_placement(12, 8)
    assert plan.gpus_per_node == [8, 4] and plan.total == 12
    assert plan.locate(0) == (0, 0) and plan.locate(7) == (0, 7) and plan.locate(8) == (1, 0)
    with pytest.raises(IndexError):
        plan.locate(12)
    assert plan.tp_layout(3, 4) == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11]]
    assert ColocatePlacement([8, 8]).tp_layout(2, 8) == [list(range(8)), list(range(8, 16))]
    # a TP-3 replica may not straddle the node boundary: bundles 6,7 stay unused on node 0
    assert ColocatePlacement([8, 8]).tp_layout(4, 3) == [[0, 1, 2], [3, 4, 5], [8, 9, 10], [11, 12, 13]]
    with pytest.raises(ValueError):
        ColocatePlacement([4]).tp_layout(2, 4)
    assert gpu_fraction("training", True) == 0.34 and gpu_fraction("sampling", False) == 1.0
    opts = pg_scheduling_options(plan, 9, "log_prob", True)
    assert opts["num_gpus"] == 0.33


def test_generate_routing_over_replicas():
    from arctic_platform_b200.common.server import route_prompts

    class Sampler:
        seen = []

        def __init__(self, rank):
            self.rank = rank

        def call(self, method, *args, **kwargs):
            if method == "generate":
                prompts, sp = args
                Sampler.seen.append((self.rank, [p[0] for p in prompts]))
                n = (sp or {}).get("n", 1)
                return [{"token_ids": [p[0] * 10 + s], "prompt_index": i, "rank": self.rank}
                        for i, p in enumerate(prompts) for s in range(n)]
            return True

        def kill(self):
            pass

    core = ArcticRLServerCore(worker_factory=lambda cfg, r, n: Sampler(r))
    job = core.initialize({"model_name": "m", "job_type": "sampling", "num_devices": 3})
    prompts = [[i] for i in range(7)]
    out = core.generate(job["job_id"], prompts, {"n": 2})["results"]
    assert [o["prompt_index"] for o in out] == [i for i in range(7) for _ in range(2)]
    assert [o["token_ids"][0] for o in out] == [i * 10 + s for i in range(7) for s in range(2)]
    assert [o["rank"] for o in out][::2] == [0, 0, 0, 1, 1, 1, 2]                     # contiguous slices
    assert route_prompts(prompts, 3, strict=True) == [0, 1, 2, 0, 1, 2, 0]
    keyed = route_prompts(prompts, 3, routing_key=["a", "b", "a", "c", "b", "a", "c"])
    assert keyed[0] == keyed[2] == keyed[5] and keyed[1] == keyed[4] and keyed[3] == keyed[6]
    assert route_prompts(prompts, 3, routing_key="same") == [route_prompts(prompts, 3, routing_key="same")[0]] * 7
    out2 = core.generate(job["job_id"], prompts, {"n": 1}, routing_key=["a", "b", "a", "c", "b", "a", "c"])["results"]
    assert [o["prompt_index"] for o in out2] == list(range(7)) and out2[0]["rank"] == out2[2]["rank"] == out2[5]["rank"]
    with pytest.raises(JobError):
        core.generate(job["job_id"], prompts, None, routing_key=[1, 2])


class _Initable(_Echo):
    def initialize(self, job_config):
        return True

    def destroy(self):
        return None


def test_watchdog_marks_a_job_failed_when_a_worker_process_is_gone():
    import time
    from arctic_platform_b200.common.local_actors import SpawnedActor
    core = ArcticRLServerCore(worker_factory=lambda cfg, r, n: SpawnedActor(_Initable))
    try:
        jid = core.initialize({"model_name": "x", "job_type": "training", "num_devices": 2})["job_id"]
        job = core.jobs[jid]
        assert core.check_workers(jid) == {"job_id": jid, "alive": [True, True], "status": "RUNNING"}
        core.start_worker_watchdog(period_s=0.1)
        core.start_worker_watchdog(period_s=0.1)                 # idempotent
        time.sleep(0.3)
        assert job.status == "RUNNING"
        job.workers[0]._proc.terminate()                         # the exact child created above
        job.workers[0]._proc.join(10)
        deadline = time.time() + 180.0                           # generous: a loaded CI box schedules the watchdog late
        while job.status != "FAILED" and time.time() < deadline:
            time.sleep(0.05)
        assert job.status == "FAILED" and "do not answer" in job.info["failure"]
        # teardown follows the state change.  The watchdog thread is joining that process right now, so this thread
        # must not join it too (two joiners race for the one waitpid): it watches the worker's own liveness probe
        deadline = time.time() + 180.0
        while job.workers[1].alive() and time.time() < deadline:
            time.sleep(0.05)
        assert not job.workers[1].alive()                        # the peer was stopped with it
    finally:
        core.stop_worker_watchdog()
        core.destroy()


def test_worker_process_ends_when_its_owner_is_gone(tmp_path):
    """A process that owns a spawned worker is ended hard (no clean-up runs); the worker notices and exits."""
    import subprocess
    import sys
    import time
    import psutil
    script = tmp_path / "owner.py"
    script.write_text(
        "import sys, time\n"
        f"sys.path.insert(0, {str(__import__('pathlib').Path(__file__).resolve().parents[1])!r})\n"
        "from arctic_platform_b200.common.local_actors import SpawnedActor\n"
        "class W:\n"
        "    def pid(self):\n"
        "        import os; return os.getpid()\n"
        "if __name__ == '__main__':\n"
        "    a = SpawnedActor(W)\n"
        "    print(a.call('pid'), flush=True)\n"
        "    time.sleep(600)\n")
    owner = subprocess.Popen([sys.executable, str(script)], stdout=subprocess.PIPE, text=True)
    try:
        child_pid = int(owner.stdout.readline())
        assert psutil.pid_exists(child_pid)
        owner.kill()                                   # the exact process started above; SIGKILL: no atexit, no cleanup
        owner.wait(10)
        for _ in range(100):
            if not psutil.pid_exists(child_pid) or psutil.Process(child_pid).status() == psutil.STATUS_ZOMBIE:
                break
            time.sleep(0.1)
        assert not psutil.pid_exists(child_pid) or psutil.Process(child_pid).status() == psutil.STATUS_ZOMBIE
    finally:
        if owner.poll() is None:
            owner.kill()


def test_hard_stop_only_asks_for_shutdown_while_buffers_are_multicast_bound(monkeypatch):
    """With ``APB_MULTIMEM=1`` a stuck rank's memory is bound to an NVSwitch multicast object shared with its peers:
    the server must not end that process, only ask it to shut down.  Without multimem it terminates as before."""
    from arctic_platform_b200.common import server as srv

    class _W:
        def __init__(self):
            self.log = []

        def terminate(self):
            self.log.append("terminate")

        def request_destroy(self):
            self.log.append("request_destroy")

        def kill(self):
            self.log.append("kill")

    monkeypatch.delenv("APB_MULTIMEM", raising=False)
    monkeypatch.delenv("NCCL_NVLS_ENABLE", raising=False)
    w = _W()
    srv._hard_stop(w)
    assert w.log == ["terminate"]
    monkeypatch.setenv("APB_MULTIMEM", "1")
    w = _W()
    srv._hard_stop(w)
    assert w.log == ["request_destroy"]
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")              # NVLS off overrides the request: plain peer mappings
    w = _W()
    srv._hard_stop(w)
    assert w.log == ["terminate"]


def test_symmetric_rendezvous_stays_off_multicast_unless_asked(monkeypatch):
    from arctic_platform_b200.parallel import symm
    monkeypatch.delenv("APB_MULTIMEM", raising=False)
    monkeypatch.delenv("TORCH_SYMM_MEM_DISABLE_MULTICAST", raising=False)
    symm._keep_rendezvous_off_multicast()
    import os
    assert os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] == "1"
    monkeypatch.delenv("TORCH_SYMM_MEM_DISABLE_MULTICAST", raising=False)
    monkeypatch.setenv("APB_MULTIMEM", "1")
    monkeypatch.delenv("NCCL_NVLS_ENABLE", raising=False)
    symm._keep_rendezvous_off_multicast()
    assert "TORCH_SYMM_MEM_DISABLE_MULTICAST" not in os.environ
