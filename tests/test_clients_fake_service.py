"""Unified client over a recording transport, Cortex transport and the stand-alone service client + CLI against an
in-memory fake of the REST service (no sockets)."""
import io

import pytest
import torch

from arctic_platform_b200.client import ArcticRLClientConfig
from arctic_platform_b200.client.client import SyncArcticRLClient, create_arctic_rl_client
from arctic_platform_b200.client.transport import JobHandles, Request, Transport
from arctic_platform_b200.client.transports import cortex as cortex_mod
from arctic_platform_b200.client.transports.cortex import CortexError, CortexTransport
from cortex_client.dss_client import (NeutrinoClient, NeutrinoError, NeutrinoTrainingEngine, SubJobConfig)
from cortex_client.dss_client import dss_neutrino_cli as cli
from tests.fake_service import FakeServiceSession


class FakeTransport(Transport):
    """Records every request and answers with canned replies."""

    def __init__(self):
        self.jobs = JobHandles(training=1, sampling=2, log_prob=3)
        self.requests = []
        self.closed = False

    def initialize(self):
        return self.jobs

    def call(self, request: Request) -> dict:
        self.requests.append(request)
        if request.op == "generate":
            return {"results": [{"token_ids": [1]} for _ in request.body["prompts"]]}
        return {"op": request.op, "job_id": request.job_id}

    async def acall(self, request: Request) -> dict:
        return self.call(request)

    def shutdown(self) -> None:
        self.closed = True


def _cfg(**kw):
    return ArcticRLClientConfig(model_name="qwen3-tiny", training_gpus=1, sampling_gpus=1, log_prob_gpus=1, **kw)


def test_unified_client_builds_the_documented_requests():
    t = FakeTransport()
    c = SyncArcticRLClient(_cfg(), transport=t)
    batch = {"input_ids": torch.ones(2, 4, dtype=torch.long)}
    c.fwd_bwd(batch, processing={"loss_fn": "grpo"})
    c.fwd_no_grad(batch, reference_model=True)
    c.fwd_no_grad(batch)
    c.step(2e-6)
    c.save_checkpoint("/x", step=3, export_hf=True)
    c.load_checkpoint(step=3)
    c.generate([[1, 2]], {"n": 2})
    ops = [(r.op, r.job_id, r.binary) for r in t.requests]
    assert ops == [("forward-backward", 1, True), ("forward", 3, True), ("forward", 1, True), ("step", 1, False),
                   ("save", 1, False), ("load-checkpoint", 1, False), ("generate", 2, True)]
    assert t.requests[0].body["processing"] == {"loss_fn": "grpo"} and "batch" in t.requests[0].body
    assert t.requests[3].body == {"learning_rate": 2e-6} and t.requests[4].body["export_hf"] is True
    t.requests.clear()
    c.sync_weights(cuda_ipc=True)
    assert [r.op for r in t.requests] == ["wake-inference", "operation", "wake-inference", "operation"]
    assert t.requests[1].body["operation_type"] == "weight-sync" and t.requests[1].body["payload"]["cuda_ipc"] is True
    assert t.requests[3].body["operation_type"] == "reset-prefix-cache"
    rc = c.reconnect_config()
    assert (rc.training_job_id, rc.sampling_job_id, rc.log_prob_job_id) == (1, 2, 3)
    with c:
        pass
    assert t.closed
    t2 = FakeTransport()
    t2.jobs = JobHandles(training=1)
    with pytest.raises(ValueError, match="No sampling job"):
        SyncArcticRLClient(_cfg(), transport=t2).generate([[1]])
    with pytest.raises(ValueError):
        ArcticRLClientConfig(model_name="m")


def test_async_client_mirrors_sync_surface():
    import asyncio
    t = FakeTransport()
    c = create_arctic_rl_client(_cfg(), blocking_calls=False) if False else None  # construction below avoids real transports
    from arctic_platform_b200.client.client import ArcticRLClient
    c = ArcticRLClient(_cfg(), transport=t)

    async def run():
        await c.fwd_bwd({"input_ids": torch.ones(1, 2, dtype=torch.long)})
        await c.step()
        return await c.generate([[3]], None)

    out = asyncio.run(run())
    assert [r.op for r in t.requests] == ["forward-backward", "step", "generate"] and out


def _cortex_cfg(**kw):
    return _cfg(backend={"type": "remote", "base_url": "http://svc", "max_retries": 3}, request_timeout=5.0,
                job_ready_timeout=5.0, **kw)


def test_cortex_transport_submit_poll_chunks_and_retries(monkeypatch):
    s = FakeServiceSession(ready_after=2, chunk_results_over=600)
    sleeps = []
    tr = CortexTransport(_cortex_cfg(), session=s, sleep=sleeps.append)
    jobs = tr.initialize()
    assert jobs.training.endswith(":s0") and jobs.sampling.endswith(":s1") and jobs.log_prob.endswith(":s2")
    assert len(sleeps) >= 1                                           # polled until RUNNING
    monkeypatch.setattr(cortex_mod, "MAX_CHUNK_BYTES", 16384)
    ids = torch.arange(4 * 2000).view(4, 2000)
    s.fail_next = [503, 429]                                          # transient: retried with back-off
    out = tr.call(Request("forward", jobs.log_prob, {"batch": {"input_ids": ids}}, binary=True))
    assert out["batch"]["log_probs"].shape == (4, 3) and out["sub_job_id"] == "s2"
    posts = [c for c in s.calls if c[0] == "POST" and c[1].endswith("/forward")]
    assert len(posts) > 3 and all(p[3].get("Content-Type") == "application/octet-stream" for p in posts)
    s.restart_chunk_groups = 1                                        # a lost group is resent under a new id
    out = tr.call(Request("forward-backward", jobs.training, {"batch": {"input_ids": ids}}, binary=True))
    assert out["avg_loss"] == 0.25 and out["metrics"]["n"] == 4
    assert tr.call(Request("step", jobs.training, {"learning_rate": 3e-6}))["metrics"]["last_lr"] == 3e-6
    with pytest.raises(CortexError, match="engine exploded"):
        tr.call(Request("fail", jobs.training, {}))
    s.fail_next = [400]
    with pytest.raises(CortexError, match="400"):
        tr.call(Request("step", jobs.training, {}))
    s.fail_next = [503] * 10
    with pytest.raises(CortexError, match="failed after 4 attempts"):
        tr.call(Request("step", jobs.training, {}))
    s.fail_next = []
    # verdicts on a chunk group: a conflict is final at once (even on a status that is otherwise retried, even wrapped by
    # a gateway), a refusal that is not about the group is not replayed, a group that keeps getting lost gives up
    from arctic_platform_b200.client.transports.cortex import ChunkGroupError
    big = Request("forward", jobs.log_prob, {"batch": {"input_ids": ids}}, binary=True)
    s.chunk_group_reply = (503, {"message": 'gateway: {"code": "chunk_group_conflict", "message": "group reused"}'})
    n0 = len(s.calls)
    with pytest.raises(ChunkGroupError, match="group reused") as e:
        tr.call(big)
    assert len(s.calls) == n0 + 1 and e.value.detail["code"] == "chunk_group_conflict" and e.value.status == 503
    s.chunk_group_reply = (400, {"detail": "malformed frame"})
    n0 = len(s.calls)
    with pytest.raises(CortexError, match="400") as e:
        tr.call(big)
    assert not isinstance(e.value, ChunkGroupError) and len(s.calls) == n0 + 1
    s.restart_chunk_groups = 10
    with pytest.raises(ChunkGroupError) as e:
        tr.call(big)
    assert e.value.detail["code"] == "chunk_group_restart"
    s.restart_chunk_groups = 0
    assert tr.call(big)["batch"]["log_probs"].shape == (4, 3)
    tr.shutdown()
    assert list(s.jobs.values())[0]["status"] == "CANCELLED"


def test_neutrino_client_engine_and_cli(tmp_path, monkeypatch):
    s = FakeServiceSession(ready_after=2)
    c = NeutrinoClient("http://svc", session=s, max_retries=2, sleep=lambda _t: None, poll_interval=0.0)
    job = c.create_job([SubJobConfig.training_job("qwen3-4b", num_gpus=8), SubJobConfig.sampling_job("qwen3-4b", num_gpus=8, tensor_parallel_size=2)])
    jid = job["job_id"]
    body = s.jobs[jid]["body"]
    assert body["sub_jobs"][0]["ds_config"]["zero_optimization"]["stage"] == 3 and body["sub_jobs"][1]["vllm_config"]["tensor_parallel_size"] == 2
    assert c.wait_for_job(jid)["status"] == "RUNNING" and c.list_jobs("RUNNING")[0]["job_id"] == jid
    with pytest.raises(ValueError):
        SubJobConfig.sampling_job("m", num_gpus=3, tensor_parallel_size=2).to_wire()
    with pytest.raises(ValueError):
        c.create_job([])
    eng = NeutrinoTrainingEngine(c, jid, loss_fn="sft")
    loss = eng({"input_ids": torch.ones(2, 8, dtype=torch.long)})
    assert loss == 0.25 and eng.step(1e-5)["last_lr"] == 1e-5 and eng.global_steps == 1
    assert eng.eval()({"input_ids": torch.ones(2, 8, dtype=torch.long)})["batch"]["log_probs"].shape == (2, 3)
    assert eng.save("/ckpt")["body"]["step"] == 1
    gen = c.generate(jid, [[1, 2, 3]], {"n": 2, "max_tokens": 4}, max_seq_len=16)
    assert len(gen["results"]) == 2
    with pytest.raises(ValueError, match="exceeds"):
        c.generate(jid, [[1] * 14], {"max_tokens": 4}, max_seq_len=16)
    rid = c.step(jid, wait=False)
    assert rid.startswith("r") and c.wait_request(rid)["metrics"]["grad_norm"] == 1.5
    with pytest.raises(NeutrinoError) as e:
        c.get_job("nope")
    assert e.value.status == 404
    assert c.get_capacity()["free_gpus"] == 8 and c.weight_sync(jid)["op"] == "weight_sync"
    # command line + log tail with its on-disk cursor
    monkeypatch.setenv("DSS_CACHE_DIR", str(tmp_path))
    out = io.StringIO()
    assert cli.main(["--url", "http://svc", "jobs", "get", jid], session=s, out=out) == 0 and '"RUNNING"' in out.getvalue()
    out = io.StringIO()
    cli.main(["--url", "http://svc", "logs", jid], session=s, out=out)
    assert out.getvalue().count("\n") == 5 and "line 4" in out.getvalue()
    s.logs.append({"ts": "t5", "level": "WARN", "message": "late"})
    out = io.StringIO()
    cli.main(["--url", "http://svc", "logs", jid], session=s, out=out)
    assert out.getvalue() == "t5 [WARN] late\n"                       # only what is new since the cached cursor
    out = io.StringIO()
    cli.main(["--url", "http://svc", "step", jid, "--lr", "2e-6"], session=s, out=out)
    assert "2e-06" in out.getvalue()
    cli.main(["--url", "http://svc", "jobs", "cancel", jid], session=s, out=io.StringIO())
    assert s.jobs[jid]["status"] == "CANCELLED"
    with pytest.raises(NeutrinoError, match="CANCELLED"):
        c.wait_for_job(jid)
