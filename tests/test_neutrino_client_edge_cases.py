"""Stand-alone service client against the in-memory service: retry policy, job life cycle, chunked uploads and
results, streaming, request failures, configuration validation."""
import pytest
import torch

from cortex_client.dss_client import NeutrinoClient, NeutrinoError, SubJobConfig
from cortex_client.dss_client import neutrino_client as nc
from tests.fake_service import FakeResponse, FakeServiceSession


def _client(session=None, **kw):
    sleeps = []
    c = NeutrinoClient("https://svc.example/api", session=session or FakeServiceSession(), sleep=sleeps.append,
                       poll_interval=0.01, **kw)
    return c, sleeps


def _job(c):
    return c.create_job([SubJobConfig.training_job("qwen3-tiny"), SubJobConfig.sampling_job("qwen3-tiny")])["job_id"]


def test_retries_transient_codes_with_growing_jittered_delays():
    c, sleeps = _client()
    c.session.fail_next = [503, 429, 500]
    assert c.get_capacity() == {"free_gpus": 8}
    assert len(sleeps) == 3 and all(0.25 <= sleeps[0] <= 0.75 for _ in [0]) and 0.5 <= sleeps[1] <= 1.5 and 1.0 <= sleeps[2] <= 3.0
    # a client error is final at once and carries status and body
    c.session.fail_next = [403]
    with pytest.raises(NeutrinoError) as e:
        c.get_capacity()
    assert e.value.status == 403 and e.value.detail == {"error": "injected"} and len(sleeps) == 3
    # gives up after max_retries + 1 attempts
    c2, sleeps2 = _client(max_retries=2)
    c2.session.fail_next = [502] * 5
    with pytest.raises(NeutrinoError, match="failed after 3 attempts"):
        c2.get_capacity()
    assert len(sleeps2) == 2


def test_connection_errors_count_as_transient():
    class Flaky(FakeServiceSession):
        def __init__(self):
            super().__init__()
            self.breaks = 2

        def request(self, *a, **k):
            if self.breaks:
                self.breaks -= 1
                raise ConnectionError("reset by peer")
            return super().request(*a, **k)
    c, sleeps = _client(Flaky())
    assert c.get_capacity()["free_gpus"] == 8 and len(sleeps) == 2


def test_headers_from_a_programmatic_access_token():
    s = FakeServiceSession()
    c = NeutrinoClient.from_pat("acct.example.com", "DB", "SCH", "secret", session=s, sleep=lambda x: None)
    c.get_capacity()
    _m, _p, _params, headers = s.calls[-1]
    assert headers["Authorization"] == "Bearer secret"
    assert headers["X-Snowflake-Authorization-Token-Type"] == "PROGRAMMATIC_ACCESS_TOKEN"
    assert c.base == "https://acct.example.com/api/v2/databases/DB/schemas/SCH/cortex-training"


def test_job_life_cycle_and_waiting():
    c, sleeps = _client(FakeServiceSession(ready_after=3))
    jid = _job(c)
    body = c.session.jobs[jid]["body"]
    assert [s["sub_job_type"] for s in body["sub_jobs"]] == ["training", "sampling"] and body["colocate"] is True
    assert body["sub_jobs"][0]["ds_config"]["zero_optimization"]["stage"] == 3
    assert c.list_jobs("PENDING")[0]["job_id"] == jid and c.list_jobs("RUNNING") == []
    job = c.wait_for_job(jid)
    assert job["status"] == "RUNNING" and sleeps == [1.0, 1.5]                     # polled three times
    c.cancel_job(jid)
    with pytest.raises(NeutrinoError, match="CANCELLED"):
        c.wait_for_job(jid)
    with pytest.raises(NeutrinoError) as e:
        c.get_job("nope")
    assert e.value.status == 404
    with pytest.raises(ValueError):
        c.create_job([])
    # a job that never starts
    c3, _ = _client(FakeServiceSession(ready_after=10 ** 9))
    with pytest.raises(NeutrinoError, match="not RUNNING"):
        c3.wait_for_job(_job(c3), timeout=-1.0)
    assert NeutrinoClient._normalize_job_status("JobStatus.running") == "RUNNING"
    assert NeutrinoClient._normalize_job_status(None) == "UNKNOWN"


def test_config_validation():
    with pytest.raises(ValueError):
        SubJobConfig.training_job("m", num_gpus=0).to_wire()
    with pytest.raises(ValueError):
        SubJobConfig.training_job("m", zero_stage=4).to_wire()
    with pytest.raises(ValueError):
        SubJobConfig.training_job("m", learning_rate=0.0).to_wire()
    with pytest.raises(ValueError):
        SubJobConfig.sampling_job("m", num_gpus=6, tensor_parallel_size=4).to_wire()
    w = SubJobConfig.sampling_job("m", num_gpus=8, tensor_parallel_size=4, extra={"seed": 3}).to_wire()
    assert w["sub_job_type"] == "sampling" and w["vllm_config"]["tensor_parallel_size"] == 4 and w["seed"] == 3


def test_large_uploads_are_chunked_and_lost_groups_are_resent(monkeypatch):
    monkeypatch.setattr(nc, "MAX_CHUNK_BYTES", 16384)
    c, _ = _client()
    jid = _job(c)
    batch = {"input_ids": torch.arange(6000).view(4, 1500)}                       # 48 kB frame: several chunks
    out = c.forward_backward(jid, batch, sub_job_id="s0")
    posts = [x for x in c.session.calls if x[0] == "POST" and x[1].endswith("/forward_backward")]
    assert len(posts) >= 3 and out["metrics"]["n"] == 4 and out["sub_job_id"] == "s0"
    assert all(p[3]["Content-Type"] == "application/octet-stream" and p[2] == {"sub_job_id": "s0"} for p in posts)
    # the server forgets the group in the middle: the whole group goes again under a new id
    c.session.restart_chunk_groups = 1
    n0 = len(c.session.calls)
    assert c.forward(jid, batch)["batch"]["log_probs"].shape == (4, 3)
    resent = [x for x in c.session.calls[n0:] if x[0] == "POST"]
    assert len(resent) >= len(posts) + 1
    # ... but not for ever
    c.session.restart_chunk_groups = 10
    with pytest.raises(NeutrinoError):
        c.forward(jid, batch)


def test_results_arrive_in_chunks_and_errors_surface():
    c, _ = _client(FakeServiceSession(chunk_results_over=16384))
    jid = _job(c)
    out = c.forward(jid, {"input_ids": torch.zeros(3000, 4, dtype=torch.long)})    # 36 kB of log-probs back
    assert out["batch"]["log_probs"].shape == (3000, 3)
    with pytest.raises(NeutrinoError, match="engine exploded"):
        c._operation(jid, "fail", {})
    with pytest.raises(NeutrinoError) as e:
        c.step("missing-job")
    assert e.value.status == 404
    with pytest.raises(NeutrinoError):
        c.wait_request("r-unknown")


def test_request_timeout_and_empty_polls():
    class Silent(FakeServiceSession):
        def _route(self, method, path, params, body, data):
            if path.startswith("/requests/"):
                return FakeResponse(200, {"events": []})
            return super()._route(method, path, params, body, data)
    c, sleeps = _client(Silent(), request_timeout=0.05)
    jid = _job(c)
    with pytest.raises(NeutrinoError, match="timed out"):
        c.step(jid)
    assert sleeps and all(s == 0.01 for s in sleeps)


def test_generate_checks_lengths_and_streams():
    c, _ = _client()
    jid = _job(c)
    res = c.generate(jid, [[1, 2, 3], [4]], {"n": 2, "max_tokens": 8}, max_seq_len=16)
    assert len(res["results"]) == 4
    with pytest.raises(ValueError, match="prompt 1"):
        c.generate(jid, [[1], list(range(12))], {"max_tokens": 8}, max_seq_len=16)
    evs = list(c.generate_stream(jid, [[1, 2]], {"max_tokens": 2}))
    assert [e["type"] for e in evs] == ["result"]
    assert c.step(jid, learning_rate=3e-6)["metrics"]["last_lr"] == 3e-6
    for call, op in ((c.weight_sync, "weight_sync"), (c.reset_prefix_cache, "reset_prefix_cache"),
                     (c.router_replay_discard, "router_replay_discard")):
        assert call(jid)["op"] == op
    assert c.save(jid, path="/ck", step=4, export_hf=True)["body"] == {"path": "/ck", "step": 4, "export_hf": True}
    assert c.load(jid, step=4)["op"] == "load"
    assert c.bootstrap_router_replay(jid, {"layer0": torch.zeros(2, 2, dtype=torch.long)})["op"] == "bootstrap_router_replay"
    assert c.fwd == c.forward_backward and c.fwd_no_grad == c.forward


def test_request_polling_log_tails_and_checkpoint_routes():
    """The status-page way of waiting for a request, cursor-paged log / scheduler-event feeds (one page, and the
    streaming generators with and without follow), checkpoint listing / export / deletion, experiment bookkeeping
    and the older forward aliases."""
    svc = FakeServiceSession(chunk_results_over=600)
    naps = []
    c = NeutrinoClient("https://svc/api", session=svc, poll_interval=0.01, sleep=naps.append)
    job = c.create_job([SubJobConfig.training_job("qwen3-tiny")])["job_id"]
    # status-page polling: plain result, chunked result, failure
    rid = c._operation(job, "step", {"learning_rate": 3e-6}, wait=False)
    assert c.poll_request(job, rid)["metrics"]["last_lr"] == 3e-6
    big = {"batch": {"input_ids": torch.zeros(4, 300, dtype=torch.int64)}}
    rid = c._operation(job, "forward", big, binary=True, wait=False)
    assert c.poll_request(job, rid)["batch"]["log_probs"].shape == (4, 3)
    rid = c._operation(job, "fail", {}, wait=False)
    import pytest
    with pytest.raises(NeutrinoError, match="failed: engine exploded"):
        c.poll_request(job, rid)
    assert c._normalize_request_status("in-progress") == "RUNNING" and c._normalize_request_status("Done") == "COMPLETED"
    assert c.cancel_request(job, "r-any")["body"] == {"request_id": "r-any"}
    # one page, then the generators
    page = c.tail_logs(job, max_lines=3)
    assert [e["message"] for e in page["entries"]] == ["line 0", "line 1", "line 2"] and not page["eof"]
    assert [e["message"] for e in c.stream_logs(job, follow=False, max_lines=2)] == [f"line {i}" for i in range(5)]
    assert [e["kind"] for e in c.stream_events(job, follow=False)] == ["SCHEDULED", "ZONE_READY", "ZONE_READY"]
    live = c.stream_logs(job, cursor="4")                        # follow: waits for new entries after the end
    assert next(live)["message"] == "line 4"
    svc.logs.append({"ts": "t5", "level": "INFO", "message": "line 5"})
    assert next(live)["message"] == "line 5" and len(naps) >= 0
    # checkpoints and bookkeeping
    assert [k["checkpoint_id"] for k in c.list_checkpoints(job)] == ["c1", "c2"]
    assert c.export_checkpoint(job, "c2")["status"] == "EXPORTING"
    c.delete_checkpoint(job, "c1")
    assert [k["checkpoint_id"] for k in c.list_checkpoints(job)] == ["c2"]
    with pytest.raises(NeutrinoError):
        c.delete_checkpoint(job, "c1")
    assert c.get_experiment_run(job) == {"experiment_name": "exp", "experiment_run_name": f"run-{job}"}
    out = c.fwd_no_grad(job, {"input_ids": torch.zeros(2, 5, dtype=torch.int64)})
    assert out["batch"]["log_probs"].shape == (2, 3)


def test_chunk_group_verdicts_become_structured_errors(monkeypatch):
    from cortex_client.dss_client.neutrino_client import (ChunkGroupConflictError, ChunkGroupRestartError,
                                                          find_chunk_group_error)
    monkeypatch.setattr(nc, "MAX_CHUNK_BYTES", 16384)
    c, _ = _client()
    jid = _job(c)
    batch = {"input_ids": torch.arange(6000).view(4, 1500)}
    # the verdict may sit inside a gateway's wrapper, as JSON embedded in a string, on a status that is otherwise retried
    wrapped = {"message": 'upstream error: {"error": {"code": "chunk_group_conflict", "message": "group g reused", '
                          '"chunk_group_id": "g"}} (request 77)'}
    c.session.chunk_group_reply = (503, wrapped)
    n0 = len(c.session.calls)
    with pytest.raises(ChunkGroupConflictError, match="group g reused") as e:
        c.forward_backward(jid, batch)
    assert e.value.detail["code"] == "chunk_group_conflict" and e.value.status == 503
    assert len(c.session.calls) == n0 + 1                          # not retried, not replayed
    c.session.chunk_group_reply = (400, {"chunk_group_id": "g", "message": "request chunk group is missing chunks"})
    with pytest.raises(ChunkGroupConflictError) as e:
        c.forward_backward(jid, batch)
    assert e.value.detail["code"] == "chunk_group_missing_chunks"
    # a restart verdict is replayed; when the replays run out the error says so
    c.session.chunk_group_reply = (409, {"code": "chunk_group_restart_required", "message": "state lost"})
    assert c.forward_backward(jid, batch)["metrics"]["n"] == 4
    c.session.restart_chunk_groups = 10
    with pytest.raises(ChunkGroupRestartError):
        c.forward_backward(jid, batch)
    assert isinstance(ChunkGroupRestartError("x"), NeutrinoError)
    assert find_chunk_group_error({"a": [1, "text {not json} more", {"b": "{}"}]}) is None
    assert find_chunk_group_error("[[[[[[[[[[[[[[[[") is None


def test_sampling_limit_is_read_from_the_job_and_cached():
    c, _ = _client()
    jid = _job(c)
    c.session.jobs[jid]["sub_jobs"] = [{"sub_job_type": "training"},
                                       {"sub_job_type": "sampling", "inference_config": {"max_seq_len": 64.0}}]
    assert c.sampling_max_seq_len(jid) == 64
    n0 = len(c.session.calls)
    assert c.sampling_max_seq_len(jid) == 64 and len(c.session.calls) == n0          # cached
    with pytest.raises(ValueError, match="max_seq_len 64"):
        c.generate(jid, [[1] * 60], {"max_tokens": 8}, validate_lengths=True)
    assert c.sampling_max_seq_len("missing-job") is None                             # failed look-up: not cached
    assert "missing-job" not in c._max_seq_len_cache


def test_training_engine_deepspeed_call_shape_and_lifecycle():
    from cortex_client.dss_client import NeutrinoTrainingEngine, SubJobConfig
    c, _ = _client()
    eng = NeutrinoTrainingEngine.from_sub_job(c, SubJobConfig.training_job("qwen3-4b", num_gpus=2), name="t", loss_fn="sft_ce")
    assert c.session.jobs[eng.job_id]["status"] == "RUNNING" and eng.module is None and eng.optimizer is None
    assert eng.lr_scheduler.get_last_lr() == [-1.0] and eng.is_gradient_accumulation_boundary()
    handle = eng.forward(input_ids=torch.ones(2, 8, dtype=torch.long))
    with pytest.raises(RuntimeError, match="twice"):
        eng.forward(input_ids=torch.ones(1, 8, dtype=torch.long))
    assert eng.backward(handle) == 0.25
    with pytest.raises(RuntimeError, match="forward"):
        eng.backward()
    assert eng.forward({"input_ids": torch.ones(3, 8, dtype=torch.long)})["input_ids"].shape[0] == 3
    eng.backward()
    eng.step(2e-5)
    assert eng.global_steps == 1 and eng.lr_scheduler.get_last_lr() == [2e-5]
    saved = eng.save_checkpoint("/ignored/dir", "tag", checkpoint_type="full")
    assert saved["op"] == "save" and saved["body"] == {"step": 1, "checkpoint_type": "full"}
    loaded = eng.load_checkpoint("ck-7", source_job_id="job-old", target_sub_job_id=f"{eng.job_id}:training:0")
    assert loaded["body"] == {"checkpoint_id": "ck-7", "source_job_id": "job-old"}
    posts = [x for x in c.session.calls if x[0] == "POST" and x[1].endswith("/load")]
    assert posts[-1][2] == {"sub_job_id": f"{eng.job_id}:training:0"}
    eng.destroy()
    assert c.session.jobs[eng.job_id]["status"] == "CANCELLED"
    eng.destroy()                                                       # a second cancel is not an error for the caller
