"""Every sub-command of the service CLI against the in-memory service; stored login state."""
import io
import json
import os
import stat

import pytest

from cortex_client.dss_client import dss_neutrino_cli as cli
from tests.fake_service import FakeServiceSession


def _run(argv, s, **kw):
    out = io.StringIO()
    rc = cli.main(argv, session=s, out=out, **kw)
    return rc, out.getvalue()


def test_job_commands_and_operations(tmp_path, monkeypatch):
    monkeypatch.setenv("DSS_CACHE_DIR", str(tmp_path / "cache"))
    monkeypatch.setenv("NEUTRINO_TUI_CACHE_DIR", str(tmp_path / "tui"))
    s = FakeServiceSession(ready_after=2)
    url = ["--url", "http://svc"]
    rc, text = _run(url + ["jobs", "create", "--model", "qwen3-4b", "--training-gpus", "8", "--sampling-gpus", "8", "--tp", "2",
                           "--name", "exp1"], s)
    jid = json.loads(text)["job_id"]
    body = s.jobs[jid]["body"]
    assert rc == 0 and body["name"] == "exp1" and [x["sub_job_type"] for x in body["sub_jobs"]] == ["training", "sampling"]
    assert body["sub_jobs"][1]["vllm_config"]["tensor_parallel_size"] == 2
    assert json.loads(_run(url + ["jobs", "list", "--status", "PENDING"], s)[1])[0]["job_id"] == jid
    assert json.loads(_run(url + ["jobs", "wait", jid], s)[1])["status"] == "RUNNING"
    assert json.loads(_run(url + ["jobs", "get", jid], s)[1])["status"] == "RUNNING"
    assert json.loads(_run(url + ["capacity"], s)[1]) == {"free_gpus": 8}
    assert json.loads(_run(url + ["step", jid, "--lr", "2e-6"], s)[1])["metrics"]["last_lr"] == 2e-6
    assert json.loads(_run(url + ["save", jid, "--path", "/ck"], s)[1])["body"]["path"] == "/ck"
    assert json.loads(_run(url + ["sync", jid], s)[1])["op"] == "weight_sync"
    # logs: the plain tail keeps a cursor, the viewer keeps entries as well
    assert _run(url + ["logs", jid], s)[1].count("\n") == 5
    s.logs.append({"ts": "t5", "level": "ERROR", "message": "boom"})
    assert _run(url + ["logs", jid], s)[1] == "t5 [ERROR] boom\n"
    rc, text = _run(url + ["tui", "logs", jid, "--level", "ERROR"], s)
    assert rc == 0 and text == "t5 [ERROR] boom\n"
    assert jid in _run(url + ["tui", "jobs"], s)[1]
    assert json.loads(_run(url + ["jobs", "cancel", jid], s)[1]) == {"cancelled": jid}
    with pytest.raises(SystemExit):
        _run(["jobs"], s)                                        # a sub-command is required


def test_login_state_is_private_and_used_last(tmp_path, monkeypatch):
    for k in ("DSS_URL", "DSS_HOST", "DSS_DATABASE", "DSS_SCHEMA", "DSS_PAT", "XDG_CONFIG_HOME"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("DSS_CONFIG_DIR", str(tmp_path))
    s = FakeServiceSession()
    with pytest.raises(SystemExit, match="login"):
        _run(["capacity"], s)
    with pytest.raises(SystemExit):
        _run(["login", "--host", "h"], s)
    rc, text = _run(["login", "--host", "acct.example.com", "--database", "DB", "--schema", "S", "--pat", "tok"], s)
    path = cli.login_state_path()
    assert rc == 0 and path == tmp_path / "login.json" and str(path) in text
    assert stat.S_IMODE(os.stat(path).st_mode) == 0o600
    assert json.loads(_run(["whoami"], s)[1]) == {"host": "acct.example.com", "database": "DB", "schema": "S", "pat": "***"}
    assert json.loads(_run(["capacity"], s)[1]) == {"free_gpus": 8}
    assert s.calls[-1][3]["Authorization"] == "Bearer tok"
    monkeypatch.setenv("DSS_URL", "http://other")                # the environment wins over the stored login
    _run(["capacity"], s)
    assert "Authorization" not in s.calls[-1][3]
    monkeypatch.delenv("DSS_URL")
    _run(["login", "--service-url", "http://svc2"], s)
    _run(["capacity"], s)
    assert "Authorization" not in s.calls[-1][3] and json.loads(_run(["whoami"], s)[1]) == {"url": "http://svc2"}
    assert _run(["logout"], s)[1] == "logged out\n" and not path.exists()
    assert json.loads(_run(["whoami"], s)[1]) == {"login": None}
    monkeypatch.delenv("DSS_CONFIG_DIR")
    monkeypatch.setenv("XDG_CONFIG_HOME", str(tmp_path / "xdg"))
    assert cli.login_state_path() == tmp_path / "xdg" / "dss-neutrino" / "login.json"


def _run2(argv, s, stdin_text=""):
    out, err = io.StringIO(), io.StringIO()
    rc = cli.main(argv, session=s, out=out, err=err, stdin=io.StringIO(stdin_text))
    return rc, out.getvalue(), err.getvalue()


def test_submit_list_checkpoints_and_data_plane_commands(tmp_path):
    s = FakeServiceSession(ready_after=1)
    url = ["--url", "http://svc", "--compact"]
    job_json = tmp_path / "job.json"
    job_json.write_text(json.dumps({"name": "from-file", "sub_jobs": [{"sub_job_type": "training", "model_name": "m"}]}))
    rc, text, _ = _run2(url + ["submit", str(job_json), "--job-id", "fixed", "--dry-run"], s)
    assert rc == 0 and json.loads(text)["job_id"] == "fixed" and not s.jobs           # nothing was sent
    rc, text, _ = _run2(url + ["submit", "-", "--wait"], s, stdin_text=job_json.read_text())
    job = json.loads(text)
    jid = job["job_id"]
    assert rc == 0 and job["status"] == "RUNNING" and "\n" not in text.strip()         # --compact: one line
    refusing = FakeServiceSession()
    refusing.fail_next = [400]
    rc, _, err = _run2(url + ["submit", str(job_json)], refusing)
    assert rc == 1 and err.startswith("error: ")
    (tmp_path / "bad.json").write_text("{not json")
    assert _run2(url + ["submit", str(tmp_path / "bad.json")], s)[0] == 1
    (tmp_path / "empty.json").write_text("{}")
    assert "sub_jobs" in _run2(url + ["submit", str(tmp_path / "empty.json")], s)[2]
    # list: oldest first
    s.jobs["a"] = {"job_id": "a", "status": "RUNNING", "created_at": "2025-03-02T00:00:00Z"}
    s.jobs["b"] = {"job_id": "b", "status": "RUNNING", "created_at": "2025-03-01T00:00:00+00:00"}
    listed = json.loads(_run2(url + ["list"], s)[1])["jobs"]
    assert [j["job_id"] for j in listed if j["job_id"] in ("a", "b")] == ["b", "a"]
    # checkpoints
    s.checkpoints = [{"checkpoint_id": "ck1"}, {"checkpoint_id": "ck2"}]
    assert len(json.loads(_run2(url + ["checkpoints", jid], s)[1])["checkpoints"]) == 2
    assert json.loads(_run2(url + ["checkpoints", jid, "--export", "ck1"], s)[1])["status"] == "EXPORTING"
    assert json.loads(_run2(url + ["checkpoints", jid, "--delete", "ck2"], s)[1])["deleted"] == "ck2"
    assert [c["checkpoint_id"] for c in s.checkpoints] == ["ck1"]
    # fwd-bwd from a readable description; without --job it is refused
    spec = tmp_path / "batch.json"
    spec.write_text(json.dumps({"payload": {"input_ids": [[1, 2, 3, 4], [5, 6, 7, 8]], "attention_mask": True}}))
    rc, _, err = _run2(url + ["fwd-bwd", str(spec)], s)
    assert rc == 1 and "--job" in err
    rc, text, _ = _run2(url + ["--job", jid, "fwd-bwd", str(spec)], s)
    reply = json.loads(text)
    assert rc == 0 and reply["result"]["metrics"]["n"] == 2 and reply["tensor_bytes"] == 3 * 8 * 8
    spec.write_text(json.dumps({"poll": False, "input_ids": [[1, 2]]}))
    assert json.loads(_run2(url + ["--job", jid, "fwd-bwd", str(spec)], s)[1])["request_id"].startswith("r")
    spec.write_text(json.dumps({"input_ids": [1, 2]}))
    assert "shape" in _run2(url + ["--job", jid, "fwd-bwd", str(spec)], s)[2]
    # generate
    gen = tmp_path / "gen.json"
    gen.write_text(json.dumps({"prompts": [[1, 2, 3], [4]], "sampling_params": {"n": 2, "max_tokens": 4}, "strict": True}))
    reply = json.loads(_run2(url + ["--job-id", jid, "generate", str(gen)], s)[1])
    assert reply["prompt_count"] == 2 and len(reply["result"]["results"]) == 4
    gen.write_text(json.dumps({"prompts": []}))
    assert _run2(url + ["--job", jid, "generate", str(gen)], s)[0] == 1
    # load / weight-sync
    reply = json.loads(_run2(url + ["--job", jid, "load", "ck1", "--source-job-id", "old", "--target-sub-job-id", "t0"], s)[1])
    assert reply["result"]["body"] == {"checkpoint_id": "ck1", "source_job_id": "old"} and reply["target_sub_job_id"] == "t0"
    assert json.loads(_run2(url + ["--job", jid, "load", "ck1", "--no-poll"], s)[1])["request_id"].startswith("r")
    reply = json.loads(_run2(url + ["--job", jid, "weight-sync", "--weight-format", "fp8"], s)[1])
    assert reply["source_sub_job_id"] == f"{jid}:training:0" and reply["target_sub_job_ids"] == [f"{jid}:sampling:0"]
    assert reply["result"]["body"]["weight_format"] == "fp8"
    # download-log
    reply = json.loads(_run2(url + ["download-log", jid, "-o", str(tmp_path / "logs")], s)[1])
    saved = reply["logs"][0]["saved_path"]
    assert open(saved).read().count("\n") == len(s.logs)


def test_connection_config_file_and_remembered_config(tmp_path, monkeypatch):
    for k in ("DSS_URL", "DSS_HOST", "DSS_DATABASE", "DSS_SCHEMA", "DSS_PAT", "DSS_CONFIG", "XDG_CONFIG_HOME"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("DSS_CONFIG_DIR", str(tmp_path / "state"))
    s = FakeServiceSession()
    cfg = tmp_path / "conn.json"
    cfg.write_text(json.dumps({"connection": {"host": "https://acct.example.com/", "pat": "tok", "db": "DB", "poll_timeout": 5}}))
    assert json.loads(_run2(["--config", str(cfg), "capacity"], s)[1]) == {"free_gpus": 8}
    assert s.calls[-1][3]["Authorization"] == "Bearer tok"
    made = cli._client_from_config(cli.load_connection_config(str(cfg)), s)
    assert made.base == "https://acct.example.com/api/v2/databases/DB/schemas/PUBLIC/cortex-training"
    assert made.request_timeout == 5.0
    got = cli.load_connection_config(str(cfg))
    assert got["database"] == "DB" and got["request_timeout"] == 5
    cfg2 = tmp_path / "typo.json"
    cfg2.write_text(json.dumps({"url": "http://svc", "databse": "x"}))
    rc, _, err = _run2(["--config", str(cfg2), "capacity"], s)
    assert rc == 1 and "databse" in err
    cfg2.write_text(json.dumps({"host": "h"}))
    assert "needs url" in _run2(["--config", str(cfg2), "capacity"], s)[2]
    cfg2.write_text(json.dumps({"url": "http://svc", "no_verify_ssl": True, "poll_interval": "fast"}))
    assert "poll_interval" in _run2(["--config", str(cfg2), "capacity"], s)[2]
    # login --config remembers the path; later commands need no flags
    assert _run2(["login", "--config", str(cfg2)], s)[0] == 1                         # a file that does not load is refused
    rc, text, _ = _run2(["login", "--config", str(cfg)], s)
    assert rc == 0 and json.loads(text)["logged_in"] is True
    n0 = len(s.calls)
    assert _run2(["capacity"], s)[0] == 0 and s.calls[n0][3]["Authorization"] == "Bearer tok"
    assert cli.jobs_oldest_first([{"job_id": 1}, {"job_id": 2}]) == [{"job_id": 2}, {"job_id": 1}]
    assert [j["job_id"] for j in cli.jobs_oldest_first([{"job_id": 1, "created_at": "garbage"},
                                                        {"job_id": 2, "created_at": "2025-01-01T00:00:00"}])] == [2, 1]
