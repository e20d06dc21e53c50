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
