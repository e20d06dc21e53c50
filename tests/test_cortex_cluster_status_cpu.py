"""GPU accounting and rendering of the cluster status view; the shipped example files stay loadable."""
import io
import json
from pathlib import Path

import pytest

from cortex_client import cluster_status as cs
from cortex_client.dss_client import batch_spec, dss_neutrino_cli as cli
from tests.fake_service import FakeServiceSession

EXAMPLES = Path(cs.__file__).parent / "examples"


def _jobs():
    return [
        {"job_id": "j1", "name": "grpo", "status": "JOB_STATE_RUNNING",
         "sub_jobs": [{"sub_job_type": "training", "num_devices": 8},
                      {"sub_job_type": "sampling", "num_devices": 8, "vllm_config": {"tensor_parallel_size": 2}}]},
        {"job_id": "j2", "status": "running", "sub_job_configs": [{"job_type": "training", "training_config": {"n_gpus": "4"}}]},
        {"job_id": "j3", "status": "PLACING", "body": {"name": "queued", "sub_jobs": [{"sub_job_type": "sampling", "n_gpus": 0.5}]}},
        {"job_id": "j4", "status": "COMPLETED", "sub_jobs": [{"sub_job_type": "training", "num_devices": 64}]},
        {"job_id": "j5", "status": "RUNNING", "n_gpus": 2},
    ]


def test_gpu_accounting():
    jobs = _jobs()
    assert [cs.job_gpus(j) for j in jobs] == [16.0, 4.0, 0.5, 64.0, 2.0]
    assert cs.sub_job_summary(jobs[0]) == "training x8 + sampling x8 (tp 2)"
    assert cs.sub_job_summary(jobs[4]) == "-"
    assert cs.normalize_status("job_state_placing") == "PLACING"
    assert cs.sub_job_gpus({"n_gpus": True, "training_config": {"n_gpus": "x"}}) == 0.0


def test_render_groups_by_state_and_totals():
    text = cs.render(_jobs(), {"free_gpus": 10, "total_gpus": 32}, now="T")
    lines = text.splitlines()
    assert lines[0] == "cluster status T"
    assert "RUNNING: 3 job(s), 22 GPU(s)" in lines and "PLACING: 1 job(s), 0.5 GPU(s)" in lines
    assert not any(line.startswith("PENDING") for line in lines) and "j4" not in text
    assert any(line.split() == ["j1", "grpo", "16", "training", "x8", "+", "sampling", "x8", "(tp", "2)"] for line in lines)
    assert lines[-1] == "free: 10 GPU(s) of 32"
    assert "RUNNING: 0 job(s), 0 GPU(s)" in cs.render([], None, now="T")


def test_main_reads_the_service_or_a_file(tmp_path):
    s = FakeServiceSession()
    s.jobs["a"] = {"job_id": "a", "status": "RUNNING", "sub_jobs": [{"sub_job_type": "training", "num_devices": 8}]}
    out = io.StringIO()
    assert cs.main(["--url", "http://svc", "--once"], session=s, out=out) == 0
    assert "RUNNING: 1 job(s), 8 GPU(s)" in out.getvalue() and "free: 8 GPU(s)" in out.getvalue()
    out, naps = io.StringIO(), []
    assert cs.main(["--url", "http://svc", "--interval", "3"], session=s, out=out, sleep=naps.append, max_refreshes=3) == 0
    assert naps == [3.0, 3.0] and out.getvalue().count("cluster status") == 3
    out = io.StringIO()
    cs.main(["--jobs-json", "-"], out=out, stdin=io.StringIO(json.dumps({"jobs": _jobs()})))
    assert "RUNNING: 3 job(s), 22 GPU(s)" in out.getvalue()
    f = tmp_path / "jobs.json"
    f.write_text(json.dumps(_jobs()[:1]))
    out = io.StringIO()
    cs.main(["--jobs-json", str(f)], out=out)
    assert "RUNNING: 1 job(s), 16 GPU(s)" in out.getvalue()
    with pytest.raises(ValueError):
        cs.load_jobs('"text"')


def test_example_files_load_with_the_tools_they_are_for(tmp_path):
    for name in ("rl_job.json", "training_job.json", "sampling_job.json"):
        out, err = io.StringIO(), io.StringIO()
        assert cli.main(["submit", str(EXAMPLES / name), "--dry-run"], out=out, err=err) == 0, err.getvalue()
        assert json.loads(out.getvalue())["sub_jobs"]
    assert cs.job_gpus(json.loads((EXAMPLES / "rl_job.json").read_text())) == 16.0
    spec = json.loads((EXAMPLES / "fwd_bwd_tokens.json").read_text())
    batch = batch_spec.build_forward_backward_kwargs(spec["payload"])
    assert set(batch) == {"input_ids", "attention_mask", "position_ids", "labels"}
    assert (batch["labels"][0, -3:] == -100).all() and batch["labels"][0, 0] == batch["input_ids"][0, 0]
    texts = json.loads((EXAMPLES / "fwd_bwd_texts.json").read_text())["payload"]
    assert batch_spec.expand_texts(texts["texts"], texts["batch_size"])[2] == texts["texts"][0]
    # the connection template becomes a valid config once its placeholders are filled in
    conn = json.loads((EXAMPLES / "connection.json.template").read_text())
    filled = tmp_path / "conn.json"
    filled.write_text(json.dumps(conn))
    assert cli.load_connection_config(str(filled))["request_timeout"] == 1800.0
    s = FakeServiceSession()
    jid = json.loads(_submit(s, EXAMPLES / "rl_job.json"))["job_id"]
    out = io.StringIO()
    assert cli.main(["--url", "http://svc", "--job", jid, "generate", str(EXAMPLES / "generate.json")], session=s, out=out) == 0
    assert len(json.loads(out.getvalue())["result"]["results"]) == 4


def _submit(s, path):
    out = io.StringIO()
    assert cli.main(["--url", "http://svc", "submit", str(path)], session=s, out=out) == 0
    return out.getvalue()
