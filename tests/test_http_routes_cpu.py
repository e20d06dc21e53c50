"""Every route of the job server, called raw (no client in between) through an in-process ASGI test client: the
sampling, weight hand-over, operation and log-prob routes, sleep / wake state, and the error codes."""
import pytest
import torch
from fastapi.testclient import TestClient

from arctic_platform_b200 import wire
from arctic_platform_b200.common.http_server import OCTET, create_app
from arctic_platform_b200.common.server import ArcticRLServerCore


@pytest.fixture(scope="module")
def api():
    with TestClient(create_app(ArcticRLServerCore(colocate=True))) as c:
        yield c


def _octet(c, path, obj, **params):
    r = c.post(path, params=params, content=wire.dumps(obj), headers={"Content-Type": OCTET})
    return r.status_code, (wire.loads(r.content) if r.status_code == 200 else r.json())


def test_all_routes(api, tmp_path):
    assert api.get("/health").json() == {"status": "ok"}
    jobs = {}
    for jt in ("sampling", "log_prob", "training"):
        r = api.post("/initialize", json={"model_name": "qwen3-tiny", "job_type": jt, "seed": 3,
                                          "vllm_config": {"max_model_len": 64},
                                          "ds_config": {"optimizer": {"params": {"lr": 1e-2}}}})
        assert r.status_code == 200, r.text
        jobs[jt] = r.json()["job_id"]
        assert r.json()["status"] == "RUNNING" and r.json()["engine"] == "b200"
    assert api.post("/initialize", json={"model_name": "qwen3-tiny", "job_type": "nonsense"}).status_code in (400, 422)
    assert {j["job_type"] for j in api.get("/status").json()["jobs"]} == set(jobs)
    assert api.get(f"/job/{jobs['training']}").json()["job_type"] == "training"
    assert api.post("/heartbeat", params={"job_id": jobs["sampling"]}).json() == {"status": "ok"}
    assert api.post("/heartbeat", params={"job_id": 999}).status_code == 404
    assert api.get(f"/job/{jobs['training']}/workers").json() == {"job_id": jobs["training"], "alive": [True], "status": "RUNNING"}
    assert api.get("/job/999/workers").status_code == 404

    # rollout, then sleep: a sleeping sampler refuses to generate until it is woken
    code, out = _octet(api, "/generate", {"prompts": [[4, 5, 6], [7, 8]], "sampling_params": {"n": 2, "max_tokens": 3}},
                       job_id=jobs["sampling"])
    assert code == 200 and len(out["results"]) == 4 and out["results"][2]["prompt_index"] == 1
    assert _octet(api, "/generate", {"prompts": [[1]]}, job_id=jobs["training"])[0] == 400          # wrong kind of job
    assert api.post("/sleep-inference", params={"job_id": jobs["sampling"], "level": 1}).json()["status"] == "sleeping"
    code, err = _octet(api, "/generate", {"prompts": [[4, 5]], "sampling_params": {"max_tokens": 2}}, job_id=jobs["sampling"])
    assert code == 409 and "asleep" in err["detail"]
    code, err = _octet(api, "/generate", {"prompts": [[]]}, job_id=jobs["sampling"])           # engine-side validation
    assert code in (400, 409)
    assert api.post("/wake-inference", params={"job_id": jobs["sampling"]}, json=["weights", "kv_cache"]).json()["status"] == "awake"
    assert api.post("/reset-prefix-cache", params={"job_id": jobs["sampling"]}).json()["status"] == "ok"

    # one optimizer step so that trainer and sampler differ, then the hand-over makes them equal again
    ids = torch.randint(3, 100, (4, 12))
    mask = torch.ones_like(ids)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -4:].contiguous(),
             "advantages": torch.randn(4, 1).expand(4, 4).contiguous(), "old_log_probs": torch.full((4, 4), -4.0)}
    code, out = _octet(api, "/forward-backward", {"batch": batch, "meta": {"response_length": 4},
                                                  "processing": {"loss_fn": "verl_grpo"}}, job_id=jobs["training"])
    assert code == 200 and "batch" not in out and "actor/pg_loss" in out["metrics"]
    st = api.post("/step", params={"job_id": jobs["training"]}, json={"learning_rate": 5e-3}).json()
    assert st["metrics"]["last_lr"] == pytest.approx(5e-3)
    assert api.post("/empty-training-cache", params={"job_id": jobs["training"]}).json()["status"] == "ok"
    wn = api.post("/weight-norm", json={"training_job_id": jobs["training"], "sampling_job_id": jobs["sampling"]}).json()
    assert wn["training_norm"] != pytest.approx(wn["sampling_norm"], rel=1e-9)
    ws = api.post("/weight-sync", json={"source_sub_job_id": jobs["training"], "target_sub_job_ids": [jobs["sampling"]]}).json()
    assert ws["status"] == "ok" and ws["strategies"] == ["in_process"]
    wn = api.post("/weight-norm", json={"training_job_id": jobs["training"], "sampling_job_id": jobs["sampling"]}).json()
    assert wn["training_norm"] == pytest.approx(wn["sampling_norm"], rel=1e-6)

    # the same four actions through /operation
    op = lambda t, sid, payload=None: api.post("/operation", json={"operation_type": t, "sub_job_id": sid, "payload": payload or {}})
    assert op("sleep-inference", jobs["sampling"], {"level": 2}).json()["status"] == "sleeping"
    assert op("wake-inference", jobs["sampling"], {"tags": ["weights"]}).json()["status"] == "awake"
    assert op("reset-prefix-cache", jobs["sampling"]).json()["status"] == "ok"
    assert op("weight-sync", jobs["training"], {"target_sub_job_ids": [jobs["log_prob"]]}).json()["status"] == "ok"
    assert op("defragment", jobs["sampling"]).status_code == 400

    # log-probs of given completions from the reference engine: equal to /forward on the same tokens
    lp = api.post("/log-probs", params={"job_id": jobs["log_prob"]},
                  json={"prompts": [[4, 5, 6], [7, 8]], "completions": [[9, 10], [11]]}).json()["log_probs"]
    assert [len(r) for r in lp] == [2, 1] and all(v < 0 for r in lp for v in r)
    # a sampling job scores with the sampler's own weights; after the hand-over above they are the trainer's, the
    # reference engine still holds the initial policy
    sl = api.post("/log-probs", params={"job_id": jobs["sampling"]},
                  json={"prompts": [[4, 5, 6], [7, 8], [4, 5, 6]], "completions": [[9, 10], [11], [12]]})
    assert sl.status_code == 200 and [len(r) for r in sl.json()["log_probs"]] == [2, 1, 1]
    tl = api.post("/log-probs", params={"job_id": jobs["training"]},
                  json={"prompts": [[4, 5, 6], [7, 8], [4, 5, 6]], "completions": [[9, 10], [11], [12]]}).json()["log_probs"]
    assert sl.json()["log_probs"][0] == pytest.approx(tl[0], abs=1e-5) and sl.json()["log_probs"][2] == pytest.approx(tl[2], abs=1e-5)
    assert api.post("/log-probs", params={"job_id": jobs["sampling"]}, json={"prompts": [[1]], "completions": [[2], [3]]}).status_code == 400
    code, fw = _octet(api, "/forward", {"batch": {"input_ids": torch.tensor([[4, 5, 6, 9, 10]]),
                                                  "attention_mask": torch.ones(1, 5, dtype=torch.long),
                                                  "response_mask": torch.ones(1, 2, dtype=torch.long)},
                                        "meta": {"response_length": 2}}, job_id=jobs["log_prob"])
    assert code == 200 and fw["batch"]["log_probs"][0].tolist() == pytest.approx(lp[0], abs=1e-5)

    # training-side sleep / wake, all three modes, and the log-prob aliases
    for mode in ("all", "non_lp", "lp_params"):
        assert api.post("/sleep-training", params={"job_id": jobs["training"], "mode": mode}).json()["mode"] == mode
        assert api.post("/wake-training", params={"job_id": jobs["training"]}).json()["status"] == "awake"
    assert api.post("/sleep-training", params={"job_id": jobs["training"], "mode": "deep"}).status_code == 400
    assert api.post("/sleep-log-prob", params={"job_id": jobs["log_prob"]}).json()["status"] == "sleeping"
    assert api.post("/wake-log-prob", params={"job_id": jobs["log_prob"]}).json()["status"] == "awake"

    # checkpoint + restart through the API: a new job id, the step counter comes back
    ck = api.post("/save", params={"job_id": jobs["training"]}, json={"path": str(tmp_path), "step": 1}).json()
    assert ck["path"].endswith("checkpoint-1") and ck["global_step"] == 1 and ck["hf_path"] is None
    assert (tmp_path / "latest").read_text().strip() == "1"
    assert api.post("/load-checkpoint", params={"job_id": jobs["training"]},
                    json={"path": str(tmp_path), "step": 7}).status_code == 404      # never saved: an error, not step 0
    rec = api.post("/recover", params={"job_id": jobs["training"]}, json={"path": str(tmp_path)}).json()
    assert rec["recovered_from"] == jobs["training"] and rec["global_steps"] == 1 and rec["job_id"] != jobs["training"]
    assert api.post("/recover", params={"job_id": jobs["training"]}).status_code == 404
    jobs["training"] = rec["job_id"]

    # teardown: one job, an unknown job, then everything
    assert api.post("/destroy", params={"job_id": jobs["log_prob"]}).json() == {"destroyed": [jobs["log_prob"]]}
    assert api.post("/destroy", params={"job_id": jobs["log_prob"]}).status_code == 404
    assert api.post("/step", params={"job_id": jobs["log_prob"]}).status_code == 404
    assert sorted(api.post("/destroy").json()["destroyed"]) == sorted([jobs["sampling"], jobs["training"]])
    assert api.get("/status").json() == {"jobs": []}
