"""HTTP server + HTTP client round trip on CPU (tiny model, real sockets on 127.0.0.1)."""
import socket
import threading
import time

import pytest
import torch

from arctic_platform_b200.common.http_server import create_app
from arctic_platform_b200.common.server import ArcticRLServerCore
from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.fixture(scope="module")
def server():
    import uvicorn
    port = _free_port()
    config = uvicorn.Config(create_app(ArcticRLServerCore()), host="127.0.0.1", port=port, log_level="error")
    srv = uvicorn.Server(config)
    t = threading.Thread(target=srv.run, daemon=True)
    t.start()
    for _ in range(100):
        if srv.started:
            break
        time.sleep(0.05)
    yield port
    srv.should_exit = True
    t.join(timeout=5)


def test_http_training_loop_and_errors(server, tmp_path):
    cfg = ArcticRLClientConfig(comm_protocol="http", host="127.0.0.1", port=server, model_name="qwen3-tiny",
                               training_gpus=1, log_prob_gpus=1, checkpoint_path=str(tmp_path),
                               ds_config={"optimizer": {"params": {"lr": 1e-3}}, "gradient_clipping": 1.0})
    c = create_arctic_rl_client(cfg)
    assert c.job_ids["training"] is not None and c.job_ids["log_prob"] is not None and c.job_ids["sampling"] is None
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2)
    B = ids.shape[0]
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:],
             "advantages": torch.randn(B, 1).expand(B, R).contiguous()}
    ref = c.call("fwd_no_grad", {"batch": batch, "meta": {}}, reference_model=True)
    assert ref["batch"]["log_probs"].shape == (B, R)
    batch["old_log_probs"] = ref["batch"]["log_probs"]
    out = c.call("fwd_bwd", {"batch": batch, "meta": {"zorro_train_enable": True}})
    assert set(out) == {"job_id", "metrics", "avg_loss"} and "actor/pg_loss" in out["metrics"]
    st = c.call("step")
    assert st["metrics"]["grad_norm"] > 0 and st["metrics"]["last_lr"] == pytest.approx(1e-3)
    norms = c.call("weight_norm")
    assert norms["training_norm"] > 0
    saved = c.call("save_checkpoint", None, 3, True)
    # the reference's contract: a self-contained <root>/checkpoint-3/ (own latest, global_step<N>/, hf/), the
    # integer step in <root>/latest, and path / hf_path / global_step in the reply
    import os
    ck = saved["path"]
    assert os.path.basename(ck) == "checkpoint-3" and saved["global_step"] == 1
    assert saved["hf_path"] == os.path.join(ck, "hf") and os.path.isdir(saved["hf_path"])
    assert open(os.path.join(ck, "latest")).read().strip() == "global_step1"
    assert os.path.isfile(os.path.join(ck, "global_step1", "mp_rank_00_model_states.pt"))
    assert open(os.path.join(os.path.dirname(ck), "latest")).read().strip() == "3"
    loaded = c.call("load_checkpoint", None, 3)
    assert loaded["global_steps"] == 1 and loaded["global_step"] == 1 and loaded["path"] == ck
    assert c.call("load_checkpoint")["global_step"] == 1             # the job root: follows <root>/latest
    assert c.call("load_checkpoint", ck)["global_step"] == 1         # the reference form: path=<root>/checkpoint-N
    with pytest.raises(RuntimeError):                                 # a step that was never saved is an error, not step 0
        c.call("load_checkpoint", None, 99)
    assert c.call("sleep_log_prob")["status"] == "sleeping" and c.call("wake_log_prob")["status"] == "awake"
    before = c.job_ids["training"]
    rec = c.call("recover_training")                     # checkpoint + restart: same weights and step counter, new id
    assert rec["recovered_from"] == before and rec["global_steps"] == 1 and c.job_ids["training"] == rec["job_id"] != before
    assert c.call("weight_norm")["training_norm"] == pytest.approx(norms["training_norm"], rel=1e-6)
    with pytest.raises(RuntimeError, match="no sampling job"):
        c.call("generate", [[1, 2, 3]])
    # reconnect: a second client attaches to the same jobs without re-initialising
    c2 = create_arctic_rl_client(c.reconnect_config())
    assert c2.job_ids == c.job_ids
    state = c2.get_server_state()
    assert {j["job_type"] for j in state["jobs"]} == {"training", "log_prob"}
    # error codes
    import requests
    base = f"http://127.0.0.1:{server}"
    assert requests.get(f"{base}/job/9999").status_code == 404
    assert requests.post(f"{base}/step", params={"job_id": 9999}).status_code == 404
    assert requests.post(f"{base}/initialize", json={"model_name": "qwen3-tiny", "job_type": "training"}).status_code == 409
    assert requests.post(f"{base}/forward", params={"job_id": c.job_ids["training"]}, data=b"junk",
                         headers={"Content-Type": "application/octet-stream"}).status_code == 400
    c.call("shutdown")
    assert requests.get(f"{base}/status").json()["jobs"] == []
