"""The whole stack in separate processes on CPU: a client launches the job server as a child process, the server
starts two rank processes (gloo), training over HTTP equals the in-process run, and everything is gone afterwards."""
import socket

import pytest
import torch

from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _payload():
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=13)
    B = ids.shape[0]
    g = torch.Generator().manual_seed(4)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:].contiguous(),
             "old_log_probs": torch.randn(B, R, generator=g) * 0.01 - 2.0,
             "advantages": torch.randn(B, 1, generator=g).expand(B, R).contiguous()}
    return {"batch": batch, "meta": {"zorro_train_enable": True, "response_length": R}}


DS = {"zero_optimization": {"stage": 3}, "gradient_clipping": 1.0, "optimizer": {"type": "AdamW", "params": {"lr": 1e-3}}}


@pytest.mark.timeout(600)
def test_client_launched_server_with_two_rank_processes():
    ref = create_arctic_rl_client(ArcticRLClientConfig(comm_protocol="local", model_name="qwen3-tiny", training_gpus=1,
                                                       sampling_gpus=0, log_prob_gpus=0, seed=7, ds_config=DS))
    want = ref.call("fwd_bwd", _payload(), {"loss_fn": "verl_grpo"})
    want_norm = ref.call("step")["metrics"]["grad_norm"]
    ref.call("shutdown")
    cfg = ArcticRLClientConfig(comm_protocol="http", backend="local", host="127.0.0.1", port=_free_port(),
                               model_name="qwen3-tiny", training_gpus=2, sampling_gpus=0, log_prob_gpus=0, seed=7,
                               ds_config=DS, startup_timeout=120)
    c = create_arctic_rl_client(cfg)
    try:
        assert c._proc is not None and c._proc.poll() is None                  # the server is this client's child
        import requests
        base = f"http://127.0.0.1:{cfg.port}"
        jid = c.job_ids["training"]
        assert requests.get(f"{base}/job/{jid}").json()["num_devices"] == 2
        assert requests.get(f"{base}/job/{jid}/workers").json()["alive"] == [True, True]
        got = c.call("fwd_bwd", _payload(), {"loss_fn": "verl_grpo"})
        assert got["avg_loss"] == pytest.approx(want["avg_loss"], rel=1e-4, abs=1e-6)
        assert c.call("step")["metrics"]["grad_norm"] == pytest.approx(want_norm, rel=1e-4)
    finally:
        proc = c._proc
        c.call("shutdown")
    proc.wait(timeout=30)
    assert proc.poll() is not None                                              # server (and with it its ranks) ended
