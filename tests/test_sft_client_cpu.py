"""SFT client: configuration rules, the requests it builds (recording transport) and a real loss-decreasing loop through
the in-process engine."""
import pytest
import torch

from arctic_platform_b200.client.transport import JobHandles, Request, Transport
from arctic_platform_b200.sft import ArcticSFTClient, ArcticSFTClientConfig
from arctic_platform_b200.sft.client import SFT_PROCESSING


class FakeTransport(Transport):
    def __init__(self, sampling=True):
        self.jobs = JobHandles(training=7, sampling=8 if sampling else None)
        self.requests = []
        self.closed = False

    def initialize(self):
        return self.jobs

    def call(self, request: Request) -> dict:
        self.requests.append(request)
        return {"results": [{"token_ids": [1]}]} if request.op == "generate" else {"op": request.op}

    async def acall(self, request):
        return self.call(request)

    def shutdown(self):
        self.closed = True


def _cfg(**kw):
    base = dict(comm_protocol="local", model_name="qwen3-tiny", training_gpus=1, checkpoint_path="/tmp/x")
    base.update(kw)
    return ArcticSFTClientConfig(**base)


def test_config_rules():
    with pytest.raises(ValueError, match="training_gpus"):
        _cfg(training_gpus=0)
    with pytest.raises(ValueError, match="checkpoint_path"):
        _cfg(checkpoint_path=None)
    rc = _cfg(training_gpus=0, checkpoint_path=None, training_job_id=3)          # reconnecting needs neither
    assert rc.training_job_id == 3
    with pytest.raises(Exception):
        ArcticSFTClientConfig(comm_protocol="local", model_name="m", training_gpus=1, checkpoint_path="/x", bogus=1)
    rl = _cfg(sampling_gpus=2, colocate=True, max_seq_len=512, ds_config={"gradient_clipping": 2.0}).to_rl_config()
    assert rl.training_gpus == 1 and rl.sampling_gpus == 2 and rl.max_seq_len == 512 and rl.backend.colocate
    assert rl.training.ds_config["gradient_clipping"] == 2.0 and rl.training.checkpoint_path == "/tmp/x"


def test_requests_built_by_every_op():
    t = FakeTransport()
    with ArcticSFTClient(_cfg(sampling_gpus=1), transport=t) as c:
        batch = {"input_ids": torch.ones(2, 4, dtype=torch.long), "labels": torch.ones(2, 4, dtype=torch.long)}
        c.fwd_bwd(batch)
        c.fwd_bwd(batch, {"loss_fn": "sft"})
        c.fwd_no_grad(batch)
        c.step(3e-5)
        c.save_checkpoint("/ck", step=9, export_hf=True, save_total_limit=2)
        c.load_checkpoint(step=9)
        c.generate([[1, 2]], {"max_tokens": 4})
        c.sleep_training("optimizer")
        c.wake_training()
        c.sleep_inference(2)
        c.wake_inference(["weights"])
        c.reset_prefix_cache()
        rc = c.reconnect_config()
    assert t.closed and (rc.training_job_id, rc.sampling_job_id) == (7, 8)
    ops = [r.op for r in t.requests]
    assert ops[:7] == ["forward-backward", "forward-backward", "forward", "step", "save", "load-checkpoint", "generate"]
    assert t.requests[0].body["processing"] == SFT_PROCESSING and t.requests[1].body["processing"] == {"loss_fn": "sft"}
    assert t.requests[2].body["meta"]["plain_packing"] is True and t.requests[2].job_id == 7
    assert t.requests[3].body == {"learning_rate": 3e-5}
    assert t.requests[4].body == {"path": "/ck", "step": 9, "export_hf": True, "save_total_limit": 2}
    assert "sleep-training" in ops and "wake-training" in ops and "sleep-inference" in ops and "wake-inference" in ops
    t2 = FakeTransport(sampling=False)
    with pytest.raises(ValueError, match="No sampling job"):
        ArcticSFTClient(_cfg(), transport=t2).generate([[1]])


def test_sft_loss_decreases_in_process(tmp_path):
    cfg = _cfg(checkpoint_path=str(tmp_path), max_seq_len=32,
               ds_config={"optimizer": {"type": "AdamW", "params": {"lr": 2e-3}}, "gradient_clipping": 1.0})
    g = torch.Generator().manual_seed(0)
    src = torch.randint(3, 50, (4, 8), generator=g)
    ids = torch.cat([src, src], 1)
    labels = ids.clone()
    labels[:, :8] = -100
    batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": labels}
    with ArcticSFTClient(cfg) as c:
        losses = []
        for _ in range(6):
            out = c.fwd_bwd(batch)
            st = c.step()
            losses.append(out["avg_loss"])
            assert st["metrics"]["grad_norm"] > 0
        assert losses[-1] < losses[0]
        saved = c.save_checkpoint(step=6)
        assert saved["tag"].endswith("6")
        nograd = c.fwd_no_grad(batch)
        assert nograd["batch"]["log_probs"].shape[0] == 4
