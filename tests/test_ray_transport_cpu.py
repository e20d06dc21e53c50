"""Ray transport of the unified client on a machine without Ray (the server state then lives in process): sync
calls from plain and from async code, async calls, pickling, reconnect without ownership."""
import asyncio
import pickle

import pytest
import torch

from arctic_platform_b200.client.client import SyncArcticRLClient, make_transport
from arctic_platform_b200.client.transport import Request
from arctic_platform_b200.client.transports.ray_actor import RayTransport
from arctic_platform_b200.sft import ArcticSFTClientConfig


def _cfg(tmp_path, **kw):
    base = dict(comm_protocol="ray", model_name="qwen3-tiny", training_gpus=1, checkpoint_path=str(tmp_path),
                max_seq_len=32, ds_config={"optimizer": {"type": "AdamW", "params": {"lr": 1e-3}}})
    base.update(kw)
    return ArcticSFTClientConfig(**base)


def _batch():
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(3, 50, (2, 12), generator=g)
    return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()}


def test_ray_protocol_selects_the_ray_transport_and_trains(tmp_path, monkeypatch):
    monkeypatch.setitem(__import__("sys").modules, "ray", None)            # no Ray: the core is hosted in process
    from arctic_platform_b200.sft import ArcticSFTClient
    with ArcticSFTClient(_cfg(tmp_path)) as c:
        t = c._rl.transport
        assert isinstance(t, RayTransport)
        first = c.fwd_bwd(_batch())["avg_loss"]
        assert c.step()["metrics"]["grad_norm"] > 0
        # the synchronous API from inside a running loop hops to a helper thread instead of nesting loops
        async def from_async_code():
            return c.fwd_no_grad(_batch())
        out = asyncio.run(from_async_code())
        assert out["batch"]["log_probs"].shape[0] == 2
        # the asynchronous entry point
        req = Request("step", t.jobs.training, {})
        assert asyncio.run(t.acall(req))["metrics"]["last_lr"] > 0
        assert first == first
        # a second transport attaches to the same state and jobs, and does not tear them down
        cc = t.config.model_copy(update={"training_job_id": t.jobs.training})
        other = RayTransport(cc, server_state=t.get_server_state())
        assert other.initialize().training == t.jobs.training
        assert other.call(Request("step", t.jobs.training, {}))["metrics"]["grad_norm"] >= 0
        other.shutdown()
        assert c.step()["metrics"]["grad_norm"] >= 0                       # still alive after the guest left
        # pickling drops the private loop and rebuilds it
        state = t.__getstate__()
        assert "_loop" not in state
        clone = RayTransport.__new__(RayTransport)
        clone.__setstate__({k: v for k, v in state.items() if k != "_state"} | {"_state": t.get_server_state()})
        assert clone.call(Request("step", t.jobs.training, {}))["metrics"]["grad_norm"] >= 0
        clone._loop.close()


def test_reconnect_needs_job_ids(tmp_path, monkeypatch):
    monkeypatch.setitem(__import__("sys").modules, "ray", None)
    from arctic_platform_b200.common.server import ArcticRLServerCore
    from arctic_platform_b200.sft import ArcticSFTClient
    with ArcticSFTClient(_cfg(tmp_path)) as c:
        t = c._rl.transport
        guest = RayTransport(t.config, server_state=ArcticRLServerCore())
        with pytest.raises(ValueError, match="needs the job ids"):
            guest.initialize()
        guest.shutdown()
