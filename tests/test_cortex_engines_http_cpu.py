"""Engine-shaped handles of the stand-alone client against a real job server on 127.0.0.1 (tiny model, CPU)."""
import socket
import threading
import time

import pytest
import torch

from arctic_platform_b200.common.http_server import create_app
from arctic_platform_b200.common.server import ArcticRLServerCore
from cortex_client.dss_client import (ArcticInferenceClient, ArcticInferenceEngine, DSSTrainingClient, DSSTrainingEngine,
                                      build_forward_backward_kwargs)
from cortex_client.dss_client.engines import EngineError, loss_mask_from_labels


@pytest.fixture(scope="module")
def server_url():
    import uvicorn
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    srv = uvicorn.Server(uvicorn.Config(create_app(ArcticRLServerCore()), host="127.0.0.1", port=port, log_level="error"))
    t = threading.Thread(target=srv.run, daemon=True)
    t.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    yield f"http://127.0.0.1:{port}"
    srv.should_exit = True
    t.join(timeout=5)


def test_loss_mask_alignment():
    labels = torch.tensor([[5, 6, -100, -100]])
    assert loss_mask_from_labels(labels, shifted=False).tolist() == [[True, True, False, False]]
    assert loss_mask_from_labels(labels, shifted=True).tolist() == [[False, True, True, False]]


def test_training_engine_drives_a_job_like_a_local_engine(server_url, tmp_path):
    engine = DSSTrainingClient(server_url).initialize(
        "qwen3-tiny", {"optimizer": {"type": "AdamW", "params": {"lr": 5e-3}}, "gradient_clipping": 1.0}, {},
        checkpoint_path=str(tmp_path))
    assert isinstance(engine, DSSTrainingEngine) and engine.module is None and engine.model_name == "qwen3-tiny"
    assert engine.is_gradient_accumulation_boundary() and list(engine.parameters()) == []
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(1, 200, (4, 24), generator=g)
    batch = build_forward_backward_kwargs({"input_ids": ids.tolist(), "labels": "input_ids", "attention_mask": True})
    losses = []
    for _ in range(4):
        handle = engine(**batch)
        with pytest.raises(RuntimeError, match="twice"):
            engine(**batch)
        loss = engine.backward(handle)
        assert loss.dim() == 0 and torch.isfinite(loss)
        losses.append(float(loss))
        metrics = engine.step()
        assert metrics["grad_norm"] > 0
    assert engine.global_steps == 4 and engine.lr_scheduler.get_last_lr() == [pytest.approx(5e-3)]
    assert losses[-1] < losses[0]                                     # the same batch four times: the loss goes down
    with pytest.raises(RuntimeError, match="without a batch"):
        engine.backward()
    ev = engine.evaluate(batch)
    assert ev["batch"]["log_probs"].shape[0] == 4
    engine.step(1e-4)
    assert engine.lr_scheduler.get_last_lr() == [pytest.approx(1e-4)]
    with pytest.raises(ValueError):
        engine.step([1e-4, 1e-5])
    with pytest.raises(TypeError):
        engine.step(1)
    saved = engine.save_checkpoint()
    assert saved["path"].endswith("checkpoint-5")
    engine.global_steps = 0
    assert engine.load_checkpoint(step=5)["global_steps"] == 5 and engine.global_steps == 5
    assert engine.job_id in engine.destroy()
    with pytest.raises(EngineError) as e:
        engine.step()
    assert e.value.status in (404, 409)


def test_next_token_labels_move_the_mask(server_url):
    engine = DSSTrainingEngine("qwen3-tiny", {"optimizer": {"params": {"lr": 1e-3}}}, None, server_url, next_token_labels=True)
    try:
        ids = torch.randint(1, 200, (2, 16), generator=torch.Generator().manual_seed(1))
        shifted = build_forward_backward_kwargs({"input_ids": ids.tolist()})                     # next-token labels
        sent = engine._server_batch(shifted)
        assert sent["loss_mask"][:, 0].sum() == 0 and sent["loss_mask"][:, 1:].all()
        a = float(engine.forward_backward(shifted))
        engine.next_token_labels = False
        aligned = build_forward_backward_kwargs({"input_ids": ids.tolist(), "labels": "input_ids"})
        b = float(engine.forward_backward(aligned))
        assert a == pytest.approx(b, rel=1e-5)                        # both forms select the same 15 targets per row
    finally:
        engine.destroy()


def test_inference_engine_generates(server_url):
    eng = ArcticInferenceClient(server_url).initialize("qwen3-tiny", {"max_model_len": 64})
    assert isinstance(eng, ArcticInferenceEngine)
    try:
        res = eng.generate([[1, 2, 3], [4, 5]], {"max_tokens": 4, "temperature": 0.0, "n": 2})
        assert len(res) == 4 and [r["prompt_index"] for r in res] == [0, 0, 1, 1]
        assert all(len(r["token_ids"]) == 4 for r in res)
        mixed = eng.generate([[1, 2, 3], [4, 5], [1, 2, 3]],
                             [{"max_tokens": 2, "temperature": 0.0}, {"max_tokens": 3, "temperature": 0.0}, None])
        assert [r["prompt_index"] for r in mixed] == [0, 1, 2]
        assert len(mixed[0]["token_ids"]) == 2 and len(mixed[1]["token_ids"]) == 3
        assert mixed[0]["token_ids"] == res[0]["token_ids"][:2]      # greedy: the same continuation
        with pytest.raises(ValueError):
            eng.generate([[1]], [{}, {}])
    finally:
        eng.destroy()
