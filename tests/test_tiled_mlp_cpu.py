"""Sequence-tiled MLP: identical outputs and gradients to the untiled block, with and without gradient
checkpointing and for a token count that does not divide into the tiles; patch switch and worker config."""
import pytest
import torch

from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.models.tiled_mlp import resolve_shards, tiled_mlp
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def test_resolve_shards():
    assert resolve_shards(0, 100, 16) == 1 and resolve_shards(None, 100, 16) == 1 and resolve_shards(1, 100, 16) == 1
    assert resolve_shards("auto", 100, 16) == 7 and resolve_shards(True, 10, 16) == 1
    assert resolve_shards(4, 100, 16) == 4 and resolve_shards(400, 100, 16) == 100


def test_tiled_function_matches_plain_and_accumulates_weight_grads():
    g = torch.Generator().manual_seed(0)
    w1 = torch.randn(24, 8, generator=g, requires_grad=True)
    w2 = torch.randn(8, 24, generator=g, requires_grad=True)
    fn = lambda t: torch.nn.functional.silu(t @ w1.t()) @ w2.t()
    x = torch.randn(37, 8, generator=g, requires_grad=True)
    up = torch.randn(37, 8, generator=g)
    fn(x).backward(up)
    want = (x.grad.clone(), w1.grad.clone(), w2.grad.clone())
    for t in (x, w1, w2):
        t.grad = None
    calls = []
    counted = lambda t: (calls.append(t.shape[0]), fn(t))[1]
    out = tiled_mlp(x, counted, 5, (w1, w2))
    assert torch.equal(out, fn(x)) and calls == [8, 8, 8, 8, 5]
    out.backward(up)
    assert calls == [8, 8, 8, 8, 5] * 2                              # every tile recomputed once in the backward
    assert torch.allclose(x.grad, want[0], atol=1e-6) and torch.allclose(w1.grad, want[1], atol=1e-5)
    assert torch.allclose(w2.grad, want[2], atol=1e-5)
    with torch.no_grad():
        calls.clear()
        tiled_mlp(x, counted, 5, (w1, w2))
        assert calls == [37]                                         # nothing to save without autograd: one pass


@pytest.mark.parametrize("checkpointing", [False, True])
def test_model_with_tiled_mlp_equals_plain_model(checkpointing):
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=3, seed=6)
    pb = build_packed_batch(ids, mask, R, dedup=True)
    grads = {}
    for shards in (0, 3, "auto"):
        m = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=2)
        m.gradient_checkpointing = checkpointing
        for blk in m.blocks:
            blk.tiled_mlp_shards = shards
        lp, _ = token_logprobs(m, pb)
        lp.mean().backward()
        grads[shards] = (lp.detach().clone(), {n: p.grad.clone() for n, p in m.named_parameters()})
    for shards in (3, "auto"):
        assert torch.equal(grads[shards][0], grads[0][0])
        for n, gref in grads[0][1].items():
            assert torch.allclose(grads[shards][1][n], gref, atol=1e-6, rtol=1e-5), n


def test_patch_switch_and_worker_config():
    from arctic_platform_b200.engine.worker import EngineWorker
    from arctic_platform_b200.models.factory import ModelSpec, PATCH_ORDER, build_model
    assert PATCH_ORDER.index("tiled_mlp") < PATCH_ORDER.index("gradient_checkpointing")
    spec = ModelSpec.from_ds_worker_config("qwen3-tiny", {"tiled_mlp": {"enable": True, "shards": 4}})
    loaded = build_model(spec)
    assert "tiled_mlp" in loaded.applied_patches and all(b.tiled_mlp_shards == 4 for b in loaded.model.blocks)
    off = build_model(ModelSpec.from_ds_worker_config("qwen3-tiny", {"tiled_mlp": {"enable": False}}))
    assert "tiled_mlp" not in off.applied_patches and all(b.tiled_mlp_shards == 0 for b in off.model.blocks)
    assert ModelSpec.from_ds_worker_config("qwen3-tiny", {"tiled_mlp": True}).patches.tiled_mlp == "auto"
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": "training", "ds_worker_config": {"tiled_mlp": 2},
                  "ds_config": {"zero_optimization": {"stage": 1}}})
    assert all(b.tiled_mlp_shards == 2 for b in w.engine.model.blocks)
