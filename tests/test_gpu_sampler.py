"""Rollout engine: paged decode (plain and forest-cascade) against full-sequence scoring with the same weights."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(cascade, graph, max_batch=16, **kw):
    from arctic_platform_b200.engine.sampler import SamplerEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    cfg = PRESETS["qwen3-tiny-d128"]
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=5, std=0.05)
    eng = SamplerEngine(cfg, "cuda", model=model, kv_cache_tokens=1 << 14, max_batch=max_batch, max_seq_len=512,
                        cascade=cascade, sync_interval=4, use_cuda_graph=graph, **kw)
    return cfg, model, eng


@pytest.mark.parametrize("cascade,graph,kw", [
    (False, False, {"split_k": False}), (True, False, {"prefix_on_tensor_cores": False, "split_k": False}),
    (True, False, {}), (True, True, {})])
def test_generate_logprobs_match_scoring(cascade, graph, kw):
    """Greedy rollouts: every reported log-prob must equal the model's own log-prob of that token when the
    whole sequence is scored in one packed forward pass, and the token must be the arg-max there."""
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    cfg, model, eng = _engine(cascade, graph, **kw)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, cfg.vocab_size, size=n).tolist() for n in (37, 64, 5)]
    outs = eng.generate(prompts, {"n": 3, "temperature": 0.0, "max_tokens": 21})
    _lib.check_status("generate")
    assert len(outs) == 9
    P, R = 64, 21
    ids = torch.zeros((9, P + R), dtype=torch.int64)
    mask = torch.zeros_like(ids)
    for i, o in enumerate(outs):
        p = prompts[o["prompt_index"]]
        assert o["prompt_len"] == len(p) and len(o["token_ids"]) == R and o["finish_reason"] == "length"
        ids[i, P - len(p):P] = torch.tensor(p)
        mask[i, P - len(p):P] = 1
        ids[i, P:] = torch.tensor(o["token_ids"])
        mask[i, P:] = 1
    # greedy rollouts of one prompt are identical
    assert outs[0]["token_ids"] == outs[1]["token_ids"] == outs[2]["token_ids"]
    pb = build_packed_batch(ids, mask, R, dedup=True).to("cuda")
    with torch.no_grad():
        lp, _ = token_logprobs(model, pb, 1.0)
    got = torch.tensor([o["logprobs"] for o in outs]).reshape(-1)
    ref = pb.scatter_to_grid(lp).cpu().reshape(-1)
    assert (got - ref).abs().max() < 0.08, (got - ref).abs().max()
    assert (got - ref).abs().mean() < 0.01


def test_sampling_is_seeded_and_diverse():
    cfg, model, eng = _engine(True, True, max_batch=32)
    prompt = list(range(10, 60))
    a = eng.generate([prompt], {"n": 8, "temperature": 1.0, "max_tokens": 12, "seed": 7})
    b = eng.generate([prompt], {"n": 8, "temperature": 1.0, "max_tokens": 12, "seed": 7})
    assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]
    assert len({tuple(o["token_ids"]) for o in a}) > 1
    assert eng.pages.free_count() == eng.num_pages


def test_more_sequences_than_slots_and_stop_tokens():
    cfg, model, eng = _engine(True, False, max_batch=8)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, cfg.vocab_size, size=20 + i).tolist() for i in range(7)]
    outs = eng.generate(prompts, {"n": 4, "temperature": 0.0, "max_tokens": 9})
    assert len(outs) == 28 and all(len(o["token_ids"]) == 9 for o in outs)
    first = outs[0]["token_ids"]
    outs2 = eng.generate(prompts[:1], {"n": 1, "temperature": 0.0, "max_tokens": 9, "stop_token_ids": [first[3]]})
    assert outs2[0]["finish_reason"] == "stop" and outs2[0]["token_ids"] == first[:first.index(first[3]) + 1]
