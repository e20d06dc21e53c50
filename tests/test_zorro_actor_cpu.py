"""The stand-alone actor harness: deduplicated and plain packing optimise the same objective."""
import pytest
import torch

from arctic_platform_b200.rl.zorro_train.actor import DeduplicatedActor, packed_ppo_policy_loss


def _batch(B=8, n=4, P=9, R=6, V=151, seed=0):
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(1, V, (B // n, P), generator=g).repeat_interleave(n, 0)
    ids = torch.cat([prompts, torch.randint(1, V, (B, R), generator=g)], 1)
    mask = torch.ones_like(ids)
    mask[:n, :3] = 0                                           # first group's prompt is left-padded
    for i in range(B):
        mask[i, P + R - (i % 3):] = 0                          # ragged responses
    return {"input_ids": ids, "attention_mask": mask,
            "old_log_probs": -torch.rand(B, R, generator=g) * 3, "advantages": torch.randn(B, R, generator=g),
            "ref_log_prob": -torch.rand(B, R, generator=g) * 3}


def test_packed_ppo_loss_values():
    lp = torch.tensor([-1.0, -2.0, -0.5])
    old = torch.tensor([-1.2, -1.0, -0.5])
    adv = torch.tensor([1.0, -1.0, 2.0])
    loss, m = packed_ppo_policy_loss(lp, old, adv, clip_ratio=0.2, kl_loss_coef=0.0)
    ratio = torch.exp(lp - old)
    want = torch.maximum(-adv * ratio, -adv * ratio.clamp(0.8, 1.2)).mean()
    assert torch.allclose(loss, want) and abs(m["actor/pg_clipfrac"] - 2 / 3) < 1e-6
    loss2, m2 = packed_ppo_policy_loss(lp, old, adv, ref_log_prob=old, kl_loss_coef=0.5)
    assert torch.allclose(loss2, want + 0.5 * (lp - old).mean()) and "actor/kl_loss" in m2


def test_dedup_actor_equals_plain_actor_and_microbatching_is_exact():
    batch = _batch()
    R = 6
    a = DeduplicatedActor("qwen3-tiny", device="cpu", dtype=torch.float32, dedup=True, max_token_len=10 ** 6)
    b = DeduplicatedActor("qwen3-tiny", device="cpu", dtype=torch.float32, dedup=False, max_token_len=10 ** 6, model=None)
    b.model.load_state_dict(a.model.state_dict())
    fa, fb = a.forward(batch, R, temperature=0.9), b.forward(batch, R, temperature=0.9)
    assert torch.allclose(fa["log_probs"], fb["log_probs"], atol=1e-4) and torch.allclose(fa["entropy"], fb["entropy"], atol=1e-4)
    assert a.last_stats["packed_tokens"] < b.last_stats["packed_tokens"] and b.last_stats["redundancy"] == 0.0
    P = batch["input_ids"].shape[1] - R
    assert float(fa["log_probs"][batch["attention_mask"][:, P:] == 0].abs().max()) == 0.0
    ma = a.compute_policy_loss_and_backward(batch, R, temperature=0.9)
    mb = b.compute_policy_loss_and_backward(batch, R, temperature=0.9)
    assert abs(ma["actor/loss"] - mb["actor/loss"]) < 1e-5
    ga = [p.grad.clone() for p in a.model.parameters()]
    for x, p in zip(ga, b.model.parameters()):
        assert torch.allclose(x, p.grad, atol=2e-5), float((x - p.grad).abs().max())
    # small token budget -> several micro-batches, same accumulated gradient
    for p in a.model.parameters():
        p.grad = None
    a.max_token_len = 40
    mc = a.compute_policy_loss_and_backward(batch, R, temperature=0.9)
    assert mc["actor/num_micro_batches"] > 1 and abs(mc["actor/loss"] - ma["actor/loss"]) < 1e-5
    for x, p in zip(ga, a.model.parameters()):
        assert torch.allclose(x, p.grad, atol=2e-5)


def test_harness_batch_convention_equivalence_and_timing():
    import torch
    from arctic_platform_b200.rl.zorro_train import harness
    b = harness.create_dummy_batch(num_prompts=3, rollouts=4, prompt_len=(6, 20), response_len=(2, 9), vocab_size=500, seed=1)
    ids, mask, R = b["input_ids"], b["attention_mask"], b["response_length"]
    P = ids.shape[1] - R
    assert ids.shape == (12, 29) and R == 9
    for row in mask:                                  # prompts left-padded, responses right-padded
        p, r = row[:P], row[P:]
        assert p.sum() >= 6 and torch.equal(p, p.sort().values) and torch.equal(r, r.sort(descending=True).values)
    assert len({tuple(x[:P].tolist()) for x in ids}) == 3
    report = harness.main(["--model", "qwen3-tiny", "--prompts", "2", "--rollouts", "3", "--prompt-len", "16",
                           "--response-len", "8", "--iters", "1", "--device", "cpu"])
    assert report["max_logprob_diff"] < 1e-4 and report["min_cosine"] > 0.9999 and report["max_rel"] < 1e-3
    assert report["tokens_dedup"] < report["tokens_plain"] and report["plain_ms"] > 0 and report["dedup_ms"] > 0
    same = harness.compare_gradients({"w": torch.ones(3)}, {"w": torch.ones(3)})
    assert same["max_abs"] == 0 and same["min_cosine"] == pytest.approx(1.0)
    assert harness.timed(lambda: None, warmup=0, iters=2) >= 0
