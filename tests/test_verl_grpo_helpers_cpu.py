"""The verl-named building blocks of the GRPO objective against plain PyTorch expressions."""
import pytest
import torch

from arctic_platform_b200.integrations.verl import grpo_loss as gl


def test_vanilla_policy_loss_matches_the_textbook_expression():
    torch.manual_seed(0)
    B, R = 4, 6
    old, new = torch.randn(B, R) * 0.3, torch.randn(B, R) * 0.3
    adv = torch.randn(B, R)
    mask = (torch.rand(B, R) > 0.3).long()
    loss, m = gl.compute_policy_loss_vanilla(old, new, adv, mask)
    ratio = torch.exp(torch.clamp(new - old, -20, 20))
    l1, l2 = -adv * ratio, -adv * torch.clamp(ratio, 0.8, 1.2)
    c1 = torch.maximum(l1, l2)
    per = torch.where(adv < 0, torch.minimum(-adv * 3.0, c1), c1)
    want = (per * mask).sum() / mask.sum()
    torch.testing.assert_close(loss, want)
    n = float(mask.sum())
    assert m["actor/pg_loss.tokens"] == n and m["actor/pg_loss.sum"] == pytest.approx(float((per * mask).sum()), rel=1e-5)
    assert m["actor/pg_clipfrac.sum"] == float(((l2 > l1) & mask.bool()).sum())
    assert m["actor/ppo_kl.sum"] == pytest.approx(float(((old - new) * mask).sum()), rel=1e-5, abs=1e-6)
    # global normalisers and importance weights
    loss2, _ = gl.compute_policy_loss_vanilla(old, new, adv, mask, global_batch_info={"dp_size": 2, "batch_num_tokens": 2 * n},
                                              rollout_is_weights=torch.full((B, R), 0.5))
    torch.testing.assert_close(loss2, 0.5 * want)
    wide = gl.VerlPolicyConfig({"clip_ratio": 0.3, "clip_ratio_c": 5.0, "use_kl_loss": True}, {"loss_mode": "vanilla"})
    assert (wide.clip_ratio_low, wide.clip_ratio_high, wide.clip_ratio_c, wide.use_kl_loss) == (0.3, 0.3, 5.0, True)
    loss3, _ = gl.compute_policy_loss_vanilla(old, new, adv, mask, config=wide)
    assert not torch.allclose(loss3, loss)
    with pytest.raises(ValueError):
        gl.VerlPolicyConfig({"clip_ratio_c": 1.0})


def test_packed_log_probs_move_to_predict_next_positions():
    # two sequences packed: lengths 5 (response 2) and 4 (response 3)
    vals = torch.arange(1.0, 10.0)
    batch = {"sequence_offsets": [5, 9], "response_lens": [2, 3]}
    out = gl.mask_and_pad_for_log_probs(vals, batch)
    assert out.tolist() == [0, 0, 0, 3, 4, 0, 6, 7, 8]
    nested = torch.nested.nested_tensor([vals[:5], vals[5:]], layout=torch.jagged)
    assert torch.equal(gl.mask_and_pad_for_log_probs(nested, batch), out)
    assert torch.equal(gl.shift_log_probs_left(nested, batch), vals) and gl.shift_log_probs_left(vals) is vals
    assert gl.masked_mean(torch.tensor([1.0, 3.0]), torch.tensor([1, 0])) == 1.0
    assert callable(gl.verl_grpo_loss) and callable(gl.kl_penalty)
