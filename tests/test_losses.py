"""Loss building blocks and registered losses on small hand-checkable inputs (CPU)."""
import math

import pytest
import torch

from arctic_platform_b200.common.registry import LOSS_FNS
from arctic_platform_b200.rl.processors import functional as F
from arctic_platform_b200.rl.processors import losses  # noqa: F401
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch


def test_masked_reductions_ignore_nan_outside_mask():
    v = torch.tensor([[1.0, float("nan")], [3.0, 5.0]])
    m = torch.tensor([[1, 0], [1, 1]])
    assert F.masked_sum(v, m).item() == 9.0
    assert F.masked_mean(v, m).item() == pytest.approx(3.0)
    assert F.masked_sum(v, m, axis=1).tolist() == [1.0, 8.0]


@pytest.mark.parametrize("mode", ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"])
def test_agg_loss_modes_padded_equals_packed(mode):
    loss = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0], [7.0, 8.0, 9.0]])
    mask = torch.tensor([[1, 1, 0], [1, 1, 1], [0, 0, 0]])
    padded = F.agg_loss(loss, mask, mode)
    flat_mask = mask.reshape(-1).bool()
    seq_ids = torch.arange(3).repeat_interleave(3)[flat_mask]
    packed = F.agg_loss(loss.reshape(-1)[flat_mask], torch.ones(int(flat_mask.sum())), mode, seq_ids=seq_ids, num_seqs=3,
                        loss_scale_factor=3 if mode.endswith("norm") else None)
    expect = {"token-mean": 18.0 / 5, "seq-mean-token-sum": (3.0 + 15.0) / 2, "seq-mean-token-mean": (1.5 + 5.0) / 2,
              "seq-mean-token-sum-norm": (3.0 + 15.0) / 2 / 3}[mode]
    assert padded.item() == pytest.approx(expect) and packed.item() == pytest.approx(expect)


def test_agg_loss_global_normalisers_and_errors():
    loss, mask = torch.ones(2, 2), torch.ones(2, 2)
    assert F.agg_loss(loss, mask, "token-mean", dp_size=2, batch_num_tokens=8).item() == pytest.approx(1.0)
    with pytest.raises(ValueError):
        F.agg_loss(loss, mask, "token-mean", dp_size=2)
    with pytest.raises(ValueError):
        F.agg_loss(loss, mask, "nope")


def test_kl_estimators_and_straight_through():
    lp = torch.tensor([-1.0, -2.0], requires_grad=True)
    ref = torch.tensor([-1.5, -1.0])
    assert torch.allclose(F.kl_penalty(lp, ref, "k1"), lp - ref)
    assert torch.allclose(F.kl_penalty(lp, ref, "abs"), (lp - ref).abs())
    assert torch.allclose(F.kl_penalty(lp, ref, "k2"), 0.5 * (lp - ref) ** 2)
    k3 = F.kl_penalty(lp, ref, "low_var_kl")
    d = ref - lp
    assert torch.allclose(k3, torch.exp(d) - d - 1)
    st = F.kl_penalty(lp, ref, "k3+")
    assert torch.allclose(st, k3)
    st.sum().backward()
    assert torch.allclose(lp.grad, (lp - ref).detach())          # gradient of the k2 estimator


def test_ppo_dual_clip_cases():
    old = torch.zeros(4)
    lp = torch.log(torch.tensor([1.5, 0.5, 5.0, 1.0]))
    adv = torch.tensor([1.0, 1.0, -1.0, 2.0])
    loss, _, clipped, lower = F.ppo_clip_token_loss(lp, old, adv)
    assert loss.tolist() == pytest.approx([-1.2, -0.5, 3.0, -2.0])
    assert clipped.tolist() == [True, False, False, False] and lower.tolist() == [False, False, True, False]


def _rl_inputs():
    ids = torch.tensor([[0, 5, 6, 7, 8, 9], [0, 5, 6, 7, 3, 0], [4, 4, 4, 2, 2, 2]])
    mask = torch.tensor([[0, 1, 1, 1, 1, 1], [0, 1, 1, 1, 1, 0], [1, 1, 1, 1, 1, 1]])
    R = 3
    pb = build_packed_batch(ids, mask, R, dedup=True)
    n = pb.labels.numel()
    torch.manual_seed(0)
    lp = (-torch.rand(n)).requires_grad_()
    batch = {"response_mask": mask[:, -R:], "old_log_probs": pb.scatter_to_grid(lp.detach() + 0.1 * torch.randn(n)),
             "advantages": torch.tensor([[1.0], [-1.0], [0.5]]).expand(3, R).contiguous(),
             "ref_log_prob": pb.scatter_to_grid(lp.detach() - 0.05)}
    return pb, lp, batch


def test_verl_grpo_matches_padded_formula():
    pb, lp, batch = _rl_inputs()
    meta = {"actor_config": {"use_kl_loss": True, "kl_loss_coef": 0.01, "kl_loss_type": "low_var_kl",
                             "entropy_coeff": 0.001}}
    ent = torch.rand(lp.numel())
    loss, metrics = LOSS_FNS["verl_grpo"]({"logprobs": lp, "entropy": ent, "packed": pb}, batch, meta, {}, "cpu")
    grid, m = pb.scatter_to_grid(lp), batch["response_mask"].bool()
    tok, _, _, _ = F.ppo_clip_token_loss(grid, batch["old_log_probs"], batch["advantages"])
    n = m.sum()
    expect = ((tok * m).sum() - 0.001 * (pb.scatter_to_grid(ent) * m).sum()
              + 0.01 * (F.kl_penalty(grid, batch["ref_log_prob"], "low_var_kl") * m).sum()) / n
    assert loss.item() == pytest.approx(expect.item(), rel=1e-5)
    assert metrics["loss.tokens"] == n.item() and metrics["loss.sum"] / n.item() == pytest.approx(loss.item(), rel=1e-5)
    for k in ("actor/pg_loss", "actor/pg_clipfrac", "actor/ppo_kl", "actor/pg_clipfrac_lower", "actor/entropy_loss", "kl_loss"):
        assert k + ".sum" in metrics and k + ".tokens" in metrics
    loss.backward()
    assert lp.grad is not None and torch.isfinite(lp.grad).all()


def test_verl_grpo_is_split_invariant():
    """Summing shard losses computed with global normalisers reproduces the unsplit loss (per-rank mean x dp)."""
    pb, lp, batch = _rl_inputs()
    full, _ = LOSS_FNS["verl_grpo"]({"logprobs": lp, "entropy": None, "packed": pb}, batch, {}, {}, "cpu")
    ntok = float(batch["response_mask"].sum())
    meta = {"dp_size": 3, "batch_num_tokens": ntok, "global_batch_size": 3.0}
    ids = torch.tensor([[0, 5, 6, 7, 8, 9], [0, 5, 6, 7, 3, 0], [4, 4, 4, 2, 2, 2]])
    mask = torch.tensor([[0, 1, 1, 1, 1, 1], [0, 1, 1, 1, 1, 0], [1, 1, 1, 1, 1, 1]])
    total = 0.0
    grid = pb.scatter_to_grid(lp.detach())
    for b in range(3):
        sub = build_packed_batch(ids[b:b + 1], mask[b:b + 1], 3)
        sub_lp = sub.gather_from_grid(grid[b:b + 1])
        sb = {k: v[b:b + 1] for k, v in batch.items()}
        l, _ = LOSS_FNS["verl_grpo"]({"logprobs": sub_lp, "entropy": None, "packed": sub}, sb, dict(meta), {}, "cpu")
        total += l.item() / 3
    assert total == pytest.approx(full.item(), rel=1e-5)


def test_grpo_and_sft_losses_run():
    pb, lp, batch = _rl_inputs()
    loss, metrics = LOSS_FNS["grpo"]({"logprobs": lp, "entropy": None, "packed": pb}, batch,
                                     {"actor_config": {"eps_clip": 0.2, "c_clip": 3.0, "behav_imp_weight_cap": 5.0}}, {}, "cpu")
    assert torch.isfinite(loss) and metrics["loss.tokens"] > 0
    from arctic_platform_b200.rl.zorro_train.layout import build_plain_packed
    ids = torch.tensor([[3, 4, 5, 6], [7, 8, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 1], [1, 1, 0, 0]])
    sp = build_plain_packed(ids, mask)
    slp = -torch.arange(1.0, sp.labels.numel() + 1)
    l_mean, m1 = LOSS_FNS["sft"]({"logprobs": slp, "packed": sp}, {"labels": ids}, {}, {}, "cpu")
    assert l_mean.item() == pytest.approx(slp.neg().mean().item()) and m1["loss.tokens"] == 4
    l_ce, _ = LOSS_FNS["sft_ce"]({"logprobs": slp, "packed": sp}, {"labels": ids}, {"dp_size": 2, "batch_num_tokens": 8}, {}, "cpu")
    assert l_ce.item() == pytest.approx(slp.neg().sum().item() / 8 * 2)
    masked = {"labels": torch.full_like(ids, -100)}
    l0, m0 = LOSS_FNS["sft"]({"logprobs": slp, "packed": sp}, masked, {}, {}, "cpu")
    assert l0.item() == 0.0 and m0["loss.tokens"] == 0
