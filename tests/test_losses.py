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


# ----------------------------------------------------------------------------- asynchronous / off-policy pieces
def test_proximal_logp_interpolates_by_staleness():
    old = torch.log(torch.tensor([0.2, 0.2, 0.2, 0.2]))
    cur = torch.log(torch.tensor([0.4, 0.4, 0.4, 0.4]))
    versions = torch.tensor([4, 3, 1, -1])                   # fresh, one behind, three behind, prompt token
    ap = F.proximal_logp_approximations(old, cur, versions, current_version=4)
    alpha = torch.tensor([0.0, 0.0, 2.0 / 3.0, 0.0])
    assert torch.allclose(ap["loglinear"], old + alpha * (cur - old))
    assert torch.allclose(ap["linear"].exp(), (1 - alpha) * 0.2 + alpha * 0.4, atol=1e-6)
    assert torch.equal(ap["rollout"], old)
    assert set(F.proximal_logp_approximations(old, cur, versions, 4, "linear")) == {"linear"}
    # resolution rules
    assert F.resolve_proximal_logp(None, "recompute", old, cur, None, None) is old
    sent = old + 0.01
    assert F.resolve_proximal_logp(sent, "metrics", old, cur, None, None) is sent
    assert torch.allclose(F.resolve_proximal_logp(None, "loglinear", old, cur, versions, 4), ap["loglinear"])
    with pytest.raises(ValueError):
        F.resolve_proximal_logp(None, "loglinear", old, cur, None, 4)
    with pytest.raises(ValueError):
        F.resolve_proximal_logp(None, "metrics", old, cur, versions, 4)
    with pytest.raises(ValueError):
        F.resolve_proximal_logp(None, "other", old, cur, versions, 4)
    with pytest.raises(RuntimeError):
        F.resolve_proximal_logp(torch.tensor([float("nan")] * 4), "recompute", old, cur, None, None)


def test_m2po_mask_drops_the_most_off_policy_tokens_first():
    prox = torch.zeros(6)
    old = torch.tensor([0.1, 2.0, 0.2, 1.0, 0.0, 5.0])      # squared gaps 0.01, 4, 0.04, 1, 0, 25
    mask = torch.tensor([1, 1, 1, 1, 1, 0]).bool()           # the largest gap is already outside the loss
    # means of the suffixes in descending order: all 5 -> 1.01, without 4 -> 0.2625, without 4 and 1 -> 0.0167
    assert F.m2po_mask(old, prox, mask, 2.0).tolist() == [True, True, True, True, True, False]
    assert F.m2po_mask(old, prox, mask, 1.0).tolist() == [True, False, True, True, True, False]
    assert F.m2po_mask(old, prox, mask, 0.1).tolist() == [True, False, True, False, True, False]
    assert F.m2po_mask(old, prox, mask, 1e-9).sum() == 1     # never empties the batch
    none = torch.zeros(6, dtype=torch.bool)
    assert torch.equal(F.m2po_mask(old, prox, none, 0.1), none)
    grid = F.m2po_mask(old.view(2, 3), prox.view(2, 3), mask.view(2, 3), 1.0)
    assert grid.shape == (2, 3) and grid.reshape(-1).tolist() == [True, False, True, True, True, False]


def test_sequence_level_ratio_matches_between_layouts():
    lr = torch.tensor([[0.1, 0.3, 0.0], [-0.2, 0.0, 0.0]])
    adv = torch.tensor([[1.0, 3.0, 9.0], [2.0, 9.0, 9.0]])
    mask = torch.tensor([[1, 1, 0], [1, 0, 0]]).bool()
    r2, a2 = F.sequence_level_ratio_and_advantages(lr, adv, mask)
    assert torch.allclose(r2, torch.tensor([[math.exp(0.2)] * 2 + [0.0], [math.exp(-0.2), 0.0, 0.0]]))
    assert torch.allclose(a2, torch.tensor([[2.0, 2.0, 0.0], [2.0, 0.0, 0.0]]))
    flat = mask.reshape(-1)
    seq_ids = torch.arange(2).repeat_interleave(3)[flat]
    r1, a1 = F.sequence_level_ratio_and_advantages(lr.reshape(-1)[flat], adv.reshape(-1)[flat], torch.ones(3).bool(),
                                                   seq_ids, 2)
    assert torch.allclose(r1, r2.reshape(-1)[flat]) and torch.allclose(a1, a2.reshape(-1)[flat])
    with pytest.raises(ValueError):
        F.sequence_level_ratio_and_advantages(lr.reshape(-1)[flat], adv.reshape(-1)[flat], torch.ones(3).bool())


def test_decoupled_ppo_reduces_to_plain_ppo_on_policy_and_caps_off_policy_tokens():
    torch.manual_seed(1)
    lp = (-torch.rand(8)).requires_grad_()
    old = lp.detach() + 0.2 * torch.randn(8)
    adv = torch.randn(8)
    mask = torch.ones(8).bool()
    loss, stat = F.ppo_actor_loss_fn(lp, old, old, adv, 0.2, mask, c_clip=3.0)
    tok, _, clipped, lower = F.ppo_clip_token_loss(lp, old, adv)
    assert loss.item() == pytest.approx(tok.mean().item(), rel=1e-6)
    assert torch.equal(stat["dual_clip_mask"], lower)
    assert torch.allclose(stat["behave_imp_weight"], torch.ones(8))
    # a proximal policy far from the behaviour policy: weight exp(prox - old), capped tokens contribute nothing
    prox = old.clone()
    prox[0] += math.log(10.0)
    prox[1] += math.log(2.0)
    loss2, stat2 = F.ppo_actor_loss_fn(lp, prox, old, adv, 0.2, mask, behav_imp_weight_cap=5.0)
    assert stat2["behave_imp_weight"][0] == 0 and stat2["behave_imp_weight"][1] == pytest.approx(2.0)
    assert not stat2["behave_mask"][0] and stat2["loss"][0] == 0
    w = torch.full((8,), 0.5)
    loss3, _ = F.ppo_actor_loss_fn(lp, old, old, adv, 0.2, mask, rollout_is_weights=w)
    loss4, _ = F.ppo_actor_loss_fn(lp, old, old, adv, 0.2, mask)
    assert loss3.item() == pytest.approx(0.5 * loss4.item(), rel=1e-6)
    with pytest.raises(ValueError):
        F.ppo_actor_loss_fn(lp, old, old, adv, 0.2, mask, c_clip=0.5)
    with pytest.raises(ValueError):
        F.ppo_actor_loss_fn(lp, old, old, adv, 0.2, mask, importance_sampling_level="word")
    loss.backward()
    assert torch.isfinite(lp.grad).all()


def test_sapo_gate_has_unit_slope_at_ratio_one_and_separate_temperatures():
    lp = torch.zeros(2, requires_grad=True)
    old = torch.zeros(2)
    adv = torch.tensor([1.0, -1.0])
    loss, stat = F.sapo_loss_fn(lp, old, adv, 1.0, 2.0, torch.ones(2).bool())
    # at ratio 1: gate = 4 / tau * 0.5 = 2 / tau
    assert stat["sapo_soft_gate"].tolist() == pytest.approx([2.0, 1.0])
    assert loss.item() == pytest.approx((-2.0 * 1.0 + 1.0 * 1.0) / 2)
    loss.backward()
    # d/dlogp of -(4/tau) sigmoid(tau (e^x - 1)) A at x = 0 is -A for every tau
    assert lp.grad.tolist() == pytest.approx([-0.5, 0.5])
    with pytest.raises(ValueError):
        F.sapo_loss_fn(lp, old, adv, 0.0, 1.0, torch.ones(2).bool())


def test_grpo_loss_options_through_the_registry():
    pb, lp, batch = _rl_inputs()
    out = {"logprobs": lp, "entropy": -lp.detach(), "packed": pb}
    base, m0 = LOSS_FNS["grpo"](out, batch, {}, {}, "cpu")
    # on-policy defaults: proximal == behaviour, so this is the verl-shaped clipped loss without dual clip
    tok, _, _, _ = F.ppo_clip_token_loss(lp, pb.gather_from_grid(batch["old_log_probs"]), pb.gather_from_grid(batch["advantages"]),
                                         clip_c=1e9)
    assert base.item() == pytest.approx(tok.mean().item(), rel=1e-5)
    assert m0["actor/behav_imp_weight.sum"] == pytest.approx(m0["loss.tokens"])
    R = batch["response_mask"].shape[1]
    versions = torch.tensor([[2, 2, 2], [0, 0, 0], [1, 1, 1]])
    # unclipped tokens give exp(lp - prox) * exp(prox - old) = exp(lp - old) whatever the proximal policy is: the
    # proximal policy only moves the centre of the clip, so the difference shows with a tight clip range
    tight, _ = LOSS_FNS["grpo"](out, batch, {}, {"eps_clip": 0.01}, "cpu")
    stale, _ = LOSS_FNS["grpo"](out, {**batch, "versions": versions}, {},
                                {"prox_logp_method": "loglinear", "current_version": 3, "eps_clip": 0.01}, "cpu")
    loose, _ = LOSS_FNS["grpo"](out, {**batch, "versions": versions}, {},
                                {"prox_logp_method": "loglinear", "current_version": 3, "eps_clip": 10.0}, "cpu")
    wide, _ = LOSS_FNS["grpo"](out, batch, {}, {"eps_clip": 10.0}, "cpu")
    assert torch.isfinite(stale) and abs(stale.item() - tight.item()) > 1e-4
    assert loose.item() == pytest.approx(wide.item(), rel=1e-5)
    with pytest.raises(ValueError):
        LOSS_FNS["grpo"](out, batch, {}, {"prox_logp_method": "loglinear", "current_version": 3}, "cpu")
    m2, mm = LOSS_FNS["grpo"](out, {**batch, "prox_log_probs": batch["old_log_probs"] + torch.randn(3, R)}, {},
                              {"m2_threshold": 0.05}, "cpu")
    assert mm["loss.tokens"] < m0["loss.tokens"]
    sapo, ms = LOSS_FNS["grpo"](out, batch, {}, {"use_sapo_loss": True}, "cpu")
    assert torch.isfinite(sapo) and ms["actor/pg_clipfrac.sum"] == 0
    with pytest.raises(ValueError):
        LOSS_FNS["grpo"](out, batch, {}, {"use_sapo_loss": True, "use_decoupled_loss": True}, "cpu")
    seq, _ = LOSS_FNS["grpo"](out, batch, {}, {"importance_sampling_level": "sequence",
                                                "loss_agg_mode": "seq-mean-token-mean"}, "cpu")
    assert torch.isfinite(seq)
    kl, _ = LOSS_FNS["grpo"](out, batch, {}, {"use_kl_loss": True, "kl_loss_coef": 0.5, "entropy_coeff": 0.1}, "cpu")
    assert kl.item() != pytest.approx(base.item())
    with pytest.raises(ValueError):
        LOSS_FNS["grpo"](out, {k: v for k, v in batch.items() if k != "ref_log_prob"}, {}, {"use_kl_loss": True}, "cpu")
    onp, _ = LOSS_FNS["grpo"](out, {k: v for k, v in batch.items() if k != "old_log_probs"}, {}, {}, "cpu")
    adv_tok = pb.gather_from_grid(batch["advantages"])
    assert onp.item() == pytest.approx(-adv_tok.mean().item(), rel=1e-5)       # ratio == 1 everywhere


@pytest.mark.parametrize("mode", ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"])
def test_ownership_split_of_sequences_adds_up_to_the_whole(mode):
    """Sequence parallelism: two ranks hold complementary parts of every sequence's tokens.  With the global
    normalisers the mean of the ranks' losses (factor dp_size = 2 ranks) equals the loss of the whole batch."""
    pb, lp, batch = _rl_inputs()
    meta = {"batch_num_tokens": float(batch["response_mask"].sum()), "global_batch_size": 3.0}
    cfg = {"loss_agg_mode": mode, "kl_loss_coef": 0.01, "use_kl_loss": True}
    whole, _ = LOSS_FNS["verl_grpo"]({"logprobs": lp, "entropy": None, "packed": pb}, batch,
                                     {**meta, "dp_size": 1, "actor_config": cfg}, {}, "cpu")
    n = lp.numel()
    owned0 = torch.arange(n) % 2 == 0
    parts = []
    for owned in (owned0, ~owned0):
        l, m = LOSS_FNS["verl_grpo"]({"logprobs": lp * owned, "entropy": None, "packed": pb, "owned": owned}, batch,
                                     {**meta, "dp_size": 2, "actor_config": cfg}, {}, "cpu")
        parts.append(l)
        assert m["loss.tokens"] == int(owned.sum())
    assert ((parts[0] + parts[1]) / 2).item() == pytest.approx(whole.item(), rel=1e-5, abs=1e-7)
    g, _ = LOSS_FNS["grpo"]({"logprobs": lp * owned0, "entropy": None, "packed": pb, "owned": owned0}, batch,
                            {**meta, "dp_size": 2}, {"loss_agg_mode": mode}, "cpu")
    assert torch.isfinite(g)
    with pytest.raises(NotImplementedError):
        LOSS_FNS["grpo"]({"logprobs": lp, "entropy": None, "packed": pb, "owned": owned0}, batch, {**meta, "dp_size": 2},
                         {"importance_sampling_level": "sequence"}, "cpu")


@pytest.mark.parametrize("mode", ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"])
def test_registered_loss_equals_the_padded_grid_formula_in_every_aggregation_mode(mode):
    pb, lp, batch = _rl_inputs()
    R = batch["response_mask"].shape[1]
    loss, _ = LOSS_FNS["verl_grpo"]({"logprobs": lp, "entropy": None, "packed": pb}, batch,
                                    {"actor_config": {"loss_agg_mode": mode}}, {}, "cpu")
    grid_lp = pb.scatter_to_grid(lp.detach())
    tok, _, _, _ = F.ppo_clip_token_loss(grid_lp, batch["old_log_probs"], batch["advantages"])
    want = F.agg_loss(tok, batch["response_mask"], mode)               # [B, R] layout: the horizon is R
    assert loss.item() == pytest.approx(want.item(), rel=1e-5)
    if mode.endswith("norm"):
        plain, _ = LOSS_FNS["verl_grpo"]({"logprobs": lp, "entropy": None, "packed": pb}, batch,
                                         {"actor_config": {"loss_agg_mode": "seq-mean-token-sum"}}, {}, "cpu")
        assert loss.item() == pytest.approx(plain.item() / R, rel=1e-5)
