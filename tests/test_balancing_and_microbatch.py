"""Sequence-length balancing, prompt groups, FFD micro-batching, packing helpers, stats tracker (CPU)."""
import pytest
import torch

from arctic_platform_b200.rl.processors.microbatch import MicroBatchSpec, ffd_allocate, split_padded_tensor_dict_into_mb_list
from arctic_platform_b200.rl.processors.packing import pack_sequences, pad_packed_for_model, unpack_sequences
from arctic_platform_b200.rl.processors.stats_tracker import DistributedStatsTracker, ReduceType
from arctic_platform_b200.rl.zorro_train import seqlen_balancing as sb
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def test_partitions_cover_and_balance():
    sizes = [9, 8, 7, 6, 5, 4, 3, 2, 1, 1, 1, 1]
    for fn in (sb.karmarkar_karp, sb.greedy_partition):
        parts = fn(sizes, 3)
        assert sorted(i for p in parts for i in p) == list(range(len(sizes)))
        loads = [sum(sizes[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= 2
        eq = fn(sizes, 3, equal_size=True)
        assert all(len(p) == 4 for p in eq)
    with pytest.raises(ValueError):
        sb.get_seqlen_balanced_partitions([1, 2], 3)
    stats = sb.log_seqlen_unbalance(sizes, sb.get_seqlen_balanced_partitions(sizes, 4), "x")
    assert stats["x/balance"] > 0.8


def test_prompt_groups_and_reorg():
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4)
    groups = sb.create_prompt_groups(ids, mask, R)
    assert sorted(len(g) for g in groups) == [4, 4, 4, 4]
    assert sorted(len(g) for g in sb.create_prompt_groups(ids, mask, R, max_group_size=3)) == [1] * 4 + [3] * 4
    with pytest.raises(ValueError):
        sb.create_prompt_groups(ids, mask, R, max_token_len=5)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:], "tag": "t"}
    out, order = sb.reorg_global_batch(batch, {"response_length": R}, 2)
    assert sorted(order.tolist()) == list(range(16)) and torch.equal(out["input_ids"], ids[order]) and out["tag"] == "t"
    from arctic_platform_b200.rl.zorro_train.layout import find_prompt_groups
    g0 = set(find_prompt_groups(out["input_ids"][:8], R).tolist())
    assert len(g0) == 2                                    # each rank received exactly two whole groups
    costs = sb.compute_group_costs([[0, 1], [2]], [10, 10, 4], [3, 5, 2], quadratic_weight=0.0)
    assert costs == [18.0, 6.0]


def test_dedup_micro_batches_respect_budget():
    ids, mask, R = make_grpo_batch(n_prompts=3, n_samples=4)
    P = ids.shape[1] - R
    mbs, rows = sb.rearrange_micro_batches_with_dedup({"input_ids": ids, "attention_mask": mask}, R, max_token_len=160)
    assert sorted(i for r in rows for i in r) == list(range(12))
    for mb in mbs:
        gid = sb.find_prompt_groups(mb["input_ids"], R)
        tokens = 0
        for g in set(gid.tolist()):
            sel = (torch.tensor(gid) == g).nonzero().squeeze(-1)
            tokens += int(mb["attention_mask"][sel[0], :P].sum()) + int(mb["attention_mask"][sel, P:].sum())
        assert tokens <= 160


def test_ffd_and_split_by_tokens():
    groups = ffd_allocate([5, 4, 3, 3, 2, 1], 6)
    assert sorted(i for g in groups for i in g) == list(range(6))
    assert all(sum([5, 4, 3, 3, 2, 1][i] for i in g) <= 6 for g in groups)
    assert len(ffd_allocate([1, 1], 10, min_groups=3, divisor=2)) == 4
    with pytest.raises(ValueError):
        ffd_allocate([7], 6)
    mask = torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0], [1, 1, 1, 1], [1, 1, 0, 0]])
    batch = {"input_ids": torch.arange(16).view(4, 4), "attention_mask": mask, "k": 1}
    mbs, idx = split_padded_tensor_dict_into_mb_list(batch, MicroBatchSpec(max_tokens_per_mb=5))
    assert sorted(i for g in idx for i in g) == [0, 1, 2, 3] and all(int(m["attention_mask"].sum()) <= 5 for m in mbs)


def test_pack_unpack_roundtrip():
    ids = torch.tensor([[0, 0, 5, 6], [7, 8, 9, 0]])
    mask = torch.tensor([[0, 0, 1, 1], [1, 1, 1, 0]])
    packed = pack_sequences({"input_ids": ids, "attention_mask": mask, "adv": ids.float() * 2})
    assert packed["input_ids"].tolist() == [[5, 6, 7, 8, 9]] and packed["position_ids"].tolist() == [[0, 1, 0, 1, 2]]
    assert packed["cu_seqlens"].tolist() == [0, 2, 5] and packed["adv"].tolist() == [[10.0, 12.0, 14.0, 16.0, 18.0]]
    padded = pad_packed_for_model(packed, multiple=4)
    assert padded["input_ids"].shape[1] == 8 and padded["cu_seq_lens_q"].tolist() == [0, 2, 5, 8]
    back = unpack_sequences(packed["input_ids"].float(), packed["_pack_meta"], fill=-1.0)
    assert back.tolist() == [[-1.0, -1.0, 5.0, 6.0], [7.0, 8.0, 9.0, -1.0]]


def test_stats_tracker_scopes_and_reduce_types():
    tr = DistributedStatsTracker("actor")
    m = torch.tensor([True, True, False, True])
    tr.denominator(tokens=m)
    tr.stat("tokens", loss=torch.tensor([1.0, 3.0, 100.0, 5.0]))
    with tr.scope("clip"):
        tr.denominator(tokens=m)
        tr.stat("tokens", ReduceType.SUM, n=torch.tensor([1.0, 0.0, 1.0, 1.0]))
    tr.scalar(lr=0.5)
    out = tr.export()
    assert out["actor/tokens"] == 3 and out["actor/loss/avg"] == pytest.approx(3.0)
    assert out["actor/loss/min"] == 1.0 and out["actor/loss/max"] == 5.0
    assert out["actor/clip/n"] == 2.0 and out["actor/lr"] == 0.5
    with pytest.raises(ValueError):
        tr.stat("missing", x=torch.zeros(1))
    with pytest.raises(ValueError):
        tr.denominator(bad=torch.ones(2))


def test_group_token_layout_and_split_by_group():
    import torch
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    from arctic_platform_b200.rl.zorro_train.reconstruct import get_group_token_layout, split_deduplicated_hidden_by_group
    from tests.test_zorro_equivalence_cpu import make_grpo_batch
    ids, mask, R = make_grpo_batch(n_prompts=3, n_samples=3, seed=9)
    pb = build_packed_batch(ids, mask, R, dedup=True)
    layout = get_group_token_layout(pb)
    assert len(layout) == pb.num_groups == 3
    assert sum(g["prompt_tokens"] + sum(g["response_tokens"]) for g in layout) == pb.total_tokens
    assert sorted(b for g in layout for b in g["sample_indices"]) == list(range(ids.shape[0]))
    P = ids.shape[1] - R
    parts = split_deduplicated_hidden_by_group(pb.input_ids, pb)
    for g in parts:
        first = g["sample_indices"][0]
        assert g["prompt_hidden"].tolist() == ids[first, :P][mask[first, :P].bool()].tolist()
        for b, resp in zip(g["sample_indices"], g["response_hiddens"]):
            assert resp.tolist() == ids[b, P:][mask[b, P:].bool()].tolist()      # the right sample's own tokens
    hid = torch.randn(pb.total_tokens, 4)
    parts = split_deduplicated_hidden_by_group(hid, pb)
    assert parts[0]["prompt_hidden"].data_ptr() == hid[layout[0]["prompt_start"]:].data_ptr()      # views, not copies
    import pytest
    with pytest.raises(ValueError):
        split_deduplicated_hidden_by_group(hid[:-1], pb)


def test_reorg_global_batch_for_a_verl_style_super_batch():
    import numpy as np
    import torch
    from arctic_platform_b200.rl.zorro_train.seqlen_balancing import reorg_global_batch_verl
    from tests.test_zorro_equivalence_cpu import make_grpo_batch
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=12, p_rng=(4, 40), r_rng=(2, 30))
    B = ids.shape[0]
    perm = torch.randperm(B, generator=torch.Generator().manual_seed(0))       # groups scattered over the batch

    class Super:
        def __init__(self):
            self.batch = {"input_ids": ids[perm].clone(), "attention_mask": mask[perm].clone(),
                          "tag": torch.arange(B)}
            self.non_tensor_batch = {"uid": np.arange(B), "names": [f"s{i}" for i in range(B)]}
    sb = Super()
    out = reorg_global_batch_verl(sb, R, world_size=2)
    assert out is sb
    order = sb.batch["tag"]
    assert sorted(order.tolist()) == list(range(B))
    assert torch.equal(sb.batch["input_ids"], ids[perm][order]) and sb.non_tensor_batch["uid"].tolist() == order.tolist()
    assert sb.non_tensor_batch["names"] == [f"s{i}" for i in order.tolist()]
    # every prompt group now sits inside one rank's half
    P = ids.shape[1] - R
    for half in (sb.batch["input_ids"][:B // 2], sb.batch["input_ids"][B // 2:]):
        prompts = {tuple(r[:P].tolist()) for r in half}
        assert len(prompts) == 2
    tiny = Super()
    tiny.batch = {k: v[:2] for k, v in tiny.batch.items()}
    before = tiny.batch["tag"].clone()
    assert reorg_global_batch_verl(tiny, R, world_size=2) is tiny and torch.equal(tiny.batch["tag"], before)

    class Reorderable(Super):
        def reorder(self, indices):
            self.seen = indices
    r = Reorderable()
    reorg_global_batch_verl(r, R, world_size=2)
    assert sorted(r.seen.tolist()) == list(range(B))
