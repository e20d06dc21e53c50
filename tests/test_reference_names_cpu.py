"""Names and helpers a program written against the reference imports beside the client API: padded <-> packed
conversions, logits-level log-prob helpers, tracker / micro-batch / profile helpers, the ``ZoRRoTrain`` class, and the
table of renamed objects that the ``arctic_platform`` alias applies."""
import importlib
import types

import pytest
import torch
import torch.nn.functional as F


def _grid(B=3, P=4, R=5, seed=0):
    g = torch.Generator().manual_seed(seed)
    mask = torch.zeros(B, P + R, dtype=torch.bool)
    for b in range(B):
        p = int(torch.randint(1, P + 1, (1,), generator=g))
        r = int(torch.randint(1, R + 1, (1,), generator=g))
        mask[b, P - p:P] = True              # prompts are left padded
        mask[b, P:P + r] = True              # responses right padded
    vals = torch.randn(B, P + R, generator=g)
    return vals, mask, P, R


def test_padded_grids_and_packed_rows_round_trip():
    from arctic_platform_b200.rl.processors import pipeline as pl

    vals, mask, P, R = _grid()
    row = pl.padded_tensor_2d_to_unpadded_tensor_1d(vals, mask)
    assert row.shape == (1, int(mask.sum()))
    assert torch.equal(row[0], torch.cat([vals[b][mask[b]] for b in range(vals.shape[0])]))
    back = pl.unpadded_tensor_1d_to_padded_tensor_2d(row, mask, pad_value=-7.0)
    assert torch.equal(back[mask], vals[mask]) and bool((back[~mask] == -7.0).all())

    resp = pl.padded_tensor_2d_full_to_unpadded_tensor_1d_response(vals, mask, P)
    assert resp.shape == (1, int(mask[:, P:].sum()))
    full = pl.unpadded_tensor_1d_response_to_padded_tensor_2d_full(resp, mask, P)
    assert full.shape == vals.shape and bool((full[:, :P] == 0).all())
    assert torch.equal(full[:, P:][mask[:, P:]], vals[:, P:][mask[:, P:]])

    d = {"a": vals.clone(), "ids": torch.arange(vals.numel()).view_as(vals), "other": torch.ones(2), "n": 3}
    pl.padded_tensor_2d_dict_to_unpadded_tensor_1d_dict(d, mask.long())           # an integer mask works too
    assert d["a"].shape == d["ids"].shape == row.shape and d["other"].shape == (2,) and d["n"] == 3
    pl.unpadded_tensor_1d_dict_to_padded_tensor_2d_dict(dd := {"a": d["a"]}, mask, 0)
    assert dd["a"].shape == vals.shape
    pl.unpadded_tensor_1d_response_dict_to_padded_tensor_2d_full_dict(rd := {"r": resp}, mask, P)
    assert rd["r"].shape == vals.shape

    with pytest.raises(ValueError, match="packed values"):
        pl.unpadded_tensor_1d_to_padded_tensor_2d(row[:, :-1], mask, 0)

    info = pl.compute_packing_info_for_batch({"attention_mask": mask, "prompts": torch.zeros(vals.shape[0], P)})
    assert info["sequence_offsets"].tolist() == mask.sum(1).cumsum(0).tolist()
    assert info["response_lens"].tolist() == mask[:, P:].sum(1).tolist()


def test_logits_level_helpers_match_log_softmax():
    from arctic_platform_b200.rl.processors.pipeline import (chunked_logprobs_and_entropy_from_logits,
                                                              fast_logprobs_and_entropy_from_logits, logprobs_from_logits)

    torch.manual_seed(0)
    logits = torch.randn(2, 7, 33, requires_grad=True)
    labels = torch.randint(0, 33, (2, 7))
    ls = torch.log_softmax(logits.detach().float(), -1)
    want_lp = ls.gather(-1, labels.unsqueeze(-1)).squeeze(-1)
    want_ent = -(ls.exp() * ls).sum(-1)

    lp = logprobs_from_logits(logits, labels)
    torch.testing.assert_close(lp.detach(), want_lp)
    lp.sum().backward()
    assert logits.grad is not None and torch.isfinite(logits.grad).all()

    lp2, ent2 = fast_logprobs_and_entropy_from_logits(logits.detach(), labels, True)
    torch.testing.assert_close(lp2, want_lp)
    torch.testing.assert_close(ent2, want_ent)
    assert fast_logprobs_and_entropy_from_logits(logits.detach(), labels, False)[1] is None

    # a budget of a few rows: the result does not depend on the block size
    lp3, ent3 = chunked_logprobs_and_entropy_from_logits(logits.detach(), labels, True, peak_mem_gib=3 * 33 * 4 / 2 ** 30)
    torch.testing.assert_close(lp3, want_lp)
    torch.testing.assert_close(ent3, want_ent)


def test_named_trackers_timing_and_export_all():
    from arctic_platform_b200.rl.processors import stats_tracker as st

    st.export_all()                                             # start clean
    with st.record_timing("time/outer"):
        st.scalar(x=2.0)
    tr = st.get("rollout")
    assert st.get("rollout") is tr and "rollout" in st.TRACKERS
    tr.scalar(y=3.0)
    out = st.export_all()
    assert out["x"] == 2.0 and out["rollout/y"] == 3.0 and out["time/outer"] >= 0.0
    assert st.export_all() == {}                                # everything was reset


def test_micro_batch_list_carries_the_reorder_indices():
    from arctic_platform_b200.rl.processors import MicroBatchList, MicroBatchSpec, split_padded_tensor_dict_into_mb_list

    batch = {"attention_mask": torch.tensor([[1, 1, 1, 0], [1, 0, 0, 0], [1, 1, 1, 1], [1, 1, 0, 0]]),
             "input_ids": torch.arange(16).view(4, 4), "tag": "x"}
    res = split_padded_tensor_dict_into_mb_list(batch, MicroBatchSpec(max_tokens_per_mb=5))
    assert isinstance(res, MicroBatchList) and len(res) == len(res.mbs) == 2
    mbs, groups = res                                            # the two-value form keeps working
    assert sorted(i for g in groups for i in g) == [0, 1, 2, 3] and all(t <= 5 for t in res.group_lens)
    cat = torch.cat([m["input_ids"] for m in mbs])
    assert torch.equal(cat[torch.tensor(res.backward_indices)], batch["input_ids"])
    assert torch.equal(batch["input_ids"][torch.tensor(res.forward_indices)], cat)
    assert mbs[0]["tag"] == "x" and res.mb_spec.max_tokens_per_mb == 5


def test_sft_target_count_and_cross_entropy_from_hidden_states():
    from arctic_platform_b200.sft.processor import count_valid_target_tokens, sft_ce_loss, sft_ce_sum_from_hidden, sft_loss

    labels = torch.tensor([[-100, 5, 6, -100], [1, 2, -100, 3]])
    assert count_valid_target_tokens({"labels": labels}) == 4    # column 0 has no predictor
    assert count_valid_target_tokens([{"labels": labels}, {"labels": labels}, {"x": 1}]) == 8
    assert count_valid_target_tokens({"input_ids": labels}) is None and count_valid_target_tokens([{}]) is None
    assert count_valid_target_tokens({"labels": torch.full((1, 3), -100)}) == 0
    assert callable(sft_loss) and callable(sft_ce_loss)

    torch.manual_seed(0)
    model = types.SimpleNamespace(lm_head=types.SimpleNamespace(weight=torch.randn(11, 8, requires_grad=True)))
    hidden = torch.randn(2, 4, 8, requires_grad=True)
    y = torch.tensor([[0, 3, -100, 4], [-100, -100, 9, 10]])
    for mode in ("compute", "memory"):
        ce, n = sft_ce_sum_from_hidden(model, hidden, y, mode=mode, peak_mem_gib=1e-6)
        logits = hidden[:, :-1] @ model.lm_head.weight.t()
        want = F.cross_entropy(logits.reshape(-1, 11).float(), y[:, 1:].reshape(-1), ignore_index=-100, reduction="sum")
        assert n == 4
        torch.testing.assert_close(ce, want, rtol=1e-5, atol=1e-5)
    ce.backward()
    assert hidden.grad is not None and model.lm_head.weight.grad is not None
    with pytest.raises(ValueError, match="mode"):
        sft_ce_sum_from_hidden(model, hidden, y, mode="none")


def test_profile_helpers(monkeypatch, capsys):
    from arctic_platform_b200.utils import sft_profile as prof

    monkeypatch.delenv("ARL_SFT_PROFILE", raising=False)
    assert prof.take_last() == {} and prof.merge_into_metrics({"a": 1}) == {"a": 1}
    prof.maybe_print("off")
    assert capsys.readouterr().out == ""

    monkeypatch.setenv("ARL_SFT_PROFILE", "1")
    prof.snapshot(reset=True)
    with prof.timed("fwd", sync_cuda=False):
        pass
    prof.maybe_print("step 1")
    assert capsys.readouterr().out.startswith("[ARL_SFT_PROFILE] step 1: fwd=")
    merged = prof.merge_into_metrics({"loss": 1.0}, extra={"rpc": 2.5})
    assert merged["loss"] == 1.0 and set(merged["_profile_ms"]) == {"fwd", "rpc"}
    assert prof.take_last() == {}                                # the merge consumed the buckets
    assert prof.format_line({"a": 1.0}) == "a=1.0ms(100%)"


def test_zorro_train_class_entry_points():
    from arctic_platform_b200.rl.zorro_train import ReconstructionInfo, ZoRRoTrain
    from arctic_platform_b200.rl.zorro_train.api import analyze_normal_batch_via_attention_mask
    from arctic_platform_b200.rl.zorro_train.harness import create_dummy_batch

    b = create_dummy_batch(num_prompts=3, rollouts=4)
    ids, mask, R = b["input_ids"], b["attention_mask"], int(b["response_length"])
    P = ids.shape[1] - R
    groups, prompts = ZoRRoTrain.find_prompt_groups(ids, R)
    assert sorted(i for g in groups for i in g) == list(range(12)) and prompts.shape == (3, P)
    for g, members in enumerate(groups):
        assert all(torch.equal(ids[m, :P], prompts[g]) for m in members)

    d_ids, d_pos, info = ZoRRoTrain.create_deduplicated_batch(ids, None, R, groups, prompts, attention_mask=mask)
    assert isinstance(info, ReconstructionInfo) and d_ids.shape == d_pos.shape and d_ids.shape[0] == 1
    assert d_ids.shape[1] == info["total_tokens"] < info["full_tokens"] == int(mask.sum())

    full = ZoRRoTrain.reconstruct_sequences(d_ids, info)
    assert torch.equal(full[0], torch.cat([ids[i][mask[i].bool()] for i in range(12)]))
    assert ZoRRoTrain.get_reconstructed_shape((1, d_ids.shape[1], 16), info) == (1, int(mask.sum()), 16)
    pos_full = ZoRRoTrain.reconstruct_position_ids(d_pos, info)[0]
    want_pos = torch.cat([torch.arange(int(mask[i].sum())) for i in range(12)])
    assert torch.equal(pos_full, want_pos)                       # every sample counts 0..len-1 once reconstructed

    resp = ZoRRoTrain.extract_unpadded_responses_from_deduped_packed_ids(d_ids, info)
    assert torch.equal(resp[0], torch.cat([ids[i, P:][mask[i, P:].bool()] for i in range(12)]))
    grid = ZoRRoTrain.pad_responses(resp, info)
    assert torch.equal(grid * mask[:, P:], ids[:, P:] * mask[:, P:])
    assert torch.equal(ZoRRoTrain.extract_padded_responses_from_deduped_packed_ids(d_ids, info), grid)
    per_sample = ZoRRoTrain.responses_in_orig_sample_order(resp, info)
    assert [t.numel() for t in per_sample] == mask[:, P:].sum(1).tolist()

    h = torch.randn(1, d_ids.shape[1], 4)
    back = ZoRRoTrain.deduplicate_sequences(ZoRRoTrain.reconstruct_sequences(h, info), info, reduce="first")
    assert torch.equal(back, h)
    summed = ZoRRoTrain.deduplicate_sequences(ZoRRoTrain.reconstruct_sequences(torch.ones(1, d_ids.shape[1]), info), info)
    assert summed.max() == 4 and summed.min() == 1               # a shared prompt row gets one gradient per rollout

    layout = ZoRRoTrain.get_group_token_layout(info)
    assert len(layout) == 3 and len(ZoRRoTrain.split_deduplicated_hidden_by_group(h, info)) == 3
    stats = analyze_normal_batch_via_attention_mask(ids, mask, R)
    assert stats["num_groups"] == 3 and stats["dedup_tokens"] == d_ids.shape[1] and 0 < stats["redundancy"] < 1
    with pytest.raises(TypeError):
        ZoRRoTrain.reconstruct_sequences(h, {"not": "info"})


def test_renamed_objects_resolve_through_the_alias():
    from arctic_platform._names import COMPAT_NAMES

    for path, names in COMPAT_NAMES.items():
        mod = importlib.import_module("arctic_platform." + path)
        for name, (where, attr) in names.items():
            assert getattr(mod, name) is getattr(importlib.import_module("arctic_platform_b200." + where), attr), (path, name)

    from arctic_platform.common.deepspeed_worker import DeepSpeedWorker
    from arctic_platform_b200.engine.worker import EngineWorker
    assert DeepSpeedWorker is EngineWorker
    from arctic_platform.rl.zorro_train.zorro_train import ZoRRoTrain
    assert hasattr(ZoRRoTrain, "create_deduplicated_batch")
    with pytest.raises(ImportError):
        from arctic_platform.rl.zorro_train.qwen_attention_patcher import QwenAttentionPatcher  # noqa: F401


def test_helper_packages_export_the_reference_names_lazily():
    import arctic_platform_b200.common as common
    import arctic_platform_b200.common.utils as cu

    for name in cu.__all__:
        assert getattr(cu, name) is not None
    assert {"JobConfig", "ray_split_batch", "http_split_batch", "combine_metric_shards", "merge_cuda_ipc_payloads",
            "record_replay_generation", "SynchronizedWallClockTimerSimple"} <= set(cu.__all__)
    shards, order = cu.ray_split_batch({"batch": {"input_ids": torch.arange(8).view(4, 2)}, "meta": {}}, 2)
    assert order is None and [s["batch"]["input_ids"].shape[0] for s in shards] == [2, 2] and shards[1]["meta"]["dp_size"] == 2
    assert callable(common.init_ray_cluster) and callable(common.primary_ip) and common.EngineWorker.__name__ == "EngineWorker"
    with pytest.raises(AttributeError):
        cu.no_such_name


def test_small_helpers_under_their_reference_names():
    from arctic_platform_b200.models.config import resolve_config
    from arctic_platform_b200.models.decoder import (DecoderLM, get_supported_targets, set_selective_activation_checkpointing,
                                                     supports_selective_activation_checkpointing)
    from arctic_platform_b200.rl.zorro_train.seqlen_balancing import ceildiv, compute_variation, roundup_divisible
    from arctic_platform_b200.testing_utils import apply_print_resets

    assert (ceildiv(7, 2), ceildiv(8, 2), roundup_divisible(7, 4), roundup_divisible(8, 4)) == (4, 4, 8, 8)
    assert compute_variation([1, 2, 3, 10]) == (10, 10.0, 3.0)
    assert apply_print_resets("10%\r50%\rdone\nnext") == "done\nnext"

    model = DecoderLM(resolve_config("qwen3-tiny"))
    blk = model.blocks[0]
    assert supports_selective_activation_checkpointing(blk) and not supports_selective_activation_checkpointing(model)
    have = get_supported_targets(blk)
    assert {"norm", "attn_proj", "mlp"} <= have
    set_selective_activation_checkpointing(blk, ["norm", "linear_attn", "norm"])     # a dense block has no linear_attn
    assert blk.ac_targets == ("norm",)
    with pytest.raises(ValueError, match="Unsupported"):
        set_selective_activation_checkpointing(blk, ["everything"])


def test_state_dict_directory_helpers(tmp_path):
    from arctic_platform_b200.models.hf_io import (get_max_layer_num, load_state_dict, load_state_dict_keys,
                                                   save_state_dict)

    sd = {"model.embed_tokens.weight": torch.randn(6, 4), "model.layers.0.w": torch.randn(4, 4).to(torch.bfloat16),
          "model.layers.11.w": torch.arange(8, dtype=torch.int64), "lm_head.weight": torch.randn(6, 4)}
    assert get_max_layer_num(sd) == 12 and get_max_layer_num({"x": 1}) == 0
    assert get_max_layer_num(sd, layer_prefix="model.language_model.layers.") == 0

    one = save_state_dict(sd, tmp_path / "one")
    assert one == ["model.safetensors"] and sorted(load_state_dict_keys(tmp_path / "one")) == sorted(sd)
    many = save_state_dict(sd, tmp_path / "many", max_shard_bytes=100)
    assert len(many) > 1 and (tmp_path / "many" / "model.safetensors.index.json").is_file()
    assert save_state_dict(sd, tmp_path / "flat", save_sharded=False, max_shard_bytes=100) == ["model.safetensors"]
    for d in ("one", "many", "flat"):
        back = load_state_dict(tmp_path / d)
        assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) and back[k].dtype == sd[k].dtype for k in sd)
    import json
    index = json.loads((tmp_path / "many" / "model.safetensors.index.json").read_text())
    assert set(index["weight_map"]) == set(sd) and set(index["weight_map"].values()) == set(many)

    assert save_state_dict(sd, tmp_path / "pt", save_format="torch") == ["pytorch_model.bin"]
    assert set(torch.load(tmp_path / "pt" / "pytorch_model.bin", weights_only=True)) == set(sd)
    with pytest.raises(ValueError, match="save_format"):
        save_state_dict(sd, tmp_path / "x", save_format="npz")
