"""Metric reducers, batch split/merge, checkpoint path helpers, registry."""
import os

import pytest
import torch

from arctic_platform_b200.common import registry
from arctic_platform_b200.common.utils import batch as B
from arctic_platform_b200.common.utils.checkpoint import prune_checkpoint_dirs, resolve_checkpoint_save_paths
from arctic_platform_b200.common.utils.metrics import (combine_metric_microbatches, combine_metric_shards,
                                                       finalize_fwd_bwd_metrics)


def test_shards_collapse_to_global_token_mean():
    shards = [{"loss.sum": 10.0, "loss.tokens": 4, "lr": 1e-3, "tag": "a", "ok": True},
              {"loss.sum": 2.0, "loss.tokens": 8, "lr": 3e-3}]
    out = combine_metric_shards(shards)
    assert out["loss"] == pytest.approx(1.0) and out["lr"] == pytest.approx(2e-3)
    assert out["tag"] == "a" and out["ok"] is True and "loss.sum" not in out
    assert combine_metric_shards([{"x.sum": 1.0, "x.tokens": 0}])["x"] == 0.0
    assert combine_metric_shards([]) == {}
    # an unpaired .sum is an ordinary number
    assert combine_metric_shards([{"y.sum": 2.0}, {"y.sum": 4.0}])["y.sum"] == pytest.approx(3.0)


def test_microbatches_keep_pairs_and_average_rest():
    out = combine_metric_microbatches([{"a.sum": 1.0, "a.tokens": 2, "g": 4.0}, {"a.sum": 3.0, "a.tokens": 2, "g": 2.0}])
    assert out == {"a.sum": 4.0, "a.tokens": 4.0, "g": 3.0}


def test_finalize_prefers_global_loss():
    m, loss = finalize_fwd_bwd_metrics([{"metrics": {"loss.sum": 6.0, "loss.tokens": 3}, "avg_loss": 100.0},
                                        {"metrics": {"loss.sum": 0.0, "loss.tokens": 3}, "avg_loss": 100.0}])
    assert loss == pytest.approx(1.0) and m["loss"] == pytest.approx(1.0)
    _, loss2 = finalize_fwd_bwd_metrics([{"metrics": {}, "avg_loss": 0.5}, {"avg_loss": 0.25}])
    assert loss2 == pytest.approx(0.75)


def test_split_merge_restore_order():
    batch = {"input_ids": torch.arange(24).view(6, 4), "attention_mask": torch.ones(6, 4, dtype=torch.long),
             "response_mask": torch.ones(6, 2), "note": "x"}
    meta = {}
    shards, order = B.split_batch_for_ranks(batch, meta, 3)
    assert order is None and len(shards) == 3 and shards[1]["input_ids"].shape == (2, 4) and shards[2]["note"] == "x"
    assert meta["dp_size"] == 3 and meta["batch_num_tokens"] == 12.0 and meta["global_batch_size"] == 6.0
    merged = B.merge_dict_shards([{"lp": s["input_ids"].float()} for s in shards])
    assert torch.equal(merged["lp"], batch["input_ids"].float())
    perm = torch.tensor([2, 0, 1])
    shuffled = {"v": torch.tensor([30.0, 10.0, 20.0])}          # row i holds original sample perm[i]
    assert torch.equal(B.restore_batch_order(shuffled, perm)["v"], torch.tensor([10.0, 20.0, 30.0]))
    mbs, _ = B.split_batch_for_ranks([batch, batch], {}, 2)
    assert len(mbs) == 2 and len(mbs[0]) == 2 and mbs[1][0]["input_ids"].shape == (3, 4)


def test_position_ids_reconstruction():
    b = {"attention_mask": torch.tensor([[0, 0, 1, 1, 1], [1, 1, 1, 0, 0]])}
    B.reconstruct_position_ids_(b)
    assert b["position_ids"].tolist() == [[0, 0, 0, 1, 2], [0, 1, 2, 0, 0]]


def test_checkpoint_paths_and_pruning(tmp_path):
    # (save_dir, prune_root): a step makes a self-contained child directory, pruning always happens under the root
    assert resolve_checkpoint_save_paths("/x/y", 12) == ("/x/y/checkpoint-12", "/x/y")
    assert resolve_checkpoint_save_paths("/x/y", None) == ("/x/y", "/x/y")
    from arctic_platform_b200.common.utils.checkpoint import resolve_checkpoint_load_path
    (tmp_path / "latest").write_text("20")
    assert resolve_checkpoint_load_path(str(tmp_path), 5, False) == str(tmp_path / "checkpoint-5")
    assert resolve_checkpoint_load_path(str(tmp_path), None, False) == str(tmp_path / "checkpoint-20")
    assert resolve_checkpoint_load_path(str(tmp_path), None, True) == str(tmp_path)      # an explicit path is taken as is
    (tmp_path / "latest").unlink()
    for s in (1, 5, 10, 20):
        (tmp_path / f"checkpoint-{s}").mkdir()
    (tmp_path / "hf").mkdir()
    (tmp_path / "checkpoint-abc").mkdir()
    removed = prune_checkpoint_dirs(str(tmp_path), 2)
    assert sorted(os.path.basename(r) for r in removed) == ["checkpoint-1", "checkpoint-5"]
    assert sorted(p.name for p in tmp_path.iterdir()) == ["checkpoint-10", "checkpoint-20", "checkpoint-abc", "hf"]
    assert prune_checkpoint_dirs(str(tmp_path), 0) == [] and prune_checkpoint_dirs(str(tmp_path / "nope"), 1) == []


def test_registry_lookup_and_dotted_fallback():
    @registry.register_loss_fn("_unit_loss")
    def f(*a):
        return 1

    assert registry.resolve_fn("_unit_loss", registry.LOSS_FNS) is f
    assert registry.resolve_fn(f, registry.LOSS_FNS) is f
    assert registry.resolve_fn("math.sqrt", registry.LOSS_FNS)(4) == 2
    with pytest.raises(KeyError):
        registry.resolve_fn("nope", registry.LOSS_FNS)
    with pytest.raises(KeyError):
        registry.resolve_fn("math.nope", registry.LOSS_FNS)


def test_env_gated_diagnostics(monkeypatch, capsys):
    import torch
    from arctic_platform_b200.common.utils.batch import log_dp_shard_tokens, rank_token_stats
    from arctic_platform_b200.utils import debug
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    batch = {"input_ids": torch.zeros(2, 4, dtype=torch.long), "attention_mask": mask, "response_mask": mask[:, 2:]}
    stats = rank_token_stats(batch, {"batch_num_tokens": 9})
    assert stats == {"valid_tokens": 5, "batch_size": 2, "seq_len_min": 2, "seq_len_max": 3, "response_mask_tokens": 1,
                     "meta_batch_num_tokens": 9}
    assert rank_token_stats({"input_ids": torch.zeros(7, dtype=torch.long), "cu_seqlens": torch.tensor([0, 3, 7])}) == \
        {"cu_seqlens_packed": 7, "packed_tokens": 7}
    monkeypatch.delenv("ARL_LOG_DP_SHARD_TOKENS", raising=False)
    log_dp_shard_tokens(3, "fwd", batch)
    assert capsys.readouterr().out == ""
    monkeypatch.setenv("ARL_LOG_DP_SHARD_TOKENS", "1")
    log_dp_shard_tokens(3, "fwd", batch)
    assert "[3] [DP-shard] fwd: batch_size=2" in capsys.readouterr().out
    # MoE dispatch counters: silent unless switched on, reset by the log call
    monkeypatch.delenv("DSS_MOE_IMBALANCE", raising=False)
    monkeypatch.delenv("APB_MOE_IMBALANCE", raising=False)
    debug.maybe_record_recv_tokens(100)
    assert debug.maybe_log_moe_imbalance(0) is None
    monkeypatch.setenv("DSS_MOE_IMBALANCE", "1")
    for n in (10, 40, 25):
        debug.maybe_record_recv_tokens(n)
    got = debug.maybe_log_moe_imbalance(0)
    assert (got["max_chunk"], got["total"], got["n_dispatch"]) == (40, 75, 3)
    assert debug.maybe_log_moe_imbalance(0)["n_dispatch"] == 0
    # a topology handle inherited from a parent process is dropped, an administrator's path is kept
    monkeypatch.setenv("NCCL_TOPO_FILE", "/proc/self/fd/17")
    assert debug.drop_stale_nccl_topo_file() == "/proc/self/fd/17"
    import os
    assert "NCCL_TOPO_FILE" not in os.environ
    monkeypatch.setenv("NCCL_TOPO_FILE", "/etc/nccl/topo.xml")
    assert debug.drop_stale_nccl_topo_file() is None and os.environ["NCCL_TOPO_FILE"] == "/etc/nccl/topo.xml"


def test_subprocess_runner_and_small_helpers(monkeypatch):
    import sys
    import pytest
    import torch
    from arctic_platform_b200 import testing_utils as tu
    r = tu.execute_subprocess_async([sys.executable, "-c", "import sys; print('hello'); print('warn', file=sys.stderr)"],
                                    quiet=True, echo=False)
    assert r.returncode == 0 and r.stdout == ["hello"] and r.stderr == ["warn"]
    with pytest.raises(RuntimeError, match="returncode 3"):
        tu.execute_subprocess_async([sys.executable, "-c", "import sys; print('x'); sys.exit(3)"], quiet=True, echo=False)
    with pytest.raises(RuntimeError, match="no output"):
        tu.execute_subprocess_async([sys.executable, "-c", "pass"], quiet=True, echo=False)
    with pytest.raises(RuntimeError, match="did not finish"):
        tu.execute_subprocess_async([sys.executable, "-c", "import time; time.sleep(30)"], timeout=1, quiet=True, echo=False)
    m = tu.make_tied_lm_head_model(16, 50)
    assert m.output_weight.shape == (50, 16) and m.lm_head.weight is m.embed and m.config.vocab_size == 50
    monkeypatch.setenv("ARL_GPU_PARTITIONED", "1")
    assert tu.gpu_partitioning_active()
    with tu.gpu_serial_lock():
        pass
    monkeypatch.delenv("ARL_GPU_PARTITIONED")
    assert not tu.gpu_partitioning_active()
    with tu.gpu_serial_lock("apb-test-lock"):
        pass


def test_request_frame_split_and_small_batch_helpers(monkeypatch):
    import io

    from arctic_platform_b200 import wire
    from arctic_platform_b200.common.utils import batch as b
    frame = wire.dumps({"batch": {"input_ids": torch.arange(12).view(4, 3), "response_mask": torch.ones(4, 2)},
                        "meta": {"temperature": 1.0}, "processing": {"loss_fn": "sft"}})
    shards, order = b.http_split_batch(frame, 2)
    assert len(shards) == 2 and order is None and shards[0]["batch"]["input_ids"].shape == (2, 3)
    assert shards[1]["meta"]["dp_size"] == 2 and shards[0]["meta"]["batch_num_tokens"] == 8.0
    assert shards[0]["processing"] == {"loss_fn": "sft"} and shards[0]["meta"] is not shards[1]["meta"]
    assert b.get_reverse_idx([2, 0, 1]) == [1, 2, 0]
    assert b.unpack_batch({"batch": 1, "meta": {"a": 1}, "processing": None}) == ({}, 1, {"a": 1}, None)
    buf = io.StringIO()
    monkeypatch.delenv("ARL_DUMP_PAYLOADS", raising=False)
    b.dump_dict_payload({"x": torch.zeros(2, 3)}, "t", buf)
    assert buf.getvalue() == ""
    monkeypatch.setenv("ARL_DUMP_PAYLOADS", "1")
    b.dump_dict_payload({"x": torch.zeros(2, 3), "y": 5}, "t", buf)
    assert "t: x = tensor(2, 3) torch.float32" in buf.getvalue() and "t: y = 5" in buf.getvalue()
    from arctic_platform_b200.common.utils.batch import combine_metric_shards, finalize_fwd_bwd_metrics
    from arctic_platform_b200.common.utils import metrics
    assert finalize_fwd_bwd_metrics is metrics.finalize_fwd_bwd_metrics and combine_metric_shards is metrics.combine_metric_shards
