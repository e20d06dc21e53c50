"""ParallelDims arithmetic, World parsing and Ulysses sequence parallelism on gloo (2 ranks, CPU)."""
import os
import socket
import tempfile

import numpy as np
import pytest
import torch

from arctic_platform_b200.parallel.parallel_dims import ParallelDims
from arctic_platform_b200.parallel.world import get_world


def test_parallel_dims_groups_and_validation():
    d = ParallelDims(dp_replicate=2, dp_shard=-1, cp=2, pp=1, ep=2, world_size=16)
    assert d.dp_shard == 4 and d.dp_size == 8 and d.seq_len_divisor == 4 and d.fsdp_gradient_divide_factor == 16
    assert d.rank_groups("cp")[:2] == [[0, 1], [2, 3]]
    assert d.rank_groups("dp_shard")[0] == [0, 2, 4, 6] and d.rank_groups("dp_replicate")[0] == [0, 8]
    assert d.rank_groups("dp_shard_cp") == [list(range(8)), list(range(8, 16))]
    assert d.rank_groups("dp_cp") == [list(range(16))]
    assert d.rank_groups("ep")[3] == [6, 7]
    for name in ParallelDims.GROUP_NAMES:                      # every name partitions the ranks
        flat = sorted(r for g in d.rank_groups(name) for r in g)
        assert flat == list(range(16)), name
    assert d.coords(13) == {"pp": 0, "dp_replicate": 1, "dp_shard": 2, "cp": 1, "dp": 6, "ep": 1}
    assert d.group_of("dp", 13) == [1, 3, 5, 7, 9, 11, 13, 15]
    p = ParallelDims(pp=2, world_size=8)
    assert p.dp_shard == 4 and p.rank_groups("pp")[0] == [0, 4]
    with pytest.raises(ValueError):
        ParallelDims(dp_replicate=3, world_size=8)
    with pytest.raises(ValueError):
        ParallelDims(dp_shard=2, cp=2, world_size=8)
    with pytest.raises(ValueError):
        ParallelDims(ep=3, world_size=8)
    with pytest.raises(KeyError):
        d.group("dp")


def test_world_from_env(monkeypatch):
    monkeypatch.setenv("RANK", "11")
    monkeypatch.setenv("WORLD_SIZE", "16")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    monkeypatch.delenv("LOCAL_RANK", raising=False)
    w = get_world(refresh=True)
    assert (w.rank, w.local_rank, w.num_nodes, w.node_rank, w.is_master) == (11, 3, 2, 1, False)
    monkeypatch.setenv("RANK", "16")
    with pytest.raises(ValueError):
        get_world(refresh=True)
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "1")
    get_world(refresh=True)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch():
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    g = torch.Generator().manual_seed(3)
    B, P, R, V = 6, 7, 5, 101
    prompts = torch.randint(1, V, (2, P), generator=g)
    ids = torch.cat([prompts.repeat_interleave(3, 0), torch.randint(1, V, (B, R), generator=g)], 1)
    mask = torch.ones_like(ids)
    mask[1, -2:] = 0
    mask[4, -1:] = 0
    mask[3:, :2] = 0                                  # left-padded second prompt
    return build_packed_batch(ids, mask, R, dedup=True)


def _sp_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.models.config import DecoderConfig
        from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
        from arctic_platform_b200.parallel.ulysses import (apply_sequence_parallelism, head_to_seq, seq_to_head,
                                                           sp_token_logprobs)
        # exchange round trip
        x = torch.arange(rank * 1000, rank * 1000 + 3 * 4 * 2, dtype=torch.float32).view(3, 4, 2)
        y = seq_to_head(x, None)
        assert y.shape == (6, 2, 2) and torch.equal(head_to_seq(y, None), x)
        cfg = DecoderConfig(vocab_size=101, hidden_size=32, intermediate_size=64, num_layers=2, num_heads=4,
                            num_kv_heads=1, head_dim=8, name="sp-test")           # 1 KV head < sp: replication path
        ref = DecoderLM(cfg).init_weights(seed=1)
        spm = DecoderLM(cfg).init_weights(seed=1)
        apply_sequence_parallelism(spm, dist.group.WORLD)
        packed = _batch()
        lp_ref, ent_ref = token_logprobs(ref, packed)
        lp_ref.sum().backward()
        lp, ent, owned = sp_token_logprobs(spm, packed, dist.group.WORLD)
        lp.sum().backward()
        grads = []
        for p in spm.parameters():                              # replicas: gradients add up over the SP group
            g = p.grad.clone() if p.grad is not None else torch.zeros_like(p)
            dist.all_reduce(g)
            grads.append(g)
        err_lp = float((lp - lp_ref[owned]).abs().max())
        err_ent = float((ent - ent_ref[owned]).abs().max())
        err_g = max(float((g - p.grad).abs().max()) for g, p in zip(grads, ref.parameters()))
        cnt = torch.tensor([int(owned.sum())])
        dist.all_reduce(cnt)
        torch.save({"lp": err_lp, "ent": err_ent, "g": err_g, "n": int(cnt), "N": int(packed.labels.numel())},
                   os.path.join(out_dir, f"s{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_ulysses_matches_single_rank_on_gloo():
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_sp_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"s{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        assert r["n"] == r["N"]                       # every prediction row is owned by exactly one rank
        assert r["lp"] < 1e-4 and r["ent"] < 1e-4 and r["g"] < 1e-3, r
