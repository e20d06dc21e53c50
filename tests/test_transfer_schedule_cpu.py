"""Static sender -> sampler-worker assignment of a weight transfer, and the coordinator's planning surface."""
import pytest
import torch

from arctic_platform_b200.rl import WeightSyncConfig, WeightSyncCoordinator
from arctic_platform_b200.rl.weight_sync import TransferSchedule


def _cover(s):
    return sorted(w for g in s.groups for w in g.workers)


def test_dp_schedule_partitions_the_workers():
    s = TransferSchedule.build("dp", training_gpus=8, inference_replicas=2, inference_tp=2)
    assert s.num_groups == 4 and s.active_sender_ranks == [0, 1, 2, 3]          # more trainers than workers
    assert _cover(s) == [(0, 0), (0, 1), (1, 0), (1, 1)] and all(g.world_size == 2 for g in s.groups)
    s = TransferSchedule.build("dp", 2, 4, 2)
    assert [g.replica_ids for g in s.groups] == [[0, 1], [2, 3]] and [g.world_size for g in s.groups] == [5, 5]
    assert len(_cover(s)) == len(set(_cover(s))) == 8                           # nobody receives twice
    s = TransferSchedule.build("dp", 3, 5, 1)
    assert [len(g.workers) for g in s.groups] == [2, 2, 1] and _cover(s) == [(r, 0) for r in range(5)]
    assert s.senders_of_worker(4, 0) == [2] and s.group_of_sender(1).workers == ((2, 0), (3, 0)) and s.group_of_sender(7) is None


def test_fsdp_schedule_every_rank_reaches_every_worker():
    s = TransferSchedule.build("fsdp", 4, 2, 2)
    assert s.num_groups == 4 and all(len(g.workers) == 4 and g.world_size == 5 for g in s.groups)
    assert s.senders_of_worker(1, 1) == [0, 1, 2, 3]
    for bad in (("zero", 1, 1, 1), ("dp", 0, 1, 1), ("dp", 1, 1, 0)):
        with pytest.raises(ValueError):
            TransferSchedule.build(*bad)


def test_coordinator_plans_and_syncs():
    cfg = WeightSyncConfig(training_sharding="dp", training_gpus=2, inference_replicas=2, inference_tp=2, base_port=30000)
    planner = WeightSyncCoordinator(cfg)
    assert planner.sender_ranks == [0, 1] and planner.num_groups == 2
    groups = planner.build_groups("10.0.0.1")
    assert [g["master_port"] for g in groups] == [30000, 30002] and groups[1]["replica_ids"] == [1]
    assert groups[0]["world_size"] == 3 and groups[0]["workers"] == [[0, 0], [0, 1]] and groups[0]["master_addr"] == "10.0.0.1"
    with pytest.raises(RuntimeError, match="push function"):
        WeightSyncCoordinator(WeightSyncConfig(training_gpus=1)).sync_weights(0, [("w", torch.ones(2))])
    pushed = []
    co = WeightSyncCoordinator(WeightSyncConfig(training_sharding="dp", training_gpus=1, inference_replicas=1), pushed.extend)
    out = co.sync_weights(0, [("a", torch.ones(2)), ("b", torch.zeros(3))], client=None, master_addr="x")
    assert out == {"num_tensors": 2, "sender": True} and [n for n, _ in pushed] == ["a", "b"]
    co.destroy()


def test_fsdp_shards_from_concurrent_ranks_are_assembled_and_bucketed():
    import threading
    pushes = []
    cfg = WeightSyncConfig(training_sharding="fsdp", training_gpus=2, inference_replicas=1, bucket_size=40)
    co = WeightSyncCoordinator(cfg, lambda bucket: pushes.append([(n, t.clone()) for n, t in bucket]))
    full = {"w": torch.arange(12.0).view(4, 3), "b": torch.arange(6.0)}
    results = {}

    def rank(r):
        shard = [(n, t.chunk(2, 0)[r]) for n, t in full.items()]
        results[r] = co.sync_weights(r, shard, timeout=30.0)

    threads = [threading.Thread(target=rank, args=(r,)) for r in (1, 0)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(30)
    assert results == {0: {"num_tensors": 2, "sender": True}, 1: {"num_tensors": 2, "sender": True}}
    got = {n: t for bucket in pushes for n, t in bucket}
    assert torch.equal(got["w"], full["w"]) and torch.equal(got["b"], full["b"])
    assert len(pushes) == 2                                             # 48 + 24 bytes do not fit one 40-byte bucket
    with pytest.raises(TimeoutError):
        co.sync_weights(0, [("w", full["w"][:2])], timeout=0.05)        # the other rank never arrives
    with pytest.raises(RuntimeError, match="twice"):
        co2 = WeightSyncCoordinator(cfg, pushes.append)
        co2._contrib[0] = {}
        co2.submit(0, [])
