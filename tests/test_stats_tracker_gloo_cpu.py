"""Statistics export over two gloo ranks: token-weighted means across ranks, and a rank without any masked element
still completes the export (it contributes neutral elements to every reduction)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _rank(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.rl.processors.stats_tracker import DistributedStatsTracker, ReduceType
        tr = DistributedStatsTracker("actor")
        vals = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]]) + 10 * rank
        mask = torch.tensor([[True, True, False], [True, False, False]]) if rank == 0 else torch.zeros(2, 3, dtype=torch.bool)
        tr.denominator(tokens=mask)
        tr.stat("tokens", kl=vals)                                   # avg + min + max
        tr.stat("tokens", ReduceType.SUM, total=vals)
        tr.stat("tokens", ReduceType.MAX, peak=vals)
        tr.scalar(lr=1e-3 * (rank + 1))
        torch.save(tr.export(reduce_group=None), os.path.join(out_dir, f"s{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_export_with_an_empty_rank():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank, args=(2, port, d), nprocs=2, join=True)
        a, b = (torch.load(os.path.join(d, f"s{r}.pt")) for r in range(2))
    assert a == b                                                     # every rank ends with the global figures
    assert a["actor/tokens"] == 3.0
    assert a["actor/kl/avg"] == pytest.approx((1 + 2 + 4) / 3) and a["actor/kl/min"] == 1.0 and a["actor/kl/max"] == 4.0
    assert a["actor/total"] == 7.0 and a["actor/peak"] == 4.0 and a["actor/lr"] == pytest.approx(1.5e-3)
