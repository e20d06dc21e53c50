"""Expert-parallel MoE over two gloo ranks (collective exchange path) equals the single-process MoE layer:
outputs per rank, input gradients, and expert-weight gradients summed over both ranks' tokens."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(seed=0):
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.moe import MoEFeedForward
    cfg = PRESETS["qwen3-moe-tiny"]
    torch.manual_seed(seed)
    moe = MoEFeedForward(cfg, "cpu", torch.float32)
    with torch.no_grad():
        for p in moe.parameters():
            p.normal_(0, 0.05)
    return cfg, moe


def _inputs(rank):
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randn(37 + 5 * rank, 256, generator=g), torch.randn(37 + 5 * rank, 256, generator=g)


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.parallel.expert_parallel import ExpertParallel
        cfg, moe = _make()
        El = cfg.num_experts // world
        with torch.no_grad():
            moe.wgu = torch.nn.Parameter(moe.wgu.data[rank * El:(rank + 1) * El].clone())
            moe.wdown = torch.nn.Parameter(moe.wdown.data[rank * El:(rank + 1) * El].clone())
        moe.ep = ExpertParallel(cfg.hidden_size, cfg.num_experts, None, "cpu", impl="collective")
        x, g = _inputs(rank)
        x.requires_grad_()
        y = moe(x)
        y.backward(g)
        torch.save({"y": y.detach(), "dx": x.grad, "dwgu": moe.wgu.grad, "dwdown": moe.wdown.grad,
                    "drouter": moe.router.grad}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_matches_single_process():
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(world, _free_port(), d), nprocs=world, join=True)
        outs = [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]
    cfg, moe = _make()
    El = cfg.num_experts // world
    for r in range(world):
        x, g = _inputs(r)
        x.requires_grad_()
        y = moe(x)
        y.backward(g)
        assert torch.allclose(y, outs[r]["y"], atol=1e-5, rtol=1e-4)
        assert torch.allclose(x.grad, outs[r]["dx"], atol=1e-5, rtol=1e-4)
    # gradients accumulated over both ranks' tokens
    for r in range(world):
        assert torch.allclose(moe.wgu.grad[r * El:(r + 1) * El], outs[r]["dwgu"], atol=1e-5, rtol=1e-4)
        assert torch.allclose(moe.wdown.grad[r * El:(r + 1) * El], outs[r]["dwdown"], atol=1e-5, rtol=1e-4)
    assert torch.allclose(moe.router.grad, outs[0]["drouter"] + outs[1]["drouter"], atol=1e-5, rtol=1e-4)
