"""Two NCCL ranks on two GPUs: the fused NVLink step (peer-load reduce-scatter + clip + AdamW + peer-store
all-gather over symmetric memory) against the torch.distributed collective implementation of the same step.
Skipped on boxes with fewer than two GPUs.  Runs with NVLS off and plain peer loads (no multimem)."""
import os
import socket
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
        from arctic_platform_b200.ops import _lib
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        from tests.test_zorro_equivalence_cpu import make_grpo_batch
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4, p_rng=(40, 200), r_rng=(10, 80), seed=9)
        B = ids.shape[0]
        sl = slice(rank * B // world, (rank + 1) * B // world)
        pb = build_packed_batch(ids[sl], mask[sl], R).to("cuda")
        adv = torch.randn(B, generator=torch.Generator().manual_seed(1))
        n_tok = pb.labels.shape[0]
        a = torch.randn(n_tok, generator=torch.Generator().manual_seed(2 + rank)).cuda()
        res = {}
        for impl in ("fused", "collective"):
            model = DecoderLM(PRESETS["qwen3-tiny-d128"], "cuda", torch.bfloat16).init_weights(seed=11)
            eng = TrainEngine(model, EngineConfig(lr=1e-3, weight_decay=0.01, max_grad_norm=0.5, impl=impl))
            norms = []
            for _ in range(2):
                lp, _ = token_logprobs(eng.model, pb, 1.0)
                eng.backward(-(lp * a).mean())
                norms.append(float(eng.step()["grad_norm"]))
            _lib.check_status(impl)
            res[impl] = (eng.param_buf.tensor.float().cpu(), eng.master.cpu(), norms)
        torch.save(res, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_fused_step_matches_collectives_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(2, port, d), nprocs=2, join=True)
        r0 = torch.load(os.path.join(d, "r0.pt"), weights_only=False)
        r1 = torch.load(os.path.join(d, "r1.pt"), weights_only=False)
    for impl in ("fused", "collective"):
        assert torch.equal(r0[impl][0], r1[impl][0]), f"{impl}: replicas diverged"
    nf, nc = r0["fused"][2], r0["collective"][2]
    assert all(abs(a - b) <= 2e-2 * abs(b) + 1e-4 for a, b in zip(nf, nc)), (nf, nc)
    assert (r0["fused"][1] - r0["collective"][1]).abs().max() < 5e-3
    assert (r0["fused"][0] - r0["collective"][0]).abs().max() < 2e-2
