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


def _tp_ep_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.moe import MoEFeedForward
        from arctic_platform_b200.ops import _lib
        from arctic_platform_b200.parallel import tensor_parallel as tp
        from arctic_platform_b200.parallel.expert_parallel import ExpertParallel
        dev = torch.device("cuda", rank)
        res = {}
        # ---- tensor parallel: all-gather -> GEMM and GEMM -> reduce-scatter fused kernels vs NCCL + matmul
        ctx = tp.TPContext(dev, None, max_rows=512, max_cols=4096)
        g = torch.Generator(device="cuda").manual_seed(5)
        for rows in (64, 256):
            K, N = 512, 768
            x_full = torch.randn(world * rows, K, device=dev, generator=g).bfloat16()
            w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
            x_local = x_full[rank * rows:(rank + 1) * rows].contiguous()
            for _ in range(2):                                   # twice: buffers and epochs are reused
                got = tp.ag_gemm(ctx, x_local, w)
            ref = tp.ag_gemm_collective(x_local, w)
            res[f"ag{rows}"] = float((got.float() - ref.float()).abs().max())
            M = world * rows
            xk = torch.randn(M, K, device=dev, generator=torch.Generator(device="cuda").manual_seed(7 + rank)).bfloat16()
            for _ in range(3):
                got = tp.gemm_rs(ctx, xk, w)
            ref = tp.gemm_rs_collective(xk, w)
            res[f"rs{rows}"] = float((got.float() - ref.float()).abs().max())
            res[f"rs{rows}_scale"] = float(ref.float().abs().max())
        # ---- expert parallel: fused dispatch/combine (training path and fused-epilogue inference path)
        cfg = PRESETS["qwen3-moe-tiny"]
        torch.manual_seed(0)
        full = MoEFeedForward(cfg, dev, torch.bfloat16)
        with torch.no_grad():
            for p in full.parameters():
                p.normal_(0, 0.05)
        El = cfg.num_experts // world
        ep_moe = MoEFeedForward(cfg, dev, torch.bfloat16)
        with torch.no_grad():
            ep_moe.router.copy_(full.router)
            ep_moe.wgu = torch.nn.Parameter(full.wgu.data[rank * El:(rank + 1) * El].clone())
            ep_moe.wdown = torch.nn.Parameter(full.wdown.data[rank * El:(rank + 1) * El].clone())
        ep_moe.ep = ExpertParallel(cfg.hidden_size, cfg.num_experts, None, dev, max_recv_rows=4096, max_pairs=4096)
        x = torch.randn(300 + 40 * rank, cfg.hidden_size, device=dev,
                        generator=torch.Generator(device="cuda").manual_seed(20 + rank)).bfloat16()
        gy = torch.randn_like(x)
        x1 = x.clone().requires_grad_()
        y_ep = ep_moe(x1)
        y_ep.backward(gy)
        x2 = x.clone().requires_grad_()
        y_full = full(x2)
        y_full.backward(gy)
        with torch.no_grad():
            y_inf = ep_moe(x)                                      # GEMM-2 epilogue scatters to the source ranks
        res["ep_y"] = float((y_ep.float() - y_full.float()).abs().max())
        res["ep_inf"] = float((y_inf.float() - y_full.float()).abs().max())
        res["ep_dx"] = float((x1.grad.float() - x2.grad.float()).abs().max())
        res["ep_scale"] = float(y_full.float().abs().max())
        # expert weight gradients: this rank's shard must equal the sum over ranks of the full model's gradient
        gfull = full.wdown.grad.float().clone()
        dist.all_reduce(gfull)
        res["ep_dw"] = float((ep_moe.wdown.grad.float() - gfull[rank * El:(rank + 1) * El]).abs().max())
        res["ep_dw_scale"] = float(gfull.abs().max())
        # the gate/up gradient reads the rows RECEIVED in the forward (saved for backward): they must not alias the
        # receive buffer, which the backward's own exchange overwrites
        gfull_gu = full.wgu.grad.float().clone()
        dist.all_reduce(gfull_gu)
        res["ep_dwgu"] = float((ep_moe.wgu.grad.float() - gfull_gu[rank * El:(rank + 1) * El]).abs().max())
        res["ep_dwgu_scale"] = float(gfull_gu.abs().max())
        _lib.check_status("tp/ep")
        torch.save(res, os.path.join(out_dir, f"t{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_tensor_parallel_and_expert_parallel_fused_kernels():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_tp_ep_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"t{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        for rows in (64, 256):
            assert r[f"ag{rows}"] < 0.05, r
            assert r[f"rs{rows}"] < 0.02 * r[f"rs{rows}_scale"] + 0.05, r
        assert r["ep_y"] < 0.03 * r["ep_scale"] + 0.02, r
        assert r["ep_inf"] < 0.03 * r["ep_scale"] + 0.02, r
        assert r["ep_dx"] < 0.05, r
        assert r["ep_dw"] < 0.03 * r["ep_dw_scale"] + 0.02, r
        assert r["ep_dwgu"] < 0.03 * r["ep_dwgu_scale"] + 0.02, r


def _zero3_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
        from arctic_platform_b200.ops import _lib
        from arctic_platform_b200.parallel.weight_sync import sync_flat
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        from tests.test_zorro_equivalence_cpu import make_grpo_batch
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=4, p_rng=(40, 200), r_rng=(10, 80), seed=9)
        B = ids.shape[0]
        sl = slice(rank * B // world, (rank + 1) * B // world)
        half = (sl.stop - sl.start) // 2
        mbs = [build_packed_batch(ids[m], mask[m], R).to("cuda")
               for m in (slice(sl.start, sl.start + half), slice(sl.start + half, sl.stop))]
        res = {}
        import dataclasses
        cfg5 = dataclasses.replace(PRESETS["qwen3-tiny-d128"], num_layers=5)   # enough blocks for the 3 staging buffers
        for name, stage, impl, overlap in (("z1", 1, "fused", True), ("z3", 3, "fused", True), ("z3n", 3, "fused", False),
                                           ("z3c", 3, "collective", True)):
            model = DecoderLM(cfg5, "cuda", torch.bfloat16).init_weights(seed=11)
            eng = TrainEngine(model, EngineConfig(lr=1e-3, weight_decay=0.01, max_grad_norm=0.5, impl=impl, zero_stage=stage,
                                                  zero3_overlap_comm=overlap))
            if stage == 3:
                # gradients reduced block by block during backward (three staging buffers) vs one full-size buffer
                assert (eng.grad_stage is not None) == (name == "z3")
            norms, losses = [], []
            for _step in range(2):
                for i, pb in enumerate(mbs):                      # two micro-batches per step (slots are re-gathered)
                    a = torch.randn(pb.labels.shape[0], generator=torch.Generator().manual_seed(2 + rank + 10 * i)).cuda()
                    lp, _ = token_logprobs(eng.model, pb, 1.0)
                    loss = -(lp * a).mean()
                    eng.backward(loss)
                    losses.append(float(loss))
                norms.append(float(eng.step()["grad_norm"]))
            with torch.no_grad():
                lp_after, _ = token_logprobs(eng.model, mbs[0], 1.0)
            full = eng.full_flat_params().float().cpu()
            if stage == 3:
                dst = torch.zeros(eng.total, dtype=torch.bfloat16, device="cuda")
                sync_flat(eng, dst)
                assert torch.equal(dst.float().cpu(), full)
                assert eng.zero3.shard_buf.tensor.numel() * world <= eng.total
            _lib.check_status(name)
            res[name] = (full, norms, losses, lp_after.float().cpu(), eng.weight_norm()["norm"])
        torch.save(res, os.path.join(out_dir, f"z{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_zero3_sharded_parameters_match_replicated_on_two_gpus():
    """Stage 3 (sharded bf16 parameters, units pulled from peers on a side stream, per-piece P2P reduce) against the
    replicated stage-1 engine: same losses, gradient norms, updated weights and weight norm."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_zero3_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"z{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        for other in ("z3", "z3n", "z3c"):
            assert all(abs(a - b) <= 2e-2 * abs(b) + 1e-4 for a, b in zip(r[other][1], r["z1"][1])), (r[other][1], r["z1"][1])
            assert all(abs(a - b) <= 2e-2 * abs(b) + 2e-3 for a, b in zip(r[other][2], r["z1"][2]))
            assert (r[other][0] - r["z1"][0]).abs().max() < 2e-2
            assert (r[other][3] - r["z1"][3]).abs().max() < 0.05
            assert abs(r[other][4] - r["z1"][4]) <= 1e-3 * r["z1"][4]
    assert torch.equal(res[0]["z3"][0], res[1]["z3"][0])


def _ulysses_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import copy
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
        from arctic_platform_b200.ops import _lib
        from arctic_platform_b200.parallel.ulysses import apply_sequence_parallelism, sp_token_logprobs
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        from tests.test_zorro_equivalence_cpu import make_grpo_batch
        cfg = PRESETS["qwen3-tiny-d128"]
        ref = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=4)
        spm = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=4)
        apply_sequence_parallelism(spm, dist.group.WORLD)
        ids, mask, R = make_grpo_batch(n_prompts=3, n_samples=3, p_rng=(60, 200), r_rng=(10, 90), seed=6)
        pb = build_packed_batch(ids, mask, R).to("cuda")
        lp_ref, _ = token_logprobs(ref, pb)
        lp_ref.sum().backward()
        lp, _, owned = sp_token_logprobs(spm, copy.copy(pb), dist.group.WORLD)
        lp.sum().backward()
        _lib.check_status("ulysses")
        err_lp = float((lp - lp_ref[owned]).abs().max())
        cos = []
        for p, q in zip(spm.parameters(), ref.parameters()):
            g = p.grad.float().clone() if p.grad is not None else torch.zeros_like(p, dtype=torch.float32)
            dist.all_reduce(g)
            cos.append(float(torch.nn.functional.cosine_similarity(g.flatten(), q.grad.float().flatten(), dim=0)))
        n = torch.tensor([int(owned.sum())], device="cuda")
        dist.all_reduce(n)
        torch.save({"lp": err_lp, "cos": min(cos), "n": int(n), "N": int(pb.labels.numel())}, os.path.join(out_dir, f"u{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_ulysses_sequence_parallel_on_two_gpus():
    """Head <-> sequence all-to-all around the tcgen05 segment attention: log-probs and (summed) gradients of the
    sequence-parallel model equal the single-GPU model's."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_ulysses_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"u{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        assert r["n"] == r["N"] and r["lp"] < 0.08 and r["cos"] > 0.97, r


def _ep_train_main(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
        from arctic_platform_b200.ops import _lib
        from arctic_platform_b200.parallel.expert_parallel import attach_expert_parallel
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        from tests.test_zorro_equivalence_cpu import make_grpo_batch
        cfg = PRESETS["qwen3-moe-tiny"]
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, p_rng=(40, 160), r_rng=(10, 60), seed=12)
        ids = ids % cfg.vocab_size
        B = ids.shape[0]
        sl = slice(rank * B // world, (rank + 1) * B // world)
        pb = build_packed_batch(ids[sl], mask[sl], R).to("cuda")
        a = torch.randn(pb.labels.shape[0], generator=torch.Generator().manual_seed(7 + rank)).cuda()
        res = {}
        for name, impl, stage in (("fused", "fused", 1), ("collective", "collective", 1), ("fused_z3", "fused", 3)):
            model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=8, std=0.05)
            attach_expert_parallel(model, world, impl=impl, max_recv_rows=8192, max_pairs=8192)
            eng = TrainEngine(model, EngineConfig(lr=1e-3, max_grad_norm=1.0, impl=impl, zero_stage=stage))
            norms = []
            for _ in range(2):
                lp, _ = token_logprobs(eng.model, pb)
                eng.backward(-(lp * a).mean())
                norms.append(float(eng.step()["grad_norm"]))
            _lib.check_status(name)
            res[name] = (eng.full_flat_params().float().cpu(), norms, eng.weight_norm()["norm"])
        torch.save(res, os.path.join(out_dir, f"p{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_expert_parallel_training_fused_matches_collective_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_ep_train_main, args=(2, _free_port(), d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"p{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        for other in ("fused", "fused_z3"):
            assert all(abs(x - y) <= 3e-2 * abs(y) + 1e-4 for x, y in zip(r[other][1], r["collective"][1])), (other, r[other][1], r["collective"][1])
            assert (r[other][0] - r["collective"][0]).abs().mean() < 2e-4
            assert abs(r[other][2] - r["collective"][2]) <= 2e-3 * r["collective"][2]


def _tp_paged_main(rank, world, port, out_dir):
    """Tensor-parallel replica of the paged CUDA engine (head shards of the KV cache, GEMM -> reduce-scatter and
    norm -> all-gather kernels in the decode loop) fed by the one-kernel weight hand-over from a ZeRO-3 trainer."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from arctic_platform_b200.engine.sampler import SamplerEngine
        from arctic_platform_b200.engine.worker import EngineWorker
        from arctic_platform_b200.models.config import PRESETS
        from arctic_platform_b200.models.decoder import DecoderLM
        from arctic_platform_b200.models.hf_io import iter_hf_tensors, load_hf_tensor
        from arctic_platform_b200.ops import _lib
        from arctic_platform_b200.parallel.tp_sampler import tp_config, tp_slice
        cfg = PRESETS["qwen3-tiny-d128"]
        job = {"model_name": "qwen3-tiny-d128", "seed": 5,
               "ds_config": {"zero_optimization": {"stage": 3}, "optimizer": {"params": {"lr": 1e-3}}}}
        tr, sm = EngineWorker(), EngineWorker()
        tr.initialize({**job, "job_type": "training"})
        sm.initialize({**job, "job_type": "sampling", "seed": 77,        # other weights: everything must arrive by the sync
                       "vllm_config": {"kv_cache_tokens": 1 << 14, "max_num_seqs": 16, "max_model_len": 512,
                                       "tensor_parallel_size": world}})
        assert isinstance(sm.sampler, SamplerEngine) and sm.sampler.tp == world
        n = tr.sync_weights_to(sm)
        _lib.check_status("tp sync")
        assert n > 0 and sm.sampler._sync_plan is not None
        # exact bf16 equality with the name-based slices of the trainer's full tensors
        ref = DecoderLM(tp_config(cfg, world), "cuda", torch.bfloat16)
        for name, t in tr.engine.iter_hf_tensors():
            load_hf_tensor(ref, name, tp_slice(name, t.detach(), cfg, rank, world))
        for (n1, a), (_n2, b) in zip(sm.sampler.model.named_parameters(), ref.named_parameters()):
            assert torch.equal(a, b), n1
        assert tr.engine.weight_norm()["norm"] == pytest.approx(sm.sampler.weight_norm()["norm"], rel=1e-3)
        # generation: the replica against a one-rank engine holding the same (full) weights
        full = DecoderLM(cfg, "cuda", torch.bfloat16)
        for name, t in tr.engine.iter_hf_tensors():
            load_hf_tensor(full, name, t.detach())
        one = SamplerEngine(cfg, "cuda", model=full, kv_cache_tokens=1 << 14, max_batch=16, max_seq_len=512)
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(1, cfg.vocab_size, (n_tok,), generator=g).tolist() for n_tok in (40, 75, 33)]
        sp = {"n": 4, "temperature": 0.0, "max_tokens": 24, "ignore_eos": True}
        res = {}
        for graph in (False, True):
            sm.sampler.use_cuda_graph = graph
            sm.sampler._graphs.clear()
            res[graph] = sm.generate(prompts, sp)
            _lib.check_status("tp generate")
        res["one"] = one.generate(prompts, sp)
        torch.save(res, os.path.join(out_dir, f"tp{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_tensor_parallel_paged_sampler_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_tp_paged_main, args=(2, _free_port(), d), nprocs=2, join=True)
        r0 = torch.load(os.path.join(d, "tp0.pt"), weights_only=False)
        r1 = torch.load(os.path.join(d, "tp1.pt"), weights_only=False)
    for graph in (False, True):
        # the ranks of a replica never diverge: identical activations, identical sampling decisions
        assert [o["token_ids"] for o in r0[graph]] == [o["token_ids"] for o in r1[graph]]
    assert [o["token_ids"] for o in r0[True]] == [o["token_ids"] for o in r0[False]]
    # against one rank: same model, different summation order -- greedy tokens agree except where two logits tie
    same = sum(a["token_ids"] == b["token_ids"] for a, b in zip(r0[False], r0["one"]))
    assert same >= int(0.75 * len(r0["one"])), same
    for a, b in zip(r0[False], r0["one"]):
        k = next((i for i, (x, y) in enumerate(zip(a["token_ids"], b["token_ids"])) if x != y), len(a["token_ids"]))
        assert a["logprobs"][:k] == pytest.approx(b["logprobs"][:k], abs=6e-2)


def _ipc_trainer(q_out, q_in, port):
    """Process A (cuda:0): a one-rank trainer that takes one optimizer step, exports its buffer and waits."""
    try:
        torch.cuda.set_device(0)
        from arctic_platform_b200.engine.worker import EngineWorker
        w = EngineWorker("cuda:0")
        w.initialize({"model_name": "qwen3-tiny-d128", "job_type": "training", "seed": 5,
                      "ds_config": {"zero_optimization": {"stage": 1}, "optimizer": {"params": {"lr": 1e-2}}}})
        info = w.export_ipc_source()
        assert info is not None and len(info["handle"]) == 64
        ref = {n: t.detach().float().cpu() for n, t in w.engine.iter_hf_tensors()}
        q_out.put((info, ref, w.weight_norm()["norm"]))
        assert q_in.get(timeout=120) == "done"               # keep the buffer alive while the reader has it mapped
    except Exception as exc:                                 # pragma: no cover - surfaced by the parent
        q_out.put(("error", repr(exc), None))
        raise


def _ipc_sampler(q_out, q_src, fp8):
    """Process B (cuda:1): a sampler that maps the trainer's buffer and runs the hand-over kernel on it."""
    try:
        torch.cuda.set_device(1)
        from arctic_platform_b200.engine.worker import EngineWorker
        from arctic_platform_b200.ops import _lib
        w = EngineWorker("cuda:1")
        vc = {"max_model_len": 256, "kv_cache_tokens": 4096, "max_num_seqs": 8}
        if fp8:
            vc["quantization"] = "fp8"
        w.initialize({"model_name": "qwen3-tiny-d128", "job_type": "sampling", "seed": 99, "vllm_config": vc})
        info, ref, norm = q_src.get(timeout=120)
        n = w.sync_from_ipc([info])
        _lib.check_status("ipc sync")
        got = {n_: t.detach().float().cpu() for n_, t in w.sampler.model.named_parameters()}
        out = w.generate([[3, 4, 5, 6]], {"temperature": 0.0, "max_tokens": 4})
        released = w.release_ipc_handles()
        q_out.put((n, w.weight_norm()["norm"], norm, released, len(out[0]["token_ids"]),
                   {k: float(v.abs().sum()) for k, v in got.items()}))
    except Exception as exc:                                 # pragma: no cover
        q_out.put(("error", repr(exc)))
        raise


@pytest.mark.timeout(300)
def test_split_placement_hand_over_through_cuda_ipc(fp8=False):
    """Trainer and sampler in DIFFERENT processes on different GPUs: the sampler maps the trainer's flat buffer
    through a CUDA IPC handle and the table kernel pulls the weights over NVLink."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    a_out, a_in, b_out = ctx.Queue(), ctx.Queue(), ctx.Queue()
    pa = ctx.Process(target=_ipc_trainer, args=(a_out, a_in, _free_port()))
    pa.start()
    first = a_out.get(timeout=180)
    assert first[0] != "error", first
    relay = ctx.Queue()
    relay.put(first)
    pb = ctx.Process(target=_ipc_sampler, args=(b_out, relay, fp8))
    pb.start()
    res = b_out.get(timeout=180)
    a_in.put("done")
    pa.join(60)
    pb.join(60)
    assert res[0] != "error", res
    n, got_norm, want_norm, released, n_tok, _sums = res
    assert n > 0 and released == 1 and n_tok == 4
    assert got_norm == pytest.approx(want_norm, rel=1e-3)
    assert pa.exitcode == 0 and pb.exitcode == 0
