"""The bf16 GPU model (all kernels) against the same module in fp32 on CPU, and ZoRRo equivalence on GPU."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _batch():
    from tests.test_zorro_equivalence_cpu import make_grpo_batch
    return make_grpo_batch(n_prompts=3, n_samples=4, p_rng=(100, 300), r_rng=(10, 150))


def _models(name="qwen3-tiny-d128"):
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    cfg = PRESETS[name]
    ref = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=3)
    gpu = DecoderLM(cfg, "cuda", torch.bfloat16)
    with torch.no_grad():
        for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
            p.copy_(q.to(torch.bfloat16))
            q.copy_(p.float().cpu())          # reference uses the bf16-rounded weights
    return cfg, ref, gpu


@pytest.mark.parametrize("name", ["qwen3-tiny-d128", "qwen3-moe-tiny"])
def test_model_forward_backward_vs_fp32(name):
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    cfg, ref, gpu = _models(name)
    ids, mask, R = _batch()
    pb = build_packed_batch(ids, mask, R, dedup=True)
    adv = torch.randn(pb.labels.shape[0])
    lp_r, ent_r = token_logprobs(ref, pb, 1.0)
    ((lp_r * adv).sum() / adv.numel()).backward()
    pbg = copy.copy(pb).to("cuda")
    lp_g, ent_g = token_logprobs(gpu, pbg, 1.0)
    ((lp_g * adv.cuda()).sum() / adv.numel()).backward()
    _lib.check_status("model")
    assert (lp_g.cpu() - lp_r).abs().max() < 0.25          # the reference's own gate vs HF (LOGPROB_ATOL)
    assert (lp_g.cpu() - lp_r).abs().mean() < 0.02
    assert (ent_g.cpu() - ent_r).abs().mean() < 0.02
    gr = dict(ref.named_parameters())
    for n, p in gpu.named_parameters():
        if "router" in n:
            continue
        a, b = p.grad.float().cpu().flatten(), gr[n].grad.flatten()
        cos = torch.nn.functional.cosine_similarity(a, b, dim=0)
        assert cos > 0.98, f"{n}: cosine {cos}"


def test_zorro_equals_full_on_gpu():
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    cfg, ref, gpu = _models()
    ids, mask, R = _batch()
    with torch.no_grad():
        lp_d, _ = token_logprobs(gpu, build_packed_batch(ids, mask, R, dedup=True).to("cuda"))
        lp_f, _ = token_logprobs(gpu, build_packed_batch(ids, mask, R, dedup=False).to("cuda"))
    _lib.check_status("zorro gpu")
    assert (lp_d - lp_f).abs().max() < 0.05
    assert (lp_d - lp_f).abs().mean() < 5e-3


def test_hybrid_family_runs_on_gpu():
    """Qwen3.5-style hybrid (gated delta-net + gated attention + shared expert) in bf16 on the GPU against fp32 on CPU:
    the projections run on the tcgen05 GEMM, the delta rule in PyTorch ops, attention (head_dim 64) on the dense path."""
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    from tests.test_zorro_equivalence_cpu import make_grpo_batch
    cfg, ref, gpu = _models("qwen3.5-moe-tiny")
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=3, p_rng=(40, 120), r_rng=(10, 60), seed=2)
    pb = build_packed_batch(ids % cfg.vocab_size, mask, R, dedup=True)
    lp_r, _ = token_logprobs(ref, pb, 1.0)
    lp_r.mean().backward()
    pbg = copy.copy(pb).to("cuda")
    lp_g, _ = token_logprobs(gpu, pbg, 1.0)
    lp_g.mean().backward()
    _lib.check_status("hybrid")
    assert (lp_g.cpu() - lp_r).abs().mean() < 0.03
    assert all(p.grad is not None and torch.isfinite(p.grad.float()).all() for p in gpu.parameters())
    gr = dict(ref.named_parameters())
    for n in ("blocks.0.linear_attn.in_qkv", "blocks.0.linear_attn.out_proj", "blocks.3.wqkv", "blocks.3.wgate"):
        a = dict(gpu.named_parameters())[n].grad.float().cpu().flatten()
        assert torch.nn.functional.cosine_similarity(a, gr[n].grad.flatten(), dim=0) > 0.95, n


def test_hybrid_sampler_on_gpu_agrees_with_teacher_forced_scoring():
    """The stateful hybrid sampler in bf16 on the GPU: the log-probs it reports while decoding token by token match
    a packed teacher-forced pass of the training model over prompt + sampled tokens."""
    import numpy as np
    from arctic_platform_b200.engine.hybrid_sampler import HybridSampler
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops.attention import AttnLayout
    cfg, _ref, gpu = _models("qwen3.5-moe-tiny")
    eng = HybridSampler(cfg, "cuda", model=gpu, max_seq_len=256)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(3, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 23)]
    res = eng.generate(prompts, {"n": 3, "temperature": 1.0, "max_tokens": 16, "seed": 1})
    _lib.check_status("hybrid sampler")
    assert len(res) == 6 and eng.prefill_tokens == 32
    diffs = []
    for r in res:
        seq = prompts[r["prompt_index"]] + r["token_ids"]
        ids = torch.tensor(seq, device="cuda")
        with torch.no_grad():
            h = gpu.forward_hidden(ids, torch.arange(len(seq), device="cuda"), AttnLayout.from_cu_seqlens(np.array([0, len(seq)])))
            lp = torch.log_softmax(gpu.logits(h).float(), -1)
        P = r["prompt_len"]
        want = lp[P - 1:len(seq) - 1].gather(1, ids[P:, None])[:, 0].cpu()
        diffs.append((want - torch.tensor(r["logprobs"])).abs())
    d = torch.cat(diffs)
    assert d.mean() < 0.03 and d.max() < 0.3, (d.mean(), d.max())


def test_tiled_mlp_on_gpu_matches_untiled():
    """Row-tiled dense MLP through the CUDA kernels (custom autograd functions re-run tile by tile inside the
    backward): same log-probs, weight gradients equal up to the order of the per-tile accumulation."""
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    ids, mask, R = _batch()
    pb = build_packed_batch(ids, mask, R).to("cuda")
    res = {}
    for shards in (0, 3):
        _cfg, _ref, gpu = _models()
        for blk in gpu.blocks:
            blk.tiled_mlp_shards = shards
        lp, _ = token_logprobs(gpu, pb, 1.0)
        lp.mean().backward()
        _lib.check_status(f"tiled mlp shards={shards}")
        res[shards] = (lp.detach().float(), {n: p.grad.float() for n, p in gpu.named_parameters() if p.grad is not None})
    assert (res[0][0] - res[3][0]).abs().max() < 1e-3
    assert set(res[0][1]) == set(res[3][1])
    for n in ("blocks.0.wgu", "blocks.0.wdown", "blocks.1.wqkv", "blocks.1.wo"):
        a, b = res[0][1][n].flatten(), res[3][1][n].flatten()
        assert torch.nn.functional.cosine_similarity(a, b, dim=0) > 0.999, n
