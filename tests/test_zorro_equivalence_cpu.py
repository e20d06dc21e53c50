"""Prompt-deduplicated forward/backward equals the ordinary packed computation (fp32, CPU)."""
import numpy as np
import torch

from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch, find_prompt_groups


def make_grpo_batch(n_prompts=3, n_samples=4, p_rng=(12, 40), r_rng=(4, 20), vocab=32000, seed=0):
    g = torch.Generator().manual_seed(seed)
    P, R = p_rng[1], r_rng[1]
    B = n_prompts * n_samples
    ids = torch.zeros((B, P + R), dtype=torch.int64)
    mask = torch.zeros((B, P + R), dtype=torch.int64)
    for p in range(n_prompts):
        pl = int(torch.randint(p_rng[0], p_rng[1] + 1, (1,), generator=g))
        prompt = torch.randint(1, vocab, (pl,), generator=g)
        for s in range(n_samples):
            b = p * n_samples + s
            rl = int(torch.randint(r_rng[0], r_rng[1] + 1, (1,), generator=g))
            ids[b, P - pl:P] = prompt
            mask[b, P - pl:P] = 1
            ids[b, P:P + rl] = torch.randint(1, vocab, (rl,), generator=g)
            mask[b, P:P + rl] = 1
    perm = torch.randperm(B, generator=g)          # rollouts of one prompt need not be adjacent
    return ids[perm], mask[perm], R


def test_grouping_and_tables():
    ids, mask, R = make_grpo_batch()
    groups = find_prompt_groups(ids, R)
    assert groups.max() + 1 == 3
    pb = build_packed_batch(ids, mask, R, dedup=True)
    full = build_packed_batch(ids, mask, R, dedup=False)
    assert pb.num_groups == 3 and full.num_groups == ids.shape[0]
    assert pb.total_tokens < full.total_tokens == int(mask.sum())
    assert torch.equal(pb.labels, full.labels) and torch.equal(pb.out_index, full.out_index)
    grid = pb.scatter_to_grid(pb.labels.float())
    assert torch.equal(grid.long() * mask[:, -R:], ids[:, -R:] * mask[:, -R:])
    # predictor rows hold the token that precedes the label in its own sample
    prev_tok = pb.input_ids[pb.pred_index]
    prev_full = full.input_ids[full.pred_index]
    assert torch.equal(prev_tok, prev_full)


def test_dedup_matches_full_forward_backward():
    torch.manual_seed(0)
    cfg = PRESETS["qwen3-tiny"]
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=1)
    ids, mask, R = make_grpo_batch()
    pb = build_packed_batch(ids, mask, R, dedup=True)
    full = build_packed_batch(ids, mask, R, dedup=False)
    adv = torch.randn(pb.labels.shape[0])

    def run(packed):
        model.zero_grad()
        lp, ent = token_logprobs(model, packed, inv_temperature=0.8)
        ((lp * adv).sum() + 0.01 * ent.sum()).backward()
        return lp.detach(), ent.detach(), {n: p.grad.clone() for n, p in model.named_parameters()}

    lp_d, ent_d, g_d = run(pb)
    lp_f, ent_f, g_f = run(full)
    assert torch.allclose(lp_d, lp_f, atol=1e-5, rtol=1e-5)
    assert torch.allclose(ent_d, ent_f, atol=1e-5, rtol=1e-5)
    for n in g_f:
        assert torch.allclose(g_d[n], g_f[n], atol=2e-5, rtol=1e-4), n


def test_matches_plain_pytorch_transformer():
    """The packed module equals a straightforward per-sequence PyTorch implementation of the same
    architecture (RMSNorm, q/k-norm, rotate-half RoPE, GQA causal attention, SwiGLU)."""
    torch.manual_seed(0)
    cfg = PRESETS["qwen3-tiny"]
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=2)
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2)
    full = build_packed_batch(ids, mask, R, dedup=False)
    lp, _ = token_logprobs(model, full)

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rope(x, pos):
        D = x.shape[-1]
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
        ang = pos.double()[:, None] * inv[None]
        c, s = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
        a, b = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    outs = []
    for b in range(ids.shape[0]):
        seq = ids[b][mask[b].bool()]
        n = seq.shape[0]
        pos = torch.arange(n)
        x = model.embed[seq]
        for blk in model.blocks:
            h = rms(x, blk.ln1)
            qkv = h @ blk.wqkv.t()
            q = qkv[:, :cfg.q_size].view(n, cfg.num_heads, cfg.head_dim)
            k = qkv[:, cfg.q_size:cfg.q_size + cfg.kv_size].view(n, cfg.num_kv_heads, cfg.head_dim)
            v = qkv[:, cfg.q_size + cfg.kv_size:].view(n, cfg.num_kv_heads, cfg.head_dim)
            q, k = rope(rms(q, blk.q_norm), pos), rope(rms(k, blk.k_norm), pos)
            rep = cfg.num_heads // cfg.num_kv_heads
            k2, v2 = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
            s = torch.einsum("qhd,khd->hqk", q, k2) / cfg.head_dim ** 0.5
            s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool), 1)[None], float("-inf"))
            a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v2).reshape(n, -1)
            x = x + a @ blk.wo.t()
            h = rms(x, blk.ln2)
            gu = h @ blk.wgu.t()
            x = x + (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ blk.wdown.t()
        logits = rms(x, model.final_norm) @ model.embed.t()
        rl = int(mask[b, -R:].sum())
        pl = n - rl
        lps = torch.log_softmax(logits[pl - 1:n - 1], -1).gather(-1, seq[pl:, None]).squeeze(-1)
        outs.append(lps)
    assert torch.allclose(lp, torch.cat(outs), atol=2e-5, rtol=1e-5)
