"""Same-box anchor for the training phases: Hugging Face Qwen3-4B (random init from config) with FlashAttention-2,
bf16, gradient checkpointing and torch's fused AdamW on the benchmark's batch -- 128 sequences of 2048 prompt +
2048 response tokens -- without prompt de-duplication (every sequence carries its own copy of the prompt, as a plain
FSDP / HF trainer processes it).

One "step" = a no-grad reference forward that scores the response tokens (log-softmax over the vocabulary, chunked)
+ forward/backward of a GRPO-style clipped objective with a low-variance KL term over ``--micro-batch`` sequences at a
time + one AdamW step.  CUDA-event timing, one warm-up step, new random tokens every step.  This is a library twin
measured on the same machine (cuBLAS GEMMs, flash_attn kernels), not the reference platform.

    python benchmarks/bench_train_torch.py [--sequences 128 --prompt-len 2048 --response-len 2048 --micro-batch 4]
                                           [--steps 1] [--no-checkpointing]

Prints one JSON line with the phase times.
"""
import argparse
import json

import torch


def chunked_logprobs(hidden, weight, labels, chunk=4096):
    """log softmax(hidden @ weight^T)[label] per row, recomputed per chunk in the backward (never holds [N, V])."""
    from torch.utils.checkpoint import checkpoint

    def piece(h, y):
        logits = (h @ weight.t()).float()
        return torch.gather(torch.log_softmax(logits, -1), 1, y[:, None])[:, 0]

    out = []
    for i in range(0, hidden.shape[0], chunk):
        h, y = hidden[i:i + chunk], labels[i:i + chunk]
        out.append(checkpoint(piece, h, y, use_reentrant=False) if torch.is_grad_enabled() else piece(h, y))
    return torch.cat(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sequences", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--response-len", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--no-checkpointing", action="store_true")
    args = ap.parse_args()
    from transformers import AutoModelForCausalLM, Qwen3Config
    dev = torch.device("cuda")
    cfg = Qwen3Config(vocab_size=151936, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True)
    torch.manual_seed(0)
    with torch.device(dev):
        model = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16, attn_implementation="flash_attention_2")
        ref = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16, attn_implementation="flash_attention_2")
    ref.load_state_dict(model.state_dict())
    ref.eval().requires_grad_(False)
    if not args.no_checkpointing:
        model.gradient_checkpointing_enable()
    model.train()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-6, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, fused=True)
    B, P, R, mb = args.sequences, args.prompt_len, args.response_len, args.micro_batch
    g = torch.Generator(device=dev).manual_seed(1)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    res = {}
    for step in range(args.steps + 1):
        ids = torch.randint(1, 151000, (B, P + R), generator=g, device=dev)
        adv = torch.randn(B, 1, generator=g, device=dev).expand(B, R)
        old = torch.full((B, R), -11.9, device=dev)
        e0, e1, e2, e3 = ev(), ev(), ev(), ev()
        e0.record()
        ref_lp = torch.empty((B, R), device=dev)
        with torch.no_grad():
            for i in range(0, B, 2 * mb):
                x = ids[i:i + 2 * mb]
                h = ref.model(input_ids=x).last_hidden_state[:, P - 1:-1].reshape(-1, cfg.hidden_size)
                ref_lp[i:i + 2 * mb] = chunked_logprobs(h, ref.lm_head.weight, x[:, P:].reshape(-1)).view(-1, R)
        e1.record()
        for i in range(0, B, mb):
            x = ids[i:i + mb]
            h = model.model(input_ids=x).last_hidden_state[:, P - 1:-1].reshape(-1, cfg.hidden_size)
            lp = chunked_logprobs(h, model.lm_head.weight, x[:, P:].reshape(-1)).view(-1, R)
            ratio = torch.exp(lp - old[i:i + mb])
            a = adv[i:i + mb]
            pg = -torch.minimum(ratio * a, ratio.clamp(0.8, 1.2) * a)
            d = ref_lp[i:i + mb] - lp
            kl = torch.exp(d) - d - 1.0
            loss = (pg + 1e-3 * kl).sum() / (B * R)
            loss.backward()
        e2.record()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        e3.record()
        torch.cuda.synchronize()
        if step > 0:
            res = {"ref_logprob_ms": e0.elapsed_time(e1), "fwd_bwd_ms": e1.elapsed_time(e2), "optimizer_ms": e2.elapsed_time(e3)}
    import transformers
    tokens = B * (P + R)
    total = sum(res.values())
    print(json.dumps({"anchor": "hf_torch_train", "transformers": transformers.__version__, "torch": torch.__version__,
                      "attention": "flash_attention_2", "gradient_checkpointing": not args.no_checkpointing,
                      "sequences": B, "tokens": tokens, "micro_batch": mb, **{k: round(v, 1) for k, v in res.items()},
                      "train_phases_ms": round(total, 1), "tokens_per_s": round(tokens / total * 1e3, 1),
                      "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}), flush=True)


if __name__ == "__main__":
    main()
