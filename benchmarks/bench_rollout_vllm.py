"""Same-box anchor for the rollout phase: vLLM (the reference's sampler, arctic_platform/common/ray_server.py:921-933)
on a random-init Qwen3-4B, one GPU, the benchmark's rollout shape.

8 prompts x n = 16 samples, 2048 prompt tokens + 2048 generated tokens, temperature 1.0, ``ignore_eos``, prefix caching
on (the 16 samples of a prompt share its KV), bf16, CUDA graphs as vLLM configures them by default.  Weights are
vLLM's ``load_format="dummy"`` random values for the Qwen3-4B architecture, prompts are random token ids: no files
or network are needed beyond a config.json written to a temporary directory.  This is a library baseline measured on
the same machine, not the reference platform (which cannot be installed here).

    python benchmarks/bench_rollout_vllm.py [--prompts 8 --samples 16 --prompt-len 2048 --max-tokens 2048] [--repeat 2]

Prints one JSON line: wall seconds of ``generate`` (best of ``--repeat`` after one warm-up call with new prompts
each time) and generated tokens/s.
"""
import argparse
import json
import os
import tempfile
import time


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompts", type=int, default=8)
    ap.add_argument("--samples", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--max-tokens", type=int, default=2048)
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.6)
    args = ap.parse_args()
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    import torch
    from transformers import Qwen3Config
    from vllm import LLM, SamplingParams

    cfg = Qwen3Config(vocab_size=151936, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True, dtype="bfloat16")
    cfg.architectures = ["Qwen3ForCausalLM"]
    d = tempfile.mkdtemp(prefix="qwen3_4b_cfg_")
    cfg.save_pretrained(d)
    # vLLM wants a tokenizer even when only token ids go in and come out: a word-level one built here, no download
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {"<unk>": 0, "<eos>": 1, **{f"t{i}": i for i in range(2, 1024)}}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="<eos>", pad_token="<eos>").save_pretrained(d)
    t0 = time.perf_counter()
    llm = LLM(model=d, tokenizer=d, runner="generate", load_format="dummy", dtype="bfloat16", enable_prefix_caching=True,
              max_model_len=args.prompt_len + args.max_tokens + 16, max_num_seqs=args.prompts * args.samples,
              gpu_memory_utilization=args.gpu_memory_utilization, seed=0)
    t_init = time.perf_counter() - t0
    sp = SamplingParams(n=args.samples, temperature=1.0, max_tokens=args.max_tokens, ignore_eos=True, detokenize=False)
    g = torch.Generator().manual_seed(0)
    best, toks = None, 0
    for it in range(args.repeat + 1):
        prompts = [{"prompt_token_ids": torch.randint(1, 151000, (args.prompt_len,), generator=g).tolist()}
                   for _ in range(args.prompts)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, use_tqdm=False)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        toks = sum(len(c.token_ids) for o in outs for c in o.outputs)
        if it > 0:
            best = dt if best is None else min(best, dt)
    import vllm
    print(json.dumps({"anchor": "vllm_rollout", "vllm": vllm.__version__, "model": "qwen3-4b (dummy weights)",
                      "prompts": args.prompts, "samples": args.samples, "prompt_len": args.prompt_len,
                      "max_tokens": args.max_tokens, "generated_tokens": toks, "generate_s": round(best, 3),
                      "tokens_per_s": round(toks / best, 1), "ms_per_decode_step": round(best / args.max_tokens * 1e3, 3),
                      "engine_init_s": round(t_init, 1)}), flush=True)


if __name__ == "__main__":
    main()
