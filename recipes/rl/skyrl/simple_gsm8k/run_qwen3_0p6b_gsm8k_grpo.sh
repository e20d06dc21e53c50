#!/usr/bin/env bash
# GSM8K GRPO on one GPU with everything colocated (trainer, reference engine and sampler share the device).
# DATA: a parquet / jsonl of rows {"prompt": [...chat messages...], "reward_model": {"ground_truth": "72"}}.
set -euo pipefail
DATA=${DATA:?path to the GSM8K prompt file}
MODEL=${MODEL:-Qwen/Qwen3-0.6B}
python -m recipes.rl.skyrl.run_loop --data "$DATA" --env gsm8k_arctic --model "$MODEL" --tokenizer "$MODEL" \
  --training-gpus 1 --sampling-gpus 1 --log-prob-gpus 1 --batch-prompts 64 --n 8 \
  --max-prompt-tokens 512 --max-tokens 1024 --lr 1e-6 --zero-stage 2 "$@"
