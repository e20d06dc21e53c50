#!/usr/bin/env bash
# Text-to-SQL GRPO on one 8-GPU node, colocated: ZeRO-3 trainer + one sampler replica per GPU, prompt de-duplication on.
# DATA is written by recipes/rl/verl/txt2sql/preprocess_bird.py (rows carry extra_info.db_path for the reward).
set -euo pipefail
DATA=${DATA:?train.parquet from preprocess_bird.py}
MODEL=${MODEL:-Qwen/Qwen3-8B}
torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 -m recipes.rl.skyrl.run_loop \
  --data "$DATA" --env bird_sql_arctic --model "$MODEL" --tokenizer "$MODEL" \
  --training-gpus 8 --sampling-gpus 8 --log-prob-gpus 8 --batch-prompts 8 --n 16 \
  --max-prompt-tokens 8192 --max-tokens 4096 --lr 1e-6 --zero-stage 3 "$@"
