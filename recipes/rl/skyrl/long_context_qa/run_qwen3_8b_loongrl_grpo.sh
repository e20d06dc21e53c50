#!/usr/bin/env bash
# Long-context multi-hop QA (answers in \boxed{}): 16K-token prompts held once per group on the packed axis.
set -euo pipefail
DATA=${DATA:?prompt file with reward_model.ground_truth}
MODEL=${MODEL:-Qwen/Qwen3-8B}
torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 -m recipes.rl.skyrl.run_loop \
  --data "$DATA" --env long_context_qa --model "$MODEL" --tokenizer "$MODEL" \
  --training-gpus 8 --sampling-gpus 8 --log-prob-gpus 8 --batch-prompts 4 --n 8 \
  --max-prompt-tokens 16384 --max-tokens 4096 --lr 1e-6 --zero-stage 3 "$@"
