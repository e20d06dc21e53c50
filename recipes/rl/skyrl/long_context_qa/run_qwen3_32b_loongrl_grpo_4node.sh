#!/usr/bin/env bash
# Long-context QA GRPO with Qwen3-32B on 4 nodes x 8 GPUs (32K-token prompts, 4K responses): ZeRO-3 over all ranks with
# the optimizer state on the host, Ulysses sequence parallelism 4 inside a node, sampler replicas of width 4.
# Run on every node with NODE_RANK and MASTER_ADDR set; DATA from `python -m recipes.rl.data.prepare_data long_context_qa`.
set -euo pipefail
DATA=${DATA:?merged/train.parquet from prepare_data.py}
MODEL=${MODEL:-Qwen/Qwen3-32B}
NNODES=${NNODES:-4}
NODE_RANK=${NODE_RANK:?0..NNODES-1}
MASTER_ADDR=${MASTER_ADDR:?address of node 0}
MASTER_PORT=${MASTER_PORT:-29500}
torchrun --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node 8 \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" -m recipes.rl.skyrl.run_loop \
  --data "$DATA" --env long_context_qa --model "$MODEL" --tokenizer "$MODEL" \
  --training-gpus $((NNODES * 8)) --sampling-gpus $((NNODES * 8)) --log-prob-gpus $((NNODES * 8)) \
  --batch-prompts 2 --n 16 --max-prompt-tokens 32768 --max-tokens 4096 --lr 1e-6 --zero-stage 3 \
  --sampler-tp 4 --sequence-parallel 4 --offload-optimizer "$@"
