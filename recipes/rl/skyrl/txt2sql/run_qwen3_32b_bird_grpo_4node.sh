#!/usr/bin/env bash
# Text-to-SQL GRPO with Qwen3-32B on 4 nodes x 8 GPUs, colocated: one SPMD rank per GPU (ZeRO-3 over all 32 ranks,
# optimizer state on the host, sampler replicas of tensor-parallel width 4), prompt de-duplication on.
# Run THIS script on every node with NODE_RANK=0..3 and the same MASTER_ADDR (node 0's address), e.g. through
# `srun` / `pdsh`; DATA as in run_qwen3_8b_bird_grpo.sh.
set -euo pipefail
DATA=${DATA:?train.parquet from preprocess_bird.py}
MODEL=${MODEL:-Qwen/Qwen3-32B}
NNODES=${NNODES:-4}
NODE_RANK=${NODE_RANK:?0..NNODES-1}
MASTER_ADDR=${MASTER_ADDR:?address of node 0}
MASTER_PORT=${MASTER_PORT:-29500}
torchrun --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node 8 \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" -m recipes.rl.skyrl.run_loop \
  --data "$DATA" --env bird_sql_arctic --model "$MODEL" --tokenizer "$MODEL" \
  --training-gpus $((NNODES * 8)) --sampling-gpus $((NNODES * 8)) --log-prob-gpus $((NNODES * 8)) \
  --batch-prompts 4 --n 16 --max-prompt-tokens 16384 --max-tokens 4096 --lr 1e-6 --zero-stage 3 \
  --sampler-tp 4 --offload-optimizer "$@"
