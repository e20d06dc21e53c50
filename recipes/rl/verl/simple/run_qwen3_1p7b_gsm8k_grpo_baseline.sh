#!/usr/bin/env bash
# A/B twin of run_qwen3_1p7b_gsm8k_grpo.sh: the same GRPO run on verl's OWN engines (FSDP trainer + vLLM rollout), no
# remote backend -- what the platform's step time and reward curve are compared against.
set -euo pipefail
MODEL=${MODEL:-Qwen/Qwen3-1.7B}
DATA=${DATA:-$HOME/data/gsm8k}

python -m verl.trainer.main_ppo \
  algorithm.adv_estimator=grpo \
  data.train_files="${DATA}/train.parquet" data.val_files="${DATA}/test.parquet" \
  data.train_batch_size=128 data.max_prompt_length=512 data.max_response_length=1024 \
  actor_rollout_ref.model.path="${MODEL}" actor_rollout_ref.model.use_remove_padding=True \
  actor_rollout_ref.actor.strategy=fsdp actor_rollout_ref.actor.optim.lr=1e-6 \
  actor_rollout_ref.actor.ppo_mini_batch_size=128 actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8 \
  actor_rollout_ref.actor.use_kl_loss=True actor_rollout_ref.actor.kl_loss_coef=0.001 \
  actor_rollout_ref.actor.kl_loss_type=low_var_kl \
  actor_rollout_ref.rollout.name=vllm actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.temperature=1.0 \
  actor_rollout_ref.rollout.gpu_memory_utilization=0.5 actor_rollout_ref.rollout.tensor_model_parallel_size=1 \
  trainer.n_gpus_per_node=1 trainer.nnodes=1 trainer.total_epochs=1 trainer.project_name=fsdp_baseline_gsm8k "$@"
