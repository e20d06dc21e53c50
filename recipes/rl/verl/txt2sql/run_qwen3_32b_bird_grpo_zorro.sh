#!/usr/bin/env bash
# Text-to-SQL (BIRD) GRPO, Qwen3-32B, 32K prompt / 4K response, 16 rollouts per prompt, 4 nodes x 8 GPUs:
# ZeRO-3 trainer, sampler TP=4, ZoRRo Train prompt deduplication (the schema-heavy prompts are ~88 % of the tokens).
# Reward: recipes/rl/rewards/bird_reward.py (execution match on the sample's SQLite database).
set -euo pipefail
PKG_DIR=$(python -c "import arctic_platform_b200.integrations.verl.register as r; print(r.config_search_path())")
export VERL_USE_EXTERNAL_MODULES=arctic_platform_b200.integrations.verl.register
MODEL=${MODEL:-Qwen/Qwen3-32B}
DATA=${DATA:-$HOME/data/bird}
ZORRO=${ZORRO:-True}

python -m verl.trainer.main_ppo \
  hydra.searchpath="[file://${PKG_DIR}]" remote_backend=arctic trainer.remote_backend=arctic \
  algorithm.adv_estimator=grpo \
  data.train_files="${DATA}/train.parquet" data.val_files="${DATA}/dev.parquet" \
  data.train_batch_size=128 data.max_prompt_length=32768 data.max_response_length=4096 \
  custom_reward_function.path=recipes/rl/rewards/bird_reward.py custom_reward_function.name=bird_reward \
  actor_rollout_ref.model.path="${MODEL}" actor_rollout_ref.model.enable_gradient_checkpointing=True \
  actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=128 \
  actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=1 \
  actor_rollout_ref.rollout.n=16 actor_rollout_ref.rollout.temperature=1.0 \
  remote_backend.colocate=True remote_backend.training_gpus=32 remote_backend.sampling_gpus=32 \
  remote_backend.log_prob_gpus=32 remote_backend.sampling_tp_size=4 remote_backend.comm_protocol=ray \
  remote_backend.weight_sync.cuda_ipc=True remote_backend.train.logits.optimization=memory \
  remote_backend.train.zorro_train.enable=${ZORRO} remote_backend.train.zorro_train.max_rollouts=16 \
  remote_backend.train.deepspeed.zero_optimization.stage=3 \
  trainer.n_gpus_per_node=8 trainer.nnodes=4 trainer.total_epochs=1 trainer.project_name=arl_b200_bird "$@"
