#!/usr/bin/env bash
# Long-context QA (16K prompt / 4K response, 2048 trajectories per step = 128 prompts x 16), Qwen3-32B, 4 nodes.
# Reward: recipes/rl/rewards/long_context_qa_reward.py.
set -euo pipefail
PKG_DIR=$(python -c "import arctic_platform_b200.integrations.verl.register as r; print(r.config_search_path())")
export VERL_USE_EXTERNAL_MODULES=arctic_platform_b200.integrations.verl.register
MODEL=${MODEL:-Qwen/Qwen3-32B}
DATA=${DATA:-$HOME/data/long_context_qa}

python -m verl.trainer.main_ppo \
  hydra.searchpath="[file://${PKG_DIR}]" remote_backend=arctic trainer.remote_backend=arctic \
  algorithm.adv_estimator=grpo \
  data.train_files="${DATA}/train.parquet" data.val_files="${DATA}/val.parquet" \
  data.train_batch_size=128 data.max_prompt_length=16384 data.max_response_length=4096 \
  custom_reward_function.path=recipes/rl/rewards/long_context_qa_reward.py \
  custom_reward_function.name=long_context_qa_reward \
  actor_rollout_ref.model.path="${MODEL}" actor_rollout_ref.actor.optim.lr=1e-6 \
  actor_rollout_ref.actor.ppo_mini_batch_size=128 actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=1 \
  actor_rollout_ref.rollout.n=16 \
  remote_backend.colocate=True remote_backend.training_gpus=32 remote_backend.sampling_gpus=32 \
  remote_backend.log_prob_gpus=32 remote_backend.sampling_tp_size=4 remote_backend.comm_protocol=ray \
  remote_backend.train.zorro_train.enable=True remote_backend.train.zorro_train.max_rollouts=16 \
  remote_backend.train.deepspeed.zero_optimization.stage=3 \
  trainer.n_gpus_per_node=8 trainer.nnodes=4 "$@"
