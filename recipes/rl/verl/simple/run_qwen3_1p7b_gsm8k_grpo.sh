#!/usr/bin/env bash
# GRPO on GSM8K with verl as the driver and this platform as the remote backend, one GPU, colocated engines.
# Needs verl and the GSM8K parquet files (see verl's examples/data_preprocess/gsm8k.py); nothing here downloads.
set -euo pipefail
PKG_DIR=$(python -c "import arctic_platform_b200.integrations.verl.register as r; print(r.config_search_path())")
export VERL_USE_EXTERNAL_MODULES=arctic_platform_b200.integrations.verl.register
MODEL=${MODEL:-Qwen/Qwen3-1.7B}
DATA=${DATA:-$HOME/data/gsm8k}

python -m verl.trainer.main_ppo \
  hydra.searchpath="[file://${PKG_DIR}]" remote_backend=arctic trainer.remote_backend=arctic \
  algorithm.adv_estimator=grpo \
  data.train_files="${DATA}/train.parquet" data.val_files="${DATA}/test.parquet" \
  data.train_batch_size=128 data.max_prompt_length=512 data.max_response_length=1024 \
  actor_rollout_ref.model.path="${MODEL}" \
  actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=128 \
  actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8 actor_rollout_ref.actor.use_kl_loss=True \
  actor_rollout_ref.actor.kl_loss_coef=0.001 actor_rollout_ref.actor.kl_loss_type=low_var_kl \
  actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.temperature=1.0 \
  remote_backend.colocate=True remote_backend.training_gpus=1 remote_backend.sampling_gpus=1 \
  remote_backend.log_prob_gpus=1 remote_backend.weight_sync.cuda_ipc=True \
  remote_backend.train.zorro_train.enable=True \
  trainer.n_gpus_per_node=1 trainer.nnodes=1 trainer.total_epochs=1 trainer.project_name=arl_b200_gsm8k "$@"
