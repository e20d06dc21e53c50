#!/usr/bin/env bash
# A/B twin of run_qwen3_32b_bird_grpo_zorro.sh on verl's own engines (FSDP with parameter offload + vLLM TP 4): the
# same data, batch, lengths, rollouts and learning rate, without the remote backend and without prompt
# de-duplication.  One 8-GPU node.
set -euo pipefail
MODEL=${MODEL:-Qwen/Qwen3-32B}
DATA=${DATA:?directory with train.parquet / test.parquet from preprocess_bird.py}
REWARD=$(python -c "import recipes.rl.rewards.bird_reward as m; print(m.__file__)")

python -m verl.trainer.main_ppo \
  algorithm.adv_estimator=grpo \
  data.train_files="${DATA}/train.parquet" data.val_files="${DATA}/test.parquet" \
  data.train_batch_size=32 data.max_prompt_length=32768 data.max_response_length=4096 \
  custom_reward_function.path="${REWARD}" custom_reward_function.name=compute_score \
  actor_rollout_ref.model.path="${MODEL}" actor_rollout_ref.model.use_remove_padding=True \
  actor_rollout_ref.model.enable_gradient_checkpointing=True \
  actor_rollout_ref.actor.strategy=fsdp actor_rollout_ref.actor.fsdp_config.param_offload=True \
  actor_rollout_ref.actor.fsdp_config.optimizer_offload=True actor_rollout_ref.actor.ulysses_sequence_parallel_size=8 \
  actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=32 \
  actor_rollout_ref.actor.use_dynamic_bsz=True actor_rollout_ref.actor.ppo_max_token_len_per_gpu=36864 \
  actor_rollout_ref.actor.use_kl_loss=False \
  actor_rollout_ref.rollout.name=vllm actor_rollout_ref.rollout.n=16 actor_rollout_ref.rollout.temperature=1.0 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=4 actor_rollout_ref.rollout.gpu_memory_utilization=0.6 \
  trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=1 trainer.project_name=fsdp_baseline_bird "$@"
