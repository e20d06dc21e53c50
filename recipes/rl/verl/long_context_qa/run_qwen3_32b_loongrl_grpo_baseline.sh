#!/usr/bin/env bash
# A/B twin of run_qwen3_32b_loongrl_grpo_zorro.sh on verl's own engines (FSDP + vLLM TP 4), 16K prompts, 4K responses,
# 16 rollouts per prompt; no remote backend, every rollout carries its own copy of the prompt through training.
set -euo pipefail
MODEL=${MODEL:-Qwen/Qwen3-32B}
DATA=${DATA:?directory with merged/train.parquet from recipes.rl.data.prepare_data long_context_qa}
REWARD=$(python -c "import recipes.rl.rewards.long_context_qa_reward as m; print(m.__file__)")

python -m verl.trainer.main_ppo \
  algorithm.adv_estimator=grpo \
  data.train_files="${DATA}/merged/train.parquet" data.val_files="${DATA}/merged/test.parquet" \
  data.train_batch_size=32 data.max_prompt_length=16384 data.max_response_length=4096 \
  custom_reward_function.path="${REWARD}" custom_reward_function.name=compute_score \
  actor_rollout_ref.model.path="${MODEL}" actor_rollout_ref.model.use_remove_padding=True \
  actor_rollout_ref.model.enable_gradient_checkpointing=True \
  actor_rollout_ref.actor.strategy=fsdp actor_rollout_ref.actor.fsdp_config.param_offload=True \
  actor_rollout_ref.actor.fsdp_config.optimizer_offload=True actor_rollout_ref.actor.ulysses_sequence_parallel_size=4 \
  actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=32 \
  actor_rollout_ref.actor.use_dynamic_bsz=True actor_rollout_ref.actor.ppo_max_token_len_per_gpu=20480 \
  actor_rollout_ref.rollout.name=vllm actor_rollout_ref.rollout.n=16 actor_rollout_ref.rollout.temperature=1.0 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=4 actor_rollout_ref.rollout.gpu_memory_utilization=0.6 \
  trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=1 trainer.project_name=fsdp_baseline_loongrl "$@"
