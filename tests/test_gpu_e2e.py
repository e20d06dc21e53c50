"""Two GRPO steps through the public client on one GPU with all three jobs colocated: rollout -> old / reference
log-probs -> forward-backward -> optimizer step -> weight hand-over.  Checks that the sampler's own log-probs agree
with the trainer's scoring of the same tokens (low KL), that the hand-over makes the weight norms equal, that the
update moves the policy and that the second rollout comes from the updated weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("stage", [2])
def test_two_step_grpo_loop_colocated(stage):
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client
    P, R, n_prompts, n = 24, 16, 3, 4
    cfg = ArcticRLClientConfig(comm_protocol="local", model_name="qwen3-tiny-d128", training_gpus=1, sampling_gpus=1,
                               log_prob_gpus=1, colocate=True, seed=3,
                               ds_config={"zero_optimization": {"stage": stage}, "gradient_clipping": 1.0,
                                          "optimizer": {"type": "AdamW", "params": {"lr": 1e-2}}},
                               vllm_config={"max_model_len": P + R + 8, "kv_cache_tokens": 1 << 14})
    client = create_arctic_rl_client(cfg)
    g = torch.Generator().manual_seed(0)
    norms, kls, losses = [], [], []
    try:
        for step in range(2):
            client.call("sync_weights")
            wn = client.call("weight_norm")
            assert wn["training_norm"] == pytest.approx(wn["sampling_norm"], rel=1e-3)
            norms.append(wn["training_norm"])
            prompts = [torch.randint(3, 200, (int(torch.randint(8, P, (1,), generator=g)),), generator=g).tolist()
                       for _ in range(n_prompts)]
            outs = client.call("generate", prompts, {"n": n, "temperature": 1.0, "max_tokens": R, "seed": step})
            B = len(outs)
            assert B == n_prompts * n
            ids = torch.zeros((B, P + R), dtype=torch.int64)
            mask = torch.zeros_like(ids)
            samp_lp = torch.zeros(B, R)
            for i, o in enumerate(outs):
                p, t = prompts[o["prompt_index"]], o["token_ids"]
                ids[i, P - len(p):P] = torch.tensor(p)
                mask[i, P - len(p):P] = 1
                ids[i, P:P + len(t)] = torch.tensor(t)
                mask[i, P:P + len(t)] = 1
                samp_lp[i, :len(t)] = torch.tensor(o["logprobs"])
            rmask = mask[:, P:].contiguous()
            rewards = torch.randn(B, generator=g).view(n_prompts, n)
            adv = ((rewards - rewards.mean(1, keepdim=True)) / (rewards.std(1, keepdim=True) + 1e-6)).reshape(B, 1)
            batch = {"input_ids": ids, "attention_mask": mask, "response_mask": rmask,
                     "advantages": adv.expand(B, R).contiguous()}
            meta = {"zorro_train_enable": True, "temperature": 1.0}
            old = client.call("fwd_no_grad", {"batch": batch, "meta": meta})["batch"]["log_probs"]
            ref = client.call("fwd_no_grad", {"batch": batch, "meta": meta}, reference_model=True)["batch"]["log_probs"]
            m = rmask.bool()
            # the sampler decoded with the weights the trainer now scores with: per-token agreement up to bf16 noise
            kls.append(float((samp_lp[m] - old[m]).abs().mean()))
            assert (ref[m] - old[m]).abs().mean() < 0.05 or step > 0        # the reference engine holds the initial policy
            batch["old_log_probs"], batch["ref_log_prob"] = old, ref
            out = client.call("fwd_bwd", {"batch": batch, "meta": meta}, {"loss_fn": "verl_grpo"})
            st = client.call("step")
            losses.append(out["avg_loss"])
            assert st["metrics"]["grad_norm"] > 0 and st["metrics"]["last_lr"] == pytest.approx(1e-2)
            _lib.check_status(f"grpo step {step}")
        client.call("sync_weights")
        wn = client.call("weight_norm")
        assert wn["training_norm"] == pytest.approx(wn["sampling_norm"], rel=1e-3)
        assert abs(wn["training_norm"] - norms[0]) / norms[0] > 1e-5          # two steps at lr 1e-2 moved the weights
        assert max(kls) < 0.05, kls
        assert all(torch.isfinite(torch.tensor(losses)))
    finally:
        client.call("shutdown")
