"""The engine's update rule against torch.optim on the same gradients: AdamW (decoupled decay) and classic Adam
(``adam_w_mode: false``, decay through the moments), with the optimizer state on the device path and on the host."""
import pytest
import torch

from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
from tests.test_zorro_equivalence_cpu import make_grpo_batch


@pytest.mark.parametrize("adam_w_mode,offload", [(True, False), (False, False), (True, True), (False, True)])
def test_update_rule_matches_torch_optim(adam_w_mode, offload):
    ds = {"optimizer": {"type": "AdamW", "params": {"lr": 2e-3, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1,
                                                    "adam_w_mode": adam_w_mode}},
          "zero_optimization": {"stage": 1, "offload_optimizer": {"device": "cpu" if offload else "none"}}}
    cfg = EngineConfig.from_ds_config(ds)
    assert cfg.adam_w_mode == adam_w_mode and cfg.max_grad_norm == 0.0
    model = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=4)
    oracle = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=4)
    eng = TrainEngine(model, cfg)
    opt_cls = torch.optim.AdamW if adam_w_mode else torch.optim.Adam
    opt = opt_cls(oracle.parameters(), lr=2e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=8)
    pb = build_packed_batch(ids, mask, R, dedup=True)
    for _ in range(3):
        lp, _ = token_logprobs(eng.model, pb)
        eng.backward(-(lp.sum() / lp.numel()))
        eng.step()
        lo, _ = token_logprobs(oracle, pb)
        opt.zero_grad()
        (-(lo.sum() / lo.numel())).backward()
        opt.step()
    worst = 0.0
    for (n, a), (_n, b) in zip(eng.model.named_parameters(), oracle.named_parameters()):
        worst = max(worst, float((a.detach() - b.detach()).abs().max()))
    assert worst < 5e-5, worst


def test_training_config_passes_adam_mode_through():
    cfg = EngineConfig.from_ds_config({}, {"optimizer": {"lr": 1e-4, "adam_w_mode": False, "weight_decay": 0.01}})
    assert cfg.adam_w_mode is False and cfg.weight_decay == 0.01
    assert EngineConfig.from_ds_config({}, {"optimizer": {"lr": 1e-4}}).adam_w_mode is True
