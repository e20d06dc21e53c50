"""The RL scoring path against explicit soft-max arithmetic on full logits: log-probs and entropy on the response
grid, temperature, prompt de-duplication on and off, ragged prompts and responses, micro-batch splitting."""
import numpy as np
import pytest
import torch

from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM
from arctic_platform_b200.ops.attention import AttnLayout
from arctic_platform_b200.rl.processors.pipeline import run_pipeline
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _oracle(model, ids, mask, R, temperature):
    """Per sample: log p(token) and entropy of the tempered distribution for every valid response token."""
    B, S = ids.shape
    P = S - R
    lp = torch.zeros(B, R)
    ent = torch.zeros(B, R)
    for b in range(B):
        seq = ids[b][mask[b].bool()]
        n_resp = int(mask[b, P:].sum())
        if n_resp == 0:
            continue
        with torch.no_grad():
            h = model.forward_hidden(seq, torch.arange(len(seq)), AttnLayout.from_cu_seqlens(np.array([0, len(seq)])))
            logp = torch.log_softmax(model.logits(h) / temperature, -1)
        first = len(seq) - n_resp                          # index of the first response token in the sequence
        rows = logp[first - 1:len(seq) - 1]
        lp[b, :n_resp] = rows.gather(1, seq[first:, None])[:, 0]
        ent[b, :n_resp] = -(rows.exp() * rows).sum(-1)
    return lp, ent


@pytest.mark.parametrize("preset", ["qwen3-tiny", "qwen3-moe-tiny", "qwen3.5-moe-tiny"])
@pytest.mark.parametrize("dedup,temperature", [(True, 1.0), (False, 1.0), (True, 0.7)])
def test_scoring_equals_explicit_softmax(preset, dedup, temperature):
    cfg = PRESETS[preset]
    eng = TrainEngine(DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=3), EngineConfig(), forward_only=True)
    ids, mask, R = make_grpo_batch(n_prompts=3, n_samples=3, seed=7)
    ids = ids % cfg.vocab_size
    mask[4, -R:] = 0                                        # one rollout with an empty response
    mask[4, -R] = 1                                         # ... and one with a single token
    mask[5, -R:] = 0
    want_lp, want_ent = _oracle(eng.model, ids, mask, R, temperature)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:].contiguous()}
    meta = {"zorro_train_enable": dedup, "temperature": temperature, "compute_entropy": True}
    r = run_pipeline(eng, batch, meta, {"loss_fn": None, "post": []}, backward=False)
    m = mask[:, -R:].bool()
    assert torch.allclose(r["batch"]["log_probs"][m], want_lp[m], atol=2e-5)
    assert torch.allclose(r["batch"]["entropy"][m], want_ent[m], atol=2e-5)
    assert float(r["batch"]["log_probs"][~m].abs().max()) == 0.0       # padding stays zero
    # share of the un-deduplicated tokens that the shared prompts save
    assert (r["metrics"]["perf/dedup_redundancy"] > 0.2) == dedup


def test_worker_micro_batches_return_the_same_grid():
    from arctic_platform_b200.engine.worker import EngineWorker
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=4, seed=8)
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": "log_prob", "seed": 2})
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:].contiguous()}
    one = w.forward_no_grad(batch, {"zorro_train_enable": True})["batch"]["log_probs"]
    four = w.forward_no_grad(batch, {"zorro_train_enable": True, "num_micro_batches": 4})["batch"]["log_probs"]
    assert one.shape == four.shape == (8, R) and torch.allclose(one, four, atol=1e-5)
    want, _ = _oracle(w.engine.model, ids, mask, R, 1.0)
    assert torch.allclose(one[mask[:, -R:].bool()], want[mask[:, -R:].bool()], atol=2e-5)
