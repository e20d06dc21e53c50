"""SFT pipeline against explicit cross entropy on the model's logits, and its edge cases: label masks, all-masked
batches, micro-batch invariance with global token counts, padding sides, and batches the client packed itself."""
import pytest
import torch
import torch.nn.functional as F

from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM
from arctic_platform_b200.ops.attention import AttnLayout
from arctic_platform_b200.sft.processor import batch_is_packed, inject_sft_global_token_meta, run_sft_pipeline

import numpy as np


def _engine(seed=1):
    model = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=seed)
    return TrainEngine(model, EngineConfig(lr=1e-3))


def _oracle_ce(model, seq):
    """Sum of next-token cross entropies of one un-padded sequence, from full logits."""
    ids = torch.tensor(seq)
    with torch.no_grad():
        h = model.forward_hidden(ids, torch.arange(len(seq)), AttnLayout.from_cu_seqlens(np.array([0, len(seq)])))
        logits = model.logits(h)
    return F.cross_entropy(logits[:-1], ids[1:], reduction="none")


def _batch(seqs, side="right", S=None):
    S = S or max(len(s) for s in seqs)
    ids = torch.zeros(len(seqs), S, dtype=torch.int64)
    mask = torch.zeros_like(ids)
    for i, s in enumerate(seqs):
        sl = slice(0, len(s)) if side == "right" else slice(S - len(s), S)
        ids[i, sl] = torch.tensor(s)
        mask[i, sl] = 1
    return ids, mask


SEQS = [[5, 9, 11, 3, 7, 21], [4, 4, 8], [30, 2, 17, 17, 6]]


@pytest.mark.parametrize("side", ["right", "left"])
def test_sft_losses_equal_explicit_cross_entropy(side):
    eng = _engine()
    ids, mask = _batch(SEQS, side)
    per_tok = [_oracle_ce(eng.model, s) for s in SEQS]
    total, n = float(sum(t.sum() for t in per_tok)), sum(len(t) for t in per_tok)
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    r = run_sft_pipeline(eng, {"input_ids": ids, "attention_mask": mask, "labels": labels}, backward=False)
    assert r["metrics"]["loss.sum"] == pytest.approx(total, rel=1e-5) and r["metrics"]["loss.tokens"] == n
    assert r["avg_loss"] == pytest.approx(total / n, rel=1e-5)             # batch_num_tokens injected: one rank
    r2 = run_sft_pipeline(eng, {"input_ids": ids, "attention_mask": mask, "labels": labels}, processing={"loss_fn": "sft"},
                          backward=False)
    assert r2["avg_loss"] == pytest.approx(total / n, rel=1e-5)
    # per-token log-probs come back on the grid at the column of the PREDICTED token
    grid = r["batch"]["log_probs"]
    for i, s in enumerate(SEQS):
        cols = mask[i].nonzero()[:, 0][1:]
        assert torch.allclose(-grid[i, cols], per_tok[i], atol=1e-5)


def test_label_mask_selects_tokens_and_all_masked_is_zero():
    eng = _engine()
    ids, mask = _batch(SEQS)
    per_tok = [_oracle_ce(eng.model, s) for s in SEQS]
    labels = torch.full_like(ids, -100)
    labels[0, 3:6] = ids[0, 3:6]                        # train on the "answer" of the first sequence only
    r = run_sft_pipeline(eng, {"input_ids": ids, "attention_mask": mask, "labels": labels}, backward=True)
    assert r["metrics"]["loss.tokens"] == 3
    assert r["metrics"]["loss.sum"] == pytest.approx(float(per_tok[0][2:5].sum()), rel=1e-5)
    lm = torch.zeros_like(ids)
    lm[1, 1:3] = 1
    eng.zero_grad()
    r = run_sft_pipeline(eng, {"input_ids": ids, "attention_mask": mask, "loss_mask": lm}, backward=False)
    assert r["metrics"]["loss.sum"] == pytest.approx(float(per_tok[1].sum()), rel=1e-5)
    # nothing to learn from: zero loss, zero gradient, no NaN
    eng.zero_grad()
    r = run_sft_pipeline(eng, {"input_ids": ids, "attention_mask": mask, "labels": torch.full_like(ids, -100)}, backward=True)
    assert r["avg_loss"] == 0.0 and r["metrics"]["loss.tokens"] == 0
    assert float(eng.grad_buf.tensor.abs().max()) == 0.0
    for fn in ("sft", "sft_ce"):
        r = run_sft_pipeline(eng, {"input_ids": ids, "attention_mask": mask, "labels": torch.full_like(ids, -100)},
                             processing={"loss_fn": fn}, backward=False)
        assert r["avg_loss"] == 0.0


def test_micro_batches_with_global_token_count_equal_one_batch():
    ids, mask = _batch(SEQS)
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    whole = _engine()
    run_sft_pipeline(whole, {"input_ids": ids, "attention_mask": mask, "labels": labels})
    g_whole = whole.grad_buf.tensor.clone()
    split = _engine()
    meta = {}
    inject_sft_global_token_meta({"input_ids": ids, "attention_mask": mask, "labels": labels}, meta)
    assert meta["batch_num_tokens"] == sum(len(s) - 1 for s in SEQS)
    for rows in ([0], [1, 2]):                          # very different token counts per micro-batch
        run_sft_pipeline(split, {"input_ids": ids[rows], "attention_mask": mask[rows], "labels": labels[rows]}, dict(meta))
    assert torch.allclose(split.grad_buf.tensor, g_whole, atol=1e-6, rtol=1e-5)
    # without the global count every micro-batch would be normalised by its own tokens: a different gradient
    local = _engine()
    for rows in ([0], [1, 2]):
        run_sft_pipeline(local, {"input_ids": ids[rows], "attention_mask": mask[rows], "labels": labels[rows]},
                         processing={"loss_fn": "sft"})
    assert not torch.allclose(local.grad_buf.tensor, g_whole, atol=1e-6, rtol=1e-3)


def test_client_packed_row_keeps_documents_apart():
    eng = _engine()
    per_tok = [_oracle_ce(eng.model, s) for s in SEQS]
    flat = [t for s in SEQS for t in s]
    pos = [i for s in SEQS for i in range(len(s))]
    batch = {"input_ids": torch.tensor([flat]), "position_ids": torch.tensor([pos])}
    assert batch_is_packed(batch) and not batch_is_packed({"position_ids": torch.arange(6)[None]})
    r = run_sft_pipeline(eng, batch, backward=False)
    n = sum(len(t) for t in per_tok)
    assert r["metrics"]["loss.tokens"] == n                      # document ends predict nothing
    assert r["metrics"]["loss.sum"] == pytest.approx(float(sum(t.sum() for t in per_tok)), rel=1e-5)
    cu = torch.tensor([0, 6, 9, 14])
    r2 = run_sft_pipeline(eng, {"input_ids": torch.tensor([flat]), "cu_seqlens": cu}, backward=False)
    assert r2["metrics"]["loss.sum"] == pytest.approx(r["metrics"]["loss.sum"], rel=1e-6)
    # labels on the packed row, with trailing padding after the last document
    padded = torch.tensor([flat + [0, 0]])
    labels = torch.full_like(padded, -100)
    labels[0, 7:9] = padded[0, 7:9]                              # the second document's two predicted tokens
    r3 = run_sft_pipeline(eng, {"input_ids": padded, "cu_seqlens": cu, "labels": labels}, backward=False)
    assert r3["metrics"]["loss.tokens"] == 2
    assert r3["metrics"]["loss.sum"] == pytest.approx(float(per_tok[1].sum()), rel=1e-5)
    # treated as ONE sequence the numbers differ: the second document would attend to the first
    one = run_sft_pipeline(eng, {"input_ids": torch.tensor([flat])}, backward=False)
    assert one["metrics"]["loss.tokens"] == len(flat) - 1
    with pytest.raises(ValueError):
        run_sft_pipeline(eng, {"input_ids": torch.tensor([flat]), "cu_seqlens": torch.tensor([0, 9, 6])}, backward=False)


def test_worker_normalises_sft_ce_over_all_micro_batches():
    """Through the worker: a list of micro-batches (client-side gradient accumulation) with very different token
    counts gives the gradient of the whole batch; the worker works out the global token count itself."""
    from arctic_platform_b200.engine.worker import EngineWorker
    ids, mask = _batch(SEQS, "left")
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    job = {"model_name": "qwen3-tiny", "job_type": "training", "seed": 5, "ds_config": {"zero_optimization": {"stage": 1}}}
    grads = []
    for parts in ([[0, 1, 2]], [[0], [1, 2]]):
        w = EngineWorker("cpu")
        w.initialize(job)
        mbs = [{"input_ids": ids[r], "attention_mask": mask[r], "labels": labels[r]} for r in parts]
        out = w.forward_backward(mbs if len(mbs) > 1 else mbs[0], {}, {"loss_fn": "sft_ce"})
        assert out["metrics"]["loss.tokens"] == sum(len(s) - 1 for s in SEQS)
        grads.append(w.engine.grad_buf.tensor.clone())
    assert torch.allclose(grads[0], grads[1], atol=1e-6, rtol=1e-5)
