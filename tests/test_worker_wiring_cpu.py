"""Options that reach the engines through the worker: token-set constraints carried by the batch, activation
offload, the one-shot profiler and memory reports."""
import os

import pytest
import torch

from arctic_platform_b200.engine.worker import EngineWorker
from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _worker(job_type="log_prob", **wc):
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": job_type, "seed": 6, "ds_worker_config": wc,
                  "ds_config": {"zero_optimization": {"stage": 1}}})
    return w


def test_action_masks_in_the_batch_constrain_the_scored_distribution():
    w = _worker()
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=3)
    B = ids.shape[0]
    rmask = mask[:, -R:].contiguous()
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": rmask}
    meta = {"zorro_train_enable": True, "compute_entropy": True}
    free = w.forward_no_grad(batch, meta)["batch"]
    # response position 0 of every rollout: only {label, 3, 4} are legal; position 1 of rollout 0: token 5 is illegal
    K = 3
    toks = torch.full((B, R, K), -1, dtype=torch.int64)
    allow = torch.full((B, R), -1, dtype=torch.int64)
    P = ids.shape[1] - R
    for b in range(B):
        toks[b, 0] = torch.tensor([int(ids[b, P]), 3, 4])
        allow[b, 0] = 1
    toks[0, 1, 0] = 5
    allow[0, 1] = 0
    con = w.forward_no_grad({**batch, "action_mask_tokens": toks, "action_mask_allow": allow}, meta)["batch"]
    lp_f, lp_c = free["log_probs"], con["log_probs"]
    assert (lp_c[:, 0] > lp_f[:, 0]).all()                         # mass of a three-token set: the label gains
    assert (con["entropy"][:, 0] < free["entropy"][:, 0]).all() and (con["entropy"][:, 0] <= torch.log(torch.tensor(3.0)) + 1e-5).all()
    assert lp_c[0, 1] >= lp_f[0, 1] - 1e-6                         # removing another token can only help the label
    untouched = rmask.bool().clone()
    untouched[:, 0] = False
    untouched[0, 1] = False
    assert torch.allclose(lp_c[untouched], lp_f[untouched], atol=1e-6)
    # a label outside its own allow list is impossible
    toks2 = toks.clone()
    toks2[1, 0] = torch.tensor([3, 4, -1])
    bad = w.forward_no_grad({**batch, "action_mask_tokens": toks2, "action_mask_allow": allow}, meta)["batch"]["log_probs"]
    assert torch.isinf(bad[1, 0]) and bad[1, 0] < 0
    # the allow flags can be left out: every position with tokens listed is an allow list
    same = w.forward_no_grad({**batch, "action_mask_tokens": torch.where(allow[..., None] == 0, -1, toks)}, meta)["batch"]["log_probs"]
    assert torch.allclose(same[:, 0], lp_c[:, 0], atol=1e-6)


def test_activation_offload_option_changes_nothing_but_where_tensors_wait():
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=2, seed=4)
    B = ids.shape[0]
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:].contiguous(),
             "advantages": torch.ones(B, R), "old_log_probs": torch.full((B, R), -3.0)}
    grads = {}
    for name, wc in (("plain", {}), ("offload", {"activation_offload": {"min_bytes": 1, "keep_last": 0}})):
        w = _worker("training", **wc)
        assert (w.activation_offload is not None) == (name == "offload")
        w.forward_backward(batch, {"zorro_train_enable": True}, {"loss_fn": "verl_grpo"})
        grads[name] = w.engine.grad_buf.tensor.clone()
        if name == "offload":
            st = w.activation_offload.stats.as_dict()
            assert st["skipped_tensors"] > 0 and st["offloaded_tensors"] == 0      # host tensors stay put; device tensors move (GPU test)
    assert torch.equal(grads["plain"], grads["offload"])
    assert _worker("training", activation_offload={"enable": False}).activation_offload is None


def test_one_shot_profiler_and_memory_report(monkeypatch, capsys, tmp_path):
    monkeypatch.setenv("APB_PROFILER", "c")
    monkeypatch.setenv("APB_PROFILER_CALL", "1")
    w = _worker()
    ids, mask, R = make_grpo_batch(n_prompts=1, n_samples=2, seed=5)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:].contiguous()}
    w.forward_no_grad(batch, {})
    out = capsys.readouterr().out
    assert "[profile] fwd:" in out and "cumulative" in out
    w.forward_no_grad(batch, {})
    assert "[profile]" not in capsys.readouterr().out               # only the chosen call is profiled
    from arctic_platform_b200.utils import debug
    monkeypatch.setattr(debug, "DISABLE_DEBUG", False)
    w.forward_no_grad(batch, {})
    out = capsys.readouterr().out
    assert "[mem][rank 0] fwd start" in out and "[mem][rank 0] fwd end" in out


def test_token_budget_micro_batches_keep_results_and_order():
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=3, seed=9, p_rng=(4, 40), r_rng=(2, 24))
    B = ids.shape[0]
    g = torch.Generator().manual_seed(1)
    batch = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, -R:].contiguous(),
             "advantages": torch.randn(B, 1, generator=g).expand(B, R).contiguous(),
             "old_log_probs": -2.0 + 0.01 * torch.randn(B, R, generator=g)}
    lp = _worker()
    whole = lp.forward_no_grad(batch, {"zorro_train_enable": True})["batch"]["log_probs"]
    budget = int(mask.sum(1).max()) * 3
    split = lp.forward_no_grad(batch, {"zorro_train_enable": True, "max_tokens_per_mb": budget})["batch"]["log_probs"]
    assert torch.allclose(split, whole, atol=1e-5)                          # same rows, same order
    plain = lp.forward_no_grad(batch, {"zorro_train_enable": False, "max_tokens_per_mb": budget})["batch"]["log_probs"]
    assert torch.allclose(plain, whole, atol=1e-5)
    with pytest.raises(ValueError):
        lp.forward_no_grad(batch, {"zorro_train_enable": False, "max_tokens_per_mb": 3})
    # training: the gradient of the whole batch, however it is cut up
    grads = {}
    for name, meta in (("whole", {}), ("budget", {"max_tokens_per_mb": budget}), ("four", {"num_micro_batches": 4})):
        w = _worker("training")
        out = w.forward_backward(batch, {"zorro_train_enable": True, **meta}, {"loss_fn": "verl_grpo"})
        grads[name] = w.engine.grad_buf.tensor.clone()
        assert out["metrics"]["loss.tokens"] == float(mask[:, -R:].sum())
    assert torch.allclose(grads["budget"], grads["whole"], atol=1e-6, rtol=1e-4)
    assert torch.allclose(grads["four"], grads["whole"], atol=1e-6, rtol=1e-4)


def test_sampler_worker_uses_the_tokenizer_that_ships_with_a_checkpoint(tmp_path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.models.hf_io import save_hf_checkpoint
    ck = tmp_path / "ck"
    save_hf_checkpoint(DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=1), ck)
    w = EngineWorker("cpu")
    w.initialize({"model_name": str(ck), "job_type": "sampling", "vllm_config": {"max_model_len": 64}})
    out = w.generate([[5, 6, 7]], {"n": 1, "max_tokens": 3, "temperature": 0.0})
    assert out[0]["text"] is None                                   # weights only: ids in, ids out
    with pytest.raises(ValueError, match="tokenizer"):
        w.generate(["hello"], {"max_tokens": 2})
    vocab = {**{f"w{i}": i for i in range(1, PRESETS["qwen3-tiny"].vocab_size)}, "[UNK]": 0}
    tk = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tk.pre_tokenizer = pre_tokenizers.Whitespace()
    PreTrainedTokenizerFast(tokenizer_object=tk, unk_token="[UNK]").save_pretrained(str(ck))
    w2 = EngineWorker("cpu")
    w2.initialize({"model_name": str(ck), "job_type": "sampling", "vllm_config": {"max_model_len": 64}})
    ids = w2.generate([[5, 6, 7]], {"n": 1, "max_tokens": 3, "temperature": 0.0})
    txt = w2.generate(["w5 w6 w7"], {"n": 1, "max_tokens": 3, "temperature": 0.0})
    assert txt[0]["token_ids"] == ids[0]["token_ids"] == out[0]["token_ids"]
    assert txt[0]["text"] == " ".join(f"w{t}" for t in txt[0]["token_ids"]) and txt[0]["prompt_len"] == 3
    quiet = w2.generate([[5, 6, 7]], {"n": 1, "max_tokens": 3, "temperature": 0.0, "detokenize": False})
    assert quiet[0]["text"] is None
    # stop strings: a one-token string ends the sequence in the sampler, a longer one cuts the decoded text
    full = ids[0]["token_ids"]
    stop_tok = full[1]
    cut = w2.generate([[5, 6, 7]], {"n": 1, "max_tokens": 3, "temperature": 0.0, "stop": f"w{stop_tok}"})
    assert cut[0]["token_ids"] == full[:full.index(stop_tok) + 1] and cut[0]["finish_reason"] == "stop"
    two = " ".join(f"w{t}" for t in full[1:3])
    cut2 = w2.generate([[5, 6, 7]], {"n": 1, "max_tokens": 3, "temperature": 0.0, "stop": [two]})
    whole = " ".join(f"w{t}" for t in full)
    assert cut2[0]["token_ids"] == full and cut2[0]["text"] == whole[:whole.find(two)] and cut2[0]["finish_reason"] == "stop"
    with pytest.raises(ValueError, match="stop strings"):
        w.generate([[5, 6, 7]], {"max_tokens": 2, "stop": "x"})
    # a training worker loaded from that directory exports checkpoints that carry the tokenizer along
    t = EngineWorker("cpu")
    t.initialize({"model_name": str(ck), "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}}})
    t.export_hf_checkpoint(str(tmp_path / "export"))
    assert (tmp_path / "export" / "tokenizer.json").exists() and (tmp_path / "export" / "config.json").exists()
    from transformers import AutoTokenizer
    assert AutoTokenizer.from_pretrained(str(tmp_path / "export"), local_files_only=True).encode("w5 w6", add_special_tokens=False) == [5, 6]


def test_log_prob_top_k_and_scoring_engine_choice():
    """``log_probs(top_k > 1)`` returns the k most likely tokens per completion position (the chosen token's own
    log-prob stays in ``log_probs``), and the server hands ``log_prob_engine`` to its log-prob jobs."""
    import torch
    from arctic_platform_b200.common.server import ArcticRLServerCore
    core = ArcticRLServerCore(log_prob_engine="vllm")
    try:
        jid = core.initialize({"model_name": "qwen3-tiny", "job_type": "log_prob", "seed": 3})["job_id"]
        assert core.jobs[jid].config["log_prob_engine"] == "vllm"
        prompts, completions = [[5, 6, 7, 8], [9, 10, 11]], [[12, 13, 14], [15, 16]]
        one = core.log_probs(jid, prompts, completions)
        top = core.log_probs(jid, prompts, completions, top_k=3)
        assert "top_log_probs" not in one and len(top["top_log_probs"]) == 2
        for rows, tops, comp in zip(top["log_probs"], top["top_log_probs"], completions):
            assert len(rows) == len(tops) == len(comp)
            for lp, cand, tok in zip(rows, tops, comp):
                assert len(cand) == 3 and max(cand.values()) >= lp - 1e-4
                if tok in cand:
                    assert cand[tok] == pytest.approx(lp, abs=1e-4)
        assert one["log_probs"][0] == pytest.approx(top["log_probs"][0], abs=1e-5)
    finally:
        core.destroy()
    with pytest.raises(ValueError):
        ArcticRLServerCore(log_prob_engine="other")
