"""Speculative decoding on the tensor-op engine: a small draft model proposes ``k`` tokens, the target model scores
them all in one pass, and the standard accept / resample rule keeps the output distribution exactly the target's.

The reference passes ``arctic_inference_config.speculative_decoding.model`` to its sampler as ``spec_model``
(arctic_platform/common/utils/server_models.py:134-165); the drafting and verification happen inside ArcticInference.
Here the same configuration key selects this sampler on the engines that recompute sequences through the training
model (CPU runs, and GPU runs that ask for it with ``vllm_config.speculative_engine = "tensor_op"``).  The paged CUDA
engine verifies one token per sequence and step and does not speculate.

One round for a sequence ``s``:

1. the draft model extends ``s`` by ``k`` tokens, sampling each from its own (temperature / top-k / top-p shaped)
   distribution ``q_i``;
2. ONE target pass over ``s + k`` tokens gives the target distributions ``p_0 .. p_k`` at the ``k + 1`` positions;
3. token ``i`` is accepted with probability ``min(1, p_i(x_i) / q_i(x_i))``; at the first rejection a replacement is
   drawn from ``max(0, p_i - q_i)`` renormalised and the round ends; if all ``k`` are accepted, a bonus token is drawn
   from ``p_k``.  Greedy decoding (temperature 0) accepts exactly the tokens the target would have produced and
   replaces the first mismatch by the target's arg-max, so its output equals plain greedy decoding token for token.

Every round therefore emits between 1 and ``k + 1`` tokens for ``k`` draft passes and one target pass.  All sequences
of a request (``n`` samples of every prompt) advance together: a draft step, and the verifying target pass, is ONE
packed forward over all sequences that are still running, so the number of model passes per round does not grow with
the number of sequences.  Requests with
distribution shaping that depends on the tokens emitted so far (penalties, ``min_tokens``, ``logit_bias``, ``min_p``)
fall back to plain decoding.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.config import DecoderConfig
from ..models.decoder import DecoderLM
from ..ops.attention import AttnLayout
from .reference_sampler import EXTRA_KEYS, LogitsProcessor, ReferenceSampler, filter_logits
from .sampler import SamplingParams


class SpeculativeSampler(ReferenceSampler):
    """``ReferenceSampler`` with a draft model.  ``stats`` accumulates ``proposed`` / ``accepted`` draft tokens,
    ``rounds`` and ``target_passes`` since construction (``acceptance_rate()`` = accepted / proposed)."""

    def __init__(self, cfg: DecoderConfig, device="cpu", model: Optional[DecoderLM] = None,
                 draft_model: Optional[DecoderLM] = None, num_speculative_tokens: int = 4, **kw):
        super().__init__(cfg, device, model=model, **kw)
        if draft_model is None:
            raise ValueError("speculative decoding needs a draft model (spec_model)")
        if draft_model.cfg.vocab_size != cfg.vocab_size:
            raise ValueError(f"draft vocabulary ({draft_model.cfg.vocab_size}) differs from the target's ({cfg.vocab_size})")
        if num_speculative_tokens < 1:
            raise ValueError("num_speculative_tokens must be at least 1")
        self.draft = draft_model
        self.k = int(num_speculative_tokens)
        self.stats: Dict[str, int] = {"proposed": 0, "accepted": 0, "rounds": 0, "target_passes": 0}

    def acceptance_rate(self) -> float:
        return self.stats["accepted"] / max(1, self.stats["proposed"])

    # ------------------------------------------------------------------ model passes
    def _logits_packed(self, model: DecoderLM, seqs: Sequence[Sequence[int]], lasts: Sequence[int]) -> List[torch.Tensor]:
        """fp32 logits of the last ``lasts[i]`` positions of every sequence, from one packed recompute pass."""
        lens = [len(s) for s in seqs]
        ids = torch.tensor([t for s in seqs for t in s], dtype=torch.int64, device=self.device)
        pos = torch.cat([torch.arange(n, device=self.device) for n in lens])
        cu = np.concatenate([[0], np.cumsum(lens)])
        h = model.forward_hidden(ids, pos, AttnLayout.from_cu_seqlens(cu))
        rows = torch.cat([torch.arange(int(cu[i + 1]) - int(lasts[i]), int(cu[i + 1]), device=self.device) for i in range(len(seqs))])
        return list(model.logits(h[rows]).float().split([int(x) for x in lasts]))

    def _logits(self, model: DecoderLM, seq: Sequence[int], last: int) -> torch.Tensor:
        return self._logits_packed(model, [seq], [last])[0]

    @staticmethod
    def _dist(logits: torch.Tensor, sp: SamplingParams) -> torch.Tensor:
        """The distribution tokens are drawn from: temperature, then top-k / top-p."""
        return torch.softmax(filter_logits(logits / sp.temperature, sp.top_k, sp.top_p), -1)

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sampling_params=None) -> List[dict]:
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else \
            SamplingParams.from_dict(sampling_params, supported=EXTRA_KEYS)
        if LogitsProcessor(sampling_params if isinstance(sampling_params, dict) else None).active:
            return super().generate(prompts, sampling_params)      # history-dependent shaping: plain decoding
        if self._asleep:
            raise RuntimeError("sampler is asleep; call wake() first")
        if sp.seed is not None:
            self.gen.manual_seed(int(sp.seed))
        stops = set(int(t) for t in sp.stop_token_ids)
        if self.eos is not None and not sp.ignore_eos:
            stops.add(int(self.eos))
        greedy = not (sp.temperature and sp.temperature > 0)
        states: List[dict] = []
        for pi, prompt in enumerate(prompts):
            if len(prompt) == 0:
                raise ValueError("empty prompt")
            if len(prompt) + sp.max_tokens > self.max_seq_len:
                raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({sp.max_tokens}) exceeds max_seq_len {self.max_seq_len}")
            for _ in range(sp.n):
                states.append({"seq": list(map(int, prompt)), "out": [], "lps": [], "reason": "length", "pi": pi,
                               "prompt_len": len(prompt)})
        running = [st for st in states if sp.max_tokens > 0]
        while running:
            ks = [min(self.k, sp.max_tokens - len(st["out"])) for st in running]
            emitted = self._rounds([st["seq"] for st in running], ks, sp, greedy)
            still = []
            for st, (toks, tok_lps) in zip(running, emitted):
                for tok, lp in zip(toks, tok_lps):
                    st["out"].append(tok)
                    st["lps"].append(lp)
                    st["seq"].append(tok)
                    if tok in stops:
                        st["reason"] = "stop"
                        break
                    if len(st["out"]) >= sp.max_tokens:
                        break
                if st["reason"] == "length" and len(st["out"]) < sp.max_tokens:
                    still.append(st)
            running = still
        return [{"token_ids": st["out"], "logprobs": st["lps"], "finish_reason": st["reason"], "prompt_len": st["prompt_len"],
                 "prompt_index": st["pi"], "text": None} for st in states]

    def _draw(self, probs: torch.Tensor) -> int:
        return int(torch.multinomial(probs.cpu(), 1, generator=self.gen))

    def _round(self, seq: List[int], k: int, sp: SamplingParams, greedy: bool):
        """One draft-and-verify round after ``seq``: the emitted tokens (1 .. k + 1) and their log-probs under the
        target's unfiltered (temperature-scaled) policy."""
        return self._rounds([seq], [k], sp, greedy)[0]

    def _rounds(self, seqs: Sequence[List[int]], ks: Sequence[int], sp: SamplingParams, greedy: bool):
        """One round for every sequence at once (``ks[i]`` draft tokens for sequence ``i``): ``max(ks)`` packed draft
        passes and one packed target pass.  Returns ``[(tokens, log-probs)]`` in the order of ``seqs``."""
        n = len(seqs)
        exts = [list(s) for s in seqs]
        draft_tokens: List[List[int]] = [[] for _ in range(n)]
        draft_probs: List[List[torch.Tensor]] = [[] for _ in range(n)]
        # 1. draft: step j extends every sequence that still has draft tokens to produce
        for j in range(max(ks)):
            idx = [i for i in range(n) if j < ks[i]]
            for i, lg in zip(idx, self._logits_packed(self.draft, [exts[i] for i in idx], [1] * len(idx))):
                lg = lg[0]
                if greedy:
                    tok = int(lg.argmax())
                    draft_probs[i].append(lg)                          # unused in greedy mode
                else:
                    q = self._dist(lg, sp)
                    tok = self._draw(q)
                    draft_probs[i].append(q)
                draft_tokens[i].append(tok)
                exts[i].append(tok)
        # 2. one target pass over every seq + drafts: distributions at the k + 1 positions after seq[-1], x_1, ..., x_k
        target = self._logits_packed(self.model, exts, [k + 1 for k in ks])
        self.stats["rounds"] += n
        self.stats["target_passes"] += 1
        self.stats["proposed"] += int(sum(ks))
        scale = sp.temperature if not greedy else 1.0
        # 3. accept / resample, sequence by sequence
        return [self._verify(target[i], draft_tokens[i], draft_probs[i], ks[i], sp, greedy, scale) for i in range(n)]

    def _verify(self, tl: torch.Tensor, drafts: List[int], qs: List[torch.Tensor], k: int, sp: SamplingParams, greedy: bool,
                scale: float):
        emitted: List[int] = []
        emitted_lps: List[float] = []

        def emit(tok: int, pos: int) -> None:
            emitted.append(tok)
            emitted_lps.append(float(torch.log_softmax(tl[pos] / scale, -1)[tok]))

        for i, x in enumerate(drafts):
            if greedy:
                best = int(tl[i].argmax())
                if best == x:
                    emit(x, i)
                    self.stats["accepted"] += 1
                    continue
                emit(best, i)
                return emitted, emitted_lps
            p, q = self._dist(tl[i], sp), qs[i]
            ratio = float(p[x]) / max(float(q[x]), 1e-30)
            if float(torch.rand((), generator=self.gen)) < min(1.0, ratio):
                emit(x, i)
                self.stats["accepted"] += 1
                continue
            resid = torch.clamp(p - q, min=0.0)
            total = float(resid.sum())
            emit(self._draw(resid / total) if total > 0 else self._draw(p), i)
            return emitted, emitted_lps
        # all k accepted: one more token from the target's distribution after the last draft
        emit(int(tl[k].argmax()) if greedy else self._draw(self._dist(tl[k], sp)), k)
        return emitted, emitted_lps

    # ------------------------------------------------------------------ weights: the target's; the draft is static
    def weight_norm(self) -> Dict[str, float]:
        out = super().weight_norm()
        out["draft_parameters"] = float(sum(p.numel() for p in self.draft.parameters()))
        return out
