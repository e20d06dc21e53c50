"""Plain PyTorch sampler with the interface of :class:`~arctic_platform_b200.engine.sampler.SamplerEngine`.

It recomputes the whole sequence at every step through the training model (no KV cache, no paging, no graphs), so
it is only for CPU runs of the full RL loop, tiny models and as the token-level oracle of the CUDA sampler (greedy
outputs must match; sampled tokens come from the same filtered distribution).  Unlike the CUDA kernel it also
implements top-k and top-p filtering."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.config import DecoderConfig
from ..models.decoder import DecoderLM
from ..ops.attention import AttnLayout
from .sampler import SamplingParams


def filter_logits(logits: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """``-inf`` outside the top-k tokens and outside the smallest set whose probability mass reaches ``top_p``."""
    if top_k and top_k > 0 and top_k < logits.shape[-1]:
        kth = torch.topk(logits, top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        srt, idx = torch.sort(logits, dim=-1, descending=True)
        probs = torch.softmax(srt, -1)
        drop = probs.cumsum(-1) - probs > top_p                   # mass BEFORE the token already exceeds top_p
        srt = srt.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    return logits


EXTRA_KEYS = ("repetition_penalty", "presence_penalty", "frequency_penalty", "min_p", "min_tokens", "logit_bias")


class LogitsProcessor:
    """Distribution shaping that the tensor-op samplers implement beyond temperature / top-k / top-p, in the order
    vLLM applies it: ``logit_bias``, repetition penalty (prompt and output tokens: positive logits divided, negative
    multiplied), presence / frequency penalties (output tokens), then -- after temperature -- ``min_p`` (tokens below
    ``min_p`` times the top probability are dropped); ``min_tokens`` keeps the stop tokens impossible until that many
    tokens were produced."""

    def __init__(self, params: Optional[dict], stop_ids: Sequence[int] = ()):
        p = dict(params or {})
        self.repetition = float(p.get("repetition_penalty") or 1.0)
        self.presence = float(p.get("presence_penalty") or 0.0)
        self.frequency = float(p.get("frequency_penalty") or 0.0)
        self.min_p = float(p.get("min_p") or 0.0)
        self.min_tokens = int(p.get("min_tokens") or 0)
        self.bias = {int(k): float(v) for k, v in (p.get("logit_bias") or {}).items()}
        self.stop_ids = [int(t) for t in stop_ids]
        self.active = (self.repetition != 1.0 or self.presence or self.frequency or self.min_p or self.min_tokens
                       or bool(self.bias))

    def before_temperature(self, logits: torch.Tensor, prompt: Sequence[int], output: Sequence[int]) -> torch.Tensor:
        """``logits [V]`` of one sequence -> adjusted copy."""
        if not self.active:
            return logits
        logits = logits.clone()
        for t, b in self.bias.items():
            if 0 <= t < logits.shape[-1]:
                logits[t] += b
        if self.repetition != 1.0:
            seen = torch.tensor(sorted(set(prompt) | set(output)), dtype=torch.long, device=logits.device)
            if seen.numel():
                v = logits[seen]
                logits[seen] = torch.where(v > 0, v / self.repetition, v * self.repetition)
        if (self.presence or self.frequency) and len(output):
            toks, counts = torch.tensor(output, dtype=torch.long, device=logits.device).unique(return_counts=True)
            logits[toks] -= self.presence + self.frequency * counts.to(logits.dtype)
        if len(output) < self.min_tokens and self.stop_ids:
            logits[torch.tensor(self.stop_ids, dtype=torch.long, device=logits.device)] = float("-inf")
        return logits

    def after_temperature(self, scaled: torch.Tensor) -> torch.Tensor:
        if not self.min_p:
            return scaled
        probs = torch.softmax(scaled, -1)
        return scaled.masked_fill(probs < self.min_p * probs.max(-1, keepdim=True).values, float("-inf"))


class ReferenceSampler:
    def __init__(self, cfg: DecoderConfig, device="cpu", model: Optional[DecoderLM] = None, max_seq_len: int = 8192,
                 seed: int = 0, eos_token_id: Optional[int] = None, **_ignored):
        self.cfg = cfg
        self.device = torch.device(device)
        self.model = model if model is not None else DecoderLM(cfg, self.device, torch.float32)
        self.max_seq_len = max_seq_len
        self.eos = eos_token_id
        self.gen = torch.Generator(device="cpu").manual_seed(seed)
        self._asleep = False

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sampling_params=None) -> List[dict]:
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else \
            SamplingParams.from_dict(sampling_params, supported=EXTRA_KEYS)
        if self._asleep:
            raise RuntimeError("sampler is asleep; call wake() first")
        if sp.seed is not None:
            self.gen.manual_seed(int(sp.seed))
        stops = set(int(t) for t in sp.stop_token_ids)
        if self.eos is not None and not sp.ignore_eos:
            stops.add(int(self.eos))
        shaper = LogitsProcessor(sampling_params if isinstance(sampling_params, dict) else None, sorted(stops))
        results: List[dict] = []
        for pi, prompt in enumerate(prompts):
            if len(prompt) == 0:
                raise ValueError("empty prompt")
            if len(prompt) + sp.max_tokens > self.max_seq_len:
                raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({sp.max_tokens}) exceeds max_seq_len {self.max_seq_len}")
            for _ in range(sp.n):
                seq = list(map(int, prompt))
                out, lps, reason = [], [], "length"
                for _t in range(sp.max_tokens):
                    ids = torch.tensor(seq, dtype=torch.int64, device=self.device)
                    layout = AttnLayout.from_cu_seqlens(np.array([0, len(seq)]))
                    h = self.model.forward_hidden(ids, torch.arange(len(seq), device=self.device), layout)[-1:]
                    logits = shaper.before_temperature(self.model.logits(h)[0].float(), prompt, out)
                    if sp.temperature and sp.temperature > 0:
                        scaled = shaper.after_temperature(logits / sp.temperature)
                        dist_logits = filter_logits(scaled, sp.top_k, sp.top_p)
                        probs = torch.softmax(dist_logits, -1).cpu()
                        tok = int(torch.multinomial(probs, 1, generator=self.gen))
                        lp = float(torch.log_softmax(scaled, -1)[tok])        # log-prob under the unfiltered policy
                    else:
                        tok = int(logits.argmax())
                        lp = float(torch.log_softmax(logits, -1)[tok])
                    out.append(tok)
                    lps.append(lp)
                    seq.append(tok)
                    if tok in stops:
                        reason = "stop"
                        break
                results.append({"token_ids": out, "logprobs": lps, "finish_reason": reason, "prompt_len": len(prompt),
                                "prompt_index": pi, "text": None})
        return results

    # ------------------------------------------------------------------ same management surface as the CUDA engine
    def load_weights(self, named_tensors) -> int:
        from ..models.hf_io import load_hf_tensor
        n = 0
        for name, t in named_tensors:
            load_hf_tensor(self.model, name, t)
            n += 1
        return n

    def weight_norm(self) -> Dict[str, float]:
        sq = sum(float(p.data.double().pow(2).sum()) for p in self.model.parameters())
        return {"norm": sq ** 0.5, "sq_sum": sq, "num_params": sum(p.numel() for p in self.model.parameters())}

    def reset_prefix_cache(self) -> None:
        return None

    def kv_bytes(self) -> int:
        return 0

    def sleep(self, level: int = 1) -> None:
        self._asleep = True

    def wake(self, tags: Optional[Sequence[str]] = None) -> None:
        self._asleep = False
