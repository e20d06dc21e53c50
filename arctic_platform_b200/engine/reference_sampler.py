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
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        if self._asleep:
            raise RuntimeError("sampler is asleep; call wake() first")
        if sp.seed is not None:
            self.gen.manual_seed(int(sp.seed))
        stops = set(int(t) for t in sp.stop_token_ids)
        if self.eos is not None and not sp.ignore_eos:
            stops.add(int(self.eos))
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
                    logits = self.model.logits(h)[0].float()
                    if sp.temperature and sp.temperature > 0:
                        scaled = logits / sp.temperature
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
