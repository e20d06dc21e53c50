"""Stateful sampler for the hybrid (gated delta-net + gated attention) model family.

The paged CUDA sampler serves plain-attention decoders.  A hybrid decoder keeps two kinds of per-sequence state:
a constant-size recurrent state (convolution window + ``S [Hv, Dk, Dv]``) in every linear-attention layer, and a
growing K/V cache only in every n-th (full-attention) layer.  This engine

* prefills every DISTINCT prompt once, in one packed forward of the training model (so training and sampling run
  the same prefill arithmetic), capturing the recurrent states and K/V rows the layers leave behind,
* gives each of a prompt's ``n`` samples a copy of the small recurrent state and of the prompt's K/V rows
  (prompt work is shared, as the reference's prefix caching does for its samplers), and
* decodes all sequences together, one token per step: ``GatedDeltaNet.step`` for the linear layers, batched
  masked attention over the cache for the full-attention layers, O(1) / O(context) per token instead of a
  recomputation of the whole sequence.

It works for any decoder configuration (a plain-attention model is the special case without linear layers), on CPU
and on a GPU; the math is tensor operations on the model's own parameters.  Interface and result records are those
of the CUDA engine (arctic_platform/common/ray_server.py:375 creates the reference's samplers)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..models.decoder import _qknorm_partial_rope, gate_up_act
from ..ops import gemm, norm
from ..ops.attention import AttnLayout
from .reference_sampler import EXTRA_KEYS, LogitsProcessor, ReferenceSampler, filter_logits
from .sampler import SamplingParams


class _State:
    """Decode state of ``B`` sequences: per linear layer ``(conv [B, K-1, C], S [B, Hv, Dk, Dv])``, per attention
    layer ``(K, V) [B, Tmax, Hkv, D]``, and the number of valid cache rows ``lens [B]``."""

    def __init__(self) -> None:
        self.linear: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.lens: Optional[torch.Tensor] = None

    def num_bytes(self) -> int:
        n = 0
        for a, b in list(self.linear.values()) + list(self.kv.values()):
            n += a.numel() * a.element_size() + b.numel() * b.element_size()
        return n


class HybridSampler(ReferenceSampler):
    def __init__(self, cfg, device="cpu", model=None, max_seq_len: int = 8192, seed: int = 0,
                 eos_token_id: Optional[int] = None, max_batch: int = 256, **_ignored):
        super().__init__(cfg, device, model=model, max_seq_len=max_seq_len, seed=seed, eos_token_id=eos_token_id)
        self.max_batch = max_batch
        self.last_state_bytes = 0
        self.prefill_tokens = 0          # prompt tokens actually computed (distinct prompts only)
        self.decode_steps = 0

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def _prefill(self, prompts: List[List[int]]):
        """One packed forward over the distinct prompts.  Returns the last-token logits ``[P, V]`` and, per layer,
        what decoding needs: ``linear[li][p] = (conv, S)`` and ``kv[li] = (k, v)`` over the packed rows."""
        m, dev = self.model, self.device
        lens = [len(p) for p in prompts]
        cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        ids = torch.tensor([t for p in prompts for t in p], dtype=torch.int64, device=dev)
        pos = torch.cat([torch.arange(n, device=dev) for n in lens])
        layout = AttnLayout.from_cu_seqlens(cu)
        for blk in m.blocks:
            if blk.linear_attn is not None:
                blk.linear_attn.capture = {}
            else:
                blk.kv_capture = []
        try:
            h = m.forward_hidden(ids, pos, layout)
            linear = {li: blk.linear_attn.capture for li, blk in enumerate(m.blocks) if blk.linear_attn is not None}
            kv = {li: blk.kv_capture[0] for li, blk in enumerate(m.blocks) if blk.linear_attn is None}
        finally:
            for blk in m.blocks:
                if blk.linear_attn is not None:
                    blk.linear_attn.capture = None
                blk.kv_capture = None
        last = torch.as_tensor(cu[1:] - 1, device=dev)
        self.prefill_tokens += int(cu[-1])
        return m.logits(h[last]).float(), linear, kv, cu

    def _spread(self, linear, kv, cu, owner: List[int], t_max: int) -> _State:
        """Decode state for sequences whose prompts are ``owner[b]`` (index into the distinct prompts)."""
        st, dev = _State(), self.device
        own = torch.as_tensor(owner, device=dev)
        B = len(owner)
        for li, cap in linear.items():
            conv = torch.stack([cap[int(cu[p + 1])][0] for p in range(len(cu) - 1)])
            S = torch.stack([cap[int(cu[p + 1])][1] for p in range(len(cu) - 1)])
            st.linear[li] = (conv[own].contiguous(), S[own].float().contiguous())
        plen = torch.as_tensor(cu[1:] - cu[:-1], device=dev)
        for li, (k, v) in kv.items():
            K = k.new_zeros((B, t_max) + tuple(k.shape[1:]))
            V = v.new_zeros((B, t_max) + tuple(v.shape[1:]))
            for b, p in enumerate(owner):
                s, e = int(cu[p]), int(cu[p + 1])
                K[b, :e - s] = k[s:e]
                V[b, :e - s] = v[s:e]
            st.kv[li] = (K, V)
        st.lens = plen[own].clone()
        return st

    # ------------------------------------------------------------------ one decode step for all sequences
    @torch.no_grad()
    def _step(self, tokens: torch.Tensor, st: _State) -> torch.Tensor:
        """``tokens [B]`` (the tokens sampled last) -> logits ``[B, V]`` for the next ones; updates ``st``."""
        m, cfg = self.model, self.cfg
        B = tokens.shape[0]
        x = F.embedding(tokens, m.embed)
        rope = m.rope(x.device)
        pos = st.lens.clone()                              # the new token's position == rows already cached
        rows = torch.arange(B, device=x.device)
        stream = None
        w_off = 1.0 if cfg.norm_one_plus else 0.0
        for li, blk in enumerate(m.blocks):
            h, stream = norm.rmsnorm(x, blk.ln1, cfg.rms_norm_eps, stream, w_off)
            if blk.linear_attn is not None:
                conv, S = st.linear[li]
                o, conv, S = blk.linear_attn.step(h, conv, S)
                st.linear[li] = (conv, S)
            else:
                qkv = gemm.linear(h, blk.wqkv)
                q, k, v = _qknorm_partial_rope(qkv, blk.q_norm, blk.k_norm, rope, pos, cfg, w_off)
                K, V = st.kv[li]
                K[rows, pos] = k
                V[rows, pos] = v
                L = int(pos.max()) + 1
                rep = cfg.num_heads // cfg.num_kv_heads
                Kh = K[:, :L].transpose(1, 2)              # [B, Hkv, L, D]
                Vh = V[:, :L].transpose(1, 2)
                if rep > 1:
                    Kh, Vh = Kh.repeat_interleave(rep, 1), Vh.repeat_interleave(rep, 1)
                mask = (torch.arange(L, device=x.device)[None, :] <= pos[:, None])[:, None, None, :]
                a = F.scaled_dot_product_attention(q[:, :, None, :].float(), Kh.float(), Vh.float(), attn_mask=mask)
                a = a[:, :, 0, :].reshape(B, -1).to(h.dtype)
                if blk.wgate is not None:
                    a = (a.float() * torch.sigmoid(gemm.linear(h, blk.wgate).float())).to(a.dtype)
                o = gemm.linear(a, blk.wo)
            o = blk.tp_reduce(o)
            h2, stream = norm.rmsnorm(o, blk.ln2, cfg.rms_norm_eps, stream, w_off)
            x = blk.mlp(h2) if blk.mlp is not None else gemm.linear(gate_up_act(h2, blk.wgu), blk.wdown)
            x = blk.tp_reduce(x)
        hf, _ = norm.rmsnorm(x, m.final_norm, cfg.rms_norm_eps, stream, w_off)
        st.lens += 1
        self.decode_steps += 1
        return m.logits(hf).float()

    # ------------------------------------------------------------------ sampling
    def _pick(self, logits: torch.Tensor, sp: SamplingParams, shaper: Optional[LogitsProcessor] = None
              ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Token and its log-probability under the unfiltered (temperature-scaled) policy, per row."""
        if sp.temperature and sp.temperature > 0:
            scaled = logits / sp.temperature
            if shaper is not None:
                scaled = shaper.after_temperature(scaled)
            probs = torch.softmax(filter_logits(scaled, sp.top_k, sp.top_p), -1).cpu()
            tok = torch.multinomial(probs, 1, generator=self.gen)[:, 0].to(logits.device)
            lp = torch.log_softmax(scaled, -1).gather(1, tok[:, None])[:, 0]
        else:
            tok = logits.argmax(-1)
            lp = torch.log_softmax(logits, -1).gather(1, tok[:, None])[:, 0]
        return tok, lp

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sampling_params=None) -> List[dict]:
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else \
            SamplingParams.from_dict(sampling_params, supported=EXTRA_KEYS)
        self._raw_params = sampling_params if isinstance(sampling_params, dict) else None
        if self._asleep:
            raise RuntimeError("sampler is asleep; call wake() first")
        if sp.seed is not None:
            self.gen.manual_seed(int(sp.seed))
        prompts = [list(map(int, p)) for p in prompts]
        for p in prompts:
            if len(p) == 0:
                raise ValueError("empty prompt")
            if len(p) + sp.max_tokens > self.max_seq_len:
                raise ValueError(f"prompt ({len(p)}) + max_tokens ({sp.max_tokens}) exceeds max_seq_len {self.max_seq_len}")
        stops = set(int(t) for t in sp.stop_token_ids)
        if self.eos is not None and not sp.ignore_eos:
            stops.add(int(self.eos))
        results: List[Optional[dict]] = [None] * (len(prompts) * sp.n)
        # waves of at most ``max_batch`` sequences; samples of one prompt stay in one wave
        per_wave = max(1, self.max_batch // max(1, sp.n))
        for w0 in range(0, len(prompts), per_wave):
            self._generate_wave(prompts, range(w0, min(len(prompts), w0 + per_wave)), sp, stops, results)
        return results            # type: ignore[return-value]

    def _generate_wave(self, prompts, wave, sp: SamplingParams, stops, results) -> None:
        distinct: Dict[Tuple[int, ...], int] = {}
        owner: List[int] = []
        seq_prompt: List[int] = []
        for pi in wave:
            key = tuple(prompts[pi])
            d = distinct.setdefault(key, len(distinct))
            owner += [d] * sp.n
            seq_prompt += [pi] * sp.n
        uniq = [list(k) for k in distinct]
        # rollout routing replay: every MoE layer logs the experts it chose, pass by pass
        want_routing = bool(getattr(self, "always_return_routing", False)
                            or (getattr(self, "_raw_params", None) and self._raw_params.get("return_routed_experts")))
        moes = [blk.mlp for blk in self.model.blocks if blk.mlp is not None] if want_routing else []
        for mm in moes:
            mm.routing_log = []
        try:
            self._run_wave(prompts, sp, stops, results, uniq, owner, seq_prompt, moes)
        finally:
            for mm in moes:
                mm.routing_log = None

    def _run_wave(self, prompts, sp, stops, results, uniq, owner, seq_prompt, moes) -> None:
        logits_p, linear, kv, cu = self._prefill(uniq)
        pre_routing = torch.stack([mm.routing_log.pop() for mm in moes], 1) if moes else None       # [T, L, k]
        step_routing: List[torch.Tensor] = []
        B = len(owner)
        t_max = max(len(u) for u in uniq) + sp.max_tokens
        st = self._spread(linear, kv, cu, owner, t_max)
        self.last_state_bytes = st.num_bytes()
        del linear, kv
        logits = logits_p[torch.as_tensor(owner, device=self.device)]
        out: List[List[int]] = [[] for _ in range(B)]
        lps: List[List[float]] = [[] for _ in range(B)]
        reason = ["length"] * B
        alive = [sp.max_tokens > 0] * B
        shaper = LogitsProcessor(getattr(self, "_raw_params", None), sorted(stops))
        for _t in range(sp.max_tokens):
            if shaper.active:
                logits = torch.stack([shaper.before_temperature(logits[b], prompts[seq_prompt[b]], out[b]) for b in range(B)])
            tok, lp = self._pick(logits, sp, shaper)
            tok_l, lp_l = tok.tolist(), lp.tolist()
            for b in range(B):
                if not alive[b]:
                    continue
                out[b].append(tok_l[b])
                lps[b].append(lp_l[b])
                if tok_l[b] in stops:
                    reason[b], alive[b] = "stop", False
            if not any(alive) or _t == sp.max_tokens - 1:
                break
            logits = self._step(tok, st)                 # finished rows keep stepping; their outputs are ignored
            if moes:
                step_routing.append(torch.stack([mm.routing_log.pop() for mm in moes], 1))           # [B, L, k]
        for b in range(B):
            pi = seq_prompt[b]
            res = {"token_ids": out[b], "logprobs": lps[b], "finish_reason": reason[b],
                   "prompt_len": len(prompts[pi]), "prompt_index": pi, "text": None}
            if moes:
                # one row per token that was FED to the model: the prompt and all drawn tokens but the last
                p = owner[b]
                rows = [pre_routing[int(cu[p]):int(cu[p + 1])]] + [s[b:b + 1] for s in step_routing[:max(0, len(out[b]) - 1)]]
                res["routed_experts"] = torch.cat(rows).to(torch.int32).cpu()
            results[pi * sp.n + (b % sp.n)] = res

    def kv_bytes(self) -> int:
        return self.last_state_bytes
