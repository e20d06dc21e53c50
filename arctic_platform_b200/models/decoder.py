"""Qwen3-style decoder on the packed token axis.

The model never sees a padded ``[B, S]`` batch: it takes ``input_ids [T]``,
``positions [T]`` and an :class:`~arctic_platform_b200.ops.attention.AttnLayout`
that says which rows attend to which key ranges.  Plain packed batches and
ZoRRo prompt-deduplicated batches differ only in that layout, so there is no
model patching step (the reference monkey-patches every attention module and the
backbone forward: arctic_platform/rl/zorro_train/qwen_model_patcher.py:255-717).

Weights are kept in the fused layouts the kernels want -- ``wqkv`` (q|k|v rows),
``wgu`` (gate/up rows interleaved so SwiGLU runs in the GEMM epilogue) -- and are
converted from / to Hugging Face names in :mod:`arctic_platform_b200.models.hf_io`.
On CPU tensors every op falls through to its fp32 PyTorch expression, which makes
this same module the numerical oracle.
"""
from __future__ import annotations

import math
from typing import Dict, Iterator, List, Optional, Tuple

import torch
from torch import nn

from ..ops import gemm, norm
from ..ops.attention import AttnLayout, segment_attention
from .config import DecoderConfig


class _GateUpSwiGLUFn(torch.autograd.Function):
    """act = silu(x Wg^T) * (x Wu^T) with Wg/Wu rows interleaved in ``wgu``; the activation is
    produced by the GEMM epilogue, the pre-activations are kept for the backward."""

    @staticmethod
    def forward(ctx, x, wgu):
        gu, act = gemm.gate_up_swiglu(x, wgu, keep_gu=True)
        ctx.save_for_backward(x, wgu, gu)
        return act

    @staticmethod
    def backward(ctx, dact):
        x, wgu, gu = ctx.saved_tensors
        from ..ops import _lib
        dact = dact.contiguous()
        dgu = torch.empty_like(gu)
        T, I2 = gu.shape
        _lib.check(_lib.cuda_lib().apb_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dact), _lib.ptr(dgu), T, I2 // 2,
                                                  _lib.stream_ptr()), "swiglu_bwd")
        dx = gemm.matmul_nn(dgu, wgu) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            acc = getattr(wgu, "grad_f32", None)
            if acc is not None:
                gemm.matmul_tn(dgu, x, out=acc, accumulate=True)
            else:
                dw = gemm.matmul_tn(dgu, x)
        return dx, dw


def gate_up_act(x: torch.Tensor, wgu: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        gu = x @ wgu.t()
        return torch.nn.functional.silu(gu[..., 0::2]) * gu[..., 1::2]
    return _GateUpSwiGLUFn.apply(x, wgu)


def _qknorm_partial_rope(qkv, wq, wk, rope, positions, cfg: DecoderConfig, w_offset: float):
    """q/k RMSNorm (optionally with the (1+w) parameterisation) and rotate-half RoPE on the first ``rotary_dim``
    dimensions of every head -- PyTorch ops; the fused kernel covers the full-rotation, plain-weight case."""
    T = qkv.shape[0]
    Hq, Hkv, D, rd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.rotary_dim
    q = qkv[:, :Hq * D].reshape(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    cos_t, sin_t = rope
    pos = positions.long()
    c, s = cos_t[pos][:, None, :rd // 2], sin_t[pos][:, None, :rd // 2]

    def one(x, w):
        xf = x.float()
        if w is not None:
            xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * (w.float() + w_offset)
        a, b, rest = xf[..., :rd // 2], xf[..., rd // 2:rd], xf[..., rd:]
        return torch.cat([a * c - b * s, b * c + a * s, rest], -1).to(x.dtype)

    return one(q, wq), one(k, wk), v


SELECTIVE_AC_TARGETS = ("norm", "attn_proj", "mlp", "routed_experts", "linear_attn")


class DecoderBlock(nn.Module):
    def __init__(self, cfg: DecoderConfig, layer_idx: int, device, dtype):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        H, D = cfg.hidden_size, cfg.head_dim
        mk = lambda *s: nn.Parameter(torch.empty(*s, device=device, dtype=dtype))
        self.ln1 = mk(H)
        self.kind = cfg.layer_type(layer_idx)
        self.w_offset = 1.0 if cfg.norm_one_plus else 0.0
        if self.kind == "linear_attention":
            from .linear_attention import GatedDeltaNet
            self.linear_attn = GatedDeltaNet(cfg, device, dtype)
            self.wqkv = self.q_norm = self.k_norm = self.wo = self.wgate = None
        else:
            self.linear_attn = None
            self.wqkv = mk(cfg.qkv_size, H)
            self.wgate = mk(cfg.q_size, H) if cfg.attn_output_gate else None
            self.q_norm = mk(D) if cfg.qk_norm else None
            self.k_norm = mk(D) if cfg.qk_norm else None
            self.wo = mk(H, cfg.q_size)
        self.kv_capture = None           # a sampler's prefill sets a list; forward appends this layer's (k, v)
        self.tp_group = None             # inference tensor parallelism: this block holds a head / column shard and
        #                                  sums the two row-parallel outputs over the group (parallel/tp_sampler.py)
        self.tiled_mlp_shards = 0        # > 1 or "auto": the dense MLP runs over row tiles (activation memory)
        self.ac_targets: Tuple[str, ...] = ()   # parts of this block under selective activation checkpointing
        self.ln2 = mk(H)
        if cfg.is_moe:
            if cfg.moe_activation == "relu2":
                from .latent_moe import LatentMoEFeedForward as MoEFeedForward
            else:
                from .moe import MoEFeedForward
            self.mlp = MoEFeedForward(cfg, device, dtype)
            self.wgu = self.wdown = None
        else:
            self.mlp = None
            self.wgu = mk(2 * cfg.intermediate_size, H)
            self.wdown = mk(H, cfg.intermediate_size)

    def forward(self, x, stream, positions, layout: AttnLayout, rope):
        """``x`` is the previous sublayer output, ``stream`` the residual stream before adding it
        (None for the first block).  Returns the MLP output and the updated stream."""
        h, stream = self._part("norm", self._norm, x, stream, self.ln1)
        if self.linear_attn is not None:
            o = self._part("linear_attn", self.linear_attn, h, layout)
        else:
            q, k, v = self._part("attn_proj", self._attn_in, h, positions, rope)
            if self.kv_capture is not None:
                self.kv_capture.append((k, v))
            if getattr(self, "sp_group", None) is not None:
                from ..parallel.ulysses import ulysses_attention
                a = ulysses_attention(q, k, v, layout, self.sp_group)
            else:
                a = segment_attention(q, k, v, layout)
            o = self._part("attn_proj", self._attn_out, a.reshape(a.shape[0], -1), h)
        o = self.tp_reduce(o)
        h2, stream = self._part("norm", self._norm, o, stream, self.ln2)
        if self.mlp is not None:
            d = self._part("routed_experts" if "routed_experts" in self.ac_targets else "mlp", self.mlp, h2)
        elif self.tiled_mlp_shards:
            from .tiled_mlp import tiled_mlp
            d = tiled_mlp(h2, self._dense_mlp, self.tiled_mlp_shards, (self.wgu, self.wdown))
        else:
            d = self._part("mlp", self._dense_mlp, h2)
        return self.tp_reduce(d), stream

    def tp_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of the row-parallel partial outputs over the tensor-parallel group (identity without one)."""
        if self.tp_group is None:
            return t
        if torch.is_grad_enabled() and t.requires_grad:
            raise RuntimeError("tensor-parallel blocks are inference-only")
        import torch.distributed as dist
        dist.all_reduce(t, group=self.tp_group)
        return t

    def _dense_mlp(self, h: torch.Tensor) -> torch.Tensor:
        return gemm.linear(gate_up_act(h, self.wgu), self.wdown)

    def _norm(self, x, stream, weight):
        return norm.rmsnorm(x, weight, self.cfg.rms_norm_eps, stream, self.w_offset)

    def _attn_in(self, h, positions, rope):
        """q/k/v projection, per-head norm and rotation."""
        cfg = self.cfg
        qkv = gemm.linear(h, self.wqkv)
        if cfg.rotary_dim != cfg.head_dim or self.w_offset:
            return _qknorm_partial_rope(qkv, self.q_norm, self.k_norm, rope, positions, cfg, self.w_offset)
        return norm.qknorm_rope(qkv, self.q_norm, self.k_norm, rope[0], rope[1], positions, cfg.num_heads,
                                cfg.num_kv_heads, cfg.head_dim, cfg.rms_norm_eps)

    def _attn_out(self, a, h):
        """Output gate (where the family has one) and output projection."""
        if self.wgate is not None:
            a = (a.float() * torch.sigmoid(gemm.linear(h, self.wgate).float())).to(a.dtype)
        return gemm.linear(a, self.wo)

    def supported_ac_targets(self) -> frozenset:
        """Selective-checkpointing targets that name a part of THIS block (same rule as the reference's
        ``get_supported_targets``, arctic_platform/model/implementations/qwen35/models/layers/checkpointing.py:97-115)."""
        out = {"norm"}
        if self.linear_attn is not None:
            out.add("linear_attn")
        else:
            out.add("attn_proj")
        out.add("routed_experts" if self.mlp is not None else "mlp")
        if self.mlp is not None:
            out.add("mlp")                                   # the whole MoE layer, router and shared expert included
        return frozenset(out)

    def _part(self, target: str, fn, *args):
        """Runs one part of the block, under activation checkpointing when selective checkpointing names it."""
        if target not in self.ac_targets or not torch.is_grad_enabled():
            return fn(*args)
        from torch.utils.checkpoint import checkpoint
        if self.mlp is not None and fn is self.mlp:
            from .moe import router_replay_scope
            ctx = lambda: (router_replay_scope(self, "capture"), router_replay_scope(self, "replay"))
            return checkpoint(fn, *args, use_reentrant=False, context_fn=ctx)
        return checkpoint(fn, *args, use_reentrant=False)


class DecoderLM(nn.Module):
    def __init__(self, cfg: DecoderConfig, device="cpu", dtype=torch.float32, max_positions: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        H = cfg.hidden_size
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, H, device=device, dtype=dtype))
        self.blocks = nn.ModuleList([DecoderBlock(cfg, i, device, dtype) for i in range(cfg.num_layers)])
        self.final_norm = nn.Parameter(torch.empty(H, device=device, dtype=dtype))
        self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(
            torch.empty(cfg.vocab_size, H, device=device, dtype=dtype))
        self._rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        self._rope_len = max_positions or min(cfg.max_position_embeddings, 40960)
        self.gradient_checkpointing = False
        # selective checkpointing: only these parts of every block are recomputed (SELECTIVE_AC_TARGETS); empty =
        # whole blocks.  ``checkpoint_freq`` = n: every n-th block (0, n, 2n, ...) is checkpointed, the rest keep
        # their activations
        self.checkpoint_targets: Tuple[str, ...] = ()
        self.checkpoint_freq = 1

    def set_activation_checkpointing(self, mode: str = "full", targets=None, freq: int = 1) -> None:
        """``mode`` ``full`` (whole blocks) or ``selective`` (``targets``, default ``["norm"]`` as in the reference's
        ``ActivationCheckpointConfig``, arctic_platform/model/implementations/qwen35/config.py:33-40).  Unknown
        target names, and names that no layer of this model has, are errors."""
        if mode not in ("full", "selective"):
            raise ValueError(f"activation checkpointing mode {mode!r}: expected 'full' or 'selective'")
        if int(freq) < 1:
            raise ValueError(f"activation checkpointing freq must be >= 1, got {freq}")
        chosen: Tuple[str, ...] = ()
        if mode == "selective":
            chosen = tuple(sorted(set(targets if targets is not None else ("norm",))))
            unknown = set(chosen) - set(SELECTIVE_AC_TARGETS)
            if unknown:
                raise ValueError(f"Unsupported selective activation checkpoint targets: {sorted(unknown)}")
            have = set().union(*(blk.supported_ac_targets() for blk in self.blocks))
            missing = set(chosen) - have
            if missing:
                raise ValueError(f"Selective activation checkpoint targets {sorted(missing)} are not supported by the "
                                 f"selected model layers. Supported targets across the model: {sorted(have)}")
        self.gradient_checkpointing = True
        self.checkpoint_targets = chosen
        self.checkpoint_freq = int(freq)

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02, on_device: Optional[bool] = None) -> "DecoderLM":
        """Deterministic normal(0, std) init keyed by parameter name, so the values do not depend on
        how the model is later sharded (norm weights are ones).  ``on_device``: draw the numbers with the device's
        own generator instead of the host's (same values on every GPU for one name and seed, different from the
        host's stream).  Default: the device for CUDA models of more than 2^28 parameters -- drawing billions of
        numbers on the host takes tens of seconds per model copy, and a colocated job builds three of them."""
        if on_device is None:
            first = next(self.parameters())
            on_device = first.is_cuda and sum(p.numel() for p in self.parameters()) > (1 << 28)
        for name, p in self.named_parameters():
            if name.endswith("A_log") or name.endswith("dt_bias"):
                p.copy_(torch.linspace(-1.0, 1.0, p.numel()).to(p.dtype))      # decays spread over the heads
                continue
            if p.dim() == 1 and not name.endswith("router_bias"):
                is_plain = name.endswith("norm_w") or not self.cfg.norm_one_plus
                p.fill_(1.0 if is_plain else 0.0)                              # (1+w) norms store w - 1
                continue
            src = p.device if (on_device and p.is_cuda) else torch.device("cpu")
            g = torch.Generator(device=src)
            g.manual_seed((hash_name(name) + seed) % (2 ** 31))
            chunk = 1 << 24
            flat = p.data.view(-1)
            for s in range(0, flat.numel(), chunk):
                n = min(chunk, flat.numel() - s)
                flat[s:s + n].copy_((torch.randn(n, generator=g, dtype=torch.float32, device=src) * std).to(p.dtype))
        return self

    def rope(self, device) -> Tuple[torch.Tensor, torch.Tensor]:
        dev = torch.device(device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        if self._rope is None or self._rope[0].device != dev:
            self._rope = norm.rope_tables(self._rope_len, self.cfg.rotary_dim, self.cfg.rope_theta, dev)
        return self._rope

    @property
    def output_weight(self) -> torch.Tensor:
        return self.embed if self.lm_head is None else self.lm_head

    # --------------------------------------------------------------- forward
    def forward_hidden(self, input_ids: torch.Tensor, positions: torch.Tensor, layout: AttnLayout,
                       routed_experts: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Final-norm hidden states ``[T, H]`` for packed ``input_ids [T]``.  ``routed_experts [T, L_moe, k]`` replays
        the expert choice recorded for every token and MoE layer elsewhere (the sampler that drew the rollout);
        entries of -1 leave the choice to the router (arctic_platform/model/implementations/qwen35/models/qwen3_5_moe/
        modeling_qwen3_5_moe.py:758-798 slices the same tensor per layer)."""
        if routed_experts is not None:
            moes = [blk.mlp for blk in self.blocks if blk.mlp is not None]
            if routed_experts.shape[0] != input_ids.shape[0] or routed_experts.shape[1] != len(moes):
                raise ValueError(f"routed_experts {tuple(routed_experts.shape)}: expected [{input_ids.shape[0]}, "
                                 f"{len(moes)}, k]")
            for i, m in enumerate(moes):
                m.routed_experts = routed_experts[:, i].to(input_ids.device)
            try:
                return self.forward_hidden(input_ids, positions, layout)
            finally:
                for m in moes:
                    m.routed_experts = None
        x = torch.nn.functional.embedding(input_ids, self.embed)
        rope = self.rope(x.device)
        positions = positions.to(torch.int32) if x.is_cuda else positions
        stream = None
        targets = tuple(self.checkpoint_targets) if self.gradient_checkpointing else ()
        freq = max(1, int(getattr(self, "checkpoint_freq", 1)))
        for li, blk in enumerate(self.blocks):
            on = self.gradient_checkpointing and li % freq == 0
            blk.ac_targets = targets if on else ()
            if on and torch.is_grad_enabled() and not self.checkpoint_targets:
                from torch.utils.checkpoint import checkpoint
                if blk.mlp is not None:
                    # the recompute replays the routing of the original pass (same expert counts, same shapes)
                    from .moe import router_replay_scope
                    ctx = lambda b=blk: (router_replay_scope(b, "capture"), router_replay_scope(b, "replay"))
                    x, stream = checkpoint(blk, x, stream, positions, layout, rope, use_reentrant=False, context_fn=ctx)
                else:
                    x, stream = checkpoint(blk, x, stream, positions, layout, rope, use_reentrant=False)
            else:
                x, stream = blk(x, stream, positions, layout, rope)
        h, _ = norm.rmsnorm(x, self.final_norm, self.cfg.rms_norm_eps, stream, 1.0 if self.cfg.norm_one_plus else 0.0)
        return h

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Full logits ``[N, V]`` in fp32 -- small inputs / tests only; training and scoring use
        :func:`arctic_platform_b200.ops.logprob.lm_head_logprobs` which never forms this tensor."""
        if hidden.is_cuda:
            return gemm.matmul_nt(hidden.contiguous(), self.output_weight, out_dtype=torch.float32)
        return hidden.float() @ self.output_weight.float().t()


def hash_name(name: str) -> int:
    h = 2166136261
    for ch in name.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


def token_logprobs(model: DecoderLM, packed, inv_temperature=1.0, with_entropy: bool = True, action_masks=None,
                   routed_experts=None):
    """Log-probabilities (and entropies) of ``packed.labels`` under ``model``; ``packed`` is a
    :class:`~arctic_platform_b200.rl.zorro_train.layout.PackedBatch` already on the model's device.
    Returns fp32 tensors of shape ``[N]`` in original sample order.  ``action_masks`` (one row per prediction)
    restricts the distribution of the constrained rows to their legal tokens."""
    from ..ops.logprob import lm_head_logprobs

    if routed_experts is not None:          # [B, S, L_moe, k] aligned with the input grid -> packed token order
        routed_experts = packed.gather_inputs(routed_experts)
    hidden = model.forward_hidden(packed.input_ids, packed.positions, packed.layout, routed_experts)
    pred = hidden.index_select(0, packed.pred_index)
    if action_masks is not None:
        from ..utils.action_masks import masked_logprobs
        return masked_logprobs(pred, model.output_weight, packed.labels, action_masks, inv_temperature, with_entropy)
    return lm_head_logprobs(pred, model.output_weight, packed.labels, inv_temperature, with_entropy)


# ----------------------------------------------------------------------------- selective checkpointing, per block
def get_supported_targets(layer: "DecoderBlock") -> frozenset:
    """Parts of ``layer`` that selective activation checkpointing can name."""
    return layer.supported_ac_targets()


def supports_selective_activation_checkpointing(layer) -> bool:
    return isinstance(layer, DecoderBlock)


def set_selective_activation_checkpointing(layer: "DecoderBlock", targets) -> None:
    """Puts the named parts of ONE block under activation checkpointing (``DecoderLM.enable_activation_checkpointing``
    does this for every block).  Unknown names raise; names of parts the block does not have are ignored, as in
    arctic_platform/model/implementations/qwen35/models/layers/checkpointing.py:118-146."""
    chosen = tuple(dict.fromkeys(targets))
    unknown = set(chosen) - set(SELECTIVE_AC_TARGETS)
    if unknown:
        raise ValueError(f"Unsupported selective activation checkpoint targets: {sorted(unknown)}")
    layer.ac_targets = tuple(t for t in chosen if t in layer.supported_ac_targets())
