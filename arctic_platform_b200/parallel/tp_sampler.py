"""Tensor-parallel sampling replicas (``vllm_config.tensor_parallel_size`` > 1) on the tensor-op decode engine.

A replica of ``tp`` ranks holds ONE copy of the decoder split Megatron-style: the q/k/v projection (and the output
gate) by heads, the output projection by the matching columns, gate/up by rows of the intermediate dimension and
down by the matching columns -- per expert for mixture-of-experts layers, and for the shared expert.  Norms, router,
embedding and LM head are replicated.  Each block sums its two row-parallel outputs over the group
(``DecoderBlock.tp_reduce``), so every rank sees the same hidden states; the K/V cache of a rank holds only its
heads (``1 / tp`` of the bytes).  All ranks of a replica receive the same ``generate`` call; rank 0 of the group
draws the tokens and broadcasts them, so the ranks cannot diverge by a last-bit difference in the logits.

Weights arrive under their Hugging Face names as FULL tensors (from a checkpoint or from the trainer's weight
hand-over) and every rank keeps its slice (:func:`tp_slice`).  The reference gets the same behaviour from its
inference engine (``tensor_parallel_size`` in ``vllm_config``, arctic_platform/common/ray_server.py:375-420); the
fused GEMM + collective kernels for the paged CUDA engine live in :mod:`arctic_platform_b200.parallel.tensor_parallel`.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Iterable, Optional, Tuple

import torch
import torch.distributed as dist

from ..engine.hybrid_sampler import HybridSampler
from ..models.config import DecoderConfig
from ..models.decoder import DecoderLM


def tp_config(cfg: DecoderConfig, tp: int) -> DecoderConfig:
    """Shapes of one rank's shard."""
    if cfg.layer_types is not None and any(t != "full_attention" for t in cfg.layer_types):
        raise NotImplementedError("tensor-parallel sampling is built for full-attention decoders; "
                                  "the recurrent layers of the hybrid family are not sharded")
    if getattr(cfg, "moe_activation", "swiglu") != "swiglu":
        raise NotImplementedError("tensor-parallel sampling is built for SwiGLU feed-forward layers")
    for what, n in (("num_heads", cfg.num_heads), ("num_kv_heads", cfg.num_kv_heads),
                    ("intermediate_size", cfg.intermediate_size if not cfg.is_moe else 0),
                    ("moe_intermediate_size", cfg.moe_intermediate_size),
                    ("shared_expert_intermediate_size", cfg.shared_expert_intermediate_size)):
        if n % tp:
            raise ValueError(f"tensor_parallel_size={tp} does not divide {what}={n}")
    return dataclasses.replace(
        cfg, num_heads=cfg.num_heads // tp, num_kv_heads=cfg.num_kv_heads // tp,
        intermediate_size=cfg.intermediate_size // tp if not cfg.is_moe else cfg.intermediate_size,
        moe_intermediate_size=cfg.moe_intermediate_size // tp,
        shared_expert_intermediate_size=cfg.shared_expert_intermediate_size // tp)


_ROWS = ("gate_proj.weight", "up_proj.weight")          # split along dim 0
_COLS = ("down_proj.weight", "o_proj.weight")           # split along dim 1


def shard_axis(name: str) -> Optional[int]:
    """Axis along which the tensor with this Hugging Face name is split, or ``None`` when it is replicated."""
    if ".self_attn." in name and name.endswith(("q_proj.weight", "k_proj.weight", "v_proj.weight")):
        return 0
    if name.endswith("shared_expert_gate.weight") or name.endswith("mlp.gate.weight"):
        return None
    if ".mlp." in name and name.endswith(_ROWS):
        return 0
    if name.endswith(_COLS):
        return 1
    return None


def tp_slice(name: str, tensor: torch.Tensor, cfg: DecoderConfig, rank: int, tp: int) -> torch.Tensor:
    """This rank's part of a full Hugging Face tensor.  Head-structured projections are cut at head boundaries
    (with an output gate the q projection interleaves [query | gate] per head: whole heads stay together)."""
    axis = shard_axis(name)
    if axis is None or tp == 1:
        return tensor
    n = tensor.shape[axis]
    if n % tp:
        raise ValueError(f"{name}: extent {n} along axis {axis} does not divide by {tp}")
    step = n // tp
    return tensor.narrow(axis, rank * step, step)


class TensorParallelSampler(HybridSampler):
    """One rank of a ``tp``-way replica.  ``model`` (optional) is a FULL model whose weights are sliced in."""

    def __init__(self, cfg: DecoderConfig, device="cpu", model: Optional[DecoderLM] = None, tp_group=None,
                 dtype: Optional[torch.dtype] = None, **kw):
        if not dist.is_initialized():
            raise RuntimeError("tensor-parallel sampling needs an initialised process group")
        self.tp_group = tp_group
        self.tp = dist.get_world_size(tp_group)
        self.tp_rank = dist.get_rank(tp_group)
        self.full_cfg = cfg
        local = tp_config(cfg, self.tp)
        dev = torch.device(device)
        dtype = dtype or (next(model.parameters()).dtype if model is not None else
                          (torch.bfloat16 if dev.type == "cuda" else torch.float32))
        shard = DecoderLM(local, dev, dtype)
        for blk in shard.blocks:
            blk.tp_group = tp_group if tp_group is not None else dist.group.WORLD
        super().__init__(local, dev, model=shard, **kw)
        self._sharded = {n for n, _ in self._named_shard_flags()}
        if model is not None:
            from ..models.hf_io import iter_hf_tensors
            self.load_weights(iter_hf_tensors(model))
        else:
            shard.init_weights(seed=kw.get("seed", 0))

    def _named_shard_flags(self) -> Iterable[Tuple[str, bool]]:
        """Parameter names of the shard model that hold a slice (everything else is replicated)."""
        for name, _p in self.model.named_parameters():
            leaf = name.split(".")[-1]
            if leaf in ("wqkv", "wgate", "wo", "wgu", "wdown", "shared_wgu", "shared_wdown"):
                yield name, True

    # ------------------------------------------------------------------ weights
    @torch.no_grad()
    def load_weights(self, named_tensors) -> int:
        from ..models.hf_io import load_hf_tensor
        n = 0
        for name, t in named_tensors:
            load_hf_tensor(self.model, name, tp_slice(name, t, self.full_cfg, self.tp_rank, self.tp))
            n += 1
        return n

    def weight_norm(self) -> Dict[str, float]:
        """Norm and size of the WHOLE model: slices are summed over the group, replicated tensors count once."""
        sq_s = sq_r = 0.0
        n_s = n_r = 0
        for name, p in self.model.named_parameters():
            v = float(p.data.double().pow(2).sum())
            if name in self._sharded:
                sq_s, n_s = sq_s + v, n_s + p.numel()
            else:
                sq_r, n_r = sq_r + v, n_r + p.numel()
        t = torch.tensor([sq_s, float(n_s)], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, group=self.tp_group)
        sq = float(t[0]) + sq_r
        return {"norm": sq ** 0.5, "sq_sum": sq, "num_params": int(t[1]) + n_r}

    # ------------------------------------------------------------------ sampling: one decision per replica
    def _pick(self, logits, sp, shaper=None):
        tok, lp = super()._pick(logits, sp, shaper)
        src = dist.get_global_rank(self.tp_group, 0) if self.tp_group is not None else 0
        dist.broadcast(tok, src=src, group=self.tp_group)
        dist.broadcast(lp, src=src, group=self.tp_group)
        return tok, lp
