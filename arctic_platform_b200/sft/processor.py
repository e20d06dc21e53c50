"""SFT step pipeline: next-token cross entropy over packed sequences with global-token normalisation
(arctic_platform/sft/processor.py:95-397 in the reference).  The heavy lifting is shared with the RL
pipeline: ``run_sft_pipeline`` packs ``[B, S]`` sequences, the fused lm-head kernel produces per-token
log-probs and ``sft`` / ``sft_ce`` (``rl/processors/losses.py``) reduce them."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..rl.processors.losses import SFT_LOSS_FNS, sft_ce_loss, sft_loss  # noqa: F401
from ..rl.processors.pipeline import run_pipeline

LOGIT_LOSS_FNS = {"sft_ce"}
SFT_GLOBAL_TOKEN_LOSS_FNS = {"sft_ce"}


def batch_is_packed(batch: Dict[str, Any]) -> bool:
    """A batch with one row and position ids that restart is already packed."""
    pos = batch.get("position_ids")
    return bool(torch.is_tensor(pos) and pos.dim() == 2 and pos.shape[0] == 1 and (pos[0, 1:] == 0).any())


def count_loss_tokens(batch: Dict[str, Any]) -> int:
    """Tokens of this shard that the loss is taken over: selected by ``loss_mask`` / ``labels != -100``, inside the
    attention mask, and PREDICTED by an earlier token of the same sequence -- the first valid token of a row (of a
    document, for a row the client packed) has no predictor whichever side the padding is on."""
    ids = batch["input_ids"] if "input_ids" in batch else batch.get("labels")
    lm = batch.get("loss_mask")
    if lm is None and batch.get("labels") is not None:
        lm = batch["labels"] != -100
    valid = batch.get("attention_mask")
    valid = valid.bool() if valid is not None else torch.ones_like(ids, dtype=torch.bool)
    sel = valid if lm is None else (lm.bool() & valid)
    first = valid & (valid.int().cumsum(1) == 1)
    if ids.dim() == 2 and ids.shape[0] == 1:
        cu, pos = batch.get("cu_seqlens"), batch.get("position_ids")
        if cu is not None:
            T = ids.shape[1]
            starts = cu.reshape(-1)[:-1].long()
            first = torch.zeros_like(valid)
            first[0, starts[starts < T]] = True
            sel = sel.clone()
            sel[0, int(cu.reshape(-1)[-1]):] = False                 # trailing padding behind the last document
        elif torch.is_tensor(pos) and pos.numel() == ids.numel():
            first = first | (pos.reshape(1, -1) == 0)
    return int((sel & ~first).sum())


def count_valid_target_tokens(batch: Any) -> Optional[int]:
    """Next-token targets the loss is taken over, for one micro-batch dict or a list of them (a gradient-accumulation
    step).  ``None`` when nothing carries ``labels`` (the caller then skips the global-token normalisation); ``0``
    when every position is masked.  Same contract as arctic_platform/sft/processor.py:60-73, counted by
    ``count_loss_tokens`` so packed rows and left padding are handled too."""
    if isinstance(batch, (list, tuple)):
        counts = [count_valid_target_tokens(mb) for mb in batch]
        counts = [c for c in counts if c is not None]
        return sum(counts) if counts else None
    if not isinstance(batch, dict) or batch.get("labels") is None:
        return None
    return count_loss_tokens(batch)


def sft_ce_sum_from_hidden(model, hidden: torch.Tensor, labels: torch.Tensor, *, mode: str = "memory",
                           peak_mem_gib: float = 4.0):
    """Summed next-token cross entropy from the last hidden states ``[B, S, H]`` and ``labels [B, S]`` (``-100`` =
    ignored) without a ``[B, S, V]`` logits tensor -> ``(ce_sum, number of valid targets)``.  ``hidden[:, :-1]``
    predicts ``labels[:, 1:]``.  Both modes of the reference (``compute`` / ``memory``,
    arctic_platform/sft/processor.py:169-238) run the lm-head kernel that produces log-probs in its epilogue;
    ``peak_mem_gib`` sizes the row chunk of its backward recompute."""
    if mode not in ("compute", "memory"):
        raise ValueError(f"sft_ce_sum_from_hidden: mode must be 'compute' or 'memory', got {mode!r}")
    from ..common.utils.tiled_logits import chunked_logprobs_entropy_from_hidden
    targets = labels[:, 1:]
    valid = targets != -100
    logprobs, _ = chunked_logprobs_entropy_from_hidden(model, hidden[:, :-1, :].contiguous(), targets.clamp_min(0).contiguous(),
                                                       temperature=1.0, calculate_entropy=False, peak_mem_gib=peak_mem_gib)
    return -(logprobs * valid.to(logprobs.dtype)).sum(), int(valid.sum())


def inject_sft_global_token_meta(batch: Dict[str, Any], meta: Dict[str, Any], group=None) -> None:
    """``meta['batch_num_tokens']`` = loss tokens over ALL ranks (one all-reduce of an int64)."""
    n = torch.tensor([count_loss_tokens(batch)], dtype=torch.int64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        n = n.to("cuda" if dist.get_backend(group) == "nccl" else "cpu")
        dist.all_reduce(n, group=group)
        meta.setdefault("dp_size", dist.get_world_size(group))
    meta["batch_num_tokens"] = float(n.item())


def run_sft_pipeline(engine, batch: Dict[str, Any], meta: Optional[dict] = None, processing: Optional[dict] = None,
                     device=None, backward: bool = True) -> Dict[str, Any]:
    meta = dict(meta or {})
    processing = {"post": [], "loss_fn": "sft_ce", **(processing or {})}
    if processing["loss_fn"] in SFT_GLOBAL_TOKEN_LOSS_FNS and "batch_num_tokens" not in meta:
        inject_sft_global_token_meta(batch, meta)
    return run_pipeline(engine, batch, meta, processing, device, backward=backward)
