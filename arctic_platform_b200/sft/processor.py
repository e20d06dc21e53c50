"""SFT step pipeline: next-token cross entropy over packed sequences with global-token normalisation
(arctic_platform/sft/processor.py:95-397 in the reference).  The heavy lifting is shared with the RL
pipeline: ``run_sft_pipeline`` packs ``[B, S]`` sequences, the fused lm-head kernel produces per-token
log-probs and ``sft`` / ``sft_ce`` (``rl/processors/losses.py``) reduce them."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..rl.processors.losses import SFT_LOSS_FNS  # noqa: F401
from ..rl.processors.pipeline import run_pipeline

LOGIT_LOSS_FNS = {"sft_ce"}
SFT_GLOBAL_TOKEN_LOSS_FNS = {"sft_ce"}


def batch_is_packed(batch: Dict[str, Any]) -> bool:
    """A batch with one row and position ids that restart is already packed."""
    pos = batch.get("position_ids")
    return bool(torch.is_tensor(pos) and pos.dim() == 2 and pos.shape[0] == 1 and (pos[0, 1:] == 0).any())


def inject_sft_global_token_meta(batch: Dict[str, Any], meta: Dict[str, Any], group=None) -> None:
    """``meta['batch_num_tokens']`` = loss tokens over ALL ranks (one all-reduce of an int64)."""
    lm = batch.get("loss_mask")
    if lm is None and batch.get("labels") is not None:
        lm = batch["labels"] != -100
    n = torch.tensor([int(lm[:, 1:].sum()) if lm is not None else 0], dtype=torch.int64)
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
