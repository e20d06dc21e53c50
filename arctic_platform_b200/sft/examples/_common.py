"""Synthetic SFT data: sequences with a learnable rule (each token is the previous one plus a per-sequence stride), so
a few dozen steps visibly lower the loss; prompts are masked out of the labels."""
from __future__ import annotations

from typing import Dict, Iterator

import torch


def make_batch(batch_size: int, seq_len: int, vocab: int, g: torch.Generator, prompt_len: int = 4) -> Dict[str, torch.Tensor]:
    start = torch.randint(3, vocab // 2, (batch_size, 1), generator=g)
    stride = torch.randint(1, 4, (batch_size, 1), generator=g)
    ids = (start + stride * torch.arange(seq_len).unsqueeze(0)) % (vocab - 3) + 3
    lens = torch.randint(seq_len // 2, seq_len + 1, (batch_size,), generator=g)
    mask = (torch.arange(seq_len).unsqueeze(0) < lens.unsqueeze(1)).long()
    labels = torch.where(mask.bool(), ids, torch.full_like(ids, -100))
    labels[:, :prompt_len] = -100                        # the loss is on the continuation only
    return {"input_ids": ids * mask, "attention_mask": mask, "labels": labels}


def batches(batch_size: int, seq_len: int, vocab: int, seed: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    g = torch.Generator().manual_seed(seed)
    while True:
        yield make_batch(batch_size, seq_len, vocab, g)
