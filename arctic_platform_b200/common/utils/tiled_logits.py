"""Per-token log-probs and entropy from hidden states without holding ``[tokens, vocab]`` logits -- the call shapes of
the reference's three "logits optimisation" modes on top of this build's single implementation.

The reference offers ``none`` (materialise the logits, then softmax), ``compute`` (materialise once, chunk the
follow-up) and ``memory`` (tile inside an autograd function and recompute in backward), sized from one memory budget
(arctic_platform/common/utils/tiled_logits.py:61-378).  Here the lm-head GEMM produces log-probs and entropy in its
epilogue (``ops/logprob.py``: online softmax over vocabulary tiles on the GPU, a row-chunked fp32 expression on CPU),
so all three entry points run that one path; their extra knobs are accepted and documented as what they mean here:

* ``peak_mem_gib`` sizes the row chunk of the backward recompute (``logits_chunk_rows``);
* ``logits_compute_in_fp32`` is always true in effect (accumulation and softmax are fp32);
* ``logits_compute_from_fp32_inputs`` upcasts the hidden states first (CPU path; the GPU kernel takes bf16 operands).

``model`` is anything with ``output_weight`` or ``lm_head.weight`` (``[vocab, hidden]``).
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch

from ...ops.logprob import lm_head_logprobs, logprobs_entropy_ref


def logits_chunk_rows(vocab_size: int, peak_mem_gib: float, bytes_per_elem: int = 4) -> int:
    """Rows whose ``[rows, vocab]`` block fits in ``peak_mem_gib`` GiB (at least 1)."""
    budget = max(1, int(peak_mem_gib * 2 ** 30))
    return max(1, budget // max(1, int(vocab_size) * int(bytes_per_elem)))


def _weight(model: Any) -> torch.Tensor:
    w = getattr(model, "output_weight", None)
    if w is None:
        head = getattr(model, "lm_head", None)
        w = getattr(head, "weight", None)
    if w is None:
        raise AttributeError("model has neither output_weight nor lm_head.weight")
    return w


def _inv_temperature(temperature, n_rows: int, device):
    if torch.is_tensor(temperature):
        t = temperature.to(device=device, dtype=torch.float32).clamp(min=1e-8)
        return (1.0 / t).reshape(-1).expand(n_rows).contiguous() if t.numel() in (1, n_rows) else 1.0 / t
    return 1.0 / max(float(temperature), 1e-8)


def lm_head_logits(model: Any, hidden_states: torch.Tensor, temperature=1.0, logits_compute_from_fp32_inputs: bool = False,
                   logits_compute_in_fp32: bool = False) -> torch.Tensor:
    """The full logits tensor (for callers that really want it: debugging, top-k inspection).  Training paths do not
    call this."""
    w = _weight(model)
    h = hidden_states.float() if logits_compute_from_fp32_inputs else hidden_states
    logits = h @ w.to(h.dtype).t()
    if logits_compute_in_fp32:
        logits = logits.float()
    inv = _inv_temperature(temperature, logits.reshape(-1, logits.shape[-1]).shape[0], logits.device)
    if torch.is_tensor(inv):
        return logits * inv.reshape(*logits.shape[:-1], 1).to(logits.dtype)
    return logits * inv if inv != 1.0 else logits


def logprobs_entropy_from_flat_logits(flat_logits: torch.Tensor, flat_labels: torch.Tensor,
                                      calculate_entropy: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``[N, V]`` logits -> log-prob of ``labels [N]`` and (optionally) the entropy of each row, fp32."""
    ls = torch.log_softmax(flat_logits.float(), dim=-1)
    lp = ls.gather(-1, flat_labels.reshape(-1, 1).long()).squeeze(-1)
    ent = -(ls.exp() * ls).sum(-1) if calculate_entropy else None
    return lp, ent


def logprobs_from_logits(logits: torch.Tensor, labels: torch.Tensor, inplace_backward: bool = True) -> torch.Tensor:
    """Log-prob of ``labels`` under ``logits [..., V]`` for callers that already hold logits (an external model);
    ``logit[label] - logsumexp`` in fp32, so no ``[..., V]`` softmax copy is made.  ``inplace_backward`` is accepted
    for call compatibility (arctic_platform/rl/processors/pipeline.py:620-647 uses it for a library CE kernel)."""
    lead = logits.shape[:-1]
    flat = logits.reshape(-1, logits.shape[-1]).float()
    picked = flat.gather(-1, labels.reshape(-1, 1).long()).squeeze(-1)
    return (picked - torch.logsumexp(flat, dim=-1)).view(*lead)


def fast_logprobs_and_entropy_from_logits(logits: torch.Tensor, labels: torch.Tensor, calculate_entropy: bool = True):
    """``logits [..., V]`` -> ``(logprobs [...], entropy [...] or None)`` in one pass."""
    lead = logits.shape[:-1]
    lp, ent = logprobs_entropy_from_flat_logits(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), calculate_entropy)
    return lp.view(*lead), (ent.view(*lead) if ent is not None else None)


def chunked_logprobs_and_entropy_from_logits(logits: torch.Tensor, labels: torch.Tensor, calculate_entropy: bool = True,
                                             peak_mem_gib: float = 4.0):
    """Same result, walking the rows in blocks whose fp32 softmax fits in ``peak_mem_gib`` GiB."""
    flat, y = logits.reshape(-1, logits.shape[-1]), labels.reshape(-1)
    rows = logits_chunk_rows(flat.shape[-1], peak_mem_gib)
    parts = [logprobs_entropy_from_flat_logits(flat[i:i + rows], y[i:i + rows], calculate_entropy)
             for i in range(0, flat.shape[0], rows)]
    if not parts:
        empty = flat.new_zeros(labels.shape, dtype=torch.float32)
        return empty, (empty.clone() if calculate_entropy else None)
    lp = torch.cat([p[0] for p in parts]).view_as(labels)
    ent = torch.cat([p[1] for p in parts]).view_as(labels) if calculate_entropy else None
    return lp, ent


def _from_hidden(model, hidden_states, labels, temperature, calculate_entropy, chunk_rows, fp32_inputs):
    w = _weight(model)
    lead = hidden_states.shape[:-1]
    h = hidden_states.reshape(-1, hidden_states.shape[-1])
    y = labels.reshape(-1)
    inv = _inv_temperature(temperature, h.shape[0], h.device)
    if h.is_cuda:
        lp, ent = lm_head_logprobs(h, w, y, inv, calculate_entropy, bwd_chunk=max(1, int(chunk_rows)))
    else:
        hh, ww = (h.float(), w.float()) if fp32_inputs else (h, w)
        lp, ent = logprobs_entropy_ref(hh, ww, y, inv, calculate_entropy, chunk=max(1, int(chunk_rows)))
    return lp.view(*lead), (ent.view(*lead) if ent is not None else None)


def tiled_logprobs_entropy_from_hidden(model, hidden_states, labels, temperature=1.0, calculate_entropy: bool = True,
                                       logits_compute_from_fp32_inputs: bool = False, logits_compute_in_fp32: bool = False):
    """Mode ``none`` of the reference; same result, no logits tensor."""
    return _from_hidden(model, hidden_states, labels, temperature, calculate_entropy, 4096, logits_compute_from_fp32_inputs)


def chunked_logprobs_entropy_from_hidden(model, hidden_states, labels, temperature=1.0, calculate_entropy: bool = True,
                                         peak_mem_gib: float = 4.0, logits_compute_from_fp32_inputs: bool = False,
                                         logits_compute_in_fp32: bool = False):
    """Mode ``compute`` of the reference: the budget sizes the row chunk of the recompute."""
    rows = logits_chunk_rows(_weight(model).shape[0], peak_mem_gib)
    return _from_hidden(model, hidden_states, labels, temperature, calculate_entropy, rows, logits_compute_from_fp32_inputs)


class TiledLogProbEntropy:
    """Mode ``memory`` of the reference, kept as a callable with the autograd function's ``apply`` signature:
    ``TiledLogProbEntropy.apply(hidden, weight, labels, temperature, calculate_entropy, peak_mem_gib)``."""

    @staticmethod
    def apply(hidden_states, weight, labels, temperature=1.0, calculate_entropy: bool = True, peak_mem_gib: float = 4.0,
              *_unused):
        from types import SimpleNamespace
        rows = logits_chunk_rows(weight.shape[0], peak_mem_gib)
        return _from_hidden(SimpleNamespace(output_weight=weight), hidden_states, labels, temperature, calculate_entropy,
                            rows, False)
