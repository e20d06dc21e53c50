"""Metric reduction across micro-batches and data-parallel ranks.

Workers report token-weighted quantities as pairs ``{name}.sum`` / ``{name}.tokens``.  Within a rank the
pairs of all micro-batches are summed (other numbers are averaged); across ranks the pairs collapse to
``sum / tokens`` -- a global token mean -- while plain numbers are averaged over the ranks that sent them
and everything else passes through from the first rank that has it.  Behaviour follows
arctic_platform/common/utils/batch.py:251-415 in the reference.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Tuple

SUM, TOK = ".sum", ".tokens"


def _is_number(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _accumulate(dicts: Iterable[dict]):
    totals: Dict[str, float] = {}
    counts: Dict[str, int] = {}
    other: Dict[str, Any] = {}
    for d in dicts:
        for k, v in (d or {}).items():
            if _is_number(v):
                totals[k] = totals.get(k, 0.0) + float(v)
                counts[k] = counts.get(k, 0) + 1
            else:
                other.setdefault(k, v)
    return totals, counts, other


def _paired_bases(totals: Dict[str, float]) -> set:
    return {k[:-len(SUM)] for k in totals if k.endswith(SUM) and k[:-len(SUM)] + TOK in totals}


def combine_metric_microbatches(per_mb: List[dict]) -> dict:
    """One rank: pairs are summed and stay pairs; other numbers become their mean over micro-batches."""
    totals, counts, other = _accumulate(per_mb)
    bases = _paired_bases(totals)
    out: Dict[str, Any] = {}
    for k, t in totals.items():
        stem = k[:-len(SUM)] if k.endswith(SUM) else k[:-len(TOK)] if k.endswith(TOK) else None
        out[k] = t if stem in bases else t / counts[k]
    for k, v in other.items():
        out.setdefault(k, v)
    return out


def combine_metric_shards(shards: List[dict]) -> dict:
    """All ranks: ``name = sum(.sum) / sum(.tokens)`` (0.0 without tokens); plain numbers are averaged."""
    totals, counts, other = _accumulate(shards)
    bases = _paired_bases(totals)
    out: Dict[str, Any] = {}
    for b in bases:
        tok = totals[b + TOK]
        out[b] = totals[b + SUM] / tok if tok > 0 else 0.0
    for k, t in totals.items():
        stem = k[:-len(SUM)] if k.endswith(SUM) else k[:-len(TOK)] if k.endswith(TOK) else None
        if stem in bases or k in out:
            continue
        out[k] = t / counts[k]
    for k, v in other.items():
        out.setdefault(k, v)
    return out


def finalize_fwd_bwd_metrics(rank_results: List[dict]) -> Tuple[dict, float]:
    """``(metrics, avg_loss)`` of one forward-backward call: the global token-mean loss when the ranks sent
    ``loss.sum``/``loss.tokens``, else the sum of the ranks' ``avg_loss``."""
    metrics = combine_metric_shards([r.get("metrics") or {} for r in rank_results])
    if "loss" in metrics:
        return metrics, float(metrics["loss"])
    return metrics, float(sum(r.get("avg_loss", 0.0) for r in rank_results))
