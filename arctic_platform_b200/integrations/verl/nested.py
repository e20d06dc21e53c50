"""verl's padding-free batches: nested-jagged tensors in, nested-jagged tensors out.

Recent verl keeps a batch without padding: ``input_ids`` (and ``position_ids``, masks, ...) are nested tensors in the
jagged layout, one row per sample holding ``prompt || response``, with ``prompts`` / ``responses`` nested alongside.
The platform's wire batch is dense (prompt left-padded to ``P``, response right-padded to ``R``) and its per-token
outputs come back as ``[B, R]`` grids aligned with the response tokens.  This module converts in both directions
without a Python loop over rows:

* ``jagged_lengths`` / ``prompt_response_lengths``: row lengths from a nested tensor or from dense masks;
* ``nested_to_padded``: jagged values -> ``[B, P + R]`` (one scatter);
* ``response_grid_to_nested``: a ``[B, R]`` grid -> nested rows of length ``prompt + response`` with the values placed
  either on the response tokens themselves (``align="response"``) or one position earlier, on the token that
  *predicts* them (``align="predict_next"``, what verl's losses index);
* ``shift_nested_left``: response-aligned nested rows -> predict-next aligned;
* ``normalize_backend_metrics``: metric values as lists of floats, the shape verl's metric reducers append.

Counterpart of ``_no_padding_2_padding_prompt_response`` (arctic_platform/integrations/verl/adapter.py:60-107) and of
the ``make_njt`` / ``shift_nested_response_aligned_to_predict_next`` / ``normalize_backend_metrics`` helpers the
reference's worker takes from verl (arctic_platform/integrations/verl/worker.py:204-291).
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Tuple

import torch


def is_nested(t: Any) -> bool:
    return torch.is_tensor(t) and bool(getattr(t, "is_nested", False))


def jagged_lengths(t: torch.Tensor) -> torch.Tensor:
    """Row lengths of a nested (jagged) tensor."""
    return t.offsets().diff().long()


def jagged_values(t: torch.Tensor) -> torch.Tensor:
    return t.values() if is_nested(t) else t


def prompt_response_lengths(data: Mapping[str, Any]) -> Tuple[torch.Tensor, torch.Tensor, int, int]:
    """``(prompt_lens, response_lens, P, R)`` of a batch whose ``prompts`` / ``responses`` are nested (``P``, ``R`` =
    ``max_prompt_len`` / ``max_response_len`` when given, else the longest row) or dense with a dense
    ``attention_mask`` (``P``, ``R`` = the padded widths)."""
    prompts, responses = data["prompts"], data["responses"]
    if is_nested(prompts):
        pl, rl = jagged_lengths(prompts), jagged_lengths(responses)
        P, R = int(data.get("max_prompt_len", -1) or -1), int(data.get("max_response_len", -1) or -1)
        return pl, rl, (int(pl.max()) if P < 0 else P), (int(rl.max()) if R < 0 else R)
    mask = data["attention_mask"]
    if is_nested(mask):
        raise ValueError("dense prompts / responses need a dense attention_mask")
    P, R = prompts.shape[1], responses.shape[1]
    return mask[:, :P].sum(1).long(), mask[:, P:P + R].sum(1).long(), P, R


def _row_index(lens: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """For jagged rows of the given lengths: (row of every element, position of every element inside its row)."""
    n = int(lens.sum())
    row = torch.repeat_interleave(torch.arange(lens.numel(), device=lens.device), lens, output_size=n)
    start = lens.cumsum(0) - lens
    return row, torch.arange(n, device=lens.device) - start[row]


def nested_to_padded(values: torch.Tensor, prompt_lens: torch.Tensor, response_lens: torch.Tensor, P: int, R: int,
                     pad_value: Any = 0) -> torch.Tensor:
    """Jagged ``prompt || response`` rows -> ``[B, P + R]``: prompts end at column ``P``, responses start there."""
    values = jagged_values(values)
    seq = prompt_lens + response_lens
    if int(seq.sum()) != values.shape[0]:
        raise ValueError(f"row lengths sum to {int(seq.sum())}, the tensor holds {values.shape[0]} elements")
    if int(prompt_lens.max()) > P or int(response_lens.max()) > R:
        raise ValueError("a row is longer than the padded prompt / response width")
    row, within = _row_index(seq)
    out = values.new_full((seq.numel(), P + R) + tuple(values.shape[1:]), pad_value)
    out[row, within + (P - prompt_lens)[row]] = values
    return out


def response_grid_to_nested(grid: torch.Tensor, prompt_lens: torch.Tensor, response_lens: torch.Tensor,
                            align: str = "predict_next") -> torch.Tensor:
    """``grid[b, k]`` = value of response token ``k`` of sample ``b`` -> nested rows of length ``prompt + response``,
    zero outside the placed values.  ``predict_next`` puts value ``k`` at position ``prompt - 1 + k``, ``response`` at
    ``prompt + k``."""
    if align not in ("predict_next", "response"):
        raise ValueError("align must be 'predict_next' or 'response'")
    if grid.dim() != 2 or grid.shape[0] != prompt_lens.numel():
        raise ValueError(f"expected a [B, R] grid for {prompt_lens.numel()} rows, got {tuple(grid.shape)}")
    if int(response_lens.max()) > grid.shape[1]:
        raise ValueError("a response is longer than the grid")
    shift = 1 if align == "predict_next" else 0
    if shift and int(prompt_lens.min()) < 1:
        raise ValueError("predict-next alignment needs at least one prompt token per row")
    seq = prompt_lens + response_lens
    flat = grid.new_zeros(int(seq.sum()))
    row, k = _row_index(response_lens)
    start = seq.cumsum(0) - seq
    flat[start[row] + prompt_lens[row] - shift + k] = grid[row, k]
    return torch.nested.nested_tensor_from_jagged(flat, offsets=torch.cat([seq.new_zeros(1), seq.cumsum(0)]))


def make_njt(data: Mapping[str, Any], grid: torch.Tensor, align: str = "predict_next") -> torch.Tensor:
    """A backend output (``[B, R]`` over the responses, or ``[B, P + R]`` over the padded sequence) as a nested tensor
    with the row layout of ``data["input_ids"]``."""
    pl, rl, P, R = prompt_response_lengths(data)
    if grid.shape[1] == P + R and grid.shape[1] != R:
        grid = grid[:, P:]
    return response_grid_to_nested(grid[:, :max(R, int(rl.max()))], pl, rl, align)


def shift_nested_left(t: torch.Tensor) -> torch.Tensor:
    """Every row moved one position to the left (the last position becomes zero): values stored on the tokens they
    belong to become values stored on the tokens that predict them."""
    vals, offs = t.values(), t.offsets()
    lens = offs.diff()
    row, within = _row_index(lens)
    out = torch.zeros_like(vals)
    keep = within >= 1
    out[(torch.arange(vals.shape[0], device=vals.device) - 1)[keep]] = vals[keep]
    return torch.nested.nested_tensor_from_jagged(out, offsets=offs)


def normalize_backend_metrics(metrics: Mapping[str, Any]) -> Dict[str, List[float]]:
    """Scalars, 0-d / 1-d tensors and lists -> lists of Python floats; anything else is dropped with its key kept
    out of the result (a metric that cannot be averaged must not break the step)."""
    out: Dict[str, List[float]] = {}
    for k, v in metrics.items():
        if torch.is_tensor(v):
            v = v.detach().float().reshape(-1).tolist()
        elif isinstance(v, (int, float)) and not isinstance(v, bool):
            v = [float(v)]
        elif isinstance(v, (list, tuple)) and all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in v):
            v = [float(x) for x in v]
        else:
            continue
        out[str(k)] = v
    return out
