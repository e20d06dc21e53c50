"""Readable JSON -> a forward-backward batch.

The command line (``dss-neutrino fwd-bwd JOB --json batch.json``) and notebooks describe a training batch as plain
JSON; this module compiles such a description into the tensor kwargs the service's training call takes and frames
them for the wire.  A description is one of

* ``{"kwargs": {...}}``: used as is; lists and ``{"data": ..., "dtype": ...}`` objects become tensors;
* ``{"input_ids": [[...]], ...}``: token ids given directly;
* ``{"texts": [...], "tokenizer": "name" | {"model_name": ..., "revision": ...}, "max_length": N, ...}``: tokenised
  here (``batch_size`` repeats the texts cyclically up to that many rows; ``padding`` defaults to ``"max_length"``).

and in the last two forms these keys shape the rest of the batch:

=====================================  ==========================================================================
``attention_mask``                     tensor data, or ``true`` / ``false`` = include one (all ones when unknown)
``include_attention_mask``             same switch as a separate key (default off)
``position_ids``                       ``true`` / ``"arange"`` = 0..S-1 per row, tensor data, or ``false``
``include_position_ids``               ``true`` = ``"arange"``
``labels`` / ``label_strategy``        ``"next_token"`` (default; row shifted left, last column ignored),
                                       ``"input_ids"`` (copy), ``"none"``, tensor data, or
                                       ``{"strategy", "ignore_index", "mask_padding"}``
``ignore_index`` / ``mask_padding``    -100 / true: targets at padded positions get the ignore index
=====================================  ==========================================================================

Contract of ``build_forward_backward_kwargs`` / ``serialize_forward_backward_args`` /
``build_forward_backward_payload`` in cortex-client/dss_client/neutrino_client.py:492-806 of the reference.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from arctic_platform_b200 import wire

DTYPES: Dict[str, torch.dtype] = {
    "bool": torch.bool, "boolean": torch.bool,
    "float": torch.float32, "float32": torch.float32, "fp32": torch.float32,
    "float64": torch.float64, "double": torch.float64,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "int": torch.int32, "int32": torch.int32, "int64": torch.int64, "long": torch.int64,
    "int8": torch.int8, "uint8": torch.uint8, "int16": torch.int16,
}
LABEL_STRATEGIES = ("next_token", "shifted_input_ids", "input_ids", "self", "none")
RESPONSE_OPTIONS = {"format": "dssst1", "delivery": "chunked"}


class BatchSpecError(ValueError):
    """A batch description that cannot be compiled; the message names the offending key."""


def _is_tensor_data(v: Any) -> bool:
    return isinstance(v, list) or (isinstance(v, dict) and "data" in v)


def to_tensor(value: Any, default_dtype: str = "long", name: str = "tensor") -> torch.Tensor:
    """``[[1, 2]]`` or ``{"data": [[1, 2]], "dtype": "float32"}`` -> tensor."""
    dtype_name = default_dtype
    if isinstance(value, dict):
        if "data" not in value:
            raise BatchSpecError(f"{name}: a tensor object needs a 'data' field")
        dtype_name = value.get("dtype") or default_dtype
        value = value["data"]
    if dtype_name not in DTYPES:
        raise BatchSpecError(f"{name}: unsupported dtype {dtype_name!r} (known: {', '.join(sorted(DTYPES))})")
    try:
        return torch.tensor(value, dtype=DTYPES[dtype_name])
    except (TypeError, ValueError, RuntimeError) as exc:
        raise BatchSpecError(f"{name}: {exc}") from exc


def _flag(spec: dict, key: str, default: bool) -> bool:
    v = spec.get(key, default)
    if not isinstance(v, bool):
        raise BatchSpecError(f"{key} must be true or false")
    return v


def _positive(v: Any, key: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise BatchSpecError(f"{key} must be a positive integer")
    return v


def _rows(t: torch.Tensor, like: Optional[torch.Tensor], name: str) -> torch.Tensor:
    if t.dim() != 2:
        raise BatchSpecError(f"{name} must have shape [batch, seq_len], got {tuple(t.shape)}")
    if like is not None and t.shape != like.shape:
        raise BatchSpecError(f"{name} has shape {tuple(t.shape)}, input_ids has {tuple(like.shape)}")
    return t.contiguous()


# --------------------------------------------------------------------------------------------- tokenisation
def default_tokenizer_loader(spec: Any):
    """``"name"`` or ``{"model_name" | "name" | "path", "trust_remote_code"?, "use_fast"?, "revision"?}`` -> tokenizer;
    a tokenizer without a pad token pads with its end-of-sequence token."""
    from transformers import AutoTokenizer
    if isinstance(spec, str):
        name, kw = spec, {}
    elif isinstance(spec, dict):
        name = spec.get("model_name") or spec.get("name") or spec.get("path")
        kw = {k: spec[k] for k in ("trust_remote_code", "use_fast", "revision") if k in spec}
    else:
        raise BatchSpecError("tokenizer must be a name or an object")
    if not isinstance(name, str) or not name:
        raise BatchSpecError("tokenizer.model_name is required")
    tok = AutoTokenizer.from_pretrained(name, **kw)
    if getattr(tok, "pad_token_id", None) is None and getattr(tok, "eos_token", None) is not None:
        tok.pad_token = tok.eos_token
    return tok


def expand_texts(texts: Any, batch_size: Any = None) -> List[str]:
    if isinstance(texts, str):
        texts = [texts]
    if not (isinstance(texts, list) and texts and all(isinstance(t, str) for t in texts)):
        raise BatchSpecError("texts must be a string or a non-empty list of strings")
    if batch_size is None:
        return list(texts)
    n = _positive(batch_size, "batch_size")
    return [texts[i % len(texts)] for i in range(n)]


def _tokenize(spec: dict, loader: Callable[[Any], Any]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    tok_spec = spec.get("tokenizer", spec.get("model_name"))
    if tok_spec is None:
        raise BatchSpecError("a batch description needs input_ids, or texts with a tokenizer")
    texts = expand_texts(spec.get("texts"), spec.get("batch_size"))
    padding = spec.get("padding", "max_length")
    kw = {"return_tensors": "pt", "padding": padding, "truncation": _flag(spec, "truncation", True),
          "add_special_tokens": _flag(spec, "add_special_tokens", True)}
    if padding == "max_length" or spec.get("max_length") is not None:
        kw["max_length"] = _positive(spec.get("max_length"), "max_length")
    enc = loader(tok_spec)(texts, **kw)
    if "input_ids" not in enc:
        raise BatchSpecError("the tokenizer returned no input_ids")
    mask = enc.get("attention_mask") if hasattr(enc, "get") else None
    return torch.as_tensor(enc["input_ids"]).long(), (torch.as_tensor(mask).long() if mask is not None else None)


# --------------------------------------------------------------------------------------------- labels / positions
def make_labels(input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor], spec: dict) -> Optional[torch.Tensor]:
    """Targets aligned with ``input_ids`` (the loss sits where ``labels != ignore_index``)."""
    want = spec.get("labels", spec.get("label_strategy", "next_token"))
    ignore = int(spec.get("ignore_index", -100))
    mask_padding = _flag(spec, "mask_padding", True)
    if _is_tensor_data(want):
        return to_tensor(want, name="labels")
    if isinstance(want, dict):
        ignore = int(want.get("ignore_index", ignore))
        mp = want.get("mask_padding", mask_padding)
        if not isinstance(mp, bool):
            raise BatchSpecError("labels.mask_padding must be true or false")
        mask_padding, want = mp, want.get("strategy", "next_token")
    if want is None or want == "none":
        return None
    if want not in LABEL_STRATEGIES:
        raise BatchSpecError(f"labels must be one of {', '.join(LABEL_STRATEGIES)} or tensor data, got {want!r}")
    valid = attention_mask.bool() if (mask_padding and attention_mask is not None) else torch.ones_like(input_ids, dtype=torch.bool)
    if want in ("input_ids", "self"):
        return torch.where(valid, input_ids, torch.full_like(input_ids, ignore))
    out = torch.full_like(input_ids, ignore)                  # next token: column j predicts token j + 1
    out[:, :-1] = torch.where(valid[:, 1:], input_ids[:, 1:], out[:, :-1])
    return out


def make_position_ids(input_ids: torch.Tensor, spec: dict) -> Optional[torch.Tensor]:
    want = spec.get("position_ids")
    if want is None and _flag(spec, "include_position_ids", False):
        want = "arange"
    if want is None or want is False:
        return None
    if want is True or want == "arange":
        b, s = input_ids.shape
        return torch.arange(s, dtype=torch.long).repeat(b, 1)
    if _is_tensor_data(want):
        return to_tensor(want, name="position_ids")
    raise BatchSpecError("position_ids must be true, false, \"arange\" or tensor data")


# --------------------------------------------------------------------------------------------- entry points
def build_forward_backward_kwargs(spec: Dict[str, Any], tokenizer_loader: Optional[Callable[[Any], Any]] = None) -> Dict[str, Any]:
    """Compiles a batch description (module docstring) into ``{"input_ids", "labels"?, "attention_mask"?,
    "position_ids"?}`` -- or, for the ``kwargs`` form, into the given keys with tensor data turned into tensors."""
    if not isinstance(spec, dict):
        raise BatchSpecError("a batch description must be a JSON object")
    if "kwargs" in spec:
        raw = spec["kwargs"]
        if not isinstance(raw, dict):
            raise BatchSpecError("kwargs must be an object")
        return {k: (to_tensor(v, name=k) if _is_tensor_data(v) else v) for k, v in raw.items()}
    given_mask = spec.get("attention_mask")
    if "input_ids" in spec:
        ids = to_tensor(spec["input_ids"], name="input_ids")
        mask = to_tensor(given_mask, name="attention_mask") if _is_tensor_data(given_mask) else None
    else:
        ids, mask = _tokenize(spec, tokenizer_loader or default_tokenizer_loader)
    ids = _rows(ids, None, "input_ids")
    if mask is not None:
        mask = _rows(mask, ids, "attention_mask")
    out: Dict[str, Any] = {"input_ids": ids}
    include_mask = given_mask if isinstance(given_mask, bool) else _flag(spec, "include_attention_mask", False)
    if include_mask:
        out["attention_mask"] = mask if mask is not None else torch.ones_like(ids)
    pos = make_position_ids(ids, spec)
    if pos is not None:
        out["position_ids"] = _rows(pos, ids, "position_ids")
    labels = make_labels(ids, mask, spec)
    if labels is not None:
        out["labels"] = _rows(labels, ids, "labels")
    return out


def serialize_forward_backward_args(args: tuple = (), kwargs: Optional[Dict[str, Any]] = None) -> bytes:
    """One DSSST1 frame ``{"args", "kwargs"}`` that asks for a chunked DSSST1 reply."""
    if not isinstance(args, tuple):
        raise BatchSpecError("args must be a tuple")
    if kwargs is not None and not isinstance(kwargs, dict):
        raise BatchSpecError("kwargs must be a dict")
    return wire.dumps({"args": list(args), "kwargs": kwargs or {}}, metadata={"response_options": dict(RESPONSE_OPTIONS)})


def build_forward_backward_payload(spec: Dict[str, Any], tokenizer_loader: Optional[Callable[[Any], Any]] = None) -> bytes:
    """``{"payload": description}`` (or the description itself) -> framed bytes; positional ``args`` pass through."""
    if not isinstance(spec, dict):
        raise BatchSpecError("the fwd-bwd JSON must be an object")
    body = spec.get("payload", spec)
    if not isinstance(body, dict):
        raise BatchSpecError("payload must be an object")
    args = body.get("args") or []
    if not isinstance(args, list):
        raise BatchSpecError("args must be a JSON list")
    return serialize_forward_backward_args(tuple(args), build_forward_backward_kwargs(body, tokenizer_loader))
