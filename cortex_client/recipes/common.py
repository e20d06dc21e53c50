"""What the hosted-service recipes share: ``key=value`` settings, metric logs, chat rendering with a loss mask on the
assistant turns, and a boxed-answer reward for math tasks.

* ``apply_overrides(settings, ["lr=3e-5", "model_name=Qwen/Qwen3-8B", ...])`` -- every key must exist on the settings
  dataclass, values are converted to the type of the default (``none`` / ``null`` for optional fields);
* ``MetricsLogger(log_path, config, wandb_project=None)`` -- ``config.json`` + one JSON line per step in
  ``metrics.jsonl``; mirrors to Weights & Biases when a project is named and the package is importable;
* ``render_chat(messages, tokenizer, max_length)`` -- token ids plus a mask that is 1 on the tokens of assistant turns
  (found by rendering the conversation prefix by prefix, so it works with any chat template);
* ``boxed_answer`` / ``math_reward`` -- the last ``\\boxed{...}`` of a completion against a reference answer.

Counterpart of cortex-client/recipes/neutrino_common.py in the reference.
"""
from __future__ import annotations

import dataclasses
import json
import os
import re
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple, get_args, get_origin, get_type_hints


# ------------------------------------------------------------------------------------------------- settings
def _convert(raw: str, hint: Any, default: Any) -> Any:
    args = get_args(hint)
    optional = get_origin(hint) is not None and type(None) in args
    if raw.lower() in ("none", "null") and (optional or default is None):
        return None
    kind = next((a for a in args if a is not type(None)), hint) if optional else hint
    if kind is bool or isinstance(default, bool):
        if raw.lower() in ("1", "true", "yes", "on"):
            return True
        if raw.lower() in ("0", "false", "no", "off"):
            return False
        raise ValueError(f"expected a boolean, got {raw!r}")
    if kind is int or (isinstance(default, int) and kind is not float):
        return int(raw)
    if kind is float or isinstance(default, float):
        return float(raw)
    if kind in (list, dict) or get_origin(kind) in (list, dict) or isinstance(default, (list, dict)):
        return json.loads(raw)
    return raw


def apply_overrides(settings: Any, items: Sequence[str]) -> Any:
    """Returns a copy of the settings dataclass with ``key=value`` items applied."""
    hints = get_type_hints(type(settings))
    fields = {f.name: f for f in dataclasses.fields(settings)}
    changes: Dict[str, Any] = {}
    for item in items:
        if "=" not in item:
            raise ValueError(f"expected key=value, got {item!r}")
        key, raw = item.split("=", 1)
        key = key.strip().lstrip("-").replace("-", "_")
        if key not in fields:
            raise ValueError(f"unknown setting {key!r} (known: {', '.join(sorted(fields))})")
        try:
            changes[key] = _convert(raw.strip(), hints.get(key, str), getattr(settings, key))
        except (ValueError, json.JSONDecodeError) as exc:
            raise ValueError(f"{key}: {exc}") from exc
    return dataclasses.replace(settings, **changes)


def client_from_settings(config_path: Optional[str], url: Optional[str] = None, session=None):
    """A service client from a connection file (``config=conn.json``) or a plain URL."""
    from ..dss_client import NeutrinoClient
    from ..dss_client.dss_neutrino_cli import _client_from_config, load_connection_config
    if config_path:
        return _client_from_config(load_connection_config(config_path), session)
    if url:
        return NeutrinoClient(url, session=session)
    raise ValueError("give config=<connection file> or url=<service URL>")


# ------------------------------------------------------------------------------------------------- metric logs
class MetricsLogger:
    def __init__(self, log_path: Optional[str], config: Optional[dict] = None, wandb_project: Optional[str] = None,
                 wandb_name: Optional[str] = None, echo=print):
        self.echo = echo
        self.path = None
        self._wandb = None
        if log_path:
            os.makedirs(os.path.expanduser(log_path), exist_ok=True)
            self.path = os.path.join(os.path.expanduser(log_path), "metrics.jsonl")
            if config is not None:
                with open(os.path.join(os.path.expanduser(log_path), "config.json"), "w", encoding="utf-8") as f:
                    json.dump(config, f, indent=1, sort_keys=True, default=str)
        if wandb_project:
            try:
                import wandb
                self._wandb = wandb.init(project=wandb_project, name=wandb_name, config=config or {})
            except Exception as exc:                      # metrics on disk are the record; the mirror is optional
                self.echo(f"wandb disabled: {exc}")

    def log(self, step: int, metrics: Dict[str, Any]) -> dict:
        rec = {"step": step, "time": round(time.time(), 3), **metrics}
        if self.path:
            with open(self.path, "a", encoding="utf-8") as f:
                f.write(json.dumps(rec, default=float) + "\n")
        if self._wandb is not None:
            self._wandb.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)
        if self.echo:
            self.echo(json.dumps(rec, default=float))
        return rec

    def close(self) -> None:
        if self._wandb is not None:
            self._wandb.finish()


# ------------------------------------------------------------------------------------------------- chat rendering
def render_chat(messages: List[Dict[str, str]], tokenizer: Any, max_length: Optional[int] = None) -> Tuple[List[int], List[int]]:
    """``(input_ids, loss_mask)``: the conversation through the tokenizer's chat template, mask 1 on the tokens each
    assistant turn adds (its content and end-of-turn marker), 0 on system / user turns and on the assistant header.
    The token range of a turn is the difference between rendering the conversation up to it with and without it, so no
    template-specific markers are assumed.  Truncation to ``max_length`` cuts the tail."""
    if not messages:
        raise ValueError("an empty conversation")
    ids: List[int] = []
    mask: List[int] = []
    for i, msg in enumerate(messages):
        upto = tokenizer.apply_chat_template(messages[:i + 1], tokenize=True, add_generation_prompt=False)
        upto = list(upto["input_ids"] if isinstance(upto, dict) else upto)
        if msg.get("role") == "assistant":
            head = tokenizer.apply_chat_template(messages[:i], tokenize=True, add_generation_prompt=True) if i else []
            head = list(head["input_ids"] if isinstance(head, dict) else head)
            start = len(head) if upto[:len(head)] == head else len(ids)
        else:
            start = len(upto)
        if upto[:len(ids)] != ids:
            raise ValueError("the chat template does not render prefixes of a conversation as prefixes of its tokens")
        new = upto[len(ids):]
        n_plain = max(0, min(len(new), start - len(ids)))
        mask += [0] * n_plain + [1] * (len(new) - n_plain)
        ids = upto
    if max_length is not None:
        ids, mask = ids[:max_length], mask[:max_length]
    return ids, mask


# ------------------------------------------------------------------------------------------------- math reward
def boxed_answer(text: str) -> Optional[str]:
    """Contents of the last ``\\boxed{...}`` (braces balanced), or None."""
    at = text.rfind("\\boxed")
    if at < 0:
        return None
    i = text.find("{", at)
    if i < 0:
        return None
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[i + 1:j]
    return None


def normalize_answer(ans: str) -> str:
    s = ans.strip().strip("$").replace("\\!", "").replace("\\,", "").replace("\\ ", "").replace(" ", "")
    s = re.sub(r"\\text\{([^}]*)\}", r"\1", s)
    s = re.sub(r"\\left|\\right", "", s).replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac")
    s = re.sub(r"^\\frac\{(-?\d+)\}\{(-?\d+)\}$", r"\1/\2", s)
    s = s.rstrip(".")
    if re.fullmatch(r"-?\d{1,3}(,\d{3})+(\.\d+)?", s):
        s = s.replace(",", "")
    try:
        f = float(s)
        return str(int(f)) if f == int(f) else repr(f)
    except ValueError:
        pass
    m = re.fullmatch(r"(-?\d+)/(-?\d+)", s)
    if m and int(m.group(2)) != 0:
        from fractions import Fraction
        fr = Fraction(int(m.group(1)), int(m.group(2)))
        return str(fr.numerator) if fr.denominator == 1 else f"{fr.numerator}/{fr.denominator}"
    return s


def math_reward(completion: str, reference: str, format_penalty: float = 0.0) -> float:
    """1 when the boxed answer equals the reference after normalisation, ``-format_penalty`` without a boxed answer."""
    got = boxed_answer(completion)
    if got is None:
        return -float(format_penalty)
    ref = boxed_answer(reference) or reference
    return 1.0 if normalize_answer(got) == normalize_answer(ref) else 0.0
