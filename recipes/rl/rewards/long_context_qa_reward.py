"""Long-context QA reward: the answer is read from ``\\boxed{...}`` (or after "Answer:"); the score is the best
token-level F1 against any gold answer, 1.0 on normalised exact match.  Counterpart of
recipes/rl/skyrl/long_context_qa/long_context_qa_reward.py in the reference."""
from __future__ import annotations

import re
import string
from collections import Counter
from typing import Iterable, Optional

_BOX = re.compile(r"\\boxed\{(.*?)\}", re.S)
_ANS = re.compile(r"[Aa]nswer\s*[:：]\s*(.+)")


def normalize(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def extract(text: str) -> Optional[str]:
    m = _BOX.findall(text)
    if m:
        return m[-1].strip()
    m = _ANS.findall(text)
    return m[-1].strip() if m else None


def f1_score(pred: str, gold: str) -> float:
    p, g = normalize(pred).split(), normalize(gold).split()
    if not p or not g:
        return float(p == g)
    common = sum((Counter(p) & Counter(g)).values())
    if common == 0:
        return 0.0
    prec, rec = common / len(p), common / len(g)
    return 2 * prec * rec / (prec + rec)


def long_context_qa_reward(completion: str, gold_answers: Iterable[str], em_only: bool = False) -> float:
    pred = extract(completion)
    if pred is None:
        return 0.0
    golds = [gold_answers] if isinstance(gold_answers, str) else list(gold_answers)
    if any(normalize(pred) == normalize(g) for g in golds):
        return 1.0
    return 0.0 if em_only else max((f1_score(pred, g) for g in golds), default=0.0)
