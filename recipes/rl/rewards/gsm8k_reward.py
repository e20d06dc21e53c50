"""GSM8K-style reward: 1.0 when the final number of the completion equals the reference answer.

Accepted answer formats, in priority order: ``#### 42``, ``\\boxed{42}``, ``The answer is 42``; with
``method="flexible"`` the last number anywhere in the text is used as a fall-back (format reward 0.1 when only the
fall-back matches nothing).  Counterpart of the reward in recipes/rl/skyrl/simple_gsm8k and verl's gsm8k scorer.
"""
from __future__ import annotations

import re
from typing import Optional

_NUM = r"-?\$?\d[\d,]*(?:\.\d+)?"
_PATTERNS = [re.compile(r"####\s*(" + _NUM + ")"), re.compile(r"\\boxed\{\s*(" + _NUM + r")\s*\}"),
             re.compile(r"[Tt]he (?:final )?answer is[:\s]*(" + _NUM + ")")]


def _norm(s: str) -> str:
    s = s.replace(",", "").replace("$", "").strip()
    if "." in s:
        s = s.rstrip("0").rstrip(".")
    return s or "0"


def extract_answer(text: str, method: str = "strict") -> Optional[str]:
    for pat in _PATTERNS:
        m = pat.findall(text)
        if m:
            return _norm(m[-1])
    if method == "flexible":
        m = re.findall(_NUM, text)
        if m:
            return _norm(m[-1])
    return None


def gsm8k_reward(completion: str, ground_truth: str, method: str = "strict", format_score: float = 0.0,
                 score: float = 1.0) -> float:
    ans = extract_answer(completion, method)
    if ans is None:
        return 0.0
    gt = extract_answer(ground_truth, "flexible") or _norm(ground_truth)
    return score if ans == gt else format_score
