"""Reward functions used by the recipes (pure Python, no GPU)."""
from .bird_reward import bird_reward, extract_sql  # noqa: F401
from .gsm8k_reward import extract_answer, gsm8k_reward  # noqa: F401
from .long_context_qa_reward import f1_score, long_context_qa_reward  # noqa: F401
