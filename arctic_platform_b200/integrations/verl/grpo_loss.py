"""The verl-shaped GRPO / PPO objective registered as ``"verl_grpo"`` (clamped log-ratio, clip 0.2/0.2, dual clip
c = 3, ``agg_loss`` with the global token count).  The implementation lives with the other losses; this module is
the import path verl recipes use (arctic_platform/integrations/verl/grpo_loss.py:415-522 in the reference)."""
from ...rl.processors.losses import verl_grpo_loss  # noqa: F401

__all__ = ["verl_grpo_loss"]
