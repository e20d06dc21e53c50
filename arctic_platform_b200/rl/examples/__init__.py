"""Runnable examples of the RL client (``python -m arctic_platform_b200.rl.examples.<name>``).  All of them default to
the tiny preset and synthetic token data, so they run on a laptop CPU; pass ``--model`` and GPU counts for real runs."""
