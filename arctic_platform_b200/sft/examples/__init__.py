"""Runnable examples of the SFT client (``python -m arctic_platform_b200.sft.examples.<name>``).  They default to the
tiny preset and synthetic token data, so they run on a CPU; pass ``--model`` and GPU counts for real runs."""
