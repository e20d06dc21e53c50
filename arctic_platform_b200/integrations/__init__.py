"""Adapters that let external RL frameworks drive this platform (verl; SkyRL recipes reuse the same client)."""
