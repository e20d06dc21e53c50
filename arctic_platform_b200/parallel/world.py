"""Process topology read from the launcher's environment (``RANK``, ``LOCAL_RANK``, ``WORLD_SIZE``,
``LOCAL_WORLD_SIZE``): the singleton every component asks for "which GPU am I".
Counterpart of arctic_platform/model/implementations/qwen35/world.py:4-43."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class World:
    rank: int
    local_rank: int
    world_size: int
    local_world_size: int

    @property
    def num_nodes(self) -> int:
        return max(1, self.world_size // max(1, self.local_world_size))

    @property
    def node_rank(self) -> int:
        return self.rank // max(1, self.local_world_size)

    @property
    def is_master(self) -> bool:
        return self.rank == 0


_world: Optional[World] = None


def get_world(refresh: bool = False) -> World:
    global _world
    if _world is None or refresh:
        ws = int(os.environ.get("WORLD_SIZE", "1"))
        lws = int(os.environ.get("LOCAL_WORLD_SIZE", str(min(ws, 8))))
        rank = int(os.environ.get("RANK", "0"))
        _world = World(rank, int(os.environ.get("LOCAL_RANK", str(rank % max(1, lws)))), ws, lws)
        if not (0 <= _world.rank < _world.world_size) or _world.world_size % _world.local_world_size:
            bad, _world = _world, None
            raise ValueError(f"inconsistent launcher environment: {bad}")
    return _world
