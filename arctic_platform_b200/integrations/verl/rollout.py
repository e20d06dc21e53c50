"""Rollout-side shims for verl: a token-in / token-out generation server and the replica descriptor verl's agent
loop schedules.  The sampling engine itself lives on the platform; these classes only translate verl's rollout
protocol (``generate(prompt_ids, sampling_params, request_id)``, ``wake_up`` / ``sleep`` by ``RolloutMode``)
into client calls.  Counterpart of arctic_platform/integrations/verl/rollout.py:55-404.
"""
from __future__ import annotations

import asyncio
import enum
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

from .adapter import ArcticRLClientWrapper


class RolloutMode(str, enum.Enum):
    HYBRID = "hybrid"          # sampler shares GPUs with training: sleep between rollouts
    COLOCATED = "colocated"    # same nodes, own GPUs: stays awake, weights synced in place
    STANDALONE = "standalone"  # own nodes


@dataclass
class TokenOutput:
    token_ids: List[int]
    log_probs: Optional[List[float]] = None
    stop_reason: Optional[str] = None
    extra: Dict[str, Any] = field(default_factory=dict)
    routed_experts: Any = None           # [fed tokens, L_moe, k] with ``enable_rollout_routing_replay``


class ArcticLLMServer:
    """One generation endpoint.  ``generate`` takes prompt token ids and returns generated token ids -- no
    tokenizer round trip (the reference's adapter decodes ids to text before calling its engine)."""

    def __init__(self, wrapper: ArcticRLClientWrapper, mode: RolloutMode = RolloutMode.HYBRID,
                 enable_rollout_routing_replay: bool = False):
        self.wrapper = wrapper
        self.mode = RolloutMode(mode)
        self._awake = True
        # ask the sampler for the experts it chose, so that training can replay them
        # (arctic_platform/integrations/verl/rollout.py:303-305)
        self.enable_rollout_routing_replay = bool(enable_rollout_routing_replay)

    async def generate(self, prompt_ids: Sequence[int], sampling_params: Optional[dict] = None,
                       request_id: Optional[str] = None, **_) -> TokenOutput:
        sp = dict(sampling_params or {})
        if "max_new_tokens" in sp:
            sp["max_tokens"] = sp.pop("max_new_tokens")
        sp.pop("logprobs", None) if sp.get("logprobs") in (None, False, 0) else None
        if self.enable_rollout_routing_replay:
            sp["return_routed_experts"] = True
        loop = asyncio.get_running_loop()
        outs = await loop.run_in_executor(None, lambda: self.wrapper.generate([list(prompt_ids)], sp, routing_key=request_id))
        o = outs[0]
        first = o["outputs"][0] if "outputs" in o else o
        return TokenOutput(list(first.get("token_ids", [])), first.get("logprobs"), first.get("finish_reason"),
                           {"request_id": request_id},
                           first.get("routed_experts") if self.enable_rollout_routing_replay else None)

    async def generate_batch(self, prompts: Sequence[Sequence[int]], sampling_params: Optional[dict] = None) -> List[TokenOutput]:
        return list(await asyncio.gather(*[self.generate(p, sampling_params, str(i)) for i, p in enumerate(prompts)]))

    async def wake_up(self, tags: Optional[List[str]] = None) -> None:
        if self.mode is RolloutMode.HYBRID and not self._awake:
            self.wrapper.wake_up_inference(tags)
        self._awake = True

    async def sleep(self, level: int = 1) -> None:
        if self.mode is RolloutMode.HYBRID and self._awake:
            self.wrapper.sleep_inference(level)
            self._awake = False

    async def reset_prefix_cache(self) -> None:
        self.wrapper.reset_prefix_cache()


@dataclass
class ArcticReplica:
    """What verl's rollout scheduler sees: one replica = one platform sampling job (its GPUs are the server's)."""
    replica_rank: int
    wrapper: ArcticRLClientWrapper
    mode: RolloutMode = RolloutMode.HYBRID
    server: Optional[ArcticLLMServer] = None
    enable_rollout_routing_replay: bool = False

    async def init(self) -> "ArcticReplica":
        self.server = ArcticLLMServer(self.wrapper, self.mode, self.enable_rollout_routing_replay)
        return self

    @property
    def server_handle(self) -> ArcticLLMServer:
        if self.server is None:
            raise RuntimeError("replica not initialised")
        return self.server

    @property
    def world_size(self) -> int:
        return self.wrapper._n_gpus("sampling")
