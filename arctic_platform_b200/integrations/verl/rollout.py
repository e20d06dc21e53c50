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
    num_preempted: Optional[int] = None
    finish_reason: Optional[str] = None  # the engine's own word ("stop" / "length" / "abort"); stop_reason is verl's


@dataclass
class RolloutServerConfig:
    """The rollout section of verl's config as far as the endpoint needs it
    (arctic_platform/integrations/verl/rollout.py:121-186, 215-250)."""
    max_model_len: Optional[int] = None      # context limit; None: not enforced here (the engine enforces its own)
    prompt_length: int = 0                   # configured prompt budget
    response_length: int = 0                 # configured response budget (default generation length)
    free_cache_engine: bool = True           # release the KV cache between rollouts (sleep / wake are no-ops when off)
    repetition_penalty: float = 1.0

    @staticmethod
    def from_verl(rollout_cfg: Optional[dict]) -> "RolloutServerConfig":
        c = dict(rollout_cfg or {})
        return RolloutServerConfig(c.get("max_model_len"), int(c.get("prompt_length", 0) or 0),
                                   int(c.get("response_length", 0) or 0), bool(c.get("free_cache_engine", True)),
                                   float(c.get("repetition_penalty", 1.0)))


def verl_stop_reason(finish_reason: Optional[str]) -> Optional[str]:
    """verl's vocabulary: an aborted request is "aborted", a natural or length stop "completed"."""
    if finish_reason == "abort":
        return "aborted"
    if finish_reason in ("stop", "length"):
        return "completed"
    return finish_reason


def resolve_max_tokens(sp: dict, prompt_len: int, cfg: RolloutServerConfig) -> int:
    """``max_tokens`` / ``max_new_tokens`` of the request (removed from ``sp``), else the configured budget, clamped
    to the context space left after the prompt.  A prompt longer than the context is an error."""
    space = None if cfg.max_model_len is None else int(cfg.max_model_len) - prompt_len
    if space is not None and space < 0:
        raise ValueError(f"Prompt length ({prompt_len}) exceeds the model's maximum context length "
                         f"({cfg.max_model_len}).")
    if "max_tokens" in sp:
        want = int(sp.pop("max_tokens"))
        sp.pop("max_new_tokens", None)
    elif "max_new_tokens" in sp:
        want = int(sp.pop("max_new_tokens"))
    else:
        want = cfg.response_length + cfg.prompt_length - prompt_len
        if want <= 0 and space is None:
            return -1                              # nothing configured: leave the engine's default
    want = max(0, want)
    return want if space is None else min(want, space)


class ArcticLLMServer:
    """One generation endpoint.  ``generate`` takes prompt token ids and returns generated token ids -- no
    tokenizer round trip (the reference's adapter decodes ids to text before calling its engine)."""

    def __init__(self, wrapper: ArcticRLClientWrapper, mode: RolloutMode = RolloutMode.HYBRID,
                 enable_rollout_routing_replay: bool = False, config: Optional[RolloutServerConfig] = None,
                 node_rank: int = 0, replica_rank: int = 0):
        self.wrapper = wrapper
        self.mode = RolloutMode(mode)
        self.config = config or RolloutServerConfig()
        self.node_rank = int(node_rank)              # only node 0 of a replica talks to the platform
        self.replica_rank = int(replica_rank)
        self.global_steps = 0                        # stamped on every output; moved on by update_weights
        self._awake = True
        # ask the sampler for the experts it chose, so that training can replay them
        # (arctic_platform/integrations/verl/rollout.py:303-305)
        self.enable_rollout_routing_replay = bool(enable_rollout_routing_replay)

    async def generate(self, prompt_ids: Sequence[int], sampling_params: Optional[dict] = None,
                       request_id: Optional[str] = None, **_) -> TokenOutput:
        sp = dict(sampling_params or {})
        prompt_ids = [int(t) for t in prompt_ids]
        max_tokens = resolve_max_tokens(sp, len(prompt_ids), self.config)
        if max_tokens >= 0:
            sp["max_tokens"] = max_tokens
        want_lp = sp.pop("logprobs", None) not in (None, False)
        if want_lp:
            sp["logprobs"] = 0                        # the sampled token's log-prob only
        if self.config.repetition_penalty != 1.0:
            sp.setdefault("repetition_penalty", self.config.repetition_penalty)
        if self.enable_rollout_routing_replay:
            sp["return_routed_experts"] = True
        loop = asyncio.get_running_loop()
        outs = await loop.run_in_executor(None, lambda: self.wrapper.generate([prompt_ids], sp, routing_key=request_id))
        o = outs[0]
        first = o["outputs"][0] if "outputs" in o else o
        reason = first.get("finish_reason")
        return TokenOutput(list(first.get("token_ids", [])), first.get("logprobs") if want_lp or first.get("logprobs") else None,
                           reason if self._raw_reasons else verl_stop_reason(reason),
                           {"request_id": request_id, "global_steps": self.global_steps},
                           first.get("routed_experts") if self.enable_rollout_routing_replay else None,
                           first.get("num_preempted"), reason)

    async def generate_batch(self, prompts: Sequence[Sequence[int]], sampling_params: Optional[dict] = None) -> List[TokenOutput]:
        return list(await asyncio.gather(*[self.generate(p, sampling_params, str(i)) for i, p in enumerate(prompts)]))

    # verl's own stop vocabulary ("completed" / "aborted") is opt-in: callers of this class that predate it read
    # the engine's finish reason from ``stop_reason``
    _raw_reasons = True

    def use_verl_stop_reasons(self, on: bool = True) -> "ArcticLLMServer":
        self._raw_reasons = not on
        return self

    def _controls_engine(self) -> bool:
        return self.node_rank == 0 and self.config.free_cache_engine

    async def wake_up(self, tags: Optional[List[str]] = None) -> None:
        """HYBRID: the sampler shares GPUs with training and comes back with its weights and KV cache; COLOCATED: the
        same without a weight hand-over, plus a prefix-cache reset; STANDALONE: never slept."""
        if not self._controls_engine() or self.mode is RolloutMode.STANDALONE:
            self._awake = True
            return
        if not self._awake:
            self.wrapper.wake_up_inference(tags if tags is not None or self.mode is RolloutMode.HYBRID
                                           else ["kv_cache", "weights"])
            if self.mode is RolloutMode.COLOCATED:
                self.wrapper.reset_prefix_cache()
        self._awake = True

    async def sleep(self, level: int = 1) -> None:
        if not self._controls_engine() or self.mode is RolloutMode.STANDALONE:
            return
        if self._awake:
            self.wrapper.sleep_inference(level)
            self._awake = False

    async def update_weights(self, global_steps: Optional[int] = None) -> Dict[str, Any]:
        """Trainer -> sampler hand-over as verl drives it in HYBRID mode: weights first (into memory the sleeping
        sampler still owns), then the KV cache comes back and cached prefixes of the old policy are dropped."""
        out = self.wrapper.update_weights()
        if self._controls_engine() and self.mode is not RolloutMode.STANDALONE and not self._awake:
            self.wrapper.wake_up_inference(["kv_cache"])
            self._awake = True
        self.wrapper.reset_prefix_cache()
        if global_steps is not None:
            self.global_steps = int(global_steps)
        return out

    async def reset_prefix_cache(self) -> None:
        self.wrapper.reset_prefix_cache()

    async def clear_kv_cache(self) -> None:
        if self.node_rank == 0:
            self.wrapper.reset_prefix_cache()

    async def abort_request(self, request_id: str) -> Dict[str, Any]:
        """Requests run to completion inside one platform call; there is nothing in flight to cancel between calls."""
        return {"request_id": request_id, "aborted": False, "reason": "requests complete within one generate call"}

    def get_server_address(self) -> Optional[str]:
        """``host:port`` of the platform server this endpoint talks to (None for an in-process client)."""
        cc = getattr(self.wrapper, "client_config", None)
        host, port = getattr(cc, "http_host", None), getattr(cc, "http_port", None)
        return f"{host}:{port}" if host and port else None


@dataclass
class ArcticReplica:
    """What verl's rollout scheduler sees: one replica = one platform sampling job (its GPUs are the server's)."""
    replica_rank: int
    wrapper: ArcticRLClientWrapper
    mode: RolloutMode = RolloutMode.HYBRID
    server: Optional[ArcticLLMServer] = None
    enable_rollout_routing_replay: bool = False
    config: Optional[RolloutServerConfig] = None
    nnodes: int = 1
    servers: List[ArcticLLMServer] = field(default_factory=list)

    async def init(self) -> "ArcticReplica":
        await self.launch_servers()
        return self

    async def launch_servers(self) -> List[ArcticLLMServer]:
        """One endpoint object per node of the replica; node 0's is the one that drives the platform (the others
        exist so that verl's per-node bookkeeping has something to hold, and never touch the engine)."""
        self.servers = [ArcticLLMServer(self.wrapper, self.mode, self.enable_rollout_routing_replay, self.config,
                                        node_rank=n, replica_rank=self.replica_rank) for n in range(max(1, self.nnodes))]
        self.server = self.servers[0]
        return self.servers

    def rollout_worker_use_gpu(self) -> bool:
        return False                 # the GPUs belong to the platform's sampling job, not to verl's rollout workers

    async def abort_request(self, request_id: str) -> Dict[str, Any]:
        return await self.server_handle.abort_request(request_id)

    @property
    def server_handle(self) -> ArcticLLMServer:
        if self.server is None:
            raise RuntimeError("replica not initialised")
        return self.server

    @property
    def world_size(self) -> int:
        return self.wrapper._n_gpus("sampling")
