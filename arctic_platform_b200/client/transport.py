"""Transport abstraction of the unified client: the client lowers every public method to a canonical
``Request(op, job_id, body, binary)``; a transport only delivers it (arctic_platform/client/transport.py:36-148)."""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

from .config import JOB_TYPES, ArcticRLClientConfig

JOB_CREATE_ORDER = ("sampling", "log_prob", "training")

OPS = frozenset({"forward-backward", "forward", "step", "save", "load-checkpoint", "generate", "log-probs",
                 "operation", "sleep-inference", "wake-inference", "sleep-training", "wake-training"})


def method_name(op: str) -> str:
    return op.replace("-", "_")


def unresolved_ops(target: object) -> list:
    """Ops of ``OPS`` for which ``target`` has no method -- lets a transport check its coverage up front."""
    return sorted(op for op in OPS if not hasattr(target, method_name(op)))


@dataclass
class JobHandles:
    training: Optional[Any] = None
    sampling: Optional[Any] = None
    log_prob: Optional[Any] = None

    @classmethod
    def from_config(cls, config: ArcticRLClientConfig) -> "JobHandles":
        return cls(config.training_job_id, config.sampling_job_id, config.log_prob_job_id)

    @property
    def any_set(self) -> bool:
        return any(getattr(self, jt) is not None for jt in JOB_TYPES)

    def set(self, job_type: str, job_id: Any) -> None:
        setattr(self, job_type, job_id)

    def require(self, job_type: str) -> Any:
        job_id = getattr(self, job_type)
        if job_id is None:
            raise ValueError(f"No {job_type} job initialized.")
        return job_id


@dataclass
class Request:
    op: str
    job_id: Optional[Any] = None
    body: Dict[str, Any] = field(default_factory=dict)
    binary: bool = False


class Transport(ABC):
    jobs: JobHandles

    @abstractmethod
    def initialize(self) -> JobHandles: ...

    @abstractmethod
    def call(self, request: Request) -> dict: ...

    @abstractmethod
    async def acall(self, request: Request) -> dict: ...

    async def aclose(self) -> None:
        return None

    @abstractmethod
    def shutdown(self) -> None: ...


def initialize_or_cleanup(transport: Transport) -> JobHandles:
    """``initialize()``; on failure ``shutdown()`` first so a launched server is not orphaned, then re-raise."""
    try:
        return transport.initialize()
    except Exception:
        try:
            transport.shutdown()
        except Exception:
            pass
        raise
