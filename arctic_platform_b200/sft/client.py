"""Supervised fine-tuning client: a thin synchronous facade over the unified RL client that defaults the
loss to next-token cross entropy (arctic_platform/sft/client.py:86-211 in the reference)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from ..client.client import SyncArcticRLClient
from .config import ArcticSFTClientConfig

SFT_PROCESSING = {"pre": [], "post": [], "loss_fn": "sft_ce", "loss_kwargs": {}}


class ArcticSFTClient:
    def __init__(self, config: ArcticSFTClientConfig, server_state: Any = None, transport=None):
        self.config = config
        self._rl = SyncArcticRLClient(config.to_rl_config(), server_state, transport)

    def fwd_bwd(self, batch: Dict[str, Any], processing: Optional[dict] = None) -> dict:
        return self._rl.fwd_bwd(batch, processing or SFT_PROCESSING)

    def fwd_no_grad(self, batch: Dict[str, Any]) -> dict:
        payload = batch if "batch" in batch else {"batch": batch}
        payload = {**payload, "meta": {**(payload.get("meta") or {}), "plain_packing": True}}
        return self._rl.fwd_no_grad(payload)

    def step(self, learning_rate: Optional[float] = None) -> dict:
        return self._rl.step(learning_rate)

    def save_checkpoint(self, path: Optional[str] = None, step: Optional[int] = None, export_hf: bool = False,
                        save_total_limit: Optional[int] = None) -> dict:
        return self._rl.save_checkpoint(path, step=step, export_hf=export_hf, save_total_limit=save_total_limit)

    def load_checkpoint(self, path: Optional[str] = None, step: Optional[int] = None) -> dict:
        return self._rl.load_checkpoint(path, step=step)

    def generate(self, prompts: List[Any], sampling_params: Optional[dict] = None) -> list:
        return self._rl.generate(prompts, sampling_params)

    def sync_weights(self, cuda_ipc=None, low_memory=None) -> dict:
        return self._rl.sync_weights(cuda_ipc, low_memory)

    def reset_prefix_cache(self) -> dict:
        return self._rl.reset_prefix_cache()

    def sleep_inference(self, level: int = 1) -> dict:
        return self._rl.sleep_inference(level)

    def wake_inference(self, tags=None) -> dict:
        return self._rl.wake_inference(tags)

    def sleep_training(self, mode: str = "all") -> dict:
        return self._rl.sleep_training(mode)

    def wake_training(self) -> dict:
        return self._rl.wake_training()

    def reconnect_config(self) -> ArcticSFTClientConfig:
        rc = self._rl.reconnect_config()
        return self.config.model_copy(update={"training_job_id": rc.training_job_id, "sampling_job_id": rc.sampling_job_id})

    def shutdown(self) -> None:
        self._rl.shutdown()

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.shutdown()


def create_arctic_sft_client(config: ArcticSFTClientConfig, server_state: Any = None) -> ArcticSFTClient:
    return ArcticSFTClient(config, server_state)
