"""CPU forwarder worker for verl.

verl schedules "workers" and dispatches trainer calls to them; with a remote backend the worker owns no GPU and
no model -- it forwards each call to the platform through ``ArcticRLClientWrapper`` and reports throughput
numbers (tokens/s, model FLOPs utilisation) the trainer logs.  ``dispatch`` records the dispatch mode verl
should use for a method (one forwarder receives the whole batch); with verl installed ``register.py`` maps these
to verl's own decorators.  Counterpart of arctic_platform/integrations/verl/worker.py:78-291.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, Optional

import torch

from .adapter import ArcticRLClientWrapper, cfg_get


def dispatch(mode: str = "ONE_TO_ALL", blocking: bool = True) -> Callable:
    def deco(fn):
        fn._dispatch = {"mode": mode, "blocking": blocking}
        return fn
    return deco


def estimate_flops_per_token(cfg, seq_len: int) -> float:
    """Training FLOPs per token (forward + backward = 3 x forward) of a dense or MoE decoder: 2 FLOPs per active
    matmul parameter per token plus causal attention ``2 * 2 * L * q_size * S / 2``."""
    H, L = cfg.hidden_size, cfg.num_layers
    attn_proj = H * cfg.qkv_size + cfg.q_size * H
    if getattr(cfg, "is_moe", False):
        mlp = 3 * H * cfg.moe_intermediate_size * cfg.num_experts_per_tok + H * cfg.num_experts
    else:
        mlp = 3 * H * cfg.intermediate_size
    dense = L * (attn_proj + mlp) + H * cfg.vocab_size
    attn = L * 2 * cfg.q_size * seq_len                          # QK^T and PV, causal half
    return 3.0 * (2.0 * dense + attn)


class ArcticRLActorRolloutRefWorker:
    def __init__(self, config: Any, role: str = "actor_rollout_ref", wrapper: Optional[ArcticRLClientWrapper] = None,
                 handle: Optional[dict] = None, peak_tflops: float = 0.0):
        self.config = config
        self.role = role
        self.wrapper = wrapper
        self._handle = handle
        self.peak_tflops = peak_tflops
        self._model_cfg = None

    @dispatch("ONE_TO_ALL")
    def init_model(self) -> None:
        if self.wrapper is None:
            self.wrapper = ArcticRLClientWrapper.from_config(self.config, handle=self._handle)
        try:
            from ...models.config import resolve_config
            self._model_cfg = resolve_config(cfg_get(self.config, "actor_rollout_ref.model.path"))
        except Exception:
            self._model_cfg = None

    def _throughput(self, data: Dict[str, Any], seconds: float, training: bool) -> Dict[str, float]:
        mask = data.get("attention_mask")
        ids = data["input_ids"]
        if getattr(ids, "is_nested", False):
            ids = ids.values().reshape(1, -1)             # padding-free: every stored token is a real token
            mask = None
            data = {**data, "input_ids": ids}
        tokens = float(mask.sum()) if torch.is_tensor(mask) and not mask.is_nested and mask.dim() == 2 else float(ids.numel())
        out = {"perf/tokens_per_s": tokens / max(seconds, 1e-9), "perf/seconds": seconds}
        if self._model_cfg is not None:
            seq = tokens / max(1, data["input_ids"].shape[0]) if data["input_ids"].dim() == 2 else tokens
            f = estimate_flops_per_token(self._model_cfg, int(seq)) * tokens * (1.0 if training else 1.0 / 3.0)
            out["perf/tflops"] = f / seconds / 1e12
            n = max(1, self.wrapper._n_gpus("training"))
            if self.peak_tflops > 0:
                out["perf/mfu"] = out["perf/tflops"] / (self.peak_tflops * n)
        return out

    @staticmethod
    def _nested_like_input(data: Dict[str, Any], out: Dict[str, Any]) -> Dict[str, Any]:
        """A padding-free batch (nested ``input_ids``) gets its per-token outputs back in the same layout: nested rows
        of ``prompt + response`` positions, each value stored on the token that predicts it.  The grids come back
        aligned with the response tokens, which is what both training modes of the platform produce."""
        from .nested import is_nested, make_njt
        if not is_nested(data.get("input_ids")):
            return out
        return {k: (make_njt(data, v, "predict_next") if torch.is_tensor(v) and v.dim() == 2 else v) for k, v in out.items()}

    @dispatch("ONE_TO_ALL")
    def compute_log_prob(self, data: Dict[str, Any]) -> Dict[str, Any]:
        t0 = time.perf_counter()
        out = self.wrapper.compute_log_prob(data, calculate_entropy=bool(data.get("calculate_entropy", False)))
        out = self._nested_like_input(data, out)
        out["metrics"] = self._throughput(data, time.perf_counter() - t0, training=False)
        return out

    @dispatch("ONE_TO_ALL")
    def compute_ref_log_prob(self, data: Dict[str, Any]) -> Dict[str, Any]:
        return self._nested_like_input(data, self.wrapper.compute_ref_log_prob(data))

    # calls verl makes on every worker that mean nothing for a forwarder: the platform owns device placement, the loss
    # function travels with each call, and engine state lives on the server
    @dispatch("ONE_TO_ALL")
    def to(self, device=None, model: bool = True, optimizer: bool = True, grad: bool = True) -> None:
        return None

    @dispatch("ONE_TO_ALL")
    def set_loss_fn(self, loss_fn=None) -> None:
        return None

    @dispatch("ONE_TO_ALL")
    def reset(self) -> None:
        return None

    @dispatch("ONE_TO_ALL", blocking=False)
    def sleep_replicas(self) -> None:
        return None

    @dispatch("ONE_TO_ALL")
    def destroy(self) -> None:
        if self.wrapper is not None:
            self.wrapper.destroy()
            self.wrapper = None

    @dispatch("ONE_TO_ALL")
    def update_actor(self, data: Dict[str, Any]) -> Dict[str, Any]:
        t0 = time.perf_counter()
        metrics = self.wrapper.update_actor(data)
        metrics.update(self._throughput(data, time.perf_counter() - t0, training=True))
        return {"metrics": metrics}

    @dispatch("ONE_TO_ALL")
    def update_weights(self):
        return self.wrapper.update_weights()

    @dispatch("ONE_TO_ALL")
    def save_checkpoint(self, local_path: Optional[str] = None, global_step: Optional[int] = None, **_):
        return self.wrapper.save_checkpoint(local_path, global_step)

    @dispatch("ONE_TO_ALL")
    def load_checkpoint(self, local_path: Optional[str] = None, global_step: Optional[int] = None, **_):
        return self.wrapper._call("load_checkpoint", local_path, global_step)

    def reconnect_handle(self) -> dict:
        return self.wrapper.reconnect_handle()
