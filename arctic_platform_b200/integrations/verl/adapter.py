"""verl ``RemoteBackend`` adapter.

``ArcticRLClientWrapper`` turns verl's trainer calls into platform client calls:

* ``compute_log_prob`` / ``compute_ref_log_prob`` -> ``fwd_no_grad`` (policy / reference engine)
* ``update_actor``  -> for every PPO epoch and mini-batch: ``fwd_bwd`` then ``step`` (one optimizer step per
  mini-batch, like verl's own ``update_policy`` loop)
* ``generate``      -> sampling engine, token ids in and out
* ``update_weights``-> ``sync_weights``; ``wake_up_inference`` / ``sleep_inference`` / ``reset_prefix_cache``;
  ``save_checkpoint``; ``destroy``

The trainer config may be an OmegaConf tree, nested dicts or attribute objects (``cfg_get`` reads all three), so
the adapter and its tests do not need verl or Hydra installed.  Batches arrive either dense (left-padded prompt +
right-padded response) or jagged (``values`` + per-sample lengths); ``no_padding_to_padded_prompt_response``
rebuilds the dense wire format.  Counterpart of arctic_platform/integrations/verl/adapter.py:60-729.
"""
from __future__ import annotations

import math
from copy import deepcopy
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ...rl.client import create_arctic_rl_client
from ...rl.config import ArcticRLClientConfig
from ...rl.local_client import run_sync

_MISSING = object()


def cfg_get(cfg: Any, path: str, default: Any = _MISSING) -> Any:
    """``cfg_get(cfg, "actor_rollout_ref.rollout.n", 1)`` over dicts, OmegaConf nodes or attribute objects."""
    cur = cfg
    for key in path.split("."):
        if cur is None:
            break
        if isinstance(cur, dict):
            cur = cur.get(key, _MISSING)
        elif hasattr(cur, "get") and not hasattr(cur, key):
            cur = cur.get(key, _MISSING)
        else:
            cur = getattr(cur, key, _MISSING)
        if cur is _MISSING:
            break
    if cur is _MISSING or cur is None:
        if default is _MISSING:
            raise KeyError(f"config key '{path}' is missing")
        return default
    return cur


def _to_plain(node: Any) -> Any:
    try:
        from omegaconf import OmegaConf
        if OmegaConf.is_config(node):
            return OmegaConf.to_container(node, resolve=True)
    except Exception:
        pass
    return deepcopy(node)


def no_padding_to_padded_prompt_response(values: torch.Tensor, prompt_lens: torch.Tensor, response_lens: torch.Tensor,
                                         max_prompt_len: int = -1, max_response_len: int = -1, pad_value: int = 0
                                         ) -> Tuple[torch.Tensor, int, int]:
    """Jagged ``values`` (all samples' ``prompt || response`` tokens concatenated) -> ``[B, P + R]`` with the prompt
    left-padded and the response right-padded.  Vectorised (one scatter) instead of a Python loop per row."""
    prompt_lens, response_lens = prompt_lens.long(), response_lens.long()
    B = prompt_lens.numel()
    P = int(prompt_lens.max()) if max_prompt_len < 0 else max_prompt_len
    R = int(response_lens.max()) if max_response_len < 0 else max_response_len
    seq = prompt_lens + response_lens
    if int(seq.sum()) != values.shape[0]:
        raise ValueError(f"lengths sum to {int(seq.sum())} but {values.shape[0]} values were given")
    if int(prompt_lens.max()) > P or int(response_lens.max()) > R:
        raise ValueError("a sample is longer than the padded prompt / response length")
    row = torch.repeat_interleave(torch.arange(B), seq)
    start = seq.cumsum(0) - seq
    within = torch.arange(values.shape[0]) - start[row]
    col = within + (P - prompt_lens)[row]                       # prompt tokens end at column P, response starts there
    out = values.new_full((B, P + R) + tuple(values.shape[1:]), pad_value)
    out[row, col] = values
    return out, P, R


def prepare_padded_batch(data: Dict[str, Any], pad_token_id: int, drop_position_ids: bool = True) -> Tuple[Dict[str, torch.Tensor], int, int]:
    """Dense wire batch from a verl batch that is either already dense (``input_ids [B, S]``, ``responses [B, R]``)
    or jagged (``input_ids`` 1-D values with ``prompt_lens`` / ``response_lens``)."""
    ids = data["input_ids"]
    if getattr(ids, "is_nested", False) or (ids.dim() == 1 and "prompt_lens" not in data and "prompts" in data):
        # verl's padding-free layout: nested rows of prompt || response (or their flat values next to dense
        # prompts / responses + mask)
        from .nested import nested_to_padded, prompt_response_lengths
        pl, rl, P, R = prompt_response_lengths(data)
        out = {"input_ids": nested_to_padded(ids, pl, rl, P, R, pad_token_id)}
        mask = data.get("attention_mask")
        if mask is None or getattr(mask, "is_nested", False):
            vals = ids.values() if getattr(ids, "is_nested", False) else ids
            mask = nested_to_padded(torch.ones_like(vals), pl, rl, P, R, 0)
        out["attention_mask"] = mask
        if not drop_position_ids and "position_ids" in data:
            out["position_ids"] = nested_to_padded(data["position_ids"], pl, rl, P, R, 0)
        return out, P, R
    if ids.dim() == 2:
        R = data["responses"].shape[1] if "responses" in data else int(data["max_response_len"])
        out = {"input_ids": ids, "attention_mask": data["attention_mask"]}
        if not drop_position_ids and "position_ids" in data:
            out["position_ids"] = data["position_ids"]
        return out, ids.shape[1] - R, R
    pl, rl = data["prompt_lens"], data["response_lens"]
    dense, P, R = no_padding_to_padded_prompt_response(ids, pl, rl, int(data.get("max_prompt_len", -1)),
                                                       int(data.get("max_response_len", -1)), pad_token_id)
    mask, _, _ = no_padding_to_padded_prompt_response(torch.ones_like(ids), pl, rl, P, R, 0)
    out = {"input_ids": dense, "attention_mask": mask}
    if not drop_position_ids and "position_ids" in data:
        out["position_ids"], _, _ = no_padding_to_padded_prompt_response(data["position_ids"], pl, rl, P, R, 0)
    return out, P, R


class ArcticRLClientWrapper:
    """verl-facing facade over the platform client."""

    backend_name = "arctic"

    def __init__(self, config: Any, client=None, handle: Optional[dict] = None, pad_token_id: int = 0):
        self.config = config
        self._backend = cfg_get(config, "remote_backend", {})
        self.pad_token_id = pad_token_id
        self.rollout_n = int(cfg_get(config, "actor_rollout_ref.rollout.n", 1))
        self.temperature = float(cfg_get(config, "actor_rollout_ref.rollout.temperature", 1.0))
        self.ppo_epochs = int(cfg_get(config, "actor_rollout_ref.actor.ppo_epochs", 1))
        self.global_steps = 0
        self.client_config = self._client_config(handle)
        self.client = client if client is not None else create_arctic_rl_client(self.client_config)

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_config(cls, main_config: Any, handle: Optional[dict] = None, **kw) -> "ArcticRLClientWrapper":
        return cls(main_config, handle=handle, **kw)

    def reconnect_handle(self) -> dict:
        """Picklable description another process can pass as ``handle=`` to attach to the same jobs."""
        rc = self.client.reconnect_config()
        return {"client_config": rc.model_dump(), "job_ids": dict(self.client.job_ids)}

    @property
    def requires_single_forwarder(self) -> bool:
        """The server fans a batch out to its own ranks, so exactly one verl worker forwards calls."""
        return True

    def _n_gpus(self, kind: str) -> int:
        return int(cfg_get(self._backend, f"{kind}_gpus", 1 if kind != "log_prob" else 0))

    def _create_ds_config(self, n_gpus: int, training: bool = True) -> Dict[str, Any]:
        """Batch sizing per OPTIMIZER step: ``train_batch_size = ppo_mini_batch_size * rollout_n`` and
        ``gradient_accumulation_steps = train_batch_size / (micro_batch * n_gpus)``; everything else in
        ``remote_backend.train.deepspeed`` passes through."""
        ds = _to_plain(cfg_get(self._backend, "train.deepspeed", {})) or {}
        micro = int(cfg_get(self.config, "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu", 1) or 1)
        mini = int(cfg_get(self.config, "actor_rollout_ref.actor.ppo_mini_batch_size", 1))
        data_bs = int(cfg_get(self.config, "data.train_batch_size", mini))
        if (data_bs * self.rollout_n) % (mini * self.rollout_n):
            raise ValueError(f"data.train_batch_size ({data_bs}) must be divisible by actor.ppo_mini_batch_size ({mini})")
        train_bs = mini * self.rollout_n
        ds.update({"train_micro_batch_size_per_gpu": micro, "train_batch_size": train_bs,
                   "gradient_accumulation_steps": max(1, train_bs // (micro * max(1, n_gpus))),
                   "sequence_parallel_size": int(cfg_get(self.config, "actor_rollout_ref.actor.fsdp_config.ulysses_sequence_parallel_size", 1))})
        lr = cfg_get(self.config, "actor_rollout_ref.actor.optim.lr", None)
        if lr is not None:
            ds.setdefault("optimizer", {}).setdefault("params", {}).setdefault("lr", float(lr))
        clip = cfg_get(self.config, "actor_rollout_ref.actor.grad_clip", None)
        if clip is not None:
            ds.setdefault("gradient_clipping", float(clip))
        if not training:
            ds.pop("data_types", None)
            ds.pop("optimizer", None)
        return ds

    def _create_ds_worker_config(self) -> Dict[str, Any]:
        z = cfg_get(self._backend, "train.zorro_train", {}) or {}
        wc = {"gradient_checkpointing": bool(cfg_get(self.config, "actor_rollout_ref.model.enable_gradient_checkpointing", True)),
              "zorro_train": {"enable": bool(cfg_get(z, "enable", False)),
                              "max_rollouts": int(cfg_get(z, "max_rollouts", self.rollout_n))},
              "logits_optimization": cfg_get(self._backend, "train.logits.optimization", "none"),
              "load_balancer": bool(cfg_get(self._backend, "train.load_balancer", True))}
        return wc

    def _client_config(self, handle: Optional[dict]) -> ArcticRLClientConfig:
        if handle is not None:
            cc = ArcticRLClientConfig(**handle["client_config"])
            ids = handle.get("job_ids", {})
            cc.training_job_id, cc.sampling_job_id, cc.log_prob_job_id = ids.get("training"), ids.get("sampling"), ids.get("log_prob")
            return cc
        n_train, n_lp = self._n_gpus("training"), self._n_gpus("log_prob")
        rollout = cfg_get(self.config, "actor_rollout_ref.rollout", {})
        vllm = {"max_model_len": int(cfg_get(rollout, "max_model_len", 0)) or
                (int(cfg_get(self.config, "data.max_prompt_length", 1024)) + int(cfg_get(self.config, "data.max_response_length", 1024))),
                "gpu_memory_utilization": float(cfg_get(rollout, "gpu_memory_utilization", 0.5)),
                "tensor_parallel_size": int(cfg_get(self._backend, "sampling_tp_size", 1))}
        return ArcticRLClientConfig(
            comm_protocol=cfg_get(self._backend, "comm_protocol", "local"),
            host=cfg_get(self._backend, "host", None), port=cfg_get(self._backend, "port", None),
            model_name=cfg_get(self.config, "actor_rollout_ref.model.path"),
            ds_config=self._create_ds_config(n_train, True),
            log_prob_ds_config=self._create_ds_config(max(1, n_lp), False) if n_lp > 0 else None,
            ds_worker_config=self._create_ds_worker_config(), vllm_config=vllm,
            training_gpus=n_train, sampling_gpus=self._n_gpus("sampling"), log_prob_gpus=n_lp,
            log_prob_engine="deepspeed", colocate=bool(cfg_get(self._backend, "colocate", True)),
            cuda_ipc=bool(cfg_get(self._backend, "weight_sync.cuda_ipc", False)),
            low_memory=bool(cfg_get(self._backend, "weight_sync.low_memory", False)),
            checkpoint_path=cfg_get(self.config, "trainer.default_local_dir", None),
            seed=int(cfg_get(self.config, "trainer.seed", 42)))

    # ------------------------------------------------------------------ calls
    def _meta(self, extra: Optional[dict] = None) -> Dict[str, Any]:
        wc = self.client_config.ds_worker_config or {}
        meta = {"temperature": self.temperature, "zorro_train_enable": bool(wc.get("zorro_train", {}).get("enable", False)),
                "zorro_train_max_rollouts": int(wc.get("zorro_train", {}).get("max_rollouts", self.rollout_n)),
                "load_balancer": bool(wc.get("load_balancer", True)), "global_steps": self.global_steps}
        meta.update(extra or {})
        return meta

    def _call(self, name: str, *args, **kwargs):
        return self.client.call(name, *args, **kwargs) if hasattr(self.client, "call") else run_sync(getattr(self.client, name)(*args, **kwargs))

    def compute_log_prob(self, data: Dict[str, Any], calculate_entropy: bool = False) -> Dict[str, torch.Tensor]:
        batch, _, R = prepare_padded_batch(data, self.pad_token_id)
        out = self._call("fwd_no_grad", {"batch": batch, "meta": self._meta({"response_length": R, "calculate_entropy": calculate_entropy})})
        res = {"old_log_probs": out["batch"]["log_probs"]}
        if calculate_entropy and "entropy" in out["batch"]:
            res["entropys"] = out["batch"]["entropy"]
        return res

    def compute_ref_log_prob(self, data: Dict[str, Any]) -> Dict[str, torch.Tensor]:
        batch, _, R = prepare_padded_batch(data, self.pad_token_id)
        out = self._call("fwd_no_grad", {"batch": batch, "meta": self._meta({"response_length": R})}, reference_model=True)
        return {"ref_log_prob": out["batch"]["log_probs"]}

    def update_actor(self, data: Dict[str, Any]) -> Dict[str, float]:
        """``ppo_epochs`` passes over the batch, each cut into mini-batches of ``ppo_mini_batch_size * rollout_n``
        samples (whole prompt groups stay together); one ``fwd_bwd`` + ``step`` per mini-batch.  Returns the reduced
        metrics (see ``update_actor_detailed`` for the loss and the token counts as well)."""
        return self.update_actor_detailed(data)["metrics"]

    # how a metric is folded over the mini-batches of one update; everything else is averaged
    METRIC_REDUCTION = {"actor/pg_clipfrac_lower": "mean", "actor/pg_clipfrac": "mean", "actor/pg_loss": "mean",
                        "actor/ppo_kl": "mean", "grad_norm": "mean", "kl_coef": "mean", "kl_loss": "mean",
                        "perf/max_memory_allocated_gb": "max", "global_tokens": "sum"}

    @staticmethod
    def _plain(obj: Any) -> Dict[str, Any]:
        """A config object as JSON-safe dict (values that do not serialise become None)."""
        import json
        if obj is None:
            return {}
        src = _to_plain(obj) if not hasattr(obj, "__dict__") or isinstance(obj, dict) else vars(obj)
        return json.loads(json.dumps(src, default=lambda o: None))

    def update_actor_detailed(self, data: Dict[str, Any]) -> Dict[str, Any]:
        """The update with everything verl's trainer reads back: ``{"loss", "metrics", "global_token_num"}``
        (arctic_platform/integrations/verl/adapter.py:268-397).  Per mini-batch the meta carries the global batch
        size of one optimizer step, the number of loss tokens in the chunk, the chunk's slice of the rollout
        importance weights, and the actor / policy-loss sections of the config."""
        batch, P, R = prepare_padded_batch(data, self.pad_token_id)
        for k in ("advantages", "old_log_probs", "ref_log_prob", "response_mask", "rollout_log_probs"):
            if k in data:
                batch[k] = data[k]
        batch.setdefault("response_mask", batch["attention_mask"][:, -R:])
        B = batch["input_ids"].shape[0]
        per_step = int(cfg_get(self.config, "actor_rollout_ref.actor.ppo_mini_batch_size",
                               max(1, B // self.rollout_n))) * self.rollout_n
        mini = max(1, min(per_step, B))
        n_mini = math.ceil(B / mini)
        actor_cfg = cfg_get(self.config, "actor_rollout_ref.actor", None)
        shared_meta = {"response_length": R, "max_prompt_len": P, "max_response_len": R, "rollout_n": self.rollout_n,
                       "pad_token_id": self.pad_token_id,
                       "calculate_entropy": bool(cfg_get(self.config, "actor_rollout_ref.actor.calculate_entropy", False)),
                       "max_token_len_per_gpu": cfg_get(self.config, "actor_rollout_ref.actor.ppo_max_token_len_per_gpu", None),
                       "actor_config": self._plain(actor_cfg),
                       "policy_loss_config": self._plain(cfg_get(self.config, "actor_rollout_ref.actor.policy_loss", None))}
        is_w = data.get("rollout_is_weights")
        token_counts = batch["attention_mask"].sum(-1).tolist()
        series: Dict[str, List[float]] = {}
        losses: List[float] = []
        last_lr = None
        for _epoch in range(self.ppo_epochs):
            for i in range(n_mini):
                sl = slice(i * mini, min(B, (i + 1) * mini))
                mb = {k: v[sl] for k, v in batch.items()}
                meta = self._meta({**shared_meta, "global_batch_size": per_step,
                                   "batch_num_tokens": int(mb["response_mask"].sum()),
                                   "rollout_is_weights": is_w[sl] if isinstance(is_w, torch.Tensor) else is_w})
                out = self._call("fwd_bwd", {"batch": mb, "meta": meta})
                st = self._call("step")
                merged = {**out.get("metrics", {}), **st.get("metrics", {})}
                if isinstance(out.get("avg_loss"), (int, float)):
                    losses.append(float(out["avg_loss"]))
                elif isinstance(merged.get("loss"), (int, float)):
                    losses.append(float(merged["loss"]))
                if isinstance(merged.get("last_lr"), (int, float)):
                    last_lr = float(merged["last_lr"])
                for k, v in merged.items():
                    if k not in ("loss",) and isinstance(v, (int, float)):
                        series.setdefault(k, []).append(float(v))
        self.global_steps += 1
        fold = {"mean": lambda v: sum(v) / len(v), "max": max, "min": min, "sum": sum}
        metrics = {k: fold[self.METRIC_REDUCTION.get(k, "mean")](v) for k, v in series.items()}
        if last_lr is not None:
            metrics["lr"] = last_lr
        loss = sum(losses) / len(losses) if losses else float("nan")
        return {"loss": loss, "metrics": metrics, "global_token_num": token_counts}

    def generate(self, prompt_ids: Sequence[Sequence[int]], sampling_params: Optional[dict] = None, routing_key=None) -> List[dict]:
        sp = {"temperature": self.temperature, "n": 1,
              "max_tokens": int(cfg_get(self.config, "data.max_response_length", 1024))}
        sp.update(sampling_params or {})
        return self._call("generate", [list(map(int, p)) for p in prompt_ids], sp)

    def update_weights(self) -> Dict[str, Any]:
        return self._call("sync_weights")

    def save_checkpoint(self, path: Optional[str] = None, step: Optional[int] = None) -> Dict[str, Any]:
        return self._call("save_checkpoint", path, self.global_steps if step is None else step)

    def wake_up_inference(self, tags: Optional[List[str]] = None):
        return self._call("wake_inference", tags)

    def sleep_inference(self, level: int = 1):
        return self._call("sleep_inference", level)

    def reset_prefix_cache(self):
        return self._call("reset_prefix_cache")

    def get_server_state(self):
        return self.client.get_server_state()

    def destroy(self) -> None:
        self._call("shutdown")
