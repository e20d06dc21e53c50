"""Engine-shaped handles on jobs of a job server reached directly over HTTP (no hosted service in between).

``DSSTrainingClient(url).initialize(model, ds_config, training_config)`` returns a ``DSSTrainingEngine`` that stands
where a local DeepSpeed engine stands in a training script: ``loss = engine(**batch); engine.backward(loss);
engine.step()`` (the forward call only remembers the batch; ``backward`` runs forward + backward on the server and
returns the loss), plus ``save_checkpoint`` / ``load_checkpoint`` / ``destroy`` and the attributes trainers look at
(``module``, ``optimizer``, ``lr_scheduler``, ``global_steps``, ``is_gradient_accumulation_boundary``).
``ArcticInferenceClient(url).initialize(model_name, vllm_config)`` returns an ``ArcticInferenceEngine`` with
``generate`` / ``destroy``.  Tensors travel as DSSST1 frames.

Routes used (``arctic_platform_b200.common.http_server``): ``/initialize``, ``/forward-backward``, ``/forward``,
``/step``, ``/save``, ``/load-checkpoint``, ``/generate``, ``/destroy``.  Counterpart of
cortex-client/dss_client/{client,engine}.py in the reference.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from arctic_platform_b200 import wire

from .neutrino_client import JobType

OCTET = {"Content-Type": "application/octet-stream"}


class EngineError(RuntimeError):
    def __init__(self, message: str, status: Optional[int] = None):
        super().__init__(message)
        self.status = status


def loss_mask_from_labels(labels: torch.Tensor, shifted: bool, ignore_index: int = -100) -> torch.Tensor:
    """Which tokens of ``input_ids`` the loss is taken over.  With labels aligned to the inputs (``labels[t]`` is
    token ``t`` or the ignore index) that is ``labels != ignore_index``; with next-token labels (``labels[t]`` is the
    target predicted AT position ``t``, i.e. token ``t + 1``) the mask moves one column to the right."""
    keep = labels != ignore_index
    if not shifted:
        return keep
    out = torch.zeros_like(keep)
    out[:, 1:] = keep[:, :-1]
    return out


class _Http:
    """The few lines of HTTP both engines share; ``session`` is anything with ``post(url, **kw)`` (``requests``)."""

    def __init__(self, server_url: str, session=None, timeout: float = 3600.0):
        self.server_url = server_url.rstrip("/")
        if session is None:
            import requests
            session = requests.Session()
        self._session = session
        self._timeout = timeout

    def _post(self, route: str, *, params: Optional[dict] = None, json: Any = None, frame: Any = None) -> Any:
        kw: Dict[str, Any] = {"params": params, "timeout": self._timeout}
        if frame is not None:
            kw.update(data=wire.dumps(frame), headers=OCTET)
        elif json is not None:
            kw["json"] = json
        resp = self._session.post(f"{self.server_url}{route}", **kw)
        if resp.status_code >= 400:
            try:
                detail = resp.json().get("detail")
            except Exception:
                detail = getattr(resp, "text", "")
            raise EngineError(f"POST {route} -> {resp.status_code}: {detail}", resp.status_code)
        ctype = str(resp.headers.get("content-type", ""))
        return wire.loads(resp.content) if ctype.startswith("application/octet-stream") else resp.json()


class _LastLR:
    """The one method of a learning-rate scheduler that training loops read for logging."""

    def __init__(self) -> None:
        self.last_lr: List[float] = [float("nan")]

    def get_last_lr(self) -> List[float]:
        return list(self.last_lr)


class DSSTrainingEngine(torch.nn.Module):
    job_type = JobType.TRAINING

    def __init__(self, model: Any, ds_config: dict, training_config: Optional[dict], dss_server_url: str,
                 lr_scheduler: Any = None, session=None, loss_fn: str = "sft_ce", next_token_labels: bool = False,
                 num_devices: int = 1, checkpoint_path: Optional[str] = None):
        super().__init__()
        self.model_name = model if isinstance(model, str) else model.config.name_or_path
        self.__dict__["module"] = None if isinstance(model, str) else model     # kept for callers; not a submodule
        self.ds_config = ds_config
        self.training_config = training_config or {}
        self.optimizer = None
        self.training_dataloader = None
        self.lr_scheduler = lr_scheduler if lr_scheduler is not None else _LastLR()
        self.global_steps = 0
        self.loss_fn = loss_fn
        self.next_token_labels = next_token_labels
        self._pending: Optional[dict] = None
        self._http = _Http(dss_server_url, session)
        body = {"model_name": self.model_name, "job_type": self.job_type.value, "num_devices": num_devices,
                "ds_config": ds_config}
        if self.training_config:                   # an (even empty) training_config outranks ds_config on the server
            body["training_config"] = self.training_config
        if checkpoint_path:
            body["checkpoint_path"] = checkpoint_path
        self.job_id = self._http._post("/initialize", json=body)["job_id"]

    # ---- the DeepSpeed-engine call shape: engine(**batch) -> handle, engine.backward(handle) -> loss
    def forward(self, *args, **kwargs):
        if self._pending is not None:
            raise RuntimeError("forward() was called twice without backward() in between")
        if args:
            if len(args) != 1 or not isinstance(args[0], dict) or kwargs:
                raise TypeError("pass the batch as keyword tensors or as one dict")
            kwargs = args[0]
        self._pending = dict(kwargs)
        return self._pending

    def backward(self, *_args, **_kwargs) -> torch.Tensor:
        if self._pending is None:
            raise RuntimeError("backward() without a batch: call the engine with the batch first")
        batch, self._pending = self._pending, None
        return self.forward_backward(batch)

    def _server_batch(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        out = dict(batch)
        labels = out.get("labels")
        if torch.is_tensor(labels) and "loss_mask" not in out:
            out["loss_mask"] = loss_mask_from_labels(labels, self.next_token_labels)
        return out

    def forward_backward(self, batch: Dict[str, Any], meta: Optional[dict] = None) -> torch.Tensor:
        """Forward + backward of one batch on the server (gradients accumulate there); returns the loss."""
        out = self._http._post("/forward-backward", params={"job_id": self.job_id},
                               frame={"batch": self._server_batch(batch), "meta": meta or {},
                                      "processing": {"pre": [], "post": [], "loss_fn": self.loss_fn, "loss_kwargs": {}}})
        self.last_metrics = out.get("metrics", {})
        return torch.tensor(float(out["avg_loss"]))

    def evaluate(self, batch: Dict[str, Any], meta: Optional[dict] = None) -> dict:
        """Forward only: ``{"batch": {"log_probs": [B, S-1...]}, "metrics": ...}`` for the same batch layout."""
        return self._http._post("/forward", params={"job_id": self.job_id},
                                frame={"batch": self._server_batch(batch), "meta": {"plain_packing": True, **(meta or {})}})

    def step(self, learning_rate: Optional[float] = None) -> dict:
        if isinstance(learning_rate, (list, tuple)):
            raise ValueError("one learning rate for all parameter groups: pass a float")
        if learning_rate is not None and not isinstance(learning_rate, float):
            raise TypeError("learning_rate must be a float")
        out = self._http._post("/step", params={"job_id": self.job_id},
                               json={"learning_rate": learning_rate} if learning_rate is not None else {})
        metrics = out.get("metrics", {})
        self.global_steps = int(out.get("global_steps", self.global_steps + 1))
        if metrics.get("last_lr") is not None and isinstance(self.lr_scheduler, _LastLR):
            lr = metrics["last_lr"]
            self.lr_scheduler.last_lr = list(lr) if isinstance(lr, (list, tuple)) else [float(lr)]
        return metrics

    def is_gradient_accumulation_boundary(self) -> bool:
        return True        # the server applies what has accumulated whenever step() is called

    def save_checkpoint(self, path: Optional[str] = None, *_args, step: Optional[int] = None, export_hf: bool = False,
                        **_kwargs) -> dict:
        return self._http._post("/save", params={"job_id": self.job_id},
                                json={"path": path, "step": step if step is not None else self.global_steps,
                                      "export_hf": export_hf})

    def load_checkpoint(self, path: Optional[str] = None, *_args, step: Optional[int] = None, **_kwargs) -> dict:
        out = self._http._post("/load-checkpoint", params={"job_id": self.job_id}, json={"path": path, "step": step})
        self.global_steps = int(out.get("global_steps", self.global_steps))
        return out

    def destroy(self) -> Any:
        out = self._http._post("/destroy", params={"job_id": self.job_id})
        return out.get("destroyed", out)


class ArcticInferenceEngine:
    """A sampling job: ``generate(prompts, sampling_params)`` with token-id prompts, results prompt-major."""

    job_type = JobType.SAMPLING

    def __init__(self, server_url: str, model_name: str, vllm_config: Optional[dict] = None, session=None,
                 num_devices: int = 1, arctic_inference_config: Optional[dict] = None):
        self._http = _Http(server_url, session)
        body: Dict[str, Any] = {"model_name": model_name, "job_type": self.job_type.value, "num_devices": num_devices}
        if vllm_config is not None:
            body["vllm_config"] = vllm_config
        if arctic_inference_config is not None:
            body["arctic_inference_config"] = arctic_inference_config
        self.job_id = self._http._post("/initialize", json=body)["job_id"]

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[dict, List[Optional[dict]], None] = None) -> List[dict]:
        if isinstance(sampling_params, list):
            # one parameter set per prompt: equal sets travel together, results return in prompt order
            if len(sampling_params) != len(prompts):
                raise ValueError("a list of sampling_params needs one entry per prompt")
            out: List[Optional[List[dict]]] = [None] * len(prompts)
            groups: Dict[str, List[int]] = {}
            import json
            for i, sp in enumerate(sampling_params):
                groups.setdefault(json.dumps(sp or {}, sort_keys=True), []).append(i)
            for key, idx in groups.items():
                res = self.generate([prompts[i] for i in idx], json.loads(key))
                per = len(res) // len(idx)
                for j, i in enumerate(idx):
                    out[i] = [{**r, "prompt_index": i} for r in res[j * per:(j + 1) * per]]
            return [r for part in out for r in (part or [])]
        body = {"prompts": [list(map(int, p)) for p in prompts], "sampling_params": sampling_params or {}}
        return self._http._post("/generate", params={"job_id": self.job_id}, frame=body)["results"]

    def destroy(self) -> Any:
        out = self._http._post("/destroy", params={"job_id": self.job_id})
        return out.get("destroyed", out)


class DSSClient:
    def __init__(self, dss_server_url: str, session=None):
        self.dss_server_url = dss_server_url
        self._session = session


class DSSTrainingClient(DSSClient):
    def initialize(self, model: Any, ds_config: dict, training_config: Optional[dict] = None, lr_scheduler: Any = None,
                   **kw) -> DSSTrainingEngine:
        return DSSTrainingEngine(model, ds_config, training_config, self.dss_server_url, lr_scheduler,
                                 session=self._session, **kw)


class ArcticInferenceClient(DSSClient):
    def initialize(self, model_name: str, vllm_config: Optional[dict] = None, **kw) -> ArcticInferenceEngine:
        return ArcticInferenceEngine(self.dss_server_url, model_name, vllm_config, session=self._session, **kw)
