"""SkyRL-side glue: the three callables a SkyRL trainer needs from a remote policy backend, built on the platform
client.  SkyRL keeps the generator / reward loop; this object scores and updates the policy and hands out the
inference endpoint.  (The reference ships shell launchers that point SkyRL at its server:
recipes/rl/skyrl/{simple_gsm8k,txt2sql,long_context_qa}.)

    backend = SkyRLArcticBackend(model="Qwen/Qwen3-1.7B", training_gpus=4, sampling_gpus=4, zorro=True)
    outs = backend.generate(prompt_token_ids, n=8, max_tokens=1024)
    metrics = backend.train_on_batch(input_ids, attention_mask, response_len, advantages)
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import torch

from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client


class SkyRLArcticBackend:
    def __init__(self, model: str, training_gpus: int = 1, sampling_gpus: int = 1, log_prob_gpus: int = 1,
                 colocate: bool = True, comm_protocol: str = "local", host: Optional[str] = None,
                 port: Optional[int] = None, lr: float = 1e-6, zero_stage: int = 3, zorro: bool = True,
                 max_model_len: int = 8192, loss_fn: str = "verl_grpo", kl_loss_coef: float = 0.001,
                 sampler_tp: int = 1, sequence_parallel: int = 1, offload_optimizer: bool = False):
        self.zorro = zorro
        self.loss_fn = loss_fn
        self.kl_loss_coef = kl_loss_coef
        self.client = create_arctic_rl_client(self.client_config(
            model, training_gpus, sampling_gpus, log_prob_gpus, colocate, comm_protocol, host, port, lr, zero_stage, zorro,
            max_model_len, sampler_tp, sequence_parallel, offload_optimizer))

    @staticmethod
    def client_config(model, training_gpus=1, sampling_gpus=1, log_prob_gpus=1, colocate=True, comm_protocol="local",
                      host=None, port=None, lr=1e-6, zero_stage=3, zorro=True, max_model_len=8192, sampler_tp=1,
                      sequence_parallel=1, offload_optimizer=False) -> ArcticRLClientConfig:
        """The platform configuration a launcher's flags stand for (kept apart so that it can be inspected without
        starting engines)."""
        zero: Dict[str, Any] = {"stage": zero_stage}
        if offload_optimizer:
            zero["offload_optimizer"] = {"device": "cpu", "pin_memory": True}
        worker: Dict[str, Any] = {"zorro_train": {"enable": zorro}}
        if sequence_parallel > 1:
            worker["sequence_parallel"] = int(sequence_parallel)
        vllm: Dict[str, Any] = {"max_model_len": max_model_len}
        if sampler_tp > 1:
            vllm["tensor_parallel_size"] = int(sampler_tp)
        kw = {"host": host, "port": port} if comm_protocol != "local" else {}
        return ArcticRLClientConfig(
            comm_protocol=comm_protocol, model_name=model, training_gpus=training_gpus, sampling_gpus=sampling_gpus,
            log_prob_gpus=log_prob_gpus, colocate=colocate,
            ds_config={"zero_optimization": zero, "gradient_clipping": 1.0, "optimizer": {"type": "AdamW", "params": {"lr": lr}}},
            ds_worker_config=worker, vllm_config=vllm, **kw)

    def generate(self, prompts: Sequence[Sequence[int]], n: int = 1, max_tokens: int = 1024, temperature: float = 1.0,
                 **extra) -> List[dict]:
        return self.client.call("generate", [list(p) for p in prompts],
                                {"n": n, "max_tokens": max_tokens, "temperature": temperature, **extra})

    def _meta(self, temperature: float) -> Dict[str, Any]:
        return {"zorro_train_enable": self.zorro, "temperature": temperature,
                "actor_config": {"use_kl_loss": self.kl_loss_coef > 0, "kl_loss_coef": self.kl_loss_coef,
                                 "kl_loss_type": "low_var_kl", "loss_agg_mode": "token-mean"}}

    def train_on_batch(self, input_ids: torch.Tensor, attention_mask: torch.Tensor, response_len: int,
                       advantages: torch.Tensor, temperature: float = 1.0, sync: bool = True) -> Dict[str, float]:
        batch = {"input_ids": input_ids, "attention_mask": attention_mask,
                 "response_mask": attention_mask[:, -response_len:].contiguous(), "advantages": advantages}
        meta = self._meta(temperature)
        batch["old_log_probs"] = self.client.call("fwd_no_grad", {"batch": batch, "meta": meta})["batch"]["log_probs"]
        if self.kl_loss_coef > 0:
            batch["ref_log_prob"] = self.client.call("fwd_no_grad", {"batch": batch, "meta": meta},
                                                     reference_model=True)["batch"]["log_probs"]
        out = self.client.call("fwd_bwd", {"batch": batch, "meta": meta}, {"loss_fn": self.loss_fn})
        st = self.client.call("step")
        if sync:
            self.client.call("sync_weights")
        return {**out["metrics"], **st["metrics"], "loss": out["avg_loss"]}

    def shutdown(self) -> None:
        self.client.call("shutdown")
