"""Per-GPU engine worker: the object a server drives for one rank of a job.

It plays the role of the reference's ``DeepSpeedWorker`` Ray actor
(arctic_platform/common/deepspeed_worker.py:107-1135) for ``training`` and ``log_prob`` jobs and of an
ArcticInference replica for ``sampling`` jobs, with the same method names and return shapes
(``{"metrics", "avg_loss", "batch"}`` for forward passes, ``{"metrics": {"last_lr", "grad_norm"}, "batch": {}}``
for ``step``).  One process owns one GPU; data-parallel ranks are peers of one ``torch.distributed`` group and
meet inside ``TrainEngine.step`` (fused NVLink kernels) -- the server only fans requests out.
"""
from __future__ import annotations

import contextlib
import os
import time
import logging
from typing import Any, Dict, Iterable, List, Optional

import torch

from ..common.utils.batch import log_dp_shard_tokens
from ..common.utils.metrics import combine_metric_microbatches
from ..utils import sft_profile
from ..models.config import DecoderConfig, resolve_config
from ..models.decoder import DecoderLM
from ..rl.processors.pipeline import run_pipeline
from .trainer import EngineConfig, TrainEngine

logger = logging.getLogger(__name__)


def split_microbatches(batch: Dict[str, torch.Tensor], n: int) -> List[Dict[str, torch.Tensor]]:
    """Splits every tensor of the batch along dim 0 into ``n`` chunks (``torch.chunk`` semantics)."""
    if n <= 1:
        return [batch]
    outs: List[Dict[str, Any]] = [dict() for _ in range(n)]
    for k, v in batch.items():
        if torch.is_tensor(v) and v.dim() > 0:
            parts = torch.chunk(v, n, dim=0)
            if len(parts) != n:
                raise ValueError(f"cannot split {k} with {v.shape[0]} rows into {n} micro-batches")
            for o, p in zip(outs, parts):
                o[k] = p
        else:
            for o in outs:
                o[k] = v
    return outs


class _ScoringView:
    """What the forward-only pipeline needs of an engine -- the model -- for a log-prob job that is served by a
    sampler's engine (``log_prob_engine = vllm``): no optimizer state, no gradient buffers."""

    def __init__(self, model):
        self.model = model

    def backward(self, _loss):
        raise RuntimeError("a log-prob job on the sampler's engine cannot train")


def _loss_free_row(batch: Dict[str, Any]) -> Dict[str, Any]:
    """One row of ``batch`` that contributes nothing to the loss (masks and labels cleared), marked ``_dummy`` so that
    its outputs are dropped: a filler pass that keeps a rank in step with its peers' collectives."""
    B = batch["input_ids"].shape[0]
    row = {k: (v[:1].clone() if torch.is_tensor(v) and v.dim() > 0 and v.shape[0] == B else v) for k, v in batch.items()}
    for k in ("response_mask", "loss_mask"):
        if k in row:
            row[k] = torch.zeros_like(row[k])
    if "labels" in row:
        row["labels"] = torch.full_like(row["labels"], -100)
    row["_dummy"] = True
    return row


# the process group a worker of this process created from the launcher's environment, and how many workers use it
_PG = {"created_here": False, "users": 0}


class EngineWorker:
    def __init__(self, device=None):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if device is None:
            # one process per GPU: the launcher (torchrun, the job server's spawned actors) names it in LOCAL_RANK
            device = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.job_type: Optional[str] = None
        self.engine: Optional[TrainEngine] = None
        self.sampler = None
        self.model_cfg: Optional[DecoderConfig] = None
        self.job_config: Dict[str, Any] = {}
        self.activation_offload = None
        self.sp = 1
        self.tp = 1                      # ranks per sampling replica (tensor parallelism)
        self._nvtx = os.environ.get("APB_NVTX", "0") == "1"

    # ------------------------------------------------------------------ lifecycle
    def initialize(self, job_config: Dict[str, Any], model: Optional[DecoderLM] = None) -> bool:
        """``job_config`` has the fields of the server-side ``JobConfig`` (model_name, job_type, ds_config,
        training_config, log_prob_config, ds_worker_config, vllm_config, seed, ...)."""
        self.job_config = dict(job_config)
        self.job_type = job_config.get("job_type", "training")
        seed = job_config.get("seed")
        seed = 42 if seed is None else int(seed)
        if job_config.get("full_determinism"):
            from ..utils.debug import enable_full_determinism
            enable_full_determinism(seed)
        self.model_cfg = model.cfg if model is not None else resolve_config(job_config["model_name"])
        dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        # strict schema, as the reference's loader: a misspelt option is an error, not a silent default
        from ..models.loader_options import LoaderOptions
        raw_lo = (job_config.get("ds_worker_config") or {}).get("loader_options") or {}
        self.loader_options = lo = LoaderOptions.from_dict(raw_lo)
        if "optimization_dtype" in raw_lo:
            if self.device.type == "cuda" and lo.optimization_dtype != "bfloat16":
                raise ValueError("loader_options.optimization_dtype='float32': the GPU kernels compute in bf16 with fp32 "
                                 "master weights and fp32 accumulation")
            if self.device.type != "cuda":
                dtype = getattr(torch, lo.optimization_dtype)
        if lo.debug is not None and model is None:
            if lo.debug.num_layers is not None:
                import dataclasses
                n = int(lo.debug.num_layers)
                lt = self.model_cfg.layer_types
                self.model_cfg = dataclasses.replace(self.model_cfg, num_layers=n,
                                                     layer_types=None if lt is None else tuple(lt[:n]))
            if lo.debug.deterministic_algorithms:
                torch.use_deterministic_algorithms(True, warn_only=True)
        tp = int((job_config.get("vllm_config") or {}).get("tensor_parallel_size", 1) or 1) \
            if self.job_type == "sampling" else 1
        if self.job_type != "sampling" or tp > 1:
            self._ensure_process_group(job_config)
        if self.job_type == "sampling" and tp > 1:
            return self._initialize_tp_sampler(job_config, model, tp, dtype, seed)
        scorer = (self.job_type == "log_prob" and job_config.get("log_prob_engine") == "vllm"
                  and self.world == 1 and self.model_cfg.layer_types is None)
        if self.job_type == "sampling" or scorer:
            from .sampler import SamplerEngine
            vc = dict(job_config.get("vllm_config") or {})
            m = model if model is not None else self._load_model(job_config, dtype, seed)
            if self.model_cfg.layer_types is not None:
                # hybrid family: recurrent state + sparse K/V layers, served by the stateful tensor-op engine
                from .hybrid_sampler import HybridSampler as SamplerEngine      # noqa: F811
            elif vc.get("enable_return_routed_experts") and self.model_cfg.is_moe:
                # rollout routing replay: the tensor-op engine records the experts chosen for every fed token
                from .hybrid_sampler import HybridSampler as SamplerEngine      # noqa: F811
            elif self.device.type != "cuda":
                from .reference_sampler import ReferenceSampler as SamplerEngine   # noqa: F811  (CPU: recompute sampler)
            spec = self._speculative_setup(job_config, vc, dtype, seed) if not scorer else None
            if spec is not None:
                from .speculative import SpeculativeSampler
                self.sampler = SpeculativeSampler(self.model_cfg, self.device, model=m, draft_model=spec["draft"],
                                                  num_speculative_tokens=spec["k"],
                                                  max_seq_len=int(vc.get("max_model_len", 8192)), seed=seed,
                                                  eos_token_id=vc.get("eos_token_id"))
                return True
            if scorer:
                # a log-prob job on the sampler's engine: it only scores (teacher-forced passes), so a token of KV
                # cache is enough; it receives weights like a sampler does
                vc.setdefault("kv_cache_tokens", 1024)
                vc.setdefault("max_num_seqs", 8)
            self.sampler = SamplerEngine(
                self.model_cfg, self.device, model=m,
                kv_cache_tokens=int(vc.get("kv_cache_tokens", 1 << 20)), max_batch=int(vc.get("max_num_seqs", 256)),
                max_seq_len=int(vc.get("max_model_len", 8192)),
                cascade=bool((job_config.get("arctic_inference_config") or {}).get("zorro_inference", {}).get("enable", True)),
                seed=seed, eos_token_id=vc.get("eos_token_id"), quantization=vc.get("quantization"))
            if vc.get("enable_return_routed_experts"):
                self.sampler.always_return_routing = True
            return True
        m = model if model is not None else self._load_model(job_config, dtype, seed)
        ep = int((job_config.get("ds_worker_config") or {}).get("expert_parallel", 1) or 1)
        if ep > 1 and m.cfg.is_moe:
            # experts sharded over the ranks of the job; tokens travel to their experts and back (peer memory on
            # GPUs, all_to_all on CPU); expert parameters become rank-local units of the engine
            from ..parallel.expert_parallel import attach_expert_parallel
            if ep != self.world:
                raise ValueError(f"expert_parallel={ep} must equal the number of ranks of the job ({self.world})")
            attach_expert_parallel(m, ep, impl="fused" if self.device.type == "cuda" else "collective")
        if self.job_type == "log_prob":
            ecfg = EngineConfig.from_ds_config(job_config.get("log_prob_config") or job_config.get("ds_config"))
            self.engine = TrainEngine(m, ecfg, forward_only=True)
            self._setup_sequence_parallel(m, int((job_config.get("ds_worker_config") or {}).get("sequence_parallel", 1) or 1))
        else:
            ecfg = EngineConfig.from_ds_config(job_config.get("ds_config"), job_config.get("training_config"))
            wc = job_config.get("ds_worker_config") or {}
            gc_cfg = wc.get("gradient_checkpointing", False)
            # the reference's spelling: training_config.ac_config = {mode, freq, targets, offload_config: {enabled,
            # keep_last_n, tensor_size_threshold}} (arctic_platform/model/implementations/qwen35/config.py:33-52)
            # It travels in ds_worker_config.loader_options (validated above) or in training_config.
            ac = lo.ac_config
            if ac is None and isinstance((job_config.get("training_config") or {}).get("ac_config"), dict):
                from ..models.loader_options import ActivationCheckpointOptions, _strict
                ac = _strict(ActivationCheckpointOptions, job_config["training_config"]["ac_config"], "training_config.ac_config")
            if ac is not None:
                gc_cfg, ao_cfg = ac.to_worker_dicts()
                if ao_cfg is not None:
                    wc = {**wc, "activation_offload": ao_cfg}
            if lo.tiled_mlp_token_chunk_size is not None and not wc.get("tiled_mlp"):
                wc = {**wc, "tiled_mlp": f"chunk:{int(lo.tiled_mlp_token_chunk_size)}"}
            ecfg.gradient_checkpointing = bool(gc_cfg.get("enable", True)) if isinstance(gc_cfg, dict) else bool(gc_cfg)
            if isinstance(gc_cfg, dict) and ecfg.gradient_checkpointing:
                m.set_activation_checkpointing(gc_cfg.get("mode", "full"), gc_cfg.get("targets"), int(gc_cfg.get("freq", 1) or 1))
            from ..models.factory import _tiled_mlp_setting
            shards = _tiled_mlp_setting(wc.get("tiled_mlp"))
            for blk in m.blocks:
                blk.tiled_mlp_shards = shards
            self.engine = TrainEngine(m, ecfg)
            self._setup_sequence_parallel(m, int(wc.get("sequence_parallel", 1) or 1))
            ao = wc.get("activation_offload")
            if ao:
                # saved activations go to pinned host memory on a side stream and come back ahead of their use
                from ..utils.activation_offload import ActivationOffload
                opts = ao if isinstance(ao, dict) else {}
                if opts.get("enable", True):
                    self.activation_offload = ActivationOffload(
                        min_bytes=int(opts.get("min_bytes", 1 << 20)), keep_last=int(opts.get("keep_last", 2)),
                        prefetch=int(opts.get("prefetch", 2)))
        return True

    def _initialize_tp_sampler(self, job_config, model, tp: int, dtype, seed) -> bool:
        """A sampling replica over ``tp`` consecutive ranks of the job: every rank keeps a head / column shard of the
        decoder (``parallel/tp_sampler.py``) and all ranks of a replica are called together."""
        import torch.distributed as dist
        from ..parallel.tp_sampler import TensorParallelSampler
        if not dist.is_initialized() or self.world % tp:
            raise ValueError(f"tensor_parallel_size={tp} needs a process group whose size ({self.world}) it divides")
        first = self.rank - self.rank % tp
        # only the members create their group: the ranks of other replicas (or of no replica) need not take part
        group = dist.new_group(list(range(first, first + tp)), use_local_synchronization=True)
        vc = dict(job_config.get("vllm_config") or {})
        full = model if model is not None else self._load_model(job_config, dtype, seed)
        paged = (self.device.type == "cuda" and not self.model_cfg.is_moe and self.model_cfg.layer_types is None
                 and self.model_cfg.head_dim == 128 and not vc.get("enable_return_routed_experts")
                 and vc.get("tp_engine", "paged") == "paged")
        if paged:
            # dense decoders on GPUs: the paged CUDA engine with head shards of the KV cache and the fused
            # GEMM -> reduce-scatter / norm -> all-gather kernels in its decode loop
            from .sampler import SamplerEngine
            self.sampler = SamplerEngine(
                self.model_cfg, self.device, model=full, tp_group=group,
                kv_cache_tokens=int(vc.get("kv_cache_tokens", 1 << 20)), max_batch=int(vc.get("max_num_seqs", 256)),
                max_seq_len=int(vc.get("max_model_len", 8192)),
                cascade=bool((job_config.get("arctic_inference_config") or {}).get("zorro_inference", {}).get("enable", True)),
                seed=seed, eos_token_id=vc.get("eos_token_id"), quantization=vc.get("quantization"))
        else:
            self.sampler = TensorParallelSampler(
                self.model_cfg, self.device, model=full, tp_group=group, dtype=dtype,
                max_batch=int(vc.get("max_num_seqs", 256)), max_seq_len=int(vc.get("max_model_len", 8192)), seed=seed,
                eos_token_id=vc.get("eos_token_id"))
        self.tp = tp
        del full                                                 # only the shard stays resident
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        return True

    def rank_info(self) -> Dict[str, Any]:
        import torch.distributed as dist
        return {"rank": self.rank, "world": self.world, "device": str(self.device),
                "process_group": dist.is_initialized(),
                "zero3": bool(self.engine is not None and getattr(self.engine, "zero3", None) is not None)}

    def _ensure_process_group(self, job_config) -> None:
        """Joins the job's data-parallel group when the launcher described one (``WORLD_SIZE`` > 1 with a
        rendezvous address) and none exists yet: NCCL on a GPU, gloo on CPU.  Sampler replicas are independent and
        call this only when they are tensor-parallel.  The reference does the same through ``deepspeed.init_distributed``
        (arctic_platform/common/deepspeed_worker.py:155)."""
        import datetime
        import os
        import torch.distributed as dist
        if dist.is_initialized():
            self.rank, self.world = dist.get_rank(), dist.get_world_size()
            if _PG["created_here"]:
                _PG["users"] += 1
                self._owns_process_group = True
            return
        if self.world <= 1 or "MASTER_ADDR" not in os.environ or "MASTER_PORT" not in os.environ:
            self.world = 1
            return
        from ..utils.debug import drop_stale_nccl_topo_file
        drop_stale_nccl_topo_file()
        timeout = datetime.timedelta(seconds=float(job_config.get("process_group_timeout_s", 600)))
        if self.device.type == "cuda":
            dist.init_process_group("nccl", rank=self.rank, world_size=self.world, timeout=timeout, device_id=self.device)
        else:
            dist.init_process_group("gloo", rank=self.rank, world_size=self.world, timeout=timeout)
        _PG["created_here"], _PG["users"] = True, 1
        self._owns_process_group = True

    def _speculative_setup(self, job_config, vc: dict, dtype, seed) -> Optional[dict]:
        """``arctic_inference_config.speculative_decoding = {model, num_speculative_tokens}`` (or ``vllm_config.spec_model``)
        names a draft model.  The tensor-op engine drafts and verifies with it (CPU runs; on a GPU when
        ``vllm_config.speculative_engine = "tensor_op"`` asks for that engine); the paged CUDA engine does not
        speculate, so there the setting is reported and ignored.  Hybrid (recurrent-state) models are not drafted for."""
        sd = dict((job_config.get("arctic_inference_config") or {}).get("speculative_decoding") or {})
        name = (sd.get("model") or vc.get("spec_model") or "").strip()
        if not name:
            return None
        tensor_op = self.device.type != "cuda" or vc.get("speculative_engine") == "tensor_op"
        if not tensor_op or self.model_cfg.layer_types is not None:
            logger.warning("speculative decoding (%s) is not available on this sampler engine; decoding without it", name)
            return None
        from pathlib import Path
        from ..models.config import resolve_config
        from ..models.conversion_cache import load_through_cache
        dcfg = resolve_config(name)
        draft = DecoderLM(dcfg, self.device, dtype)
        path = Path(name)
        if path.is_dir() and any(path.glob("*.safetensors")):
            load_through_cache(draft, path, cache_dir=job_config.get("weight_conversion_cache_dir"))
        else:
            draft.init_weights(seed=seed + 1)
        draft.eval()
        return {"draft": draft, "k": int(sd.get("num_speculative_tokens") or vc.get("num_speculative_tokens") or 4)}

    def _load_model(self, job_config, dtype, seed) -> DecoderLM:
        from pathlib import Path
        from ..models.conversion_cache import load_through_cache
        m = DecoderLM(self.model_cfg, self.device, dtype)
        path = Path(str(job_config["model_name"]))
        lo = getattr(self, "loader_options", None)
        random_init = bool(lo is not None and lo.debug is not None and lo.debug.random_init)
        if path.is_dir() and any(path.glob("*.safetensors")) and not random_init:
            # converted once per node when a cache directory is configured, else straight from the shards
            load_through_cache(m, path, cache_dir=job_config.get("weight_conversion_cache_dir")
                               or (lo.weight_conversion_cache_dir if lo is not None else None))
            m.source_dir = str(path)                 # exports take the tokenizer files from here
        else:
            m.init_weights(seed=seed)     # no checkpoint on disk: deterministic random initialisation
        return m

    def destroy(self) -> None:
        self.engine = None
        self.sampler = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        import torch.distributed as dist
        if getattr(self, "_owns_process_group", False):
            self._owns_process_group = False
            _PG["users"] -= 1
            if _PG["users"] <= 0 and dist.is_initialized():      # the last engine of this process that used it
                dist.destroy_process_group()
                _PG["created_here"] = False

    # ------------------------------------------------------------------ forward / backward / step
    def _forward_maybe_backward(self, batch, meta, processing, backward: bool) -> Dict[str, Any]:
        engine = self.engine
        if engine is None and self.sampler is not None and not backward and self.job_type == "log_prob":
            engine = _ScoringView(self.sampler.model)      # log-prob job served by the sampler's engine and weights
        if engine is None:
            raise RuntimeError("worker has no training/log-prob engine")
        t0 = time.perf_counter()
        row_order = None
        if isinstance(batch, (list, tuple)):
            mbs = list(batch)                               # client-side gradient-accumulation split
        elif (meta or {}).get("max_tokens_per_mb"):
            mbs, row_order = self._split_by_token_budget(batch, meta, processing)
        else:
            n_mb = int((meta or {}).get("num_micro_batches", 1) or 1)
            mbs = split_microbatches(batch, n_mb)
        meta = self._with_sft_global_tokens(mbs, meta, processing)
        meta = self._with_rl_global_counts(mbs, meta, processing)
        per_mb, outs = [], []
        from ..utils.debug import MemoryHistory, ProfilerContext, nvtx_range, see_memory_usage
        tag = "fwd_bwd" if backward else "fwd"
        self._calls = getattr(self, "_calls", 0) + 1
        prof_type = os.environ.get("APB_PROFILER", "none") if self._calls == int(os.environ.get("APB_PROFILER_CALL", "2")) else "none"
        see_memory_usage(f"{tag} start")
        mem_hist = MemoryHistory(prof_type == "none" and os.environ.get("APB_MEMORY_HISTORY") == "1"
                                 and self._calls == int(os.environ.get("APB_PROFILER_CALL", "2")),
                                 os.environ.get("APB_PROFILER_DIR", "/tmp/apb-prof"), f"{tag}-memory-rank{self.rank}")
        with mem_hist, ProfilerContext(prof_type, os.environ.get("APB_PROFILER_DIR", "/tmp/apb-prof"), f"{tag}-rank{self.rank}") as prof:
            for i, mb in enumerate(mbs):
                if isinstance(mb, dict):
                    log_dp_shard_tokens(self.rank, f"{tag} micro-batch {i}", mb, meta)
                offload = self.activation_offload if backward else None
                with nvtx_range(f"{tag}/mb{i}", enabled=self._nvtx), (offload or contextlib.nullcontext()):
                    r = run_pipeline(engine, mb, meta, processing, self.device, backward=backward, return_tensors=True)
                if offload is not None:
                    offload.release()
                per_mb.append(r["metrics"])
                if not (isinstance(mb, dict) and mb.get("_dummy")):
                    outs.append(r)                           # a filler pass has no rows of the caller's batch
        if prof.report and self.rank == 0:
            print(f"[profile] {tag}: {prof.report}", flush=True)
        if mem_hist.path:
            print(f"[profile] {tag}: allocator history in {mem_hist.path}", flush=True)
        see_memory_usage(f"{tag} end")
        metrics = combine_metric_microbatches(per_mb)
        result: Dict[str, Any] = {"metrics": metrics, "avg_loss": sum(o["avg_loss"] for o in outs)}
        if not backward:
            keys = outs[0].get("batch", {}).keys()
            result["batch"] = {k: torch.cat([o["batch"][k] for o in outs], 0) for k in keys}
            if row_order is not None:                      # micro-batches were formed by size: back to the caller's order
                inv = torch.empty_like(row_order)
                inv[row_order] = torch.arange(row_order.numel())
                result["batch"] = {k: v[inv] for k, v in result["batch"].items()}
        metrics["_profile_ms"] = {"fwd_bwd" if backward else "fwd_total": (time.perf_counter() - t0) * 1e3}
        sft_profile.merge_into(metrics)          # per-phase buckets when ARL_SFT_PROFILE=1
        if backward:
            from ..utils.debug import maybe_log_moe_imbalance
            maybe_log_moe_imbalance(self.rank)
        return result

    def _setup_sequence_parallel(self, model, sp: int) -> None:
        """Ulysses groups of ``sp`` consecutive ranks.  Every rank of a group receives the same batch and works on
        its slice of the packed token axis; ZeRO and the gradient mean still span all ranks."""
        self.sp = 1
        if sp <= 1:
            return
        import torch.distributed as dist
        if not dist.is_initialized() or self.world % sp:
            raise ValueError(f"sequence_parallel={sp} needs a process group whose size ({self.world}) it divides")
        from ..parallel.ulysses import apply_sequence_parallelism
        mine = None
        for g0 in range(0, self.world, sp):                    # every rank creates every group, in the same order
            grp = dist.new_group(list(range(g0, g0 + sp)))
            if g0 <= self.rank < g0 + sp:
                mine = grp
        apply_sequence_parallelism(model, mine)
        self.sp = sp

    def _split_by_token_budget(self, batch, meta, processing):
        """Micro-batches of at most ``meta['max_tokens_per_mb']`` tokens (first-fit decreasing).  With prompt
        de-duplication whole prompt groups stay together and the shared prompt counts once; every data-parallel rank
        ends up with the same number of micro-batches.  Returns the micro-batches and the row permutation they
        follow (arctic_platform/rl/processors/pipeline.py:502-606 in the reference)."""
        from ..rl.processors.losses import SFT_LOSS_FNS
        from ..rl.processors.microbatch import MicroBatchSpec, split_padded_tensor_dict_into_mb_list
        from ..rl.processors.pipeline import response_length_of
        from ..rl.zorro_train.seqlen_balancing import rearrange_micro_batches_with_dedup
        budget = int(meta["max_tokens_per_mb"])
        group = getattr(self.engine, "group", None)
        if "attention_mask" not in batch:
            batch = {**batch, "attention_mask": torch.ones_like(batch["input_ids"])}
        sft = (processing or {}).get("loss_fn") in SFT_LOSS_FNS or bool(meta.get("plain_packing"))
        if not sft and meta.get("zorro_train_enable", True):
            mbs, rows = rearrange_micro_batches_with_dedup(batch, response_length_of(batch, meta), budget,
                                                            meta.get("max_rollouts"), dp_group=group)
        else:
            mbs, rows = split_padded_tensor_dict_into_mb_list(batch, MicroBatchSpec(budget), group)
        # every rank must run the same number of passes (the ZeRO-3 gathers and the gradient reduction are
        # collectives): a rank whose rows fit into fewer micro-batches pads with loss-free copies of its first row
        import torch.distributed as dist
        if dist.is_initialized() and self.engine.world > 1:
            n = torch.tensor([len(mbs)], dtype=torch.int64)
            n = n.to(self.device if dist.get_backend(group) == "nccl" else "cpu")
            dist.all_reduce(n, op=dist.ReduceOp.MAX, group=group)
            while len(mbs) < int(n):
                mbs.append(_loss_free_row(batch))
        return mbs, torch.tensor([i for r in rows for i in r], dtype=torch.long)

    def _with_rl_global_counts(self, mbs, meta, processing):
        """Several micro-batches and no normalisers from the client: the policy losses then need the token and
        sequence counts of the WHOLE batch (all micro-batches, all ranks), or every micro-batch would be averaged on
        its own and the accumulated gradient would scale with the number of micro-batches."""
        from ..rl.processors.losses import SFT_LOSS_FNS
        loss_fn = (processing or {}).get("loss_fn")
        if (len(mbs) <= 1 or not loss_fn or loss_fn in SFT_LOSS_FNS or "batch_num_tokens" in (meta or {})
                or not all(isinstance(mb, dict) and "response_mask" in mb for mb in mbs)):
            return meta
        import torch.distributed as dist
        meta = dict(meta or {})
        t = torch.tensor([float(sum(int(mb["response_mask"].sum()) for mb in mbs)),
                          # loss-free filler micro-batches (appended so that all ranks run the same number of
                          # passes) are not sequences of the batch: the seq-mean modes divide by real rows only
                          float(sum(mb["input_ids"].shape[0] for mb in mbs if not mb.get("_dummy")))],
                         dtype=torch.float64)
        group = getattr(self.engine, "group", None)
        if dist.is_initialized() and self.engine.world > 1:
            t = t.to(self.device if dist.get_backend(group) == "nccl" else "cpu")
            dist.all_reduce(t, group=group)
            t = t / self.sp                                    # the ranks of a sequence-parallel group hold the same rows
            meta.setdefault("dp_size", self.engine.world // self.sp)
        meta["batch_num_tokens"], meta["global_batch_size"] = float(t[0]), float(t[1])
        return meta

    def _with_sft_global_tokens(self, mbs, meta, processing):
        """Cross-entropy losses normalised by the GLOBAL token count need that count before the first micro-batch
        runs: loss tokens of all this rank's micro-batches, summed over the data-parallel ranks (one all-reduce of
        an int64), plus ``dp_size``.  A client that sends ``batch_num_tokens`` itself is left alone
        (arctic_platform/common/deepspeed_worker.py:404-441 does the same before its SFT pipeline)."""
        from ..sft.processor import SFT_GLOBAL_TOKEN_LOSS_FNS, count_loss_tokens
        if (processing or {}).get("loss_fn") not in SFT_GLOBAL_TOKEN_LOSS_FNS or "batch_num_tokens" in (meta or {}):
            return meta
        import torch.distributed as dist
        meta = dict(meta or {})
        n = torch.tensor([sum(count_loss_tokens(mb) for mb in mbs if isinstance(mb, dict))], dtype=torch.int64)
        group = getattr(self.engine, "group", None)
        if dist.is_initialized() and self.engine.world > 1:
            n = n.to(self.device if dist.get_backend(group) == "nccl" else "cpu")
            dist.all_reduce(n, group=group)
            n = n // self.sp
            meta.setdefault("dp_size", self.engine.world // self.sp)
        meta["batch_num_tokens"] = float(n.item())
        return meta

    def forward_backward(self, batch, meta=None, processing=None) -> Dict[str, Any]:
        return self._forward_maybe_backward(batch, meta, processing, backward=True)

    def forward_no_grad(self, batch, meta=None, processing=None) -> Dict[str, Any]:
        processing = {"post": ["compute_entropy_and_logprobs"], "loss_fn": None, **(processing or {})}
        return self._forward_maybe_backward(batch, meta, processing, backward=False)

    def step(self, learning_rate: Optional[float] = None) -> Dict[str, Any]:
        if learning_rate is not None:
            self.engine.cfg.lr = float(learning_rate)
        with sft_profile.timed("step"):
            out = self.engine.step()
            gn = float(out["grad_norm"])
        return sft_profile.merge_into({"metrics": {"last_lr": out["last_lr"], "grad_norm": gn}, "batch": {}})

    def compute_log_probs(self, input_ids: torch.Tensor) -> torch.Tensor:
        """``log softmax(logits)[next token]`` for every position of unpadded ``input_ids [B, S]``:
        a ``[B, S-1]`` CPU tensor (arctic_platform/common/deepspeed_worker.py:638-652 in the reference)."""
        batch = {"input_ids": input_ids, "attention_mask": torch.ones_like(input_ids)}
        r = run_pipeline(self.engine, batch, {"plain_packing": True}, {"loss_fn": None, "post": []}, self.device,
                         backward=False)
        return r["batch"]["log_probs"][:, 1:]

    @torch.no_grad()
    def score_completions(self, prompts, completions, top_k: int = 1):
        """Log-probability of every completion token given its prompt, under this worker's CURRENT weights -- the
        sampler's when the worker hosts one (what the rollouts were drawn from), else the engine's.  One packed
        pass; identical prompts are computed once.  ``top_k`` > 1 also returns, per completion position, the ``k``
        most likely tokens with their log-probs (``{"log_probs": rows, "top_log_probs": [[{token: lp}]]}``), which
        the reference takes from its sampler's ``prompt_logprobs`` (arctic_platform/common/http_server.py:949)."""
        from ..models.decoder import token_logprobs
        from ..rl.zorro_train.layout import build_packed_batch
        model = self._target_model()
        if self.sampler is not None and getattr(self.sampler, "_asleep", False):
            raise RuntimeError("sampler is asleep; call wake() first")
        P = max(len(p) for p in prompts)
        R = max(len(c) for c in completions)
        ids = torch.zeros((len(prompts), P + R), dtype=torch.int64)
        mask = torch.zeros_like(ids)
        for i, (p, c) in enumerate(zip(prompts, completions)):
            if len(p) == 0:
                raise ValueError("empty prompt")
            ids[i, P - len(p):P] = torch.tensor(p)
            mask[i, P - len(p):P] = 1
            ids[i, P:P + len(c)] = torch.tensor(c)
            mask[i, P:P + len(c)] = 1
        pk = build_packed_batch(ids, mask, R, dedup=True).to(self.device)
        was_training = model.training
        model.eval()
        lp, _ = token_logprobs(model, pk, 1.0, with_entropy=False)
        grid = pk.scatter_to_grid(lp.float()).cpu()
        rows = [grid[i, :len(c)].tolist() for i, c in enumerate(completions)]
        if int(top_k) <= 1:
            model.train(was_training)
            return rows
        # the whole distribution at the prediction rows, a chunk of rows at a time
        k = int(top_k)
        h = model.forward_hidden(pk.input_ids, pk.positions, pk.layout).index_select(0, pk.pred_index)
        W = model.output_weight
        N = h.shape[0]
        top_lp = torch.empty((N, k), dtype=torch.float32, device=h.device)
        top_id = torch.empty((N, k), dtype=torch.int64, device=h.device)
        for r0 in range(0, N, 2048):
            z = torch.log_softmax((h[r0:r0 + 2048].float() @ W.float().t()), -1)
            top_lp[r0:r0 + 2048], top_id[r0:r0 + 2048] = torch.topk(z, k, dim=-1)
        model.train(was_training)
        R_ = pk.response_length
        lp_grid = torch.zeros((len(prompts) * R_, k), dtype=torch.float32)
        id_grid = torch.zeros((len(prompts) * R_, k), dtype=torch.int64)
        oi = pk.out_index.cpu()
        lp_grid[oi], id_grid[oi] = top_lp.cpu(), top_id.cpu()
        lp_grid, id_grid = lp_grid.view(len(prompts), R_, k), id_grid.view(len(prompts), R_, k)
        tops = [[{int(t): float(v) for t, v in zip(id_grid[i, j].tolist(), lp_grid[i, j].tolist())}
                 for j in range(len(c))] for i, c in enumerate(completions)]
        return {"log_probs": rows, "top_log_probs": tops}

    # ------------------------------------------------------------------ rollout
    def _tokenizer_for(self):
        """The checkpoint's tokenizer when ``model_name`` is a directory that ships one (local files only); ``None``
        for presets and weight-only directories.  Loaded on first use."""
        if not hasattr(self, "_tokenizer"):
            self._tokenizer = None
            from pathlib import Path
            path = Path(str(self.job_config.get("tokenizer") or self.job_config.get("model_name", "")))
            if path.is_dir() and any((path / f).exists() for f in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model")):
                try:
                    from transformers import AutoTokenizer
                    self._tokenizer = AutoTokenizer.from_pretrained(str(path), local_files_only=True)
                except Exception as exc:  # noqa: BLE001 - generation by token ids still works
                    import logging
                    logging.getLogger(__name__).warning("could not load the tokenizer under %s: %s", path, exc)
        return self._tokenizer

    def generate(self, prompts, sampling_params=None) -> List[dict]:
        """Token ids in, token ids out.  With a tokenizer beside the checkpoint, text prompts are accepted too and
        every result carries its decoded ``text`` (the reference's samplers return text the same way)."""
        if self.sampler is None:
            raise RuntimeError("worker has no sampling engine")
        tok = self._tokenizer_for() if prompts and (any(isinstance(p, str) for p in prompts)
                                                      or (sampling_params or {}).get("detokenize", True)) else None
        if any(isinstance(p, str) for p in prompts):
            if tok is None:
                raise ValueError("text prompts need a tokenizer beside the checkpoint (or job_config['tokenizer'])")
            prompts = [tok.encode(p, add_special_tokens=False) if isinstance(p, str) else p for p in prompts]
        sp = {k: v for k, v in (sampling_params or {}).items() if k != "detokenize"} if isinstance(sampling_params, dict) \
            else sampling_params
        text_stops: List[str] = []
        if isinstance(sp, dict) and sp.get("stop"):
            # stop STRINGS: one-token strings end the sequence in the sampler itself; longer ones cut the decoded text
            if tok is None:
                raise ValueError("stop strings need a tokenizer beside the checkpoint; use stop_token_ids")
            stops = [sp["stop"]] if isinstance(sp["stop"], str) else list(sp["stop"])
            ids = list(sp.get("stop_token_ids") or [])
            for st in stops:
                enc = tok.encode(st, add_special_tokens=False)
                if len(enc) == 1:
                    ids.append(int(enc[0]))
                else:
                    text_stops.append(st)
            sp = {**{k: v for k, v in sp.items() if k != "stop"}, "stop_token_ids": ids}
        outs = self.sampler.generate(prompts, sp)
        if tok is not None:
            skip = bool(sp.get("skip_special_tokens", True)) if isinstance(sp, dict) else True
            for o in outs:
                o["text"] = tok.decode(o["token_ids"], skip_special_tokens=skip)
                cuts = [o["text"].find(st) for st in text_stops if st in o["text"]]
                if cuts:
                    o["text"] = o["text"][:min(cuts)]
                    o["finish_reason"] = "stop"
        return outs

    # ------------------------------------------------------------------ weights
    def iter_weights(self):
        return self.engine.iter_hf_tensors()

    def get_parameter_names(self) -> List[str]:
        from ..models.hf_io import hf_param_names
        return hf_param_names(self.model_cfg)

    def max_param_bytes(self) -> int:
        """Size of the largest single weight under its Hugging Face name: what a receiver has to be able to stage
        when weights arrive one tensor at a time."""
        return max(t.numel() * t.element_size() for _n, t in self.engine.iter_hf_tensors())

    def export_hf_checkpoint(self, path: str) -> List[str]:
        """Hugging Face safetensors + ``config.json`` under ``path`` without the optimizer files.  Under ZeRO-3
        every rank takes part in the gather; rank 0 writes (arctic_platform/common/deepspeed_worker.py:602-636)."""
        import torch.distributed as dist
        from ..models.hf_io import save_hf_checkpoint
        files: List[str] = []
        sharded = getattr(self.engine, "zero3", None) is not None
        tensors = None
        if sharded:
            tensors = [(n, t.detach().to("cpu").clone() if self.rank == 0 else None) for n, t in self.engine.iter_hf_tensors()]
        if self.rank == 0:
            files = save_hf_checkpoint(self.engine.model, path, tensors=tensors)
        if dist.is_initialized() and self.world > 1:
            dist.barrier()
        return files

    def gather_and_save_state_dict(self, path: str) -> Dict[str, Any]:
        """All ranks gather, rank 0 writes one safetensors file (the hand-over file of the ``cpu_file`` strategy)."""
        import torch.distributed as dist
        from ..models.hf_io import write_safetensors
        tensors = {n: (t.detach().to("cpu").clone() if self.rank == 0 else None) for n, t in self.engine.iter_hf_tensors()}
        out = {"path": path, "num_tensors": len(tensors), "bytes": 0}
        if self.rank == 0:
            write_safetensors(path, tensors, {"format": "pt"})
            out["bytes"] = sum(t.numel() * t.element_size() for t in tensors.values())
        if dist.is_initialized() and self.world > 1:
            dist.barrier()
        return out

    def release_ipc_handles(self) -> int:
        """Unmaps the trainer buffers a split-placement sampler opened through CUDA IPC (``sync_from_ipc``); engines
        that share a process hand weights over with a kernel and hold none.  Returns how many were released."""
        return self.release_ipc()

    def weight_norm(self) -> Dict[str, float]:
        return self.sampler.weight_norm() if self.sampler is not None else self.engine.weight_norm()

    def get_named_weight(self, name: str) -> torch.Tensor:
        for n, t in self.engine.iter_hf_tensors():
            if n == name:
                return t.detach().to("cpu")
        raise KeyError(name)

    def load_named_weight(self, name: str, tensor: torch.Tensor) -> None:
        self.load_weights([(name, tensor)])

    def _target_model(self):
        return self.sampler.model if self.sampler is not None else self.engine.model

    def load_weights(self, named_tensors) -> int:
        """Copies ``(hf_name, tensor)`` pairs into this worker's model (sampler or forward-only engine)."""
        from ..models.hf_io import load_hf_tensor
        if self.sampler is not None and hasattr(self.sampler, "tp"):
            return self.sampler.load_weights(named_tensors)      # full tensors in, this rank's slices kept
        n = 0
        model = self._target_model()
        for name, t in named_tensors:
            load_hf_tensor(model, name, t)
            n += 1
        if self.sampler is not None and hasattr(self.sampler, "weights_updated"):
            self.sampler.weights_updated()
        return n

    def get_weights(self, only_rank: Optional[int] = None) -> Optional[List]:
        """Every weight under its Hugging Face name as CPU tensors: one call, one pass over the parameters (one
        gather of the shards under ZeRO-3) -- the bulk strategy of a cross-process sync.  With ``only_rank`` every
        rank still takes part in the gather but only that rank copies the tensors out; the others return None."""
        if only_rank is not None and self.rank != only_rank:
            for _ in self.engine.iter_hf_tensors():
                pass
            return None
        return [(n, t.detach().to("cpu", copy=True)) for n, t in self.engine.iter_hf_tensors()]

    def weight_buckets(self, bucket_bytes: int = 256 << 20) -> List[List[str]]:
        """Names grouped so that each group is at most ``bucket_bytes`` (one tensor may exceed it alone)."""
        from ..models.hf_io import hf_param_names
        sizes = {n: t.numel() * t.element_size() for n, t in self.engine.iter_hf_tensors()}
        out, cur, tot = [], [], 0
        for n in hf_param_names(self.model_cfg):
            if cur and tot + sizes[n] > bucket_bytes:
                out.append(cur)
                cur, tot = [], 0
            cur.append(n)
            tot += sizes[n]
        if cur:
            out.append(cur)
        return out

    def get_weight_bucket(self, names: List[str]) -> List:
        want = set(names)
        return [(n, t.detach().to("cpu", copy=True)) for n, t in self.engine.iter_hf_tensors() if n in want]

    def save_weights_to_path(self, path: str) -> Dict[str, Any]:
        """Writes the weights as one safetensors file (a tmpfs path makes this the shared-memory hand-over)."""
        from ..models.hf_io import write_safetensors
        tensors = {n: t.detach().to("cpu") for n, t in self.engine.iter_hf_tensors()}
        write_safetensors(path, tensors, {"format": "pt"})
        return {"path": path, "num_tensors": len(tensors), "bytes": sum(t.numel() * t.element_size() for t in tensors.values())}

    def load_weights_from_path(self, path: str) -> int:
        from ..models.hf_io import read_safetensors
        return self.load_weights(read_safetensors(path))

    def sync_weights_to(self, dst: "EngineWorker") -> int:
        """Pushes this (training) worker's parameters into ``dst`` (a sampling or log-prob worker of the
        same process).  Same device and layout: one flat-gather kernel; otherwise tensor by tensor under
        their Hugging Face names.  Returns the number of tensors covered."""
        from ..models.hf_io import hf_param_names
        from ..parallel import weight_sync
        n_table = self._sync_by_table(dst)
        if n_table is not None:
            return n_table
        if dst.sampler is not None and getattr(dst.sampler, "tp", 1) > 1:
            # tensor-parallel replica: a different layout per rank, so the tensors travel under their names
            return dst.sampler.load_weights((n, t.detach()) for n, t in self.engine.iter_hf_tensors())
        dst_model = dst.sampler.model if dst.sampler is not None else dst.engine.model
        n_names = len(hf_param_names(self.model_cfg))
        dst_engine = dst.engine if dst.sampler is None else None
        if dst_engine is not None and getattr(dst_engine, "zero3", None) is not None:
            # the target keeps its parameters as shards too: hand it a full copy and let it cut its own shard
            dst_engine.load_full_flat(self.engine.full_flat_params())
            return n_names
        if any(u.local_only for u in self.engine.units):
            # expert parallelism: no rank holds all experts, so there is no flat buffer to copy -- every rank gathers
            # the expert shards layer by layer and fills its target under the Hugging Face names
            n = weight_sync.sync_state_dict(((n, t.detach()) for n, t in self.engine.iter_hf_tensors()), dst_model)
            if dst.sampler is not None and hasattr(dst.sampler, "weights_updated"):
                dst.sampler.weights_updated()
            return n
        if self.engine.on_cuda and next(dst_model.parameters()).device == self.device:
            flat = getattr(dst_model, "_flat_params", None)
            if flat is None or flat.numel() != self.engine.total:
                flat = weight_sync.flatten_like(dst_model, self.engine)
            weight_sync.sync_flat(self.engine, flat)
            if dst.sampler is not None and hasattr(dst.sampler, "weights_updated"):
                dst.sampler.weights_updated()
            return n_names
        return weight_sync.sync_state_dict(((n, t.detach()) for n, t in self.engine.iter_hf_tensors()), dst_model)

    def _sync_by_table(self, dst: "EngineWorker") -> Optional[int]:
        """One kernel for a CUDA sampler of the same process whose layout differs from the trainer's: a
        tensor-parallel shard (head / column slices) and / or block-scaled fp8 matrices.  The table names, for every
        128 x 128 tile of the sampler's tensors, where it lives in the trainer (ZeRO-3 piece of which rank, or the
        replicated buffer).  Returns the tensor count, or ``None`` when this route does not apply."""
        from ..models.hf_io import hf_param_names
        from ..parallel import weight_sync
        sm = dst.sampler
        if sm is None or not self.engine.on_cuda or not hasattr(sm, "_sync_plan"):
            return None
        tp, fp8 = int(getattr(sm, "tp", 1)), bool(getattr(sm, "fp8", False))
        if tp == 1 and not fp8:
            return None                         # same layout: the flat kernel below is the shortest path
        if self.model_cfg.is_moe or any(u.local_only for u in self.engine.units):
            return None
        if next(sm.model.parameters()).device != self.device:
            return None
        layout = weight_sync.trainer_layout(self.engine)
        key = (layout["total"], layout["world"], layout["zero3"] is not None, sm.tp_rank, tp, fp8, True)
        plan = sm._sync_plan
        if plan is None or plan.layout_key != key:
            plan = weight_sync.build_sync_plan(layout, sm.model, full_cfg=sm.full_cfg, tp_rank=sm.tp_rank, tp=tp, fp8=fp8)
            sm._sync_plan = plan
        ptrs, src_rank = weight_sync.engine_source(self.engine)
        weight_sync.run_sync_plan(plan, ptrs, src_rank)
        if fp8:
            # the block-scaled copies came out of the same pass: nothing to re-quantise before the next rollout
            sm._fp8_w = [{n: plan.fp8[(li, n)] for n in weight_sync.FP8_MATRICES} for li in range(sm.cfg.num_layers)]
            sm._graphs.clear()
            sm._fp8_stale = False
        return len(hf_param_names(self.model_cfg))

    # ------------------------------------------------------------------ split placement: hand-over through CUDA IPC
    def export_ipc_source(self) -> Optional[Dict[str, Any]]:
        """Trainer side of the split-placement hand-over: an IPC handle of this rank's flat bf16 parameter buffer
        plus its layout, for a sampler in ANOTHER process of the node to map and read over NVLink
        (``sync_from_ipc``).  ``None`` when the storage cannot be exported that way -- ZeRO-3 shards and the
        symmetric-memory buffers of multi-rank fused engines are not legacy-IPC allocations -- and the caller falls
        back to shipping tensors.  The reference's counterpart is ``sync_weights_cuda_ipc``
        (arctic_platform/common/utils/weight_sync.py:47-142)."""
        from ..parallel import weight_sync
        eng = self.engine
        if eng is None or not eng.on_cuda or getattr(eng, "zero3", None) is not None:
            return None
        if any(u.local_only for u in eng.units):
            return None
        try:
            handle, offset = weight_sync.export_ipc(eng.param_buf.tensor)
        except Exception:
            return None
        torch.cuda.synchronize(self.device)               # the optimizer step that wrote the buffer has finished
        return {"handle": handle, "offset": offset, "layout": weight_sync.trainer_layout(eng),
                "device": int(self.device.index or 0)}

    def sync_from_ipc(self, sources: List[Dict[str, Any]]) -> int:
        """Sampler side: maps the trainer buffers named by ``sources`` (once per handle), builds the tile table for
        this replica's layout (tensor-parallel shard, fp8 copies) and runs the one hand-over kernel on them.  Returns
        the number of tensors covered."""
        from ..models.hf_io import hf_param_names
        from ..parallel import weight_sync
        sm = self.sampler
        if sm is None or self.device.type != "cuda" or not hasattr(sm, "_sync_plan"):
            raise RuntimeError("sync_from_ipc needs the paged CUDA sampler")
        maps = self.__dict__.setdefault("_ipc_maps", {})
        ptrs = []
        for src in sources:
            key = bytes(src["handle"])
            if key not in maps:
                maps[key] = (weight_sync.open_ipc(key, int(src["offset"])), int(src["offset"]))
            ptrs.append(maps[key][0])
        layout = sources[0]["layout"]
        tp, fp8 = int(getattr(sm, "tp", 1)), bool(getattr(sm, "fp8", False))
        key = (layout["total"], layout["world"], layout["zero3"] is not None, sm.tp_rank, tp, fp8, "ipc")
        plan = sm._sync_plan
        if plan is None or plan.layout_key != key:
            plan = weight_sync.build_sync_plan(layout, sm.model, full_cfg=sm.full_cfg, tp_rank=sm.tp_rank, tp=tp, fp8=fp8)
            plan.layout_key = key
            sm._sync_plan = plan
        weight_sync.run_sync_plan(plan, ptrs, 0)
        torch.cuda.synchronize(self.device)               # the trainer may write its buffer again after this returns
        if fp8:
            sm._fp8_w = [{n: plan.fp8[(li, n)] for n in weight_sync.FP8_MATRICES} for li in range(sm.cfg.num_layers)]
            sm._graphs.clear()
            sm._fp8_stale = False
        elif hasattr(sm, "weights_updated"):
            sm.weights_updated()
        return len(hf_param_names(self.model_cfg))

    def release_ipc(self) -> int:
        """Unmaps every trainer buffer this worker has opened (before the trainer frees them)."""
        from ..parallel import weight_sync
        maps = self.__dict__.pop("_ipc_maps", {})
        for addr, off in maps.values():
            weight_sync.close_ipc(addr, off)
        return len(maps)

    def sleep_inference(self, level: int = 1) -> None:
        if self.sampler is not None:
            self.sampler.sleep(level)

    def has_sampler(self) -> bool:
        return self.sampler is not None

    def wake_inference(self, tags=None) -> None:
        if self.sampler is not None:
            self.sampler.wake(tags)

    def reset_prefix_cache(self) -> None:
        if self.sampler is not None:
            self.sampler.reset_prefix_cache()

    # ------------------------------------------------------------------ sleep / wake
    def offload_to_cpu(self) -> None:
        if self.engine is not None:
            self.engine.offload_states(("optimizer", "grads"))

    def offload_non_lp_states(self) -> None:
        if self.engine is not None:
            self.engine.offload_states(("optimizer",))

    def offload_lp_params(self) -> None:
        return None

    def backload_to_gpu(self) -> None:
        if self.engine is not None:
            self.engine.reload_states()

    def empty_cache(self, force: bool = False) -> None:
        """Returns the allocator's cached blocks to the driver -- what a sampler in ANOTHER process needs before it
        wakes.  A sampler in this process takes the freed blocks from the shared allocator directly, so the call is
        skipped then (``force`` overrides)."""
        if self.device.type == "cuda":
            import gc
            from ..utils import memory_budget
            gc.collect()
            if force or not memory_budget.shares_allocator(self.device):
                torch.cuda.empty_cache()

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, path: str, tag: Optional[str] = None, export_hf: bool = False) -> Dict[str, Any]:
        from .checkpoint import save_checkpoint
        return save_checkpoint(self.engine, path, tag, export_hf=export_hf)

    def load_checkpoint(self, path: str, tag: Optional[str] = None, strict: bool = False) -> int:
        from .checkpoint import load_checkpoint
        return load_checkpoint(self.engine, path, tag, strict=strict)
