"""Checkpoints in the DeepSpeed directory layout, written without DeepSpeed.

``save_checkpoint(engine, save_dir, tag)`` produces what ``engine.save_checkpoint(save_dir, tag)`` of a
DeepSpeed bf16 ZeRO engine leaves on disk (the reference saves exactly that,
arctic_platform/common/deepspeed_worker.py:578-600)::

    <save_dir>/latest                                            text file with the tag
    <save_dir>/<tag>/mp_rank_00_model_states.pt                  rank 0: module weights + engine state
    <save_dir>/<tag>/bf16_zero_pp_rank_<r>_mp_rank_00_optim_states.pt   every rank: its optimizer partition
    <save_dir>/hf/                                               optional Hugging Face safetensors export

The model-states file keeps the DeepSpeed keys (``module``, ``param_shapes``, ``global_steps``,
``dp_world_size``, ``mp_world_size``, ``ds_config``, ``ds_version``, ``lr_scheduler``...), with the module
stored under Hugging Face parameter names; the optimizer file keeps ``optimizer_state_dict`` with
``zero_stage``, ``partition_count``, ``base_optimizer_state`` (``exp_avg`` / ``exp_avg_sq`` / ``step``) and
``single_partition_of_fp32_groups``.  The flat partition follows THIS engine's unit layout (recorded under
``b200_layout`` and checked on load), which is what makes a resume bit-exact.  DeepSpeed itself could not resume
from these optimizer files -- its flat groups follow the order of ``module.parameters()`` -- so between this
engine and any other the interchange format is the ``hf/`` safetensors export, not the optimizer partition.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

DS_VERSION = "0.19.2+b200"



def _load_pt(path):
    """Reads a checkpoint file as DATA: tensors, numbers, strings and containers only (``weights_only=True``), which
    is all this engine writes.  A file that needs arbitrary unpickling (e.g. written by another framework with
    custom classes inside) is refused unless ``APB_TRUST_CHECKPOINT_PICKLES=1`` says the file is trusted -- loading a
    pickle runs whatever code it names."""
    import os
    import pickle
    try:
        return torch.load(path, map_location="cpu", weights_only=True)
    except pickle.UnpicklingError as exc:
        if os.environ.get("APB_TRUST_CHECKPOINT_PICKLES") == "1":
            return torch.load(path, map_location="cpu", weights_only=False)
        raise RuntimeError(f"{path} holds objects beyond tensors and plain containers ({exc}); set "
                           f"APB_TRUST_CHECKPOINT_PICKLES=1 to load it if you trust its origin") from exc

def _barrier(engine) -> None:
    if engine.world > 1 and dist.is_initialized():
        dist.barrier(group=engine.group)


def _layout_of(engine) -> Dict[str, Any]:
    return {"total": engine.total, "units": [(u.name, u.offset, u.length) for u in engine.units],
            "param_slices": {k: (o, n, tuple(s)) for k, (o, n, s) in engine.param_slices.items()}}


def save_checkpoint(engine, save_dir: str, tag: Optional[str] = None, export_hf: bool = False) -> Dict[str, Any]:
    if hasattr(engine, "require_awake"):
        engine.require_awake("save_checkpoint")      # a sleeping engine's optimizer tensors are empty placeholders
    tag = tag or f"global_step{engine.global_steps}"
    root = Path(save_dir)
    d = root / tag
    d.mkdir(parents=True, exist_ok=True)
    files = []
    module = None
    collective_export = getattr(engine, "zero3", None) is not None or any(u.local_only for u in engine.units)
    if collective_export:
        # stage 3 / expert parallelism: materialising the weights is a collective gather -- every rank takes part,
        # rank 0 keeps the result
        gathered = ((n, t.detach().to("cpu").clone() if engine.rank == 0 else None) for n, t in engine.iter_hf_tensors())
        module = OrderedDict(gathered)
    if engine.rank == 0:
        if module is None:
            module = OrderedDict((n, t.detach().to("cpu").clone()) for n, t in engine.iter_hf_tensors())
        state = {
            "module": module, "buffer_names": [n for n, _b in engine.model.named_buffers()], "optimizer": None,
            "buffers": OrderedDict((n, b.detach().to("cpu").clone()) for n, b in engine.model.named_buffers()),
            "param_shapes": [OrderedDict((n, t.shape) for n, t in module.items())],
            "frozen_param_shapes": None, "frozen_param_fragments": None, "shared_params": {},
            "lr_scheduler": {"type": engine.cfg.scheduler.type, "warmup_steps": engine.cfg.scheduler.warmup_steps,
                             "total_steps": engine.cfg.scheduler.total_steps,
                             "min_lr_ratio": engine.cfg.scheduler.min_lr_ratio, "last_step": engine.global_steps},
            "data_sampler": None, "random_ltd": None, "sparse_tensor_module_names": [],
            "skipped_steps": 0, "global_steps": engine.global_steps, "global_samples": 0,
            "micro_steps": engine.micro_steps,
            "dp_world_size": engine.world, "mp_world_size": 1,
            "ds_config": {"zero_optimization": {"stage": engine.cfg.zero_stage}, "bf16": {"enabled": True},
                          "gradient_accumulation_steps": engine.cfg.gradient_accumulation_steps,
                          "gradient_clipping": engine.cfg.max_grad_norm},
            "ds_version": DS_VERSION,
            "b200_layout": _layout_of(engine),
        }
        f = d / "mp_rank_00_model_states.pt"
        torch.save(state, f)
        files.append(str(f))
    if not engine.forward_only:
        host = lambda t: t.detach().to("cpu").clone()
        optim = {
            "optimizer_state_dict": {
                "zero_stage": engine.cfg.zero_stage, "partition_count": [engine.world], "loss_scaler": None,
                "dynamic_loss_scale": False, "overflow": False, "clip_grad": engine.cfg.max_grad_norm,
                "base_optimizer_state": {
                    "state": {0: {"exp_avg": host(engine.exp_avg), "exp_avg_sq": host(engine.exp_avg_sq),
                                  "step": engine.global_steps}},
                    "param_groups": [{"lr": engine.cfg.lr, "betas": tuple(engine.cfg.betas), "eps": engine.cfg.eps,
                                      "weight_decay": engine.cfg.weight_decay, "params": [0]}]},
                "single_partition_of_fp32_groups": [host(engine.master)],
                "group_paddings": [0],
            },
            "ds_config": {"zero_optimization": {"stage": engine.cfg.zero_stage}},
            "ds_version": DS_VERSION,
        }
        f = d / f"bf16_zero_pp_rank_{engine.rank}_mp_rank_00_optim_states.pt"
        torch.save(optim, f)
        files.append(str(f))
    _barrier(engine)
    if engine.rank == 0:
        (root / "latest").write_text(tag)
        if export_hf:
            from ..models.hf_io import save_hf_checkpoint
            tensors = module.items() if collective_export else None   # gathered above
            files += [str(root / "hf" / x) for x in save_hf_checkpoint(engine.model, root / "hf", tensors=tensors)]
    _barrier(engine)
    return {"path": str(d), "tag": tag, "files": files, "global_step": engine.global_steps,
            "hf_path": str(root / "hf") if export_hf else None}


def _locate(load_dir: str, tag: Optional[str]) -> Optional[Path]:
    """The directory that holds ``mp_rank_00_model_states.pt``: ``load_dir/<tag>``, the tag named by
    ``load_dir/latest``, or ``load_dir`` itself when it is a tag directory."""
    root = Path(load_dir)
    if tag is not None:
        return root / tag
    if (root / "mp_rank_00_model_states.pt").is_file():
        return root
    latest = root / "latest"
    if latest.is_file():
        name = latest.read_text().strip()
        for cand in (root / name, root / f"global_step{name}", root / f"checkpoint-{name}"):
            if (cand / "mp_rank_00_model_states.pt").is_file():
                return cand
            if (cand / "latest").is_file():                      # a job root: descend into its newest checkpoint
                return _locate(str(cand), None)
        return root / name
    return None


def load_checkpoint(engine, load_dir: str, tag: Optional[str] = None, strict: bool = False) -> int:
    """Restores module weights, optimizer partition, learning-rate schedule and step counters; returns
    ``global_steps``.  A directory without any checkpoint returns 0 (a fresh start) unless ``strict`` is set or a
    tag was named, in which case it raises ``FileNotFoundError``."""
    if hasattr(engine, "require_awake"):
        engine.require_awake("load_checkpoint")
    d = _locate(load_dir, tag)
    if d is None:
        if strict:
            raise FileNotFoundError(f"no checkpoint under {load_dir} (no 'latest' file and no model-states file)")
        return 0
    ms = d / "mp_rank_00_model_states.pt"
    if not ms.exists():
        raise FileNotFoundError(f"{ms} not found")
    state = _load_pt(ms)
    if state.get("dp_world_size", 1) != engine.world and not engine.forward_only:
        raise ValueError(f"checkpoint was written with {state.get('dp_world_size')} data-parallel ranks, this job has "
                         f"{engine.world}; use the hf/ export to change the world size")
    saved_layout = state.get("b200_layout")
    if saved_layout is not None and not engine.forward_only:
        mine = _layout_of(engine)
        if int(saved_layout.get("total", -1)) != mine["total"] or \
                [tuple(u) for u in saved_layout.get("units", [])] != [tuple(u) for u in mine["units"]]:
            raise ValueError("the checkpoint's optimizer partition was written for a different parameter layout "
                             f"({saved_layout.get('total')} vs {mine['total']} flat elements); load the hf/ export instead")
    from ..models.hf_io import load_hf_tensor
    if getattr(engine, "zero3", None) is not None:
        # stage 3: load into a temporary full buffer, then cut this rank's shard out of it
        full = torch.empty(engine.total, dtype=engine.param_dtype, device=engine.device)
        saved = {}
        for u in engine.units:
            for name, p in u.params:
                o, n, shape = engine.param_slices[name]
                saved[name] = p.data
                p.data = full[o:o + n].view(shape)
        try:
            for name, t in state["module"].items():
                load_hf_tensor(engine.model, name, t)
        finally:
            for u in engine.units:
                for name, p in u.params:
                    p.data = saved[name]
        engine.load_full_flat(full)
    else:
        for name, t in state["module"].items():
            load_hf_tensor(engine.model, name, t)
    bufs = dict(engine.model.named_buffers())
    for name, t in (state.get("buffers") or {}).items():       # e.g. the routers' load-balancing bias
        if name in bufs:
            bufs[name].copy_(t.to(bufs[name].device))
    engine.global_steps = int(state.get("global_steps", 0))
    engine.micro_steps = int(state.get("micro_steps", 0))
    if not engine.forward_only:
        f = d / f"bf16_zero_pp_rank_{engine.rank}_mp_rank_00_optim_states.pt"
        osd = _load_pt(f)["optimizer_state_dict"]
        base = osd["base_optimizer_state"]["state"][0]
        part = osd["single_partition_of_fp32_groups"][0]
        if part.numel() != engine.master.numel():
            raise ValueError(f"optimizer partition of {part.numel()} elements does not fit this rank's "
                             f"{engine.master.numel()} (different world size or ZeRO stage)")
        engine.master.copy_(part)
        engine.exp_avg.copy_(base["exp_avg"])
        engine.exp_avg_sq.copy_(base["exp_avg_sq"])
        groups = osd["base_optimizer_state"].get("param_groups") or []
        if groups and "lr" in groups[0]:
            engine.cfg.lr = float(groups[0]["lr"])
        sched = state.get("lr_scheduler") or {}
        if sched.get("type"):
            from .trainer import SchedulerConfig
            engine.cfg.scheduler = SchedulerConfig(str(sched["type"]), int(sched.get("warmup_steps", 0)),
                                                   int(sched.get("total_steps", 0)), float(sched.get("min_lr_ratio", 0.0)))
    _barrier(engine)
    return engine.global_steps
