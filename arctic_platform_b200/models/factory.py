"""Model specification, loader registry and patch pipeline.

``ModelSpec`` -> ``build_model(spec)`` mirrors arctic_platform/model/{config,factory,loader,patch}.py in the
reference (``ModelSpec``, ``register_loader``, ``resolve_loader_name``, ``LoadedModel``, ``PATCH_ORDER``), but
the patches are *switches on a native model* rather than monkey patches of Hugging Face modules:

* ``liger``        -> the fused RMSNorm / RoPE / SwiGLU kernels are always on for CUDA tensors (no-op here),
* ``zorro_train``  -> recorded on the model (``model.zorro``) and consumed by the pipeline's layout builder,
* ``gradient_checkpointing`` -> ``model.gradient_checkpointing = True``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from .config import DecoderConfig, resolve_config
from .decoder import DecoderLM

PATCH_ORDER = ("liger", "zorro_train", "tiled_mlp", "gradient_checkpointing")


def _tiled_mlp_setting(v) -> Any:
    """``tiled_mlp`` of the worker config: ``True`` / ``"auto"`` / an int / ``{"enable": ..., "shards": ...}``."""
    if isinstance(v, dict):
        if not v.get("enable", True):
            return 0
        v = v.get("shards", "auto")
    if v is True:
        return "auto"
    return v or 0


@dataclass
class ZorroTrainPatch:
    response_len: int = 0
    max_token_len: int = 0
    rollout_n: int = 1
    temperature: float = 1.0
    use_unpad: bool = True
    world_size: int = 1
    logits_optimization: str = "memory"          # none | memory | compute (all map to the fused lm-head kernel)
    logits_optimization_peak_mem_size_in_gib: float = 4.0
    logits_compute_from_fp32_inputs: bool = False
    logits_compute_in_fp32: bool = True

    def __post_init__(self):
        if self.logits_optimization not in ("none", "memory", "compute"):
            raise ValueError(f"logits_optimization must be none|memory|compute, got {self.logits_optimization!r}")


@dataclass
class ParallelismConfig:
    expert_parallel: int = 1
    sequence_parallel: int = 1


@dataclass
class Patches:
    liger: bool = True
    zorro_train: Optional[ZorroTrainPatch] = None
    gradient_checkpointing: bool = False
    tiled_mlp: Any = 0                     # row tiles of the dense MLP: an int, "auto" (ceil(tokens / hidden)) or 0


@dataclass
class ModelSpec:
    model_path_or_name: str
    dtype: str = "bfloat16"
    attn_implementation: Optional[str] = None       # accepted for compatibility; attention is always the tcgen05 kernel
    loader: Optional[str] = None
    parallelism: ParallelismConfig = field(default_factory=ParallelismConfig)
    patches: Patches = field(default_factory=Patches)
    loader_options: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_ds_worker_config(model_name: str, ds_worker_config: Optional[dict]) -> "ModelSpec":
        """Bridge from the free-form worker config dict: gradient checkpointing defaults to on, ``zorro_train``
        sub-dict becomes a :class:`ZorroTrainPatch`."""
        wc = dict(ds_worker_config or {})
        z = wc.get("zorro_train")
        patches = Patches(liger=bool(wc.get("liger", True)),
                          zorro_train=ZorroTrainPatch(**{k: v for k, v in z.items() if k != "enable"})
                          if isinstance(z, dict) and z.get("enable", True) else None,
                          gradient_checkpointing=bool(wc.get("gradient_checkpointing", True)),
                          tiled_mlp=_tiled_mlp_setting(wc.get("tiled_mlp")))
        par = ParallelismConfig(expert_parallel=int(wc.get("expert_parallel", 1)),
                                sequence_parallel=int(wc.get("sequence_parallel", 1)))
        return ModelSpec(model_name, dtype=wc.get("dtype", "bfloat16"), attn_implementation=wc.get("attn_implementation"),
                         parallelism=par, patches=patches, loader_options=dict(wc.get("loader_options") or {}))


@dataclass
class LoaderContext:
    spec: ModelSpec
    _cfg: Optional[DecoderConfig] = None

    @property
    def hf_config(self) -> DecoderConfig:
        if self._cfg is None:
            self._cfg = resolve_config(self.spec.model_path_or_name)
        return self._cfg


@dataclass
class LoadedModel:
    model: DecoderLM
    applied_patches: List[str] = field(default_factory=list)


_LOADERS: Dict[str, Tuple[Callable, Optional[Callable], bool]] = {}
_LOADER_OPTIONS: Dict[str, Any] = {}


def register_loader(name: str, matches: Optional[Callable[[LoaderContext], bool]] = None, default: bool = False,
                    options: Any = None):
    """``options``: a class with ``from_dict(dict)`` that validates ``ModelSpec.loader_options`` for this loader
    (arctic_platform/model/loader.py:83-107 registers a pydantic model for the same purpose)."""
    def deco(fn):
        _LOADERS[name] = (fn, matches, default)
        _LOADER_OPTIONS[name] = options
        return fn
    return deco


def is_registered_loader(name: str) -> bool:
    return name in _LOADERS


def select_loader(ctx: LoaderContext) -> Callable:
    """The loader function ``build_model`` would call for this context (explicit ``spec.loader``, else the one
    loader whose ``matches`` accepts the context, else the default)."""
    return _LOADERS[resolve_loader_name(ctx)][0]


# user patches: callables ``patch(model, ctx)`` that run after the built-in switches, in registration order, when the
# spec asks for them (``ModelSpec.loader_options["patches"] = [name, ...]``) -- arctic_platform/model/patch.py:40-49
_USER_PATCHES: Dict[str, Callable] = {}


def register_patch(name: str):
    def deco(fn):
        if name in PATCH_ORDER or name in _USER_PATCHES:
            raise ValueError(f"patch {name!r} is already registered")
        _USER_PATCHES[name] = fn
        return fn
    return deco


def get_loader_options_model(name: str):
    """The options schema registered for a loader, or ``None``."""
    if name not in _LOADERS:
        raise KeyError(f"unknown loader {name!r} (known: {sorted(_LOADERS)})")
    return _LOADER_OPTIONS.get(name)


def resolve_loader_name(ctx: LoaderContext) -> str:
    if ctx.spec.loader:
        if ctx.spec.loader not in _LOADERS:
            raise KeyError(f"unknown loader {ctx.spec.loader!r} (known: {sorted(_LOADERS)})")
        return ctx.spec.loader
    hits = [n for n, (_, m, _) in _LOADERS.items() if m is not None and m(ctx)]
    if len(hits) == 1:
        return hits[0]
    if len(hits) > 1:
        raise ValueError(f"several loaders match this model: {hits}; set ModelSpec.loader")
    defaults = [n for n, (_, _, d) in _LOADERS.items() if d]
    if not defaults:
        raise ValueError("no loader matches and no default loader is registered")
    return defaults[0]


def _torch_dtype(name: str) -> torch.dtype:
    return {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[name]


def _options_schema():
    from .loader_options import LoaderOptions
    return LoaderOptions


@register_loader("dense", default=True, options=_options_schema())
def _load_dense(ctx: LoaderContext, device, seed: int) -> DecoderLM:
    if ctx.spec.parallelism.expert_parallel > 1:
        raise ValueError("the dense loader does not take expert_parallel > 1")
    return _instantiate(ctx, device, seed)


@register_loader("moe", matches=lambda c: c.hf_config.is_moe, options=_options_schema())
def _load_moe(ctx: LoaderContext, device, seed: int) -> DecoderLM:
    model = _instantiate(ctx, device, seed)
    if ctx.spec.parallelism.expert_parallel > 1:
        from ..parallel.expert_parallel import attach_expert_parallel
        attach_expert_parallel(model, ctx.spec.parallelism.expert_parallel)
    return model


def _instantiate(ctx: LoaderContext, device, seed: int) -> DecoderLM:
    from pathlib import Path
    from .conversion_cache import load_through_cache
    dev = torch.device(device)
    dtype = _torch_dtype(ctx.spec.dtype) if dev.type == "cuda" else torch.float32
    cfg = ctx.hf_config
    debug = ctx.spec.loader_options.get("debug") or {}
    if debug.get("num_layers") is not None:                    # test-only: a shallower model of the same family
        import dataclasses
        n, lt = int(debug["num_layers"]), cfg.layer_types
        cfg = dataclasses.replace(cfg, num_layers=n, layer_types=None if lt is None else tuple(lt[:n]))
    model = DecoderLM(cfg, dev, dtype)
    p = Path(ctx.spec.model_path_or_name)
    if p.is_dir() and any(p.glob("*.safetensors")) and not debug.get("random_init"):
        load_through_cache(model, p, cache_dir=ctx.spec.loader_options.get("weight_conversion_cache_dir"))
        model.source_dir = str(p)
    else:
        model.init_weights(seed=seed)
    return model


def apply_patches(model: DecoderLM, patches: Patches) -> List[str]:
    """Applies the enabled switches in ``PATCH_ORDER``; idempotent (a second call adds nothing)."""
    done = list(getattr(model, "_applied_patches", []))
    for name in PATCH_ORDER:
        if name in done:
            continue
        if name == "liger" and patches.liger:
            done.append(name)
        elif name == "zorro_train" and patches.zorro_train is not None:
            model.zorro = patches.zorro_train
            done.append(name)
        elif name == "tiled_mlp" and patches.tiled_mlp:
            for blk in model.blocks:
                blk.tiled_mlp_shards = patches.tiled_mlp
            done.append(name)
        elif name == "gradient_checkpointing" and patches.gradient_checkpointing:
            model.gradient_checkpointing = True
            done.append(name)
    model._applied_patches = done
    return done


def build_model(spec: ModelSpec, parallel_groups: Optional[dict] = None, device="cpu", seed: int = 42) -> LoadedModel:
    ctx = LoaderContext(spec)
    name = resolve_loader_name(ctx)
    fn, _, _ = _LOADERS[name]
    schema = _LOADER_OPTIONS.get(name)
    opts = schema.from_dict(spec.loader_options) if schema is not None else None     # raises on unknown / bad options
    model = fn(ctx, device, seed)
    applied = apply_patches(model, spec.patches)
    for pname in getattr(opts, "patches", None) or []:
        if pname not in _USER_PATCHES:
            raise KeyError(f"unknown patch {pname!r} (registered: {sorted(_USER_PATCHES)})")
        if pname not in applied:
            _USER_PATCHES[pname](model, ctx)
            applied.append(pname)
            model._applied_patches = applied
    ac = getattr(opts, "ac_config", None)
    if ac is not None:
        model.set_activation_checkpointing(ac.mode, ac.targets, ac.freq)
        if "gradient_checkpointing" not in applied:
            applied.append("gradient_checkpointing")
            model._applied_patches = applied
    chunk = getattr(opts, "tiled_mlp_token_chunk_size", None)
    if chunk is not None and "tiled_mlp" not in applied:
        for blk in model.blocks:
            blk.tiled_mlp_shards = f"chunk:{int(chunk)}"
        applied.append("tiled_mlp")
        model._applied_patches = applied
    return LoadedModel(model, applied)
