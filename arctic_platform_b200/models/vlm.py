"""Vision-language checkpoints on the text-only training path.

A composite checkpoint (``Qwen3VL*`` / ``Qwen3.5*`` with a vision tower) keeps its language model under
``model.language_model.*``, its vision encoder under ``model.visual.*`` and nests the decoder's hyper-parameters in
``text_config``.  Post-training here updates the language model only, so the platform

* reads the decoder configuration out of the composite ``config.json`` (:func:`text_config_of`),
* maps tensor names between the composite layout and the plain decoder layout (:func:`text_name` /
  :func:`composite_name`),
* carries every tensor that is not part of the language model (the vision tower, multi-token-prediction heads)
  through load -> train -> export untouched (:class:`PassthroughTensors`), and
* renames tensors for an inference engine that wraps the language model once more (:func:`sampler_name`).

Same registry and helpers as arctic_platform/model/implementations/qwen35/vlm.py:14-106 and the sampler rename of
arctic_platform/model/implementations/qwen35/deepspeed_integration.py:195-208."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterator, Optional, Tuple

import torch


@dataclass(frozen=True)
class VLMModelInfo:
    """Where a model family keeps its two halves (dotted attribute paths == tensor-name prefixes)."""
    vision_encoder_attr: str
    language_model_attr: str


VLM_REGISTRY: Dict[str, VLMModelInfo] = {
    mt: VLMModelInfo("model.visual", "model.language_model")
    for mt in ("qwen3_vl", "qwen3_vl_moe", "qwen3_5", "qwen3_5_moe")
}

DEFAULT_LAYER_PREFIX = "model.layers."
# tensors of a composite checkpoint that are neither language model nor vision tower but still travel with it
_PASSTHROUGH_PREFIXES = ("mtp.", "model.mtp.")


def _model_type(cfg: Any) -> Optional[str]:
    if isinstance(cfg, dict):
        return cfg.get("model_type")
    return getattr(cfg, "model_type", None)


def vlm_info(cfg: Any) -> Optional[VLMModelInfo]:
    mt = _model_type(cfg)
    return VLM_REGISTRY.get(mt) if mt else None


def is_vlm_architecture(cfg: Any) -> bool:
    """True when the checkpoint behind ``cfg`` has a vision half.  A raw ``config.json`` dict: a registered family
    that nests ``text_config`` / ``vision_config``; the platform's decoder configuration: its ``vlm_layout`` flag;
    any other configuration object: a registered ``model_type``."""
    if isinstance(cfg, dict):
        return vlm_info(cfg) is not None and ("vision_config" in cfg or "text_config" in cfg)
    if hasattr(cfg, "vlm_layout"):
        return bool(cfg.vlm_layout)
    return vlm_info(cfg) is not None


def get_layer_prefix(cfg: Any, override: Optional[str] = None) -> str:
    """Name prefix of the decoder layers' tensors."""
    if override is not None:
        return override
    if not is_vlm_architecture(cfg):
        return DEFAULT_LAYER_PREFIX
    info = vlm_info(cfg) or VLM_REGISTRY["qwen3_5_moe"]
    return info.language_model_attr + ".layers."


def _resolve(obj: Any, dotted: str) -> Any:
    for part in dotted.split("."):
        obj = getattr(obj, part, None)
        if obj is None:
            return None
    return obj


def get_language_model(model: Any, override: Optional[str] = None) -> Any:
    """The module that owns the decoder layers: a configured path, the registry's path, ``model.model`` of a wrapped
    text model, or the model itself (the platform's own decoder has no wrapper)."""
    if override is not None:
        found = _resolve(model, override)
        if found is None:
            raise ValueError(f"language_model_attr={override!r} does not resolve on this model")
        return found
    info = vlm_info(getattr(model, "config", None) or getattr(model, "cfg", None))
    if info is not None:
        found = _resolve(model, info.language_model_attr)
        if found is not None:
            return found
    return getattr(model, "model", model)


def get_vision_encoder(model: Any, override: Optional[str] = None) -> Any:
    """The vision encoder module, or ``None`` on the text-only path."""
    if override is not None:
        found = _resolve(model, override)
        if found is None:
            raise ValueError(f"vision_encoder_attr={override!r} does not resolve on this model")
        return found
    info = vlm_info(getattr(model, "config", None) or getattr(model, "cfg", None))
    return _resolve(model, info.vision_encoder_attr) if info is not None else None


# ----------------------------------------------------------------------------- configuration
def text_config_of(d: Dict[str, Any]) -> Tuple[Dict[str, Any], bool]:
    """``(decoder configuration, is_composite)`` of a ``config.json`` dict.  A composite configuration nests the
    decoder under ``text_config``; ``tie_word_embeddings`` may sit on either level."""
    if "text_config" not in d:
        return d, False
    text = dict(d["text_config"])
    if "tie_word_embeddings" not in text and "tie_word_embeddings" in d:
        text["tie_word_embeddings"] = d["tie_word_embeddings"]
    text.setdefault("model_type", (d.get("model_type") or "qwen3") + "_text")
    return text, True


def composite_config(text: Dict[str, Any], extra: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    """Inverse of :func:`text_config_of`: re-nests ``text`` into the composite dict it came from (``extra`` holds
    the top level without its ``text_config``)."""
    out = dict(extra or {})
    out["text_config"] = text
    if "tie_word_embeddings" in text:
        out.setdefault("tie_word_embeddings", text["tie_word_embeddings"])
    return out


# ----------------------------------------------------------------------------- tensor names
def text_name(name: str, info: VLMModelInfo = VLM_REGISTRY["qwen3_5_moe"]) -> Optional[str]:
    """Composite tensor name -> plain decoder name (``model.language_model.layers.0...`` -> ``model.layers.0...``);
    ``None`` for tensors outside the language model (vision tower, multi-token-prediction heads)."""
    lm = info.language_model_attr + "."
    if name.startswith(lm):
        return "model." + name[len(lm):]
    if name.startswith(info.vision_encoder_attr + ".") or name.startswith(_PASSTHROUGH_PREFIXES):
        return None
    return name                                    # lm_head.weight and plain text checkpoints


def composite_name(name: str, info: VLMModelInfo = VLM_REGISTRY["qwen3_5_moe"]) -> str:
    """Plain decoder name -> composite name."""
    if name.startswith("model.") and not name.startswith(info.language_model_attr + ".") \
            and not name.startswith(info.vision_encoder_attr + "."):
        return info.language_model_attr + "." + name[len("model."):]
    return name


def sampler_name(name: str, info: VLMModelInfo = VLM_REGISTRY["qwen3_5_moe"]) -> str:
    """Composite name -> the layout of an inference engine whose VLM class holds ``visual`` and a complete causal
    LM under ``language_model``."""
    vis, lm = info.vision_encoder_attr + ".", info.language_model_attr + "."
    if name.startswith(vis):
        return "visual." + name[len(vis):]
    if name.startswith(lm):
        return "language_model.model." + name[len(lm):]
    if name.startswith("lm_head."):
        return "language_model." + name
    raise KeyError(f"no inference-engine name for composite tensor {name!r}")


class PassthroughTensors:
    """Tensors of a composite checkpoint that training never touches.  They are kept on the host in the dtype they
    were read in and written back unchanged by the exporter, so a trained checkpoint is a drop-in replacement for
    the one that was loaded."""

    def __init__(self) -> None:
        self.tensors: Dict[str, torch.Tensor] = {}

    def add(self, name: str, tensor: torch.Tensor) -> None:
        self.tensors[name] = tensor.detach().to("cpu").clone()

    def __len__(self) -> int:
        return len(self.tensors)

    def __iter__(self) -> Iterator[Tuple[str, torch.Tensor]]:
        return iter(sorted(self.tensors.items()))

    def num_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())
