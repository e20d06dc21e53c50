"""Composite (vision + language) checkpoints on the text-only path: configuration nesting, tensor-name mapping, and
a load -> train -> export round trip that carries the vision tower through unchanged."""
import json

import pytest
import torch

from arctic_platform_b200.models import vlm
from arctic_platform_b200.models.config import PRESETS, DecoderConfig, resolve_config
from arctic_platform_b200.models.decoder import DecoderLM
from arctic_platform_b200.models.hf_io import (iter_hf_tensors, load_hf_checkpoint, read_safetensors, save_hf_checkpoint,
                                               write_safetensors)


def test_registry_and_names():
    assert vlm.is_vlm_architecture({"model_type": "qwen3_5_moe", "text_config": {}, "vision_config": {}})
    assert not vlm.is_vlm_architecture({"model_type": "qwen3_5_moe"})           # text-only export of the family
    assert not vlm.is_vlm_architecture({"model_type": "qwen3"})
    assert vlm.get_layer_prefix({"model_type": "qwen3"}) == "model.layers."
    assert vlm.get_layer_prefix({"model_type": "qwen3_vl", "vision_config": {}}) == "model.language_model.layers."
    assert vlm.get_layer_prefix({"model_type": "qwen3"}, override="x.") == "x."
    n = "model.language_model.layers.3.self_attn.q_proj.weight"
    assert vlm.text_name(n) == "model.layers.3.self_attn.q_proj.weight"
    assert vlm.composite_name(vlm.text_name(n)) == n
    assert vlm.text_name("model.visual.blocks.0.attn.qkv.weight") is None and vlm.text_name("mtp.fc.weight") is None
    assert vlm.text_name("lm_head.weight") == "lm_head.weight" == vlm.composite_name("lm_head.weight")
    assert vlm.text_name("model.layers.0.mlp.gate.weight") == "model.layers.0.mlp.gate.weight"
    assert vlm.sampler_name(n) == "language_model.model.layers.3.self_attn.q_proj.weight"
    assert vlm.sampler_name("model.visual.merger.norm.weight") == "visual.merger.norm.weight"
    assert vlm.sampler_name("lm_head.weight") == "language_model.lm_head.weight"
    with pytest.raises(KeyError):
        vlm.sampler_name("something.else")


def test_module_lookup():
    class Box:
        pass
    m = Box()
    m.config = Box()
    m.config.model_type = "qwen3_5_moe"
    m.model = Box()
    m.model.visual, m.model.language_model = "V", "L"
    assert vlm.get_vision_encoder(m) == "V" and vlm.get_language_model(m) == "L"
    assert vlm.get_language_model(m, override="model.visual") == "V"
    with pytest.raises(ValueError):
        vlm.get_language_model(m, override="model.nothing")
    with pytest.raises(ValueError):
        vlm.get_vision_encoder(m, override="nope")
    text = Box()
    text.config = Box()
    text.config.model_type = "qwen3"
    text.model = "inner"
    assert vlm.get_language_model(text) == "inner" and vlm.get_vision_encoder(text) is None
    own = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32)
    assert vlm.get_language_model(own) is own and vlm.get_vision_encoder(own) is None


def test_composite_checkpoint_round_trip(tmp_path):
    base = PRESETS["qwen3.5-moe-tiny"]
    src = DecoderLM(base, "cpu", torch.float32).init_weights(seed=5)
    # write the tiny model as a composite checkpoint: nested config, composite names, a fake vision tower
    text_cfg = base.to_hf_dict()
    text_cfg.pop("architectures")
    text_cfg["model_type"] = "qwen3_5_moe_text"
    tie = text_cfg.pop("tie_word_embeddings")
    comp = {"architectures": ["Qwen3_5MoeForConditionalGeneration"], "model_type": "qwen3_5_moe", "text_config": text_cfg,
            "vision_config": {"depth": 2, "hidden_size": 32, "patch_size": 16}, "image_token_id": 7,
            "tie_word_embeddings": tie}
    ck = tmp_path / "vlm"
    ck.mkdir()
    (ck / "config.json").write_text(json.dumps(comp))
    g = torch.Generator().manual_seed(1)
    extra = {"model.visual.patch_embed.proj.weight": torch.randn(32, 3, 2, 16, 16, generator=g).to(torch.bfloat16),
             "model.visual.blocks.0.attn.qkv.weight": torch.randn(96, 32, generator=g),
             "mtp.fc.weight": torch.randn(8, 16, generator=g)}
    tensors = {vlm.composite_name(n): t.detach().clone() for n, t in iter_hf_tensors(src)}
    assert any(k.startswith("model.language_model.layers.0.") for k in tensors)
    write_safetensors(ck / "model.safetensors", {**tensors, **extra}, {"format": "pt"})

    cfg = resolve_config(str(ck))
    assert cfg.vlm_layout and vlm.is_vlm_architecture(cfg) and cfg.model_type == "qwen3_5_moe_text"
    assert cfg.layer_types == base.layer_types and cfg.tie_word_embeddings == tie
    assert vlm.get_layer_prefix(cfg) == "model.language_model.layers."
    model = DecoderLM(cfg, "cpu", torch.float32).init_weights(seed=99)
    n = load_hf_checkpoint(model, ck)
    assert n == len(tensors) and len(model.passthrough) == 3
    for (na, a), (nb, b) in zip(iter_hf_tensors(src), iter_hf_tensors(model)):
        assert na == nb and torch.equal(a, b)

    # "train": change a language-model weight, export, and read the export back
    with torch.no_grad():
        model.final_norm.add_(0.25)
    out = tmp_path / "out"
    save_hf_checkpoint(model, out)
    cfg2 = json.loads((out / "config.json").read_text())
    assert cfg2["model_type"] == "qwen3_5_moe" and cfg2["vision_config"]["depth"] == 2 and cfg2["image_token_id"] == 7
    assert cfg2["text_config"]["model_type"] == "qwen3_5_moe_text" and "layer_types" in cfg2["text_config"]
    back = dict(read_safetensors(out / "model.safetensors"))
    assert set(back) == set(tensors) | set(extra)
    for k, t in extra.items():
        assert back[k].dtype == t.dtype and torch.equal(back[k], t)
    assert torch.equal(back["model.language_model.norm.weight"], tensors["model.language_model.norm.weight"] + 0.25)
    # and the export loads again as a composite
    again = DecoderLM(resolve_config(str(out)), "cpu", torch.float32)
    load_hf_checkpoint(again, out)
    assert torch.equal(again.final_norm, model.final_norm) and len(again.passthrough) == 3


def test_plain_config_is_untouched():
    cfg = DecoderConfig.from_hf_dict(PRESETS["qwen3-tiny"].to_hf_dict())
    assert not cfg.vlm_layout and cfg.composite_extra is None and "text_config" not in cfg.to_hf_dict()
