"""``ds_worker_config.loader_options``: the strict schema and what the worker does with each option."""
import pytest
import torch

from arctic_platform_b200.models.loader_options import ActivationCheckpointOptions, LoaderOptions
from arctic_platform_b200.models.tiled_mlp import resolve_shards


def test_defaults_and_nested_blocks():
    lo = LoaderOptions.from_dict(None)
    assert lo.optimization_dtype == "bfloat16" and lo.ac_config is None and lo.debug is None
    lo = LoaderOptions.from_dict({"ac_config": {"mode": "selective", "freq": 2, "offload_config": {"enabled": False}},
                                  "debug": {"random_init": True, "num_layers": 1}, "tiled_mlp_token_chunk_size": 256})
    assert isinstance(lo.ac_config, ActivationCheckpointOptions) and lo.ac_config.targets == ["norm"]
    assert lo.ac_config.to_worker_dicts() == ({"mode": "selective", "freq": 2, "targets": ["norm"]}, None)
    assert lo.debug.random_init and lo.debug.num_layers == 1
    gc, ao = ActivationCheckpointOptions(offload_config={"enabled": True, "keep_last_n": 3}).to_worker_dicts()
    assert gc["mode"] == "full" and ao == {"keep_last": 3, "min_bytes": 1 << 20}


@pytest.mark.parametrize("bad,match", [
    ({"seq_length": 4096}, "unknown option"),
    ({"optimization_dtype": "float16"}, "optimization_dtype"),
    ({"ep_comm_backend": "nccl"}, "ep_comm_backend"),
    ({"fused_lm_head_token_chunk_size": "big"}, "fused_lm_head_token_chunk_size"),
    ({"fp32_lm_head": True}, "cannot combine fused_cross_entropy"),
    ({"fused_lm_head_token_chunk_size": 1024}, "cannot combine fused_cross_entropy"),
    ({"ac_config": {"mode": "some"}}, "ac_config.mode"),
    ({"ac_config": {"target": ["norm"]}}, "unknown option"),
    ({"ac_config": {"offload_config": {"keep": 1}}}, "unknown option"),
    ({"ac_config": {"mode": "selective", "offload_config": {"enabled": True}}}, "requires ac_config.mode='full'"),
    ({"debug": {"layers": 2}}, "unknown option"),
    ({"tiled_mlp_token_chunk_size": 0}, "tiled_mlp_token_chunk_size"),
])
def test_schema_rejects(bad, match):
    with pytest.raises(ValueError, match=match):
        LoaderOptions.from_dict(bad)


def test_fp32_head_is_allowed_without_the_fused_cross_entropy():
    lo = LoaderOptions.from_dict({"fused_cross_entropy": False, "fp32_lm_head": True, "fused_lm_head_token_chunk_size": 512})
    assert lo.fp32_lm_head and lo.fused_lm_head_token_chunk_size == 512


def test_token_chunk_tiles():
    assert resolve_shards("chunk:256", 1000, 64) == 4 and resolve_shards("chunk:4096", 1000, 64) == 1


def test_worker_applies_the_options(tmp_path):
    from arctic_platform_b200.engine.worker import EngineWorker
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.models.hf_io import save_hf_checkpoint
    src = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=5)
    save_hf_checkpoint(src, tmp_path / "ckpt")
    base = {"model_name": str(tmp_path / "ckpt"), "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}}}
    w = EngineWorker("cpu")
    w.initialize({**base, "ds_worker_config": {"loader_options": {
        "ac_config": {"mode": "selective", "targets": ["mlp", "norm"], "freq": 2}, "tiled_mlp_token_chunk_size": 128,
        "weight_conversion_cache_dir": str(tmp_path / "cache")}}})
    m = w.engine.model
    assert m.checkpoint_targets == ("mlp", "norm") and m.checkpoint_freq == 2 and m.gradient_checkpointing
    assert all(b.tiled_mlp_shards == "chunk:128" for b in m.blocks)
    assert torch.equal(m.embed.data, src.embed.data) and any((tmp_path / "cache").iterdir())
    # debug: random weights instead of the checkpoint, truncated depth
    w2 = EngineWorker("cpu")
    w2.initialize({**base, "ds_worker_config": {"loader_options": {"debug": {"random_init": True, "num_layers": 1},
                                                                   "optimization_dtype": "bfloat16"}}})
    m2 = w2.engine.model
    assert len(m2.blocks) == 1 and m2.embed.dtype == torch.bfloat16 and not torch.equal(m2.embed.data.float(), src.embed.data)
    with pytest.raises(ValueError, match="unknown option"):
        EngineWorker("cpu").initialize({**base, "ds_worker_config": {"loader_options": {"atn": "sdpa"}}})


def test_model_builder_validates_and_applies_the_options():
    from arctic_platform_b200.models.factory import ModelSpec, build_model, get_loader_options_model
    assert get_loader_options_model("dense") is LoaderOptions and get_loader_options_model("moe") is LoaderOptions
    with pytest.raises(KeyError):
        get_loader_options_model("nope")
    spec = ModelSpec("qwen3.5-moe-tiny", loader_options={"debug": {"num_layers": 2, "random_init": True},
                                                         "ac_config": {"mode": "selective", "targets": ["linear_attn"]},
                                                         "tiled_mlp_token_chunk_size": 64})
    loaded = build_model(spec)
    m = loaded.model
    assert len(m.blocks) == 2 and m.cfg.layer_types == ("linear_attention", "linear_attention")
    assert m.checkpoint_targets == ("linear_attn",) and m.gradient_checkpointing
    assert "gradient_checkpointing" in loaded.applied_patches and "tiled_mlp" in loaded.applied_patches
    with pytest.raises(ValueError, match="unknown option"):
        build_model(ModelSpec("qwen3-tiny", loader_options={"sequence_len": 8}))
    with pytest.raises(ValueError, match="not supported by the selected model layers"):
        build_model(ModelSpec("qwen3-tiny", loader_options={"ac_config": {"mode": "selective", "targets": ["linear_attn"]}}))
