"""Code written against the reference's package name runs unchanged: ``arctic_platform.*`` is this build."""
import importlib

import pytest


def test_reference_import_paths_resolve_to_the_same_modules():
    import arctic_platform
    import arctic_platform_b200
    from arctic_platform import wire
    from arctic_platform.rl import ArcticRLClientConfig, create_arctic_rl_client
    import arctic_platform.common.registry as reg
    from arctic_platform_b200 import wire as real_wire
    from arctic_platform_b200.common import registry as real_reg
    from arctic_platform_b200.rl import create_arctic_rl_client as real_create
    assert wire is real_wire and reg is real_reg and create_arctic_rl_client is real_create
    assert reg.LOSS_FNS is real_reg.LOSS_FNS                          # one registry, not two
    assert importlib.import_module("arctic_platform.integrations.verl.adapter") is \
        importlib.import_module("arctic_platform_b200.integrations.verl.adapter")
    # modules the reference keeps elsewhere
    from arctic_platform.common.deepspeed_worker import EngineWorker
    from arctic_platform.common.utils.debug import see_memory_usage
    from arctic_platform_b200.engine.worker import EngineWorker as RealWorker
    assert EngineWorker is RealWorker and callable(see_memory_usage)
    assert arctic_platform.rl is arctic_platform_b200.rl
    with pytest.raises(ImportError):
        importlib.import_module("arctic_platform.no_such_module")
    # and it works end to end
    c = create_arctic_rl_client(ArcticRLClientConfig(comm_protocol="local", model_name="qwen3-tiny", training_gpus=0,
                                                     sampling_gpus=1, log_prob_gpus=0, vllm_config={"max_model_len": 32}))
    assert len(c.call("generate", [[3, 4]], {"n": 1, "max_tokens": 2})) == 1
    c.call("shutdown")


def test_reference_shim_paths_and_ipc_merge():
    # the reference keeps back-compat shims under rl/ for code that moved to common/: both spellings work here too
    from arctic_platform.rl.server import ArcticRLServerCore
    from arctic_platform_b200.common.server import ArcticRLServerCore as Real
    assert ArcticRLServerCore is Real
    assert importlib.import_module("arctic_platform.rl.ray_cluster") is importlib.import_module("arctic_platform_b200.common.ray_cluster")
    assert importlib.import_module("arctic_platform.rl.deepspeed_worker") is importlib.import_module("arctic_platform_b200.engine.worker")
    for leaf, real in (("batch", "common.utils.batch"), ("ray_pg", "common.utils.ray_pg"), ("server_models", "common.utils.server_models"),
                       ("debug", "utils.debug"), ("record_replay", "utils.record_replay"), ("cuda_ipc", "common.utils.cuda_ipc")):
        assert importlib.import_module(f"arctic_platform.rl.utils.{leaf}") is importlib.import_module(f"arctic_platform_b200.{real}")
    from arctic_platform.common.ray_server import create_arctic_rl_ray_server_state
    assert callable(create_arctic_rl_ray_server_state)

    from arctic_platform.common.utils.cuda_ipc import merge_cuda_ipc_payloads, merge_ipc_sources
    layout = {"total": 100, "world": 2, "zero3": None, "params": {"a": (0, 10, (10,))}}
    srcs = [{"handle": b"h0", "offset": 0, "layout": layout, "device": 0}, {"handle": b"h1", "offset": 0, "layout": layout, "device": 1}]
    merged = merge_ipc_sources(srcs)
    assert [s["device"] for s in merged] == [0, 1] and merged[0] is not srcs[0]
    assert merge_ipc_sources([srcs[0], None]) is None and merge_ipc_sources([]) is None
    assert merge_cuda_ipc_payloads(srcs) == {"sources": merged, "num_ranks": 2, "num_params": 1}
    assert merge_cuda_ipc_payloads([None, None])["sources"] is None
    with pytest.raises(ValueError, match="same buffer"):
        merge_ipc_sources([srcs[0], dict(srcs[0])])
    with pytest.raises(ValueError, match="another parameter layout"):
        merge_ipc_sources([srcs[0], {**srcs[1], "layout": {**layout, "total": 99}}])
    with pytest.raises(ValueError, match="2 trainer ranks"):
        merge_ipc_sources([srcs[0]])
    with pytest.raises(ValueError, match="offset"):
        merge_ipc_sources([{"handle": b"x", "layout": layout}, srcs[1]])


def test_package_level_names_of_the_reference_resolve(tmp_path):
    import arctic_platform.rl as rl
    import arctic_platform.rl.processors as proc
    import arctic_platform.sft as sft
    from arctic_platform_b200.common import registry
    for name in ("create_arctic_rl_client", "ArcticRLClientConfig", "WeightSyncConfig", "WeightSyncCoordinator", "run_pipeline",
                 "run_sft_pipeline", "register_loss_fn", "register_post_processor", "grpo_loss", "sft_loss", "pack_sequences",
                 "unpack_sequences"):
        assert getattr(rl, name) is not None, name
    assert rl.register_loss_fn is registry.register_loss_fn and rl.run_sft_pipeline is sft.run_sft_pipeline
    for name in ("POST_PROCESSORS", "LOSS_FNS", "register_post_processor", "register_loss_fn", "run_pipeline", "pack_sequences",
                 "unpack_sequences", "pad_packed_for_model", "DEFAULT_MAX_TOKENS_PER_MB", "MicroBatchSpec",
                 "split_padded_tensor_dict_into_mb_list", "DistributedStatsTracker", "ReduceType", "DEFAULT_TRACKER",
                 "denominator", "stat", "scalar", "scope", "export", "masked_normalization", "agg_loss", "kl_penalty",
                 "ppo_actor_loss_fn", "sapo_loss_fn", "grpo_loss", "verl_grpo_loss", "sft_loss", "sft_ce_loss",
                 "ProxLogpMethod", "ProxApproxMethod", "PROX_LOGP_METHOD_RECOMPUTE", "PROX_LOGP_METHOD_LOGLINEAR",
                 "PROX_LOGP_METHOD_METRICS", "PROX_APPROX_METHOD_LOGLINEAR", "PROX_APPROX_METHOD_LINEAR",
                 "PROX_APPROX_METHOD_ROLLOUT", "PROX_APPROX_METHODS_ALL", "compute_prox_logp_approximations",
                 "_resolve_proximal_logp", "_compute_sequence_level_ratio_and_advantages", "LOGIT_LOSS_FNS", "SFT_LOSS_FNS",
                 "run_sft_pipeline"):
        assert getattr(proc, name) is not None, name
    assert {"verl_grpo", "grpo", "sft", "sft_ce"} <= set(proc.LOSS_FNS) and proc.LOSS_FNS is registry.LOSS_FNS
    assert "compute_entropy_and_logprobs" in proc.POST_PROCESSORS
    with pytest.raises(AttributeError):
        proc.no_such_name
    with pytest.raises(AttributeError):
        rl.no_such_name
    for name in ("ArcticSFTClient", "ArcticSFTClientConfig", "LOGIT_LOSS_FNS", "SFT_LOSS_FNS", "create_arctic_sft_client",
                 "run_sft_pipeline", "sft_ce_loss", "sft_loss"):
        assert getattr(sft, name) is not None, name
    c = sft.create_arctic_sft_client(sft.ArcticSFTClientConfig(comm_protocol="local", model_name="qwen3-tiny", training_gpus=1,
                                                               checkpoint_path=str(tmp_path)))
    try:
        import torch
        out = c.fwd_bwd({"input_ids": torch.randint(1, 100, (2, 8)), "attention_mask": torch.ones(2, 8, dtype=torch.long)})
        assert "avg_loss" in out
    finally:
        c.shutdown()


def test_model_package_paths_and_patch_registry():
    import arctic_platform
    for path in arctic_platform._MOVED:                                   # every declared move resolves
        assert importlib.import_module(f"arctic_platform.{path}") is not None, path
    from arctic_platform.model import (LoadedModel, LoaderContext, ModelSpec, Patches, build_model, register_patch,
                                       select_loader)
    from arctic_platform.model.loader import is_registered_loader
    from arctic_platform.model.implementations.qwen35.parallel_dims import ParallelDims
    from arctic_platform_b200.parallel.parallel_dims import ParallelDims as Real
    assert ParallelDims is Real and is_registered_loader("dense") and not is_registered_loader("nope")
    seen = []

    @register_patch("count_blocks_for_test")
    def _count(model, ctx):
        seen.append((len(model.blocks), ctx.spec.model_path_or_name))

    with pytest.raises(ValueError):
        register_patch("count_blocks_for_test")(lambda m, c: None)
    with pytest.raises(ValueError):
        register_patch("liger")(lambda m, c: None)
    spec = ModelSpec("qwen3-tiny", patches=Patches(gradient_checkpointing=True),
                     loader_options={"patches": ["count_blocks_for_test"]})
    assert callable(select_loader(LoaderContext(spec)))
    loaded = build_model(spec)
    assert isinstance(loaded, LoadedModel) and seen and seen[0][1] == "qwen3-tiny"
    assert loaded.applied_patches[-1] == "count_blocks_for_test" and "gradient_checkpointing" in loaded.applied_patches
    with pytest.raises(KeyError, match="unknown patch"):
        build_model(ModelSpec("qwen3-tiny", loader_options={"patches": ["missing"]}))
    with pytest.raises(ValueError, match="patches"):
        build_model(ModelSpec("qwen3-tiny", loader_options={"patches": "count_blocks_for_test"}))


# every module path the reference package has (files under its package directory), as import names below the package
_ALL_REFERENCE_MODULES = """
_dependency_groups client client.client client.config client.examples client.examples.sft_example client.sft_client
client.sft_config client.transport client.transports client.transports.cortex client.transports.onprem
client.transports.onprem_http client.transports.onprem_ray common common.deepspeed_worker common.http_server
common.ray_cluster common.ray_server common.registry common.server common.utils common.utils.batch
common.utils.checkpoint common.utils.cuda_ipc common.utils.debug common.utils.ray_pg common.utils.record_replay
common.utils.server_models common.utils.sft_profile common.utils.tiled_logits common.utils.weight_sync integrations
integrations.verl integrations.verl.adapter integrations.verl.grpo_loss integrations.verl.register
integrations.verl.rollout integrations.verl.worker model model.config model.factory model.implementations
model.implementations.qwen35 model.implementations.qwen35.config model.implementations.qwen35.config_validation
model.implementations.qwen35.conversion_cache model.implementations.qwen35.deepspeed_integration
model.implementations.qwen35.distributed model.implementations.qwen35.distributed.deepep
model.implementations.qwen35.distributed.expert_parallel model.implementations.qwen35.gpu
model.implementations.qwen35.gpu.action_masks model.implementations.qwen35.gpu.activation_offload
model.implementations.qwen35.gpu.debug model.implementations.qwen35.gpu.router_replay_recompute
model.implementations.qwen35.gpu.tiled_mlp model.implementations.qwen35.logging_utils
model.implementations.qwen35.model_builder model.implementations.qwen35.models
model.implementations.qwen35.models.base model.implementations.qwen35.models.layers
model.implementations.qwen35.models.layers.checkpointing model.implementations.qwen35.models.layers.lm_head
model.implementations.qwen35.models.layers.moe model.implementations.qwen35.models.layers.rotary_emb
model.implementations.qwen35.models.qwen3_5_moe
model.implementations.qwen35.models.qwen3_5_moe.configuration_qwen3_5_moe
model.implementations.qwen35.models.qwen3_5_moe.converting_qwen3_5_moe
model.implementations.qwen35.models.qwen3_5_moe.modeling_qwen3_5_moe model.implementations.qwen35.parallel_dims
model.implementations.qwen35.sequence_parallel model.implementations.qwen35.vlm
model.implementations.qwen35.weights model.implementations.qwen35.world model.loader model.loaders
model.loaders.huggingface model.loaders.qwen3_5_moe model.patch model.patches model.patches.gradient_checkpointing
model.patches.liger model.patches.zorro_train rl rl.client rl.config rl.deepspeed_worker
rl.examples.inference_example rl.examples.local_server_example rl.examples.weight_sync_example rl.http_client
rl.http_server rl.processors rl.processors.functional rl.processors.grpo rl.processors.microbatch
rl.processors.packing rl.processors.pipeline rl.processors.sft rl.processors.stats_tracker rl.processors.verl_grpo
rl.ray_client rl.ray_cluster rl.ray_server rl.server rl.utils rl.utils.batch rl.utils.cuda_ipc rl.utils.debug
rl.utils.ray_pg rl.utils.record_replay rl.utils.server_models rl.weight_sync rl.zorro_train rl.zorro_train.actor
rl.zorro_train.demo rl.zorro_train.module_patcher rl.zorro_train.qwen_attention_patcher
rl.zorro_train.qwen_model_patcher rl.zorro_train.seqlen_balancing rl.zorro_train.test_perf rl.zorro_train.tests
rl.zorro_train.zorro_train sft sft.client sft.config sft.examples sft.examples.run_sft_ckpt_resume_demo
sft.examples.run_sft_generate_demo sft.examples.run_sft_http_demo sft.examples.sft_example sft.processor
testing_utils wire
""".split()


def test_every_module_path_of_the_reference_package_imports():
    import importlib

    missing = []
    for name in _ALL_REFERENCE_MODULES:
        try:
            importlib.import_module("arctic_platform." + name)
        except ImportError as exc:
            missing.append(f"{name}: {exc}")
    assert not missing, missing
    assert len(_ALL_REFERENCE_MODULES) == 135
