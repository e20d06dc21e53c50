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
