"""Import-compatibility alias: ``arctic_platform.<x>`` resolves to ``arctic_platform_b200.<x>``.

Code written against the reference platform (``from arctic_platform.rl import ArcticRLClientConfig,
create_arctic_rl_client``; ``from arctic_platform import wire``; ``arctic_platform.integrations.verl...``) runs on this
build without edits.  The alias is a meta-path finder, so every sub-module is the SAME module object under both names
(no second copy, registries and singletons stay single)."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

_TARGET = "arctic_platform_b200"
_ALIAS = __name__

# where the reference keeps a module under a different path than this build
_MOVED = {
    "common.deepspeed_worker": "engine.worker",
    "common.utils.debug": "utils.debug",
    "common.utils.sft_profile": "utils.sft_profile",
    "common.utils.record_replay": "utils.record_replay",
    "rl.zorro_train.zorro_train": "rl.zorro_train.layout",
    "model": "models",
    "model.config": "models.factory",
    "model.factory": "models.factory",
    "model.loader": "models.factory",
    "model.patch": "models.factory",
    "model.loaders": "models",
    "model.loaders.huggingface": "models.hf_io",
    "model.loaders.qwen3_5_moe": "models.loader_options",
    "model.patches": "models",
    "model.patches.liger": "ops.norm",
    "model.patches.zorro_train": "rl.zorro_train.layout",
    "model.patches.gradient_checkpointing": "models.decoder",
    "model.implementations": "models",
    "model.implementations.qwen35": "models",
    "model.implementations.qwen35.config": "models.config",
    "model.implementations.qwen35.config_validation": "models.config",
    "model.implementations.qwen35.conversion_cache": "models.conversion_cache",
    "model.implementations.qwen35.deepspeed_integration": "engine.trainer",
    "model.implementations.qwen35.distributed": "parallel",
    "model.implementations.qwen35.distributed.deepep": "parallel.expert_parallel",
    "model.implementations.qwen35.distributed.expert_parallel": "parallel.expert_parallel",
    "model.implementations.qwen35.gpu": "utils",
    "model.implementations.qwen35.gpu.action_masks": "utils.action_masks",
    "model.implementations.qwen35.gpu.activation_offload": "utils.activation_offload",
    "model.implementations.qwen35.gpu.debug": "utils.debug",
    "model.implementations.qwen35.gpu.router_replay_recompute": "models.moe",
    "model.implementations.qwen35.gpu.tiled_mlp": "models.tiled_mlp",
    "model.implementations.qwen35.logging_utils": "utils.debug",
    "model.implementations.qwen35.model_builder": "models.factory",
    "model.implementations.qwen35.parallel_dims": "parallel.parallel_dims",
    "model.implementations.qwen35.sequence_parallel": "parallel.ulysses",
    "model.implementations.qwen35.models": "models",
    "model.implementations.qwen35.models.base": "models.decoder",
    "model.implementations.qwen35.models.layers": "models",
    "model.implementations.qwen35.models.layers.checkpointing": "models.decoder",
    "model.implementations.qwen35.models.layers.lm_head": "ops.logprob",
    "model.implementations.qwen35.models.layers.moe": "models.moe",
    "model.implementations.qwen35.models.layers.rotary_emb": "models.decoder",
    "model.implementations.qwen35.models.qwen3_5_moe": "models",
    "model.implementations.qwen35.models.qwen3_5_moe.configuration_qwen3_5_moe": "models.config",
    "model.implementations.qwen35.models.qwen3_5_moe.converting_qwen3_5_moe": "models.hf_io",
    "model.implementations.qwen35.models.qwen3_5_moe.modeling_qwen3_5_moe": "models.decoder",
    "model.implementations.qwen35.vlm": "models.vlm",
    "client.examples": "sft.examples",
    "client.examples.sft_example": "sft.examples.sft_example",
    "model.implementations.qwen35.weights": "models.hf_io",
    "model.implementations.qwen35.world": "parallel.world",
    "rl.processors.grpo": "rl.processors.losses",
    "rl.processors.sft": "sft.processor",
    "rl.processors.verl_grpo": "rl.processors.losses",
    "rl.zorro_train.demo": "rl.zorro_train.harness",
    "rl.zorro_train.tests": "rl.zorro_train.harness",
    "rl.zorro_train.test_perf": "rl.zorro_train.harness",
    "rl.zorro_train.module_patcher": "rl.zorro_train.layout",
    "rl.zorro_train.qwen_attention_patcher": "rl.zorro_train.layout",
    "rl.zorro_train.qwen_model_patcher": "rl.zorro_train.layout",
    "client.sft_client": "sft.client",
    "client.sft_config": "sft.config",
    "client.transports.onprem_http": "client.transports.onprem",
    "client.transports.onprem_ray": "client.transports.ray_actor",
    # the reference's own back-compat shims under rl/ (its code moved to common/)
    "rl.server": "common.server",
    "rl.ray_cluster": "common.ray_cluster",
    "rl.ray_server": "common.ray_server",
    "rl.deepspeed_worker": "engine.worker",
    "rl.utils": "common.utils",
    "rl.utils.batch": "common.utils.batch",
    "rl.utils.cuda_ipc": "common.utils.cuda_ipc",
    "rl.utils.ray_pg": "common.utils.ray_pg",
    "rl.utils.server_models": "common.utils.server_models",
    "rl.utils.debug": "utils.debug",
    "rl.utils.record_replay": "utils.record_replay",
}


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, real_name: str, alias_path: str = ""):
        self.real_name = real_name
        self.alias_path = alias_path

    def create_module(self, spec):
        mod = importlib.import_module(self.real_name)
        self._real_spec = mod.__spec__
        return mod

    def exec_module(self, module):
        # already executed under its real name; the import machinery has just stamped the alias spec on it -- put the
        # real one back, the module's own relative imports go by it
        module.__spec__ = self._real_spec
        from ._names import COMPAT_NAMES
        for name, (where, attr) in COMPAT_NAMES.get(self.alias_path, {}).items():
            if name not in vars(module):
                setattr(module, name, getattr(importlib.import_module(f"{_TARGET}.{where}"), attr))


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        rest = fullname[len(_ALIAS) + 1:]
        real = _TARGET + "." + _MOVED.get(rest, rest)
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        mod = importlib.import_module(real)
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real, rest), is_package=hasattr(mod, "__path__"))


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())

_pkg = importlib.import_module(_TARGET)
__version__ = getattr(_pkg, "__version__", "0.1.0")


def __getattr__(name):                      # ``from arctic_platform import wire`` / ``arctic_platform.rl``
    try:
        return importlib.import_module(f"{_ALIAS}.{name}")
    except ImportError:
        return getattr(_pkg, name)
