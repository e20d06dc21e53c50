"""Model families (dense / MoE / hybrid decoders), their configs, loaders and the model factory."""

# the factory surface the reference exports from its ``model`` package (arctic_platform/model/__init__.py:21-48),
# resolved on first use so that importing ``models`` stays light
_FACTORY_NAMES = ("LoadedModel", "LoaderContext", "ModelSpec", "ParallelismConfig", "Patches", "ZorroTrainPatch",
                  "apply_patches", "build_model", "register_loader", "register_patch", "select_loader",
                  "is_registered_loader", "get_loader_options_model", "resolve_loader_name")


def __getattr__(name):
    if name in _FACTORY_NAMES:
        from . import factory
        value = getattr(factory, name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
