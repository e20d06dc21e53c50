"""``dss_client``: the import name the reference's stand-alone client installs (cortex-client/dss_client).

``from dss_client import NeutrinoClient, wire`` and ``import dss_client.neutrino_client`` resolve to
``cortex_client.dss_client`` -- the same module objects under both names, so exception classes and caches are not
duplicated.  Modules the reference splits differently are redirected: ``client`` / ``engine`` -> ``engines``,
``neutrino_engine`` / ``common`` -> ``neutrino_client``, ``wire`` -> the platform's wire codec."""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

_ALIAS = __name__
_TARGET = "cortex_client.dss_client"
_MOVED = {
    "client": _TARGET + ".engines",
    "engine": _TARGET + ".engines",
    "neutrino_engine": _TARGET + ".neutrino_client",
    "common": _TARGET + ".neutrino_client",
    "wire": "arctic_platform_b200.wire",
}


class _Loader(importlib.abc.Loader):
    def __init__(self, real_name: str):
        self.real_name = real_name

    def create_module(self, spec):
        mod = importlib.import_module(self.real_name)
        self._real_spec = mod.__spec__
        return mod

    def exec_module(self, module):
        module.__spec__ = self._real_spec          # the module's own relative imports go by its real spec


class _Finder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_ALIAS + "."):
            return None
        rest = fullname[len(_ALIAS) + 1:]
        real = _MOVED.get(rest, f"{_TARGET}.{rest}")
        try:
            if importlib.util.find_spec(real) is None:
                return None
        except (ImportError, ValueError):
            return None
        mod = importlib.import_module(real)
        return importlib.util.spec_from_loader(fullname, _Loader(real), is_package=hasattr(mod, "__path__"))


if not any(isinstance(f, _Finder) for f in sys.meta_path):
    sys.meta_path.insert(0, _Finder())

_pkg = importlib.import_module(_TARGET)
__version__ = getattr(_pkg, "__version__", "0.1.0")
__all__ = [n for n in dir(_pkg) if not n.startswith("_")] + ["wire"]


def __getattr__(name):
    if name in _MOVED or importlib.util.find_spec(f"{_TARGET}.{name}") is not None:
        try:
            return importlib.import_module(f"{_ALIAS}.{name}")
        except ImportError:
            pass
    return getattr(_pkg, name)
