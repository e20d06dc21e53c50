"""``python setup.py build_ext --inplace`` (or ``pip install -e .``) compiles the native libraries in-tree:
``nvcc -gencode arch=compute_100a,code=sm_100a`` for the kernels, ``g++`` for the host runtime.  Everything else is
declared in ``pyproject.toml``."""
import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_ext import build_ext
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent


def _native_build(force: bool = False) -> None:
    # loaded by path: importing the package would pull in torch, which a build environment may not have
    spec = importlib.util.spec_from_file_location("_apb_build", ROOT / "arctic_platform_b200" / "_build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all(force=force)


class BuildNative(build_ext):
    def run(self):
        _native_build(force=bool(getattr(self, "force", False)))


class BuildPyWithNative(build_py):
    def run(self):
        _native_build()
        super().run()


setup(cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative})
