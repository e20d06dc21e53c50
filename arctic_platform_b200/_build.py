"""In-tree build of the native libraries.

Two shared objects are produced under ``arctic_platform_b200/_C``:

* ``libapb200.so``    -- every CUDA kernel of the package, compiled by ``nvcc`` for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``), exported through
  ``extern "C"`` entry points that take raw device pointers and a stream.
* ``libapb200_rt.so`` -- the host runtime (KV page allocator, sequence packing,
  ZoRRo index tables, bucket planner), plain C++17, usable without a GPU.

The objects are rebuilt only when a source (or a header) is newer than the
library.  ``nvcc`` cross-compiles, so the build works on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "_C"
OBJ_DIR = PKG_DIR.parent / "build" / "obj"

CUDA_LIB = OUT_DIR / "libapb200.so"
RT_LIB = OUT_DIR / "libapb200_rt.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _newest_mtime(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def cuda_sources():
    return sorted(CSRC.glob("*.cu"))


def _headers():
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _compile_one(src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    deps = [src] + _headers()
    if obj.exists() and obj.stat().st_mtime >= _newest_mtime(deps):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    srcs = cuda_sources()
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    if (not force and CUDA_LIB.exists()
            and CUDA_LIB.stat().st_mtime >= _newest_mtime(srcs + _headers())):
        return CUDA_LIB
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose), srcs))
    cmd = [_nvcc(), "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-cudart", "static"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return CUDA_LIB


def build_runtime(force: bool = False) -> Path:
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cpp"))
    if not srcs:
        raise RuntimeError("no C++ runtime sources found")
    if (not force and RT_LIB.exists()
            and RT_LIB.stat().st_mtime >= _newest_mtime(srcs + _headers())):
        return RT_LIB
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-I", str(CSRC),
           "-o", str(RT_LIB), *map(str, srcs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{res.stdout}\n{res.stderr}")
    return RT_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force=force, verbose=verbose)
    build_runtime(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(CUDA_LIB, RT_LIB)
