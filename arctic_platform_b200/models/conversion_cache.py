"""Node-local cache of checkpoints converted to the engine's parameter layout.

Loading a Hugging Face checkpoint means fusing q/k/v, interleaving gate/up, stacking experts and converting dtypes,
tensor by tensor.  With eight workers per node starting at once that work (and the read of the source shards from a
network file system) would run eight times.  The cache keeps the converted parameters as ONE raw file in the order
of ``model.named_parameters()`` plus an index; the first process on a node that needs it converts under an
exclusive ``flock`` and publishes the directory with an atomic rename, everyone else maps the file.

* where: ``<cache root>/<checkpoint dir name>-<sha1 of its resolved path, 12 hex>/<format tag>``; the cache root is
  the ``cache_dir`` argument or ``$APB_WEIGHT_CONVERSION_CACHE_DIR``; without either nothing is cached.
* ready: the index parses, names the data file, and the data file has the recorded size.
* stale: the index records the (name, shape) list of the model and size + mtime of every source shard; any
  difference rebuilds.

Reference behaviour: arctic_platform/model/implementations/qwen35/conversion_cache.py:17-121 (HF -> training layout
snapshot guarded by fcntl, temporary directory + ``os.replace``)."""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import shutil
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

import numpy as np
import torch

CACHE_DIR_ENV = "APB_WEIGHT_CONVERSION_CACHE_DIR"
CACHE_SCOPE_ENV = "APB_WEIGHT_CONVERSION_CACHE_SCOPE"
INDEX_NAME = "flat.index.json"
DATA_NAME = "flat.bin"
PASSTHROUGH_NAME = "passthrough.safetensors"

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def resolve_cache_path(source: Path, fmt: str, cache_dir: Optional[str] = None) -> Optional[Path]:
    root = cache_dir or os.environ.get(CACHE_DIR_ENV)
    if not root:
        return None
    source = Path(source)
    key = hashlib.sha1(str(source.resolve()).encode()).hexdigest()[:12]
    return Path(root) / f"{source.name}-{key}" / fmt


def cache_is_node_local(path: Path) -> bool:
    """Whether every node has to build its own copy.  ``$APB_WEIGHT_CONVERSION_CACHE_SCOPE`` = ``node`` / ``shared``
    decides; ``auto`` (default) treats ``/tmp``, ``/dev/shm`` and ``/data-fast`` as node-local."""
    scope = os.environ.get(CACHE_SCOPE_ENV, "auto").lower()
    if scope in ("node", "node-local", "local"):
        return True
    if scope in ("global", "shared"):
        return False
    try:
        resolved = Path(path).resolve()
    except OSError:
        resolved = Path(path).absolute()
    roots = (Path("/tmp"), Path("/dev/shm"), Path("/data-fast"))
    return any(resolved == r or r in resolved.parents for r in roots)


def _source_fingerprint(source: Path) -> List[List[Any]]:
    return [[f.name, f.stat().st_size, int(f.stat().st_mtime)] for f in sorted(Path(source).glob("*.safetensors"))]


def _layout(model) -> List[List[Any]]:
    return [[n, list(p.shape)] for n, p in model.named_parameters()]


def read_index(path: Path) -> Optional[Dict[str, Any]]:
    try:
        idx = json.loads((Path(path) / INDEX_NAME).read_text())
    except (OSError, json.JSONDecodeError):
        return None
    return idx if isinstance(idx, dict) and "params" in idx and "dtype" in idx else None


def cache_ready(path: Path, model=None, source: Optional[Path] = None, dtype: Optional[torch.dtype] = None) -> bool:
    idx = read_index(path)
    if idx is None:
        return False
    data = Path(path) / DATA_NAME
    if not data.is_file() or data.stat().st_size != idx.get("bytes", -1):
        return False
    if idx.get("passthrough") and not (Path(path) / PASSTHROUGH_NAME).is_file():
        return False
    if model is not None and [[n, s] for n, _o, s in idx["params"]] != _layout(model):
        return False
    if dtype is not None and _DTYPES.get(idx["dtype"]) != dtype:
        return False
    if source is not None and idx.get("source") != _source_fingerprint(source):
        return False
    return True


def _write_cache(model, source: Path, path: Path, dtype: torch.dtype, convert: Callable[[Any, Path], Any]) -> None:
    from .hf_io import write_safetensors
    tmp = path.with_name(f"{path.name}.tmp-pid{os.getpid()}")
    for stale in (tmp, path):
        if stale.exists():
            shutil.rmtree(stale)
    tmp.mkdir(parents=True)
    convert(model, source)                                  # fills the model's parameters from the source shards
    params, off = [], 0
    esize = torch.empty(0, dtype=dtype).element_size()
    with open(tmp / DATA_NAME, "wb") as f:
        for name, p in model.named_parameters():
            t = p.detach().to("cpu", dtype).contiguous()
            f.write(t.view(torch.uint8).reshape(-1).numpy().tobytes())
            params.append([name, off, list(p.shape)])
            off += t.numel() * esize
    passthrough = getattr(model, "passthrough", None)
    if passthrough is not None and len(passthrough):
        write_safetensors(tmp / PASSTHROUGH_NAME, dict(iter(passthrough)), {"format": "pt"})
    idx = {"dtype": str(dtype).replace("torch.", ""), "bytes": off, "params": params,
           "passthrough": bool(passthrough is not None and len(passthrough)), "source": _source_fingerprint(source)}
    (tmp / INDEX_NAME).write_text(json.dumps(idx))
    os.replace(tmp, path)


def _read_cache(model, path: Path) -> int:
    from .hf_io import read_safetensors
    from .vlm import PassthroughTensors
    idx = read_index(path)
    dtype = _DTYPES[idx["dtype"]]
    esize = torch.empty(0, dtype=dtype).element_size()
    raw = np.memmap(Path(path) / DATA_NAME, dtype=np.uint8, mode="r")
    params = dict(model.named_parameters())
    with torch.no_grad():
        for name, off, shape in idx["params"]:
            n = int(np.prod(shape)) if shape else 1
            chunk = torch.from_numpy(np.array(raw[off:off + n * esize], copy=True)).view(dtype).view(shape)
            params[name].copy_(chunk.to(params[name].dtype))
    if idx.get("passthrough"):
        model.passthrough = PassthroughTensors()
        for name, t in read_safetensors(Path(path) / PASSTHROUGH_NAME):
            model.passthrough.add(name, t)
    return len(idx["params"])


def load_through_cache(model, source, cache_dir: Optional[str] = None, dtype: Optional[torch.dtype] = None,
                       convert: Optional[Callable[[Any, Path], Any]] = None) -> Dict[str, Any]:
    """Fills ``model`` from the checkpoint directory ``source``, through the cache when one is configured.
    Returns ``{"cache": path or None, "built": bool}``; ``built`` is true for the one process that converted."""
    from .hf_io import load_hf_checkpoint
    convert = convert or load_hf_checkpoint
    source = Path(source)
    dtype = dtype or next(model.parameters()).dtype
    fmt = f"apb-flat-{str(dtype).replace('torch.', '')}"
    path = resolve_cache_path(source, fmt, cache_dir)
    if path is None:
        convert(model, source)
        return {"cache": None, "built": False}
    path.parent.mkdir(parents=True, exist_ok=True)
    built = False
    with open(path.parent / f".{path.name}.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not cache_ready(path, model, source, dtype):
                _write_cache(model, source, path, dtype, convert)
                built = True
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    if not built:
        _read_cache(model, path)
    return {"cache": str(path), "built": built}
