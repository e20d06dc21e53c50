"""DSSST1 wire format: one frame = one safetensors blob.

::

    u64 little-endian header length | JSON header | tensor bytes

The header's ``__metadata__`` carries two JSON strings: ``dss`` -- the structure
skeleton ``{"v": "DSSST1", "tree": ...}`` that says where each tensor sits in the
original nested dict/list/tuple -- and, optionally, ``op`` -- free-form operation
metadata (chunk descriptors, router replay handles, ...).  The format and the
tree tags (``t`` tensor, ``j`` JSON leaf, ``d`` dict, ``l`` list, ``u`` tuple) are
those of the reference (arctic_platform/wire.py:35-131) so that either side can
talk to the other; the implementation here writes and parses the safetensors
container itself (a frame is assembled with one ``bytearray`` and tensors are
views into the received buffer) and never touches pickle.

Oversized frames are cut into byte-range chunk frames, each again a DSSST1 frame
holding a 1-D uint8 ``payload`` and a descriptor (arctic_platform/wire.py:236-382).
"""
from __future__ import annotations

import hashlib
import json
import struct
import uuid
from typing import Any, Dict, List, Optional, Tuple

import torch

WIRE_FORMAT_VERSION = "DSSST1"

_STRUCT_KEY = "dss"
_OP_KEY = "op"
_EMPTY_KEY = "__dss_empty__"
_ROOT_KEY = "__root__"
_PAYLOAD_KEY = "payload"
_CHUNK_KEYS = {"request": "request_chunk", "result": "result_chunk"}
_HEADER_LIMIT = 64 * 1024 * 1024
_CHUNK_OVERHEAD = 8192
_PICKLE_MAGIC = (b"\x80\x02", b"\x80\x03", b"\x80\x04", b"\x80\x05")
_ZIP_MAGIC = b"PK\x03\x04"


class WireError(ValueError):
    """Malformed, truncated or foreign payload."""


# safetensors dtype names <-> torch dtypes
_DTYPE_TO_NAME = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8",
    torch.uint8: "U8", torch.bool: "BOOL",
}
for _name, _attr in (("F8_E4M3", "float8_e4m3fn"), ("F8_E5M2", "float8_e5m2"), ("U16", "uint16"),
                     ("U32", "uint32"), ("U64", "uint64")):
    if hasattr(torch, _attr):
        _DTYPE_TO_NAME[getattr(torch, _attr)] = _name
_NAME_TO_DTYPE = {v: k for k, v in _DTYPE_TO_NAME.items()}


# --------------------------------------------------------------------------- container
def _pack_container(tensors: Dict[str, torch.Tensor], metadata: Dict[str, str]) -> bytes:
    """Writes a safetensors blob (tensors sorted by dtype alignment then name, as the
    upstream writer does, so byte-for-byte layout matches)."""
    def sort_key(item):
        name, t = item
        return (-t.element_size(), name)

    entries = sorted(tensors.items(), key=sort_key)
    header: Dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs: List[memoryview] = []
    for name, t in entries:
        raw = t.contiguous().view(torch.uint8).reshape(-1) if t.numel() else torch.empty(0, dtype=torch.uint8)
        nbytes = raw.numel()
        if t.dtype not in _DTYPE_TO_NAME:
            raise WireError(f"dtype {t.dtype} cannot be carried by DSSST1")
        header[name] = {"dtype": _DTYPE_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(memoryview(raw.numpy()) if nbytes else memoryview(b""))
    hbytes = json.dumps(header, separators=(",", ":"), ensure_ascii=False).encode("utf-8")
    pad = (-len(hbytes)) % 8
    hbytes += b" " * pad
    out = bytearray(8 + len(hbytes) + offset)
    struct.pack_into("<Q", out, 0, len(hbytes))
    out[8:8 + len(hbytes)] = hbytes
    pos = 8 + len(hbytes)
    for b in blobs:
        n = b.nbytes
        out[pos:pos + n] = b
        pos += n
    return bytes(out)


def _parse_header(data) -> Tuple[Dict[str, Any], int]:
    if len(data) < 8:
        raise WireError("payload too short to be a DSSST1 safetensors blob")
    (hlen,) = struct.unpack_from("<Q", data, 0)
    if hlen <= 0 or hlen > _HEADER_LIMIT or 8 + hlen > len(data):
        raise WireError("invalid DSSST1 safetensors header length")
    try:
        header = json.loads(bytes(data[8:8 + hlen]).decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise WireError(f"DSSST1 header is not JSON: {exc}") from exc
    if not isinstance(header, dict):
        raise WireError("DSSST1 header must be a JSON object")
    return header, 8 + hlen


def _unpack_container(data: bytes) -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    header, base = _parse_header(data)
    meta = header.pop("__metadata__", None) or {}
    body = memoryview(data)[base:]
    # one writable copy of the body; every tensor is a view into it
    storage = torch.frombuffer(bytearray(body), dtype=torch.uint8) if len(body) else torch.empty(0, dtype=torch.uint8)
    out: Dict[str, torch.Tensor] = {}
    for name, info in header.items():
        try:
            dtype = _NAME_TO_DTYPE[info["dtype"]]
            shape = [int(s) for s in info["shape"]]
            lo, hi = (int(x) for x in info["data_offsets"])
        except (KeyError, TypeError, ValueError) as exc:
            raise WireError(f"bad tensor entry {name!r}: {exc}") from exc
        if lo < 0 or hi < lo or hi > len(body):
            raise WireError(f"tensor {name!r} points outside the frame")
        numel = 1
        for s in shape:
            numel *= s
        esize = torch.empty(0, dtype=dtype).element_size()
        if numel * esize != hi - lo:
            raise WireError(f"tensor {name!r} size does not match its shape")
        if numel == 0:
            out[name] = torch.empty(shape, dtype=dtype)
        elif lo % esize == 0:
            out[name] = storage[lo:hi].view(dtype).reshape(shape)
        else:
            out[name] = storage[lo:hi].clone().view(dtype).reshape(shape)
    return out, meta


# --------------------------------------------------------------------------- tree codec
def _has_tensor(obj: Any) -> bool:
    stack = [obj]
    while stack:
        cur = stack.pop()
        if torch.is_tensor(cur):
            return True
        if isinstance(cur, dict):
            stack.extend(cur.values())
        elif isinstance(cur, (list, tuple)):
            stack.extend(cur)
    return False


class _TreeEncoder:
    def __init__(self) -> None:
        self.tensors: Dict[str, torch.Tensor] = {}
        self._storages: set = set()

    def _child(self, path: str, key: str) -> str:
        return f"{path}.{key}" if path else key

    def visit(self, obj: Any, path: str) -> list:
        if torch.is_tensor(obj):
            return self._tensor(obj, path)
        if isinstance(obj, dict):
            if not _has_tensor(obj):
                return ["j", obj]
            items = []
            for k, v in obj.items():
                if not isinstance(k, str):
                    raise WireError(f"DSSST1 dict keys must be strings, got {type(k)!r}")
                items.append([k, self.visit(v, self._child(path, k))])
            return ["d", items]
        if isinstance(obj, tuple):
            return ["u", [self.visit(v, self._child(path, str(i))) for i, v in enumerate(obj)]]
        if isinstance(obj, list):
            if not _has_tensor(obj):
                return ["j", obj]
            return ["l", [self.visit(v, self._child(path, str(i))) for i, v in enumerate(obj)]]
        return ["j", obj]

    def _tensor(self, t: torch.Tensor, path: str) -> list:
        key = path or _ROOT_KEY
        t = t.detach()
        if t.device.type != "cpu":
            t = t.cpu()
        t = t.contiguous()
        node: list = ["t", key]
        if t.dim() == 0:
            t = t.reshape(1)
            node.append({"scalar": True})
        self.tensors[key] = t
        return node


def _decode_tree(node: list, tensors: Dict[str, torch.Tensor]) -> Any:
    tag = node[0]
    if tag == "t":
        try:
            t = tensors[node[1]]
        except KeyError as exc:
            raise WireError(f"tensor {node[1]!r} named by the structure is missing") from exc
        if len(node) > 2 and isinstance(node[2], dict) and node[2].get("scalar"):
            return t.reshape(())
        return t
    if tag == "j":
        return node[1]
    if tag == "d":
        return {k: _decode_tree(child, tensors) for k, child in node[1]}
    if tag == "l":
        return [_decode_tree(child, tensors) for child in node[1]]
    if tag == "u":
        return tuple(_decode_tree(child, tensors) for child in node[1])
    raise WireError(f"unknown DSSST1 node tag {tag!r}")


# --------------------------------------------------------------------------- public codec
def dumps(obj: Any, *, metadata: Optional[dict] = None) -> bytes:
    """Serialises ``obj`` (nested dict/list/tuple of tensors and JSON values) to one frame."""
    enc = _TreeEncoder()
    tree = enc.visit(obj, "")
    tensors = enc.tensors
    if not tensors:
        tensors = {_EMPTY_KEY: torch.zeros(1, dtype=torch.uint8)}
    header = {_STRUCT_KEY: json.dumps({"v": WIRE_FORMAT_VERSION, "tree": tree})}
    if metadata:
        header[_OP_KEY] = json.dumps(metadata)
    return _pack_container(tensors, header)


def _as_bytes(data: Any, who: str) -> bytes:
    if not isinstance(data, (bytes, bytearray, memoryview)):
        raise WireError(f"DSSST1 {who} expects bytes")
    return bytes(data)


def loads(data: Any) -> Any:
    """Inverse of :func:`dumps`.  Pickle / ``torch.save`` payloads are refused, never executed."""
    data = _as_bytes(data, "loads")
    try:
        tensors, meta = _unpack_container(data)
    except WireError as exc:
        if data[:2] in _PICKLE_MAGIC or data[:4] == _ZIP_MAGIC:
            raise WireError("refusing to deserialize a legacy pickle/torch.save payload; "
                            "the peer must use the DSSST1 safetensors wire protocol") from exc
        raise WireError(f"not a valid DSSST1 safetensors payload: {exc}") from exc
    raw = meta.get(_STRUCT_KEY)
    if raw is None:
        raise WireError("DSSST1 structure missing from safetensors header")
    info = json.loads(raw)
    if info.get("v") != WIRE_FORMAT_VERSION:
        raise WireError(f"unsupported DSSST1 wire version {info.get('v')!r}")
    tensors.pop(_EMPTY_KEY, None)
    return _decode_tree(info["tree"], tensors)


def read_metadata(data: Any) -> dict:
    """Operation metadata of a frame without touching tensor bytes; ``{}`` for foreign bytes."""
    data = _as_bytes(data, "read_metadata")
    try:
        header, _ = _parse_header(data)
        raw = (header.get("__metadata__") or {}).get(_OP_KEY)
        return json.loads(raw) if raw else {}
    except (WireError, ValueError):
        return {}


# --------------------------------------------------------------------------- chunking
def _chunk_key(kind: str) -> str:
    try:
        return _CHUNK_KEYS[kind]
    except KeyError:
        raise WireError(f"unknown byte chunk kind {kind!r}") from None


def _chunk_frames(frame: bytes, kind: str, operation, group_id, payload_size: int) -> List[bytes]:
    digest = hashlib.sha256(frame).hexdigest()
    total = (len(frame) + payload_size - 1) // payload_size
    frames = []
    for idx in range(total):
        desc: Dict[str, Any] = {"chunk_idx": idx, "total_chunks": total, "frame_sha256": digest,
                                "frame_size_bytes": len(frame)}
        if group_id is not None:
            desc["chunk_group_id"] = group_id
        if operation is not None:
            desc["operation"] = operation
        piece = frame[idx * payload_size:(idx + 1) * payload_size]
        payload = torch.frombuffer(bytearray(piece), dtype=torch.uint8)
        frames.append(dumps({_PAYLOAD_KEY: payload}, metadata={_chunk_key(kind): desc}))
    return frames


def encode_byte_chunks(frame: Any, *, kind: str, operation: Optional[str] = None, max_bytes: int = 0,
                       chunk_group_id: Optional[str] = None) -> List[bytes]:
    """Splits ``frame`` so that every returned frame is at most ``max_bytes`` long
    (``[frame]`` itself when it already fits or no limit is given)."""
    frame = _as_bytes(frame, "encode_byte_chunks")
    _chunk_key(kind)
    if max_bytes <= 0 or len(frame) <= max_bytes:
        return [frame]
    group_id = None
    if kind == "request":
        group_id = chunk_group_id or str(uuid.uuid4())
    size = max(1, max_bytes - _CHUNK_OVERHEAD)
    while True:
        frames = _chunk_frames(frame, kind, operation, group_id, size)
        if max(len(f) for f in frames) <= max_bytes:
            return frames
        if size == 1:
            raise WireError("max_bytes is too small to hold one DSSST1 byte chunk frame")
        size = max(1, size // 2)


def read_byte_chunk_metadata(frame: Any) -> Optional[dict]:
    meta = read_metadata(frame)
    for kind, key in _CHUNK_KEYS.items():
        if key in meta:
            desc = dict(meta[key])
            desc["kind"] = kind
            return desc
    return None


def decode_byte_chunks(chunks: List[bytes], *, kind: Optional[str] = None) -> bytes:
    """Reassembles chunk frames (any order) into the original frame, verifying every
    descriptor field, the size and the SHA-256 of the result."""
    if not chunks:
        raise WireError("decode_byte_chunks requires at least one frame")
    descs = [read_byte_chunk_metadata(c) for c in chunks]
    if len(chunks) == 1 and descs[0] is None:
        return bytes(chunks[0])
    if any(d is None for d in descs):
        raise WireError("decode_byte_chunks received a frame without byte chunk metadata")
    first = descs[0]
    if kind is not None and first["kind"] != kind:
        raise WireError(f"expected {kind} chunks, got {first['kind']} chunks")
    total = int(first.get("total_chunks"))
    if len(chunks) != total:
        raise WireError(f"expected {total} byte chunks, got {len(chunks)}")
    parts: Dict[int, bytes] = {}
    for chunk, d in zip(chunks, descs):
        if d["kind"] != first["kind"]:
            raise WireError("mixed byte chunk kinds")
        for field in ("total_chunks", "frame_sha256", "frame_size_bytes", "chunk_group_id", "operation"):
            if d.get(field) != first.get(field):
                raise WireError(f"byte chunk {field} differs across frames")
        idx = int(d.get("chunk_idx"))
        if not 0 <= idx < total:
            raise WireError("byte chunk_idx out of range")
        if idx in parts:
            raise WireError("duplicate byte chunk_idx")
        payload = loads(chunk).get(_PAYLOAD_KEY)
        if not torch.is_tensor(payload) or payload.dtype != torch.uint8 or payload.dim() != 1:
            raise WireError("byte chunk payload must be a 1-D uint8 tensor")
        parts[idx] = payload.numpy().tobytes()
    missing = sorted(set(range(total)) - set(parts))
    if missing:
        raise WireError(f"missing byte chunks: {missing}")
    frame = b"".join(parts[i] for i in range(total))
    if len(frame) != int(first.get("frame_size_bytes")):
        raise WireError("reassembled frame size mismatch")
    if hashlib.sha256(frame).hexdigest() != first.get("frame_sha256"):
        raise WireError("reassembled frame sha256 mismatch")
    return frame


def encode_result_chunks(result: Any, *, max_bytes: int = 0) -> List[bytes]:
    return encode_byte_chunks(dumps(result), kind="result", max_bytes=max_bytes)


def decode_result_chunks(chunks: List[bytes]) -> Any:
    return loads(decode_byte_chunks(chunks, kind="result"))


# ------------------------------------------------------------------ chunk-group verdicts in error replies
CHUNK_GROUP_RESTART_CODES = {"chunk_group_restart_required", "chunk_group_restart"}
CHUNK_GROUP_CONFLICT_CODES = {"chunk_group_conflict", "chunk_group_missing_chunks"}


def find_chunk_group_error(body: Any, _depth: int = 0) -> Optional[dict]:
    """The chunk-group error object inside an error reply, or None.  Gateways wrap the service's JSON reply in their
    own (``{"message": "upstream said: {...}"}``), sometimes more than once, so the search descends into dicts,
    lists and JSON objects embedded in strings.  The returned dict always carries ``code``."""
    if _depth > 8:
        return None
    if isinstance(body, dict):
        code = body.get("code") or body.get("error")
        if isinstance(code, str) and code in CHUNK_GROUP_RESTART_CODES | CHUNK_GROUP_CONFLICT_CODES:
            return {**body, "code": code}
        if body.get("chunk_group_id") and str(body.get("message", "")).endswith("missing chunks"):
            return {**body, "code": "chunk_group_missing_chunks"}
        children = list(body.values())
    elif isinstance(body, list):
        children = body
    elif isinstance(body, str) and ("{" in body or "[" in body):
        import json
        dec, children, i = json.JSONDecoder(), [], 0
        while i < len(body):
            if body[i] in "{[":
                try:
                    obj, end = dec.raw_decode(body, i)
                except ValueError:
                    i += 1
                    continue
                children.append(obj)
                i = end
            else:
                i += 1
    else:
        return None
    for child in children:
        hit = find_chunk_group_error(child, _depth + 1)
        if hit is not None:
            return hit
    return None
