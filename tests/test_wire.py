"""DSSST1 wire format: round trips, structure tags, safety checks and byte chunking."""
import json
import pickle
import struct

import pytest
import torch

from arctic_platform_b200 import wire


def _eq(a, b):
    if torch.is_tensor(a):
        return torch.is_tensor(b) and a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b)
    if isinstance(a, dict):
        return isinstance(b, dict) and a.keys() == b.keys() and all(_eq(a[k], b[k]) for k in a)
    if isinstance(a, (list, tuple)):
        return type(a) is type(b) and len(a) == len(b) and all(_eq(x, y) for x, y in zip(a, b))
    return a == b


def test_roundtrip_nested_structures():
    obj = {"batch": {"input_ids": torch.arange(12).view(3, 4), "mask": torch.ones(3, 4, dtype=torch.bool)},
           "meta": {"lr": 1e-3, "names": ["a", "b"], "flag": True, "none": None},
           "list": [torch.zeros(2, dtype=torch.bfloat16), {"x": torch.tensor(3.5)}, 7],
           "tuple": (torch.tensor([1, 2], dtype=torch.int32), "s"), "scalar": torch.tensor(5)}
    out = wire.loads(wire.dumps(obj))
    assert _eq(obj, out)
    assert out["scalar"].dim() == 0


def test_root_tensor_and_empty_payloads():
    t = torch.randn(4, 3)
    assert torch.equal(wire.loads(wire.dumps(t)), t)
    assert wire.loads(wire.dumps({"a": 1})) == {"a": 1}
    assert wire.loads(wire.dumps([])) == []
    z = wire.loads(wire.dumps({"e": torch.zeros(0, 5)}))
    assert z["e"].shape == (0, 5)


def test_header_layout_is_safetensors_with_dss_metadata():
    frame = wire.dumps({"x": torch.ones(2)}, metadata={"op": "fwd"})
    (hlen,) = struct.unpack("<Q", frame[:8])
    header = json.loads(frame[8:8 + hlen])
    meta = header["__metadata__"]
    assert json.loads(meta["dss"])["v"] == "DSSST1"
    assert json.loads(meta["dss"])["tree"] == ["d", [["x", ["t", "x"]]]]
    assert wire.read_metadata(frame) == {"op": "fwd"}
    assert header["x"]["dtype"] == "F32" and header["x"]["shape"] == [2]


def test_interoperates_with_safetensors_package():
    st = pytest.importorskip("safetensors.torch")
    frame = wire.dumps({"a": {"b": torch.arange(6, dtype=torch.int64)}, "c": torch.ones(3, dtype=torch.bfloat16)})
    loaded = st.load(frame)
    assert torch.equal(loaded["a.b"], torch.arange(6)) and loaded["c"].dtype == torch.bfloat16
    theirs = st.save({"a.b": torch.arange(6, dtype=torch.int64)},
                     metadata={"dss": json.dumps({"v": "DSSST1", "tree": ["d", [["a", ["d", [["b", ["t", "a.b"]]]]]]]})})
    assert torch.equal(wire.loads(theirs)["a"]["b"], torch.arange(6))


def test_rejects_pickle_zip_and_garbage():
    with pytest.raises(wire.WireError, match="pickle"):
        wire.loads(pickle.dumps({"a": 1}, protocol=4))
    with pytest.raises(wire.WireError, match="pickle"):
        wire.loads(b"PK\x03\x04" + b"\x00" * 64)
    with pytest.raises(wire.WireError):
        wire.loads(b"\x01\x02")
    with pytest.raises(wire.WireError):
        wire.loads("not bytes")
    with pytest.raises(wire.WireError):
        wire.dumps({1: torch.ones(1)})
    assert wire.read_metadata(b"garbage-bytes-that-are-long-enough") == {}


def test_version_mismatch_and_missing_structure():
    st = pytest.importorskip("safetensors.torch")
    with pytest.raises(wire.WireError, match="structure missing"):
        wire.loads(st.save({"x": torch.ones(1)}))
    bad = st.save({"x": torch.ones(1)}, metadata={"dss": json.dumps({"v": "DSSST9", "tree": ["t", "x"]})})
    with pytest.raises(wire.WireError, match="unsupported"):
        wire.loads(bad)


def test_byte_chunks_roundtrip_any_order():
    frame = wire.dumps({"w": torch.randn(5000)})
    chunks = wire.encode_byte_chunks(frame, kind="request", operation="forward-backward", max_bytes=6000)
    assert len(chunks) > 1 and all(len(c) <= 6000 for c in chunks)
    desc = wire.read_byte_chunk_metadata(chunks[0])
    assert desc["kind"] == "request" and desc["operation"] == "forward-backward" and desc["chunk_group_id"]
    assert wire.decode_byte_chunks(list(reversed(chunks)), kind="request") == frame
    assert wire.encode_byte_chunks(frame, kind="result", max_bytes=0) == [frame]
    assert wire.decode_byte_chunks([frame]) == frame
    obj = {"r": torch.arange(3000)}
    assert _eq(wire.decode_result_chunks(wire.encode_result_chunks(obj, max_bytes=5000)), obj)


def test_byte_chunk_validation():
    frame = wire.dumps({"w": torch.randn(4000)})
    chunks = wire.encode_byte_chunks(frame, kind="result", max_bytes=5000)
    with pytest.raises(wire.WireError, match="expected"):
        wire.decode_byte_chunks(chunks[:-1])
    with pytest.raises(wire.WireError, match="duplicate"):
        wire.decode_byte_chunks(chunks[:-1] + [chunks[0]])
    with pytest.raises(wire.WireError, match="request chunks"):
        wire.decode_byte_chunks(chunks, kind="request")
    other = wire.encode_byte_chunks(wire.dumps({"w": torch.randn(4000)}), kind="result", max_bytes=5000)
    with pytest.raises(wire.WireError, match="differs"):
        wire.decode_byte_chunks(chunks[:-1] + [other[-1]])
    with pytest.raises(wire.WireError, match="too small"):
        wire.encode_byte_chunks(frame, kind="result", max_bytes=64)
    with pytest.raises(wire.WireError, match="kind"):
        wire.encode_byte_chunks(frame, kind="bogus", max_bytes=10)
