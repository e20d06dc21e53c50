"""Converted-checkpoint cache: one conversion per cache directory however many processes start together, stale
caches rebuilt, parameters and carried-through tensors identical to a direct load."""
import json
import multiprocessing as mp
import os

import torch

from arctic_platform_b200.models import conversion_cache as cc
from arctic_platform_b200.models.config import PRESETS
from arctic_platform_b200.models.decoder import DecoderLM
from arctic_platform_b200.models.hf_io import load_hf_checkpoint, save_hf_checkpoint


def _make_checkpoint(path, seed=4):
    src = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32).init_weights(seed=seed)
    save_hf_checkpoint(src, path)
    return src


def _counting_convert(counter_file):
    def convert(model, source):
        with open(counter_file, "a") as f:
            f.write("x")
        return load_hf_checkpoint(model, source)
    return convert


def _proc(ck, cache, counter, out):
    torch.set_num_threads(1)
    m = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    info = cc.load_through_cache(m, ck, cache_dir=cache, convert=_counting_convert(counter))
    flat = torch.cat([p.detach().reshape(-1) for p in m.parameters()])
    torch.save({"built": info["built"], "sum": float(flat.double().sum()), "flat": flat}, out)


def test_cache_paths_and_scope(tmp_path, monkeypatch):
    monkeypatch.delenv(cc.CACHE_DIR_ENV, raising=False)
    assert cc.resolve_cache_path(tmp_path / "m", "fmt") is None
    monkeypatch.setenv(cc.CACHE_DIR_ENV, str(tmp_path / "root"))
    p = cc.resolve_cache_path(tmp_path / "m", "fmt")
    assert p.parent.parent == tmp_path / "root" and p.name == "fmt" and p.parent.name.startswith("m-")
    assert p != cc.resolve_cache_path(tmp_path / "other" / "m", "fmt")          # same name, different source
    monkeypatch.setenv(cc.CACHE_SCOPE_ENV, "shared")
    assert not cc.cache_is_node_local("/tmp/x")
    monkeypatch.setenv(cc.CACHE_SCOPE_ENV, "node")
    assert cc.cache_is_node_local("/mnt/nfs/x")
    monkeypatch.setenv(cc.CACHE_SCOPE_ENV, "auto")
    assert cc.cache_is_node_local("/tmp/x/y") and not cc.cache_is_node_local("/mnt/nfs/x")


def test_no_cache_dir_loads_directly(tmp_path, monkeypatch):
    monkeypatch.delenv(cc.CACHE_DIR_ENV, raising=False)
    src = _make_checkpoint(tmp_path / "ck")
    m = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    assert cc.load_through_cache(m, tmp_path / "ck") == {"cache": None, "built": False}
    for a, b in zip(src.parameters(), m.parameters()):
        assert torch.equal(a, b)


def test_one_conversion_for_concurrent_loaders_and_rebuild_when_stale(tmp_path):
    ck, cache, counter = tmp_path / "ck", tmp_path / "cache", tmp_path / "count"
    src = _make_checkpoint(ck)
    ctx = mp.get_context("spawn")
    outs = [tmp_path / f"o{i}.pt" for i in range(3)]
    procs = [ctx.Process(target=_proc, args=(str(ck), str(cache), str(counter), str(o))) for o in outs]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = [torch.load(o, weights_only=False) for o in outs]
    assert counter.read_text() == "x" and sum(r["built"] for r in res) == 1
    want = torch.cat([p.detach().reshape(-1) for p in src.parameters()])
    for r in res:
        assert torch.equal(r["flat"], want)
    path = cc.resolve_cache_path(ck, "apb-flat-float32", str(cache))
    m = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    assert cc.cache_ready(path, m, ck, torch.float32)
    assert not cc.cache_ready(path, m, ck, torch.bfloat16)
    # a truncated data file, a broken index and a changed source are all "not ready"
    idx = json.loads((path / cc.INDEX_NAME).read_text())
    with open(path / cc.DATA_NAME, "r+b") as f:
        f.truncate(idx["bytes"] - 4)
    assert not cc.cache_ready(path)
    info = cc.load_through_cache(m, ck, cache_dir=str(cache), convert=_counting_convert(counter))
    assert info["built"] and counter.read_text() == "xx" and cc.cache_ready(path, m, ck)
    (path / cc.INDEX_NAME).write_text("{not json")
    assert not cc.cache_ready(path)
    cc.load_through_cache(m, ck, cache_dir=str(cache), convert=_counting_convert(counter))
    _make_checkpoint(ck, seed=9)                                   # new weights at the same path
    os.utime(ck / "model.safetensors", (1, 1))
    assert not cc.cache_ready(path, m, ck)
    m2 = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    assert cc.load_through_cache(m2, ck, cache_dir=str(cache))["built"]
    m3 = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    assert not cc.load_through_cache(m3, ck, cache_dir=str(cache))["built"]
    for a, b in zip(m2.parameters(), m3.parameters()):
        assert torch.equal(a, b)
    assert not torch.equal(torch.cat([p.detach().reshape(-1) for p in m3.parameters()]), want)


def test_cache_keeps_carried_through_tensors(tmp_path):
    from arctic_platform_b200.models.vlm import PassthroughTensors

    def convert(model, source):
        load_hf_checkpoint(model, source)
        model.passthrough = PassthroughTensors()
        model.passthrough.add("model.visual.w", torch.arange(6, dtype=torch.bfloat16).view(2, 3))
    _make_checkpoint(tmp_path / "ck")
    a = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    assert cc.load_through_cache(a, tmp_path / "ck", cache_dir=str(tmp_path / "c"), convert=convert)["built"]
    b = DecoderLM(PRESETS["qwen3-moe-tiny"], "cpu", torch.float32)
    assert not cc.load_through_cache(b, tmp_path / "ck", cache_dir=str(tmp_path / "c"), convert=convert)["built"]
    (name, t), = list(b.passthrough)
    assert name == "model.visual.w" and t.dtype == torch.bfloat16 and torch.equal(t, a.passthrough.tensors[name])
