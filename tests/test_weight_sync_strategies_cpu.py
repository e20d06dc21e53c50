"""Trainer -> sampler weight hand-over: in-process copy, bulk RPC, bucketed (low memory) RPC and the safetensors file
path all leave the sampler with the trainer's weights (checked with the fp64 weight norm and a bit-exact compare)."""
import pytest
import torch

from arctic_platform_b200.common.utils import weight_sync as ws
from arctic_platform_b200.engine.worker import EngineWorker


class RemoteLike:
    """Actor that only offers ``call`` (like a worker in another process)."""

    def __init__(self, worker):
        self._w = worker

    def call(self, method, *a, **kw):
        return getattr(self._w, method)(*a, **kw)


def _worker(job_type, seed):
    w = EngineWorker(device="cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": job_type, "seed": seed,
                  "ds_config": {"optimizer": {"params": {"lr": 1e-3}}}, "vllm_config": {"max_model_len": 64}})
    return w


@pytest.fixture(scope="module")
def trainer():
    return _worker("training", 1)


def _flat(worker):
    m = worker.sampler.model if worker.sampler is not None else worker.engine.model
    return torch.cat([p.data.reshape(-1).float() for p in m.parameters()])


@pytest.mark.parametrize("strategy", ["bulk", "low_mem", "cpu_file", "in_process"])
def test_strategies_transfer_identical_weights(trainer, strategy, tmp_path):
    sampler = _worker("sampling", 2)
    assert abs(sampler.weight_norm()["norm"] - trainer.weight_norm()["norm"]) > 1e-3
    src, dst = RemoteLike(trainer), RemoteLike(sampler)
    if strategy == "bulk":
        n = ws.sync_weights_bulk(src, dst, staged=True)
    elif strategy == "low_mem":
        buckets = trainer.weight_buckets(64 << 10)
        assert len(buckets) > 3 and sum(len(b) for b in buckets) == len(trainer.get_parameter_names())
        n = ws.sync_weights_low_mem(src, dst, bucket_bytes=64 << 10)
    elif strategy == "cpu_file":
        n = ws.sync_weights_cpu_file(src, dst, directory=str(tmp_path))
        assert list(tmp_path.iterdir()) == []                         # the hand-over file is removed
    else:
        from arctic_platform_b200.common.server import InProcessActor
        r = ws.sync_pair(InProcessActor(trainer), InProcessActor(sampler))
        assert r["strategy"] == "in_process"
        n = r["num_tensors"]
    assert n == len(trainer.get_parameter_names())
    assert torch.equal(_flat(sampler), _flat(trainer))
    assert sampler.weight_norm()["norm"] == pytest.approx(trainer.weight_norm()["norm"], rel=1e-9)


def test_sync_pair_picks_by_flags(trainer):
    sampler = _worker("sampling", 3)
    src, dst = RemoteLike(trainer), RemoteLike(sampler)
    assert ws.sync_pair(src, dst)["strategy"] == "bulk"
    assert ws.sync_pair(src, dst, low_memory=True)["strategy"] == "low_mem"
    assert ws.sync_pair(src, dst, via_file=True)["strategy"] == "cpu_file"


def test_worker_export_helpers(tmp_path):
    from arctic_platform_b200.engine.worker import EngineWorker
    from arctic_platform_b200.models.hf_io import read_safetensors
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}}})
    sizes = {n: t.numel() * t.element_size() for n, t in w.engine.iter_hf_tensors()}
    assert w.max_param_bytes() == max(sizes.values())
    files = w.export_hf_checkpoint(str(tmp_path / "hf"))
    assert files and (tmp_path / "hf" / "config.json").exists()
    got = {}
    for f in files:
        got.update(dict(read_safetensors(tmp_path / "hf" / f)))
    assert set(got) == set(w.get_parameter_names())
    out = w.gather_and_save_state_dict(str(tmp_path / "w.safetensors"))
    assert out["num_tensors"] == len(sizes) and out["bytes"] == sum(sizes.values())
    assert set(dict(read_safetensors(tmp_path / "w.safetensors"))) == set(sizes)
    assert w.release_ipc_handles() == 0


def test_cuda_ipc_strategy_is_tried_first_and_falls_back():
    """``cuda_ipc=True`` between workers of different processes: the source is asked for an IPC handle of its flat
    buffer and the target runs the hand-over kernel on it; a source that cannot export (CPU engine, sharded or
    symmetric-memory storage) or a target without the paged CUDA sampler falls back to shipping tensors."""
    calls = []

    class Src:
        def __init__(self, info):
            self.info = info

        def call(self, name, *a):
            calls.append(("src", name))
            if name == "export_ipc_source":
                return self.info
            if name == "get_weights":
                return [("w", torch.zeros(2))]
            raise AssertionError(name)

    class Dst:
        def __init__(self, ok=True):
            self.ok = ok

        def call(self, name, *a):
            calls.append(("dst", name))
            if name == "has_sampler":
                return True
            if name == "sync_from_ipc":
                if not self.ok:
                    raise RuntimeError("sync_from_ipc needs the paged CUDA sampler")
                assert a[0][0]["handle"] == b"h" * 64
                return 7
            if name == "load_weights":
                return len(a[0])
            return None

    info = {"handle": b"h" * 64, "offset": 0, "layout": {}, "device": 0}
    r = ws.sync_pair(Src(info), Dst(), cuda_ipc=True)
    assert r == {"strategy": "cuda_ipc", "num_tensors": 7}
    order = [c for c in calls if c[0] == "dst"]
    assert [c[1] for c in order] == ["has_sampler", "wake_inference", "sync_from_ipc", "wake_inference", "reset_prefix_cache"]
    calls.clear()
    assert ws.sync_pair(Src(None), Dst(), cuda_ipc=True)["strategy"] == "bulk"          # nothing to export
    assert ws.sync_pair(Src(info), Dst(ok=False), cuda_ipc=True)["strategy"] == "bulk"  # target cannot map
    assert ws.sync_pair(Src(info), Dst())["strategy"] == "bulk"                         # not asked for
    # a CPU trainer has nothing to export
    from arctic_platform_b200.engine.worker import EngineWorker
    w = EngineWorker("cpu")
    w.initialize({"model_name": "qwen3-tiny", "job_type": "training", "ds_config": {"zero_optimization": {"stage": 1}}})
    assert w.export_ipc_source() is None and w.release_ipc_handles() == 0
