"""Optimizer state on the host (``zero_optimization.offload_optimizer.device: cpu``): the native single-pass AdamW
against plain fp32 tensor arithmetic, and engines with and without the offload taking identical steps."""

import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from arctic_platform_b200.ops import _lib


def _torch_adamw(w, m, v, g, lr, b1, b2, eps, wd, bias1, bias2, gscale):
    g = g * gscale
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    w = w * (1 - lr * wd) - lr * (m / bias1) / ((v / bias2).sqrt() + eps)
    return w, m, v


@pytest.mark.parametrize("n,threads", [(1, 1), (1037, 1), (300_001, 0), (300_001, 3), (70_000, 64)])
def test_native_host_adamw_matches_tensor_arithmetic(n, threads):
    gen = torch.Generator().manual_seed(n)
    w = torch.randn(n, generator=gen)
    m = torch.randn(n, generator=gen) * 0.1
    v = torch.rand(n, generator=gen) * 0.01
    g = torch.randn(n, generator=gen)
    hp = dict(lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.1, bias1=1 - 0.9 ** 3, bias2=1 - 0.95 ** 3, gscale=0.37)
    rw, rm, rv = _torch_adamw(w, m, v, g, **hp)
    out = torch.empty(n, dtype=torch.bfloat16)
    rt = _lib.rt_lib()
    w2, m2, v2 = w.clone(), m.clone(), v.clone()
    rc = rt.apb_rt_cpu_adamw(w2.data_ptr(), m2.data_ptr(), v2.data_ptr(), g.data_ptr(), out.data_ptr(), n, hp["lr"],
                             hp["b1"], hp["b2"], hp["eps"], hp["wd"], hp["bias1"], hp["bias2"], hp["gscale"], threads)
    assert rc == 0
    assert torch.allclose(m2, rm, rtol=1e-6, atol=1e-7) and torch.allclose(v2, rv, rtol=1e-6, atol=1e-9)
    assert torch.allclose(w2, rw, rtol=1e-5, atol=1e-6)
    assert torch.equal(out, w2.to(torch.bfloat16))            # round-to-nearest-even, as the tensor cast
    assert rt.apb_rt_cpu_sumsq(g.data_ptr(), n) == pytest.approx(float(g.double().pow(2).sum()), rel=1e-12)


def test_native_host_adamw_rejects_bad_arguments_and_handles_specials():
    rt = _lib.rt_lib()
    x = torch.zeros(4)
    assert rt.apb_rt_cpu_adamw(None, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 4, 1e-3, 0.9, 0.999, 1e-8, 0.0,
                               1.0, 1.0, 1.0, 1) == -1
    assert rt.apb_rt_cpu_adamw(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 4, 1e-3, 0.9, 0.999, 1e-8,
                               0.0, 0.0, 1.0, 1.0, 1) == -1
    # the low-precision copy is optional, and a NaN gradient stays a NaN parameter instead of turning into infinity
    w, m, v = torch.ones(4), torch.zeros(4), torch.zeros(4)
    g = torch.tensor([0.0, 1.0, float("nan"), -1.0])
    out = torch.empty(4, dtype=torch.bfloat16)
    assert rt.apb_rt_cpu_adamw(w.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), out.data_ptr(), 4, 1e-1, 0.9, 0.999,
                               1e-8, 0.0, 0.1, 0.001, 1.0, 1) == 0
    assert torch.isnan(out[2]) and torch.isnan(w[2])
    assert float(w[0]) == 1.0 and float(w[1]) < 1.0 < float(w[3])


def _engine(stage, offload, seed=7):
    from arctic_platform_b200.engine.trainer import EngineConfig, TrainEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    model = DecoderLM(PRESETS["qwen3-tiny"], "cpu", torch.float32).init_weights(seed=seed)
    ds = {"optimizer": {"type": "AdamW", "params": {"lr": 1e-3, "weight_decay": 0.01}}, "gradient_clipping": 0.5,
          "zero_optimization": {"stage": stage, "offload_optimizer": {"device": "cpu" if offload else "none"}}}
    cfg = EngineConfig.from_ds_config(ds)
    assert cfg.offload_optimizer == offload
    return TrainEngine(model, cfg)


@pytest.mark.parametrize("stage", [1, 3])
def test_offloaded_engine_takes_the_same_steps(stage):
    from arctic_platform_b200.engine.checkpoint import load_checkpoint, save_checkpoint
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    from tests.test_zorro_equivalence_cpu import make_grpo_batch
    ids, mask, R = make_grpo_batch(n_prompts=2, n_samples=3, seed=11)
    engines = {off: _engine(stage, off) for off in (False, True)}
    assert engines[True].opt_on_host and not engines[False].opt_on_host
    assert engines[True].master.device.type == "cpu" and engines[True]._host_grad is not None
    norms = {False: [], True: []}
    for _step in range(3):
        for off, eng in engines.items():
            pb = build_packed_batch(ids, mask, R, dedup=True)
            lp, _ = token_logprobs(eng.model, pb)
            eng.backward(-(lp.sum() / lp.numel()))
            norms[off].append(float(eng.step()["grad_norm"]))
    # Adam divides by sqrt(v): where a gradient is almost zero, the last bit of the moments decides the step, so the
    # two orders of floating-point operations agree closely on average and loosely on the worst element
    assert norms[True] == pytest.approx(norms[False], rel=1e-4)
    a, b = engines[False], engines[True]
    diff = (a.full_flat_params() - b.full_flat_params()).abs()
    assert diff.mean() < 1e-6 and diff.max() < 1e-3
    assert (a.master - b.master).abs().mean() < 1e-6 and (a.exp_avg - b.exp_avg).abs().mean() < 1e-6
    # sleep / wake leave host-resident state where it is; a checkpoint round trip restores it
    b.offload_states(("optimizer",))
    b.reload_states()
    with tempfile.TemporaryDirectory() as d:
        save_checkpoint(b, d, "t", export_hf=False)
        c = _engine(stage, True, seed=3)
        assert load_checkpoint(c, d, "t") == 3
        assert torch.equal(c.master, b.master) and torch.equal(c.exp_avg_sq, b.exp_avg_sq)
        assert torch.equal(c.full_flat_params(), b.full_flat_params())


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arctic_platform_b200.models.decoder import token_logprobs
        from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
        from tests.test_zorro_equivalence_cpu import make_grpo_batch
        ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=5)
        B = ids.shape[0]
        sl = slice(rank * B // world, (rank + 1) * B // world)
        res = {}
        for off in (False, True):
            eng = _engine(3, off)
            assert eng.zero3 is not None and eng.opt_on_host == off
            norms = []
            for _step in range(2):
                pb = build_packed_batch(ids[sl], mask[sl], R, dedup=True)
                lp, _ = token_logprobs(eng.model, pb)
                eng.backward(-(lp.sum() / lp.numel()))
                norms.append(float(eng.step()["grad_norm"]))
            res[off] = {"norms": norms, "full": eng.full_flat_params().clone(), "master": eng.master.clone()}
        torch.save(res, os.path.join(out_dir, f"o{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_offloaded_zero3_on_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank_main, args=(2, port, d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"o{r}.pt"), weights_only=False) for r in range(2)]
    for r in res:
        assert r[True]["norms"] == pytest.approx(r[False]["norms"], rel=1e-4)
        diff = (r[True]["full"] - r[False]["full"]).abs()
        assert diff.mean() < 1e-6 and diff.max() < 1e-3
        assert (r[True]["master"] - r[False]["master"]).abs().mean() < 1e-6
    assert torch.equal(res[0][True]["full"], res[1][True]["full"])
