"""Gated delta-net layers under sequence sharding: every rank runs only its own rows; the convolution history and the
recurrent state cross the rank boundaries as small all-gathers (state as an affine map).  Two gloo ranks against one
process, values and gradients."""
import os
import socket
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer_and_inputs(cu):
    import dataclasses
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.linear_attention import GatedDeltaNet
    from arctic_platform_b200.ops.attention import AttnLayout
    cfg = dataclasses.replace(PRESETS["qwen3.5-moe-tiny"], hidden_size=64)
    torch.manual_seed(0)
    layer = GatedDeltaNet(cfg, "cpu", torch.float32)
    for n, p in layer.named_parameters():
        p.data.normal_(0, 0.3 if p.dim() > 1 else 0.5)
    layer.norm_w.data.fill_(1.0)
    T = cu[-1]
    x = torch.randn(T, cfg.hidden_size, generator=torch.Generator().manual_seed(1))
    w = torch.randn(T, cfg.hidden_size, generator=torch.Generator().manual_seed(2))
    return layer, x, w, AttnLayout.from_cu_seqlens(np.array(cu))


def _cp_main(rank, world, port, out_dir, cu):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        layer, x, w, layout = _layer_and_inputs(cu)
        layer.sp_group = dist.group.WORLD
        rows = x.shape[0] // world
        xl = x[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        assert layer._context_parallel_ok(xl, layout)
        y = layer(xl, layout)
        (y * w[rank * rows:(rank + 1) * rows]).sum().backward()
        grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
        for gten in grads.values():
            dist.all_reduce(gten)
        torch.save({"y": y.detach(), "dx": xl.grad, "grads": grads}, os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _check(cu, world=2):
    layer, x, w, layout = _layer_and_inputs(cu)
    xr = x.clone().requires_grad_(True)
    want = layer(xr, layout)
    (want * w).sum().backward()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_cp_main, args=(world, _free_port(), d, cu), nprocs=world, join=True)
        res = [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]
    y = torch.cat([r["y"] for r in res])
    dx = torch.cat([r["dx"] for r in res])
    tol = lambda ref: 2e-4 * float(ref.abs().max()) + 1e-6
    assert float((y - want).abs().max()) < tol(want)
    assert float((dx - xr.grad).abs().max()) < tol(xr.grad)
    for n, p in layer.named_parameters():
        assert float((res[0]["grads"][n] - p.grad).abs().max()) < tol(p.grad), n


def test_sequence_crossing_the_rank_boundary_and_sequences_inside_one_rank():
    # 3 sequences over 2 x 100 rows: the second one (60..150) crosses the boundary, the others do not
    _check([0, 60, 150, 200])


def test_one_sequence_spanning_every_rank():
    # a single sequence over 3 ranks: the middle rank neither starts nor ends it (three local passes)
    _check([0, 210], world=3)


def test_boundary_on_a_sequence_start_and_short_carry():
    # a sequence starts exactly on the boundary; another one has only 2 rows (< conv history) before the boundary
    _check([0, 98, 100, 160, 200])


def test_state_map_composes():
    from arctic_platform_b200.models.linear_attention import (delta_rule_transition, gated_delta_rule_chunked,
                                                              gated_delta_rule_recurrent)
    g = torch.Generator().manual_seed(4)
    T, H, Dk, Dv = 150, 2, 16, 24
    q, k = torch.randn(T, H, Dk, generator=g), torch.randn(T, H, Dk, generator=g)
    v = torch.randn(T, H, Dv, generator=g)
    gate, beta = -torch.rand(T, H, generator=g) * 0.2, torch.rand(T, H, generator=g)
    S0 = torch.randn(H, Dk, Dv, generator=g)
    _, want = gated_delta_rule_recurrent(q, k, v, gate, beta, S0)
    _, C = gated_delta_rule_chunked(q, k, v, gate, beta, None)
    P = delta_rule_transition(q, k, gate, beta)
    assert float((P @ S0 + C - want).abs().max()) < 1e-4 * float(want.abs().max())
