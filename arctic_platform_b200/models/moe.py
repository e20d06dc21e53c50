"""Token-choice top-k mixture of experts (Qwen3-MoE layout).

Router: fp32 softmax over ``E`` logits, top-k, optional renormalisation of the kept
probabilities (arctic_platform/model/implementations/qwen35/models/layers/moe.py:226-269
in the reference).  Experts: SwiGLU FFNs stacked as ``wgu [E, 2*I, H]`` (gate/up rows
interleaved) and ``wdown [E, H, I]``.

Single-GPU / data-parallel execution sorts the routed (token, expert) pairs by expert and
runs ONE grouped tcgen05 GEMM per projection through the GEMM kernel's tile table (the
reference calls ``torch._grouped_mm`` three times, ``moe.py:133-148``).  Expert-parallel
execution (experts sharded over ranks, dispatch/combine over NVLink) lives in
:mod:`arctic_platform_b200.parallel.expert_parallel` and reuses :func:`grouped_ffn`.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
from torch import nn

from ..ops import gemm
from .config import DecoderConfig


def route_topk(logits: torch.Tensor, k: int, renorm: bool, score_func: str = "softmax", route_scale: float = 1.0,
               expert_bias: Optional[torch.Tensor] = None, routed_experts: Optional[torch.Tensor] = None,
               n_group: int = 1, topk_group: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token-choice routing in fp32.  Returns ``(weights [T, k] fp32, experts [T, k] int64)``.

    * ``score_func``: softmax over the experts or independent sigmoids;
    * ``expert_bias [E]`` shifts the scores for the SELECTION only, the weights are the unbiased scores
      (aux-loss-free load balancing);
    * ``n_group`` / ``topk_group``: group-limited routing -- a token may only pick experts from its ``topk_group``
      best groups (a group's quality is the sum of its two best biased scores);
    * ``routed_experts [T, k]`` replays a decision taken elsewhere (an earlier pass over the same tokens, an
      inference engine): the weights are gathered from the current scores, nothing is re-selected.
    (arctic_platform/model/implementations/qwen35/models/layers/moe.py:196-269, NemotronHRouter in the same file)."""
    x = logits.float()
    if score_func == "softmax":
        scores = torch.softmax(x, dim=-1)
    elif score_func == "sigmoid":
        scores = torch.sigmoid(x)
    else:
        raise NotImplementedError(f"Unknown score function {score_func}")
    # The decision is taken without autograd and the weights are ALWAYS a gather from the scores: a fresh decision
    # and a replayed one then build the same graph (same saved tensors), which activation checkpointing checks.
    if routed_experts is not None:
        if routed_experts.shape[-1] != k:
            raise ValueError(f"routed_experts has {routed_experts.shape[-1]} experts per token, the router keeps {k}")
        idx = routed_experts.to(torch.int64)
        if bool((idx < 0).any()):
            # tokens without a recorded decision (marked -1) route themselves
            with torch.no_grad():       # a decision only: the graph must not depend on whether a replay was partial
                _w, own = route_topk(logits, k, renorm, score_func, route_scale, expert_bias, None, n_group, topk_group)
            idx = torch.where(idx < 0, own, idx)
    else:
        with torch.no_grad():
            pick = scores if expert_bias is None else scores + expert_bias.float()
            if n_group > 1:
                T, E = pick.shape
                grouped = pick.view(T, n_group, E // n_group)
                quality = grouped.topk(min(2, E // n_group), dim=-1).values.sum(-1)        # [T, n_group]
                best = quality.topk(topk_group, dim=-1).indices
                allowed = torch.zeros_like(quality, dtype=torch.bool).scatter_(1, best, True)
                pick = grouped.masked_fill(~allowed[:, :, None], float("-inf")).view(T, E)
            if pick.is_cuda and n_group <= 1 and pick.shape[-1] <= 512:
                # one kernel: scores, selection bias, k rounds of arg-max (no sort, no host round trip)
                from ..ops.rl_ops import moe_route
                idx = moe_route(x, k, score_func, expert_bias)
            else:
                idx = torch.topk(pick, k, dim=-1).indices
    w = scores.gather(-1, idx)
    if renorm:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    if route_scale != 1.0:
        w = w * route_scale
    return w, idx


def _expert_histogram(idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Tokens per expert ``[E]`` (int64) without ``torch.bincount``, which sizes its result from the data and therefore
    synchronises with the host."""
    flat = idx.reshape(-1).to(torch.int64)
    return torch.zeros(num_experts, dtype=torch.int64, device=flat.device).scatter_add_(0, flat, torch.ones_like(flat))


def build_group_tiles(counts: torch.Tensor, n_out: int, device, bn: int = 128) -> torch.Tensor:
    """Tile table ``[n, 4] = (m0, m_end, b_row_offset, n_tile)`` for a grouped GEMM whose group ``e``
    owns ``counts[e]`` consecutive rows and the ``e``-th ``n_out``-row slab of the stacked B."""
    counts_l = counts.tolist()
    tiles = []
    row = 0
    n_tiles = (n_out + bn - 1) // bn
    for e, c in enumerate(counts_l):
        for m0 in range(row, row + c, 128):
            for nt in range(n_tiles):
                tiles.append((m0, row + c, e * n_out, nt))
        row += c
    if not tiles:
        return torch.zeros((0, 4), dtype=torch.int32, device=device)
    return torch.tensor(tiles, dtype=torch.int32).to(device)


_GROUPED_DEV = {}


def _grouped_dev_fns():
    if not _GROUPED_DEV:
        import ctypes as c
        from ..ops import _lib
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        _GROUPED_DEV["tiles"] = _lib.declare("apb_moe_group_tiles", [vp, i, i, i, vp, vp, i, i, vp, vp, vp])
        _GROUPED_DEV["gemm"] = _lib.declare("apb_gemm_bf16_grouped_dev",
                                            [vp, vp, vp, i, i, i, ll, ll, ll, i, f, vp, ll, vp, i, vp, ll, vp])
    return _GROUPED_DEV


def device_group_tiles(counts: torch.Tensor, rows: int, n_out1: int, n_out2: int):
    """Tile tables of the two grouped expert GEMMs built by a kernel from ``counts [E]`` (int32, on the GPU): no copy
    of the histogram to the host.  Returns ``(tiles1, tiles2, n_tiles [2], max1, max2)``; the tables are sized for the
    worst case (every expert may add one partial 128-row block) and ``n_tiles`` holds the live sizes on the device."""
    from ..ops import _lib
    E = counts.numel()
    max_blocks = (rows + 127) // 128 + E
    max1, max2 = max_blocks * ((n_out1 + 127) // 128), max_blocks * ((n_out2 + 127) // 128)
    dev = counts.device
    t1 = torch.empty((max1, 4), dtype=torch.int32, device=dev)
    t2 = torch.empty((max2, 4), dtype=torch.int32, device=dev)
    n_tiles = torch.empty(2, dtype=torch.int32, device=dev)
    _lib.check(_grouped_dev_fns()["tiles"](_lib.ptr(counts), E, n_out1, n_out2, _lib.ptr(t1), _lib.ptr(t2), max1, max2,
                                           _lib.ptr(n_tiles), None, _lib.stream_ptr()), "apb_moe_group_tiles")
    return t1, t2, n_tiles, max1, max2


class MoEPlan:
    """Device-side plan of one expert-layer call in the PADDED expert-major row layout: expert ``e`` owns rows
    ``[seg_start[e], seg_start[e + 1])``, a multiple of 64 of them, the rows past its ``counts[e]`` tokens holding
    zeros.  Padding makes every expert's rows a whole number of 64-row K blocks, which is what lets the weight
    gradients run as ONE grouped GEMM per weight (each tile walks the K blocks of its expert) instead of a host loop
    over experts.  Everything here is written by ``moe_plan_kernel`` from the histogram on the GPU: no number of it
    ever reaches the host.  ``rows_cap`` (host) bounds the rows in use: pairs + 63 per expert, rounded to 128."""

    def __init__(self, counts: torch.Tensor, num_pairs: int, H: int, I: int, rows_cap: Optional[int] = None):
        from ..ops import _lib
        import ctypes as c
        E = counts.numel()
        dev = counts.device
        self.E, self.H, self.I = E, H, I
        self.counts = counts
        self.rows_cap = (num_pairs + 63 * E + 127) // 128 * 128 if rows_cap is None else int(rows_cap)
        blocks = self.rows_cap // 128 + E
        I2 = 2 * I
        t = lambda n: (n + 127) // 128
        self.max_tiles = [blocks * t(I2), blocks * t(H), blocks * t(I), blocks * t(H)]
        sizes = self.max_tiles + [E * t(H) * t(I), E * t(I2) * t(H)]
        self.wgrad_tiles = sizes[4:]
        self.maps = [torch.empty((n, 4), dtype=torch.int32, device=dev) for n in sizes]
        self.exts = [torch.empty((n, 4), dtype=torch.int32, device=dev) for n in sizes]
        self.seg_start = torch.empty(E + 1, dtype=torch.int32, device=dev)
        self.n_tiles = torch.empty(4, dtype=torch.int32, device=dev)
        fn = _plan_fns()["plan"]
        arr = c.c_void_p * 6
        _lib.check(fn(_lib.ptr(counts), E, H, I, arr(*[m.data_ptr() for m in self.maps]),
                      arr(*[x.data_ptr() for x in self.exts]), (c.c_int * 4)(*self.max_tiles), _lib.ptr(self.seg_start),
                      _lib.ptr(self.n_tiles), _lib.stream_ptr()), "apb_moe_plan")
        from ..utils import checked
        if checked.active_for(counts):
            seg = self.seg_start.to(torch.int64)
            checked.check_cu_seqlens(seg, name="moe_plan.seg_start")
            checked.check_range("moe_plan.seg_start", seg, 0, self.rows_cap + 1)
            if bool((seg % 64 != 0).any()):
                raise checked.TableError("moe_plan.seg_start: an expert's rows do not start at a multiple of 64")
            cap = torch.tensor(self.max_tiles, dtype=torch.int64, device=self.n_tiles.device)
            if bool((self.n_tiles.to(torch.int64) > cap).any()):
                raise checked.TableError(f"moe_plan: tile counts {self.n_tiles.tolist()} exceed the tables {self.max_tiles}")

    def padded_rows(self, sorted_expert: torch.Tensor) -> torch.Tensor:
        """Padded row of every pair of an expert-sorted list (``sorted_expert [P]`` int64, ascending)."""
        c64 = self.counts.to(torch.int64)
        first = c64.cumsum(0) - c64
        P = sorted_expert.numel()
        within = torch.arange(P, device=sorted_expert.device) - first[sorted_expert]
        return self.seg_start.to(torch.int64)[sorted_expert] + within


_PLAN_FNS = {}


def _plan_fns():
    if not _PLAN_FNS:
        import ctypes as c
        from ..ops import _lib
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        _PLAN_FNS["plan"] = _lib.declare("apb_moe_plan", [vp, i, i, i, vp, vp, vp, vp, vp, vp])
        _PLAN_FNS["gemm"] = _lib.declare("apb_gemm_bf16_grouped_ext",
                                         [vp, vp, vp, i, i, i, ll, ll, ll, i, i, i, f, vp, vp, i, vp, ll, ll, vp])
    return _PLAN_FNS


def _grouped_ext(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, plan: MoEPlan, g: int, b_n_rows=0, b_k_rows=0):
    from ..ops import _lib
    live = g < 4
    _lib.check(_plan_fns()["gemm"](_lib.ptr(A), _lib.ptr(B), _lib.ptr(C), M, N, K, lda, ldb, ldc, a_mn, b_mn, epi, 1.0,
                                   _lib.ptr(plan.maps[g]), _lib.ptr(plan.exts[g]),
                                   plan.max_tiles[g] if live else plan.wgrad_tiles[g - 4],
                                   _lib.ptr(plan.n_tiles[g:]) if live else None, b_n_rows, b_k_rows,
                                   _lib.stream_ptr()), f"grouped expert GEMM {g}")


class _GroupedFFNPaddedFn(torch.autograd.Function):
    """Expert FFN over the padded expert-major layout of :class:`MoEPlan`, forward AND backward as grouped tcgen05
    GEMMs driven by device tables: two forward GEMMs (gate/up with the SwiGLU epilogue, down), two data-gradient
    GEMMs against the K-major view of the stacked weights and two weight-gradient GEMMs whose tiles walk the rows of
    their expert -- six launches and one SwiGLU-backward kernel per layer, none of them sized on the host."""

    @staticmethod
    def forward(ctx, x_pad, wgu, wdown, plan: MoEPlan):
        from ..ops import _lib
        E, I2, H = wgu.shape
        I = I2 // 2
        R = x_pad.shape[0]
        gu = torch.empty((R, I2), device=x_pad.device, dtype=x_pad.dtype)
        act = torch.empty((R, I), device=x_pad.device, dtype=x_pad.dtype)
        y = torch.empty((R, H), device=x_pad.device, dtype=x_pad.dtype)
        fn = _grouped_dev_fns()["gemm"]
        w1, w2 = wgu.view(E * I2, H), wdown.view(E * H, I)
        _lib.check(fn(_lib.ptr(x_pad), _lib.ptr(w1), _lib.ptr(gu), R, I2, H, x_pad.stride(0), w1.stride(0), gu.stride(0),
                      gemm.EPI_SWIGLU, 1.0, _lib.ptr(act), act.stride(0), _lib.ptr(plan.maps[0]), plan.max_tiles[0],
                      _lib.ptr(plan.n_tiles), E * I2, _lib.stream_ptr()), "grouped gate/up")
        _lib.check(fn(_lib.ptr(act), _lib.ptr(w2), _lib.ptr(y), R, H, I, act.stride(0), w2.stride(0), y.stride(0),
                      gemm.EPI_BF16, 1.0, None, 0, _lib.ptr(plan.maps[1]), plan.max_tiles[1], _lib.ptr(plan.n_tiles[1:]),
                      E * H, _lib.stream_ptr()), "grouped down")
        ctx.save_for_backward(x_pad, wgu, wdown, gu, act)
        ctx.plan = plan
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _lib
        x_pad, wgu, wdown, gu, act = ctx.saved_tensors
        plan = ctx.plan
        E, I2, H = wgu.shape
        I = I2 // 2
        R = x_pad.shape[0]
        dy = dy.contiguous()
        dev = x_pad.device
        acc_gu = getattr(wgu, "grad_f32", None)
        acc_dn = getattr(wdown, "grad_f32", None)
        dwgu = acc_gu if acc_gu is not None else torch.zeros(wgu.shape, device=dev, dtype=torch.float32)
        dwdn = acc_dn if acc_dn is not None else torch.zeros(wdown.shape, device=dev, dtype=torch.float32)
        w1, w2 = wgu.view(E * I2, H), wdown.view(E * H, I)
        dact = torch.empty_like(act)
        dgu = torch.empty_like(gu)
        dx = torch.empty_like(x_pad)
        # d act = dY @ Wdown[e]: the stacked [E * H, I] weight read K-major, K offset e * H per tile
        _grouped_ext(dy, w2, dact, R, I, H, dy.stride(0), w2.stride(0), dact.stride(0), 0, 1, gemm.EPI_BF16, plan, 2,
                     b_k_rows=E * H)
        # dWdown[e] += dY[rows of e]^T @ act[rows of e]
        _grouped_ext(dy, act, dwdn.view(E * H, I), H, I, R, dy.stride(0), act.stride(0), I, 1, 1, gemm.EPI_F32_ACCUM,
                     plan, 4)
        _lib.check(_lib.cuda_lib().apb_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dact), _lib.ptr(dgu), R, I, _lib.stream_ptr()),
                   "swiglu_bwd")
        _grouped_ext(dgu, w1, dx, R, H, I2, dgu.stride(0), w1.stride(0), dx.stride(0), 0, 1, gemm.EPI_BF16, plan, 3,
                     b_k_rows=E * I2)
        _grouped_ext(dgu, x_pad, dwgu.view(E * I2, H), I2, H, R, dgu.stride(0), x_pad.stride(0), H, 1, 1,
                     gemm.EPI_F32_ACCUM, plan, 5)
        return (dx, None if acc_gu is not None else dwgu.to(wgu.dtype),
                None if acc_dn is not None else dwdn.to(wdown.dtype), None)


def padded_plan_supported(x: torch.Tensor, wgu: torch.Tensor) -> bool:
    """The padded device-planned path needs the GPU, bf16 and at most 512 experts (one block builds the plan)."""
    E, I2, H = wgu.shape
    return (x.is_cuda and x.dtype == torch.bfloat16 and E <= 512 and H % 8 == 0 and (I2 // 2) % 8 == 0
            and os.environ.get("APB_MOE_PADDED", "1") != "0")


class _GroupedFFNFn(torch.autograd.Function):
    """y[r] = W_down[e(r)] (silu(W_g[e(r)] x[r]) * (W_u[e(r)] x[r])) for rows sorted by expert.  ``counts`` on the
    GPU (int32): the forward builds its tile tables with a kernel and never synchronises with the host; ``counts`` on
    the host: tables built in Python (the expert-parallel path, which knows its row counts already)."""

    @staticmethod
    def forward(ctx, x, wgu, wdown, counts):
        from ..ops import _lib
        E, I2, H = wgu.shape
        I = I2 // 2
        R = x.shape[0]
        gu = torch.empty((R, I2), device=x.device, dtype=x.dtype)
        act = torch.empty((R, I), device=x.device, dtype=x.dtype)
        y = torch.empty((R, H), device=x.device, dtype=x.dtype)
        if R > 0 and counts.is_cuda:
            t1, t2, n_tiles, max1, max2 = device_group_tiles(counts, R, I2, H)
            fn = _grouped_dev_fns()["gemm"]
            w1, w2 = wgu.view(E * I2, H), wdown.view(E * H, I)
            _lib.check(fn(_lib.ptr(x), _lib.ptr(w1), _lib.ptr(gu), R, I2, H, x.stride(0), w1.stride(0), gu.stride(0),
                          gemm.EPI_SWIGLU, 1.0, _lib.ptr(act), act.stride(0), _lib.ptr(t1), max1, _lib.ptr(n_tiles),
                          E * I2, _lib.stream_ptr()), "grouped gate/up")
            _lib.check(fn(_lib.ptr(act), _lib.ptr(w2), _lib.ptr(y), R, H, I, act.stride(0), w2.stride(0), y.stride(0),
                          gemm.EPI_BF16, 1.0, None, 0, _lib.ptr(t2), max2, _lib.ptr(n_tiles[1:]), E * H,
                          _lib.stream_ptr()), "grouped down")
        elif R > 0:
            t1 = build_group_tiles(counts, I2, x.device)
            t2 = build_group_tiles(counts, H, x.device)
            gemm.gemm_raw(x, wgu.view(E * I2, H), gu, M=R, N=I2, K=H, epi=gemm.EPI_SWIGLU, out2=act, tile_map=t1,
                          b_rows=E * I2, bn=128)
            gemm.gemm_raw(act, wdown.view(E * H, I), y, M=R, N=H, K=I, tile_map=t2, b_rows=E * H, bn=128)
        ctx.save_for_backward(x, wgu, wdown, gu, act, counts)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops import _lib
        x, wgu, wdown, gu, act, counts = ctx.saved_tensors
        counts = counts.cpu()                 # the per-expert loops below are driven from the host (one copy per layer)
        E, I2, H = wgu.shape
        I = I2 // 2
        R = x.shape[0]
        dy = dy.contiguous()
        dx = torch.zeros_like(x)
        acc_gu = getattr(wgu, "grad_f32", None)
        acc_dn = getattr(wdown, "grad_f32", None)
        dwgu = acc_gu if acc_gu is not None else torch.zeros(wgu.shape, device=x.device, dtype=torch.float32)
        dwdn = acc_dn if acc_dn is not None else torch.zeros(wdown.shape, device=x.device, dtype=torch.float32)
        if R > 0:
            # d act = dy @ Wdown[e]   (grouped, B stored [H, I] per expert -> MN-major B over the stacked rows)
            dact = torch.empty_like(act)
            dgu = torch.empty_like(gu)
            row = 0
            for e, c in enumerate(counts.tolist()):
                if c == 0:
                    continue
                sl = slice(row, row + c)
                gemm.matmul_nn(dy[sl], wdown[e], out=dact[sl])
                gemm.matmul_tn(dy[sl], act[sl], out=dwdn[e], accumulate=True)
                row += c
            _lib.check(_lib.cuda_lib().apb_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dact), _lib.ptr(dgu), R, I,
                                                      _lib.stream_ptr()), "swiglu_bwd")
            row = 0
            for e, c in enumerate(counts.tolist()):
                if c == 0:
                    continue
                sl = slice(row, row + c)
                gemm.matmul_nn(dgu[sl], wgu[e], out=dx[sl])
                gemm.matmul_tn(dgu[sl], x[sl], out=dwgu[e], accumulate=True)
                row += c
        return (dx, None if acc_gu is not None else dwgu.to(wgu.dtype),
                None if acc_dn is not None else dwdn.to(wdown.dtype), None)


def grouped_ffn(x_sorted: torch.Tensor, wgu: torch.Tensor, wdown: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Expert FFN over rows already sorted by expert; ``counts [E]`` rows per expert (CPU or GPU int64)."""
    if not x_sorted.is_cuda:
        outs, row = [], 0
        for e, c in enumerate(counts.tolist()):
            xe = x_sorted[row:row + c]
            gu = xe @ wgu[e].t()
            outs.append((torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ wdown[e].t())
            row += c
        return torch.cat(outs) if outs else x_sorted.new_zeros((0, wdown.shape[1]))
    if counts.is_cuda and counts.numel() <= 512:
        return _GroupedFFNFn.apply(x_sorted.contiguous(), wgu, wdown, counts.to(torch.int32))
    return _GroupedFFNFn.apply(x_sorted.contiguous(), wgu, wdown, counts.cpu())


class MoEFeedForward(nn.Module):
    def __init__(self, cfg: DecoderConfig, device, dtype):
        super().__init__()
        self.cfg = cfg
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.router = nn.Parameter(torch.empty(E, H, device=device, dtype=dtype))
        self.wgu = nn.Parameter(torch.empty(E, 2 * I, H, device=device, dtype=dtype))
        self.wdown = nn.Parameter(torch.empty(E, H, I, device=device, dtype=dtype))
        S = cfg.shared_expert_intermediate_size
        if S > 0:       # dense expert every token passes through, scaled by a per-token sigmoid gate
            self.shared_wgu = nn.Parameter(torch.empty(2 * S, H, device=device, dtype=dtype))
            self.shared_wdown = nn.Parameter(torch.empty(H, S, device=device, dtype=dtype))
            self.shared_gate = nn.Parameter(torch.empty(1, H, device=device, dtype=dtype))
        else:
            self.shared_wgu = self.shared_wdown = self.shared_gate = None
        self.ep = None  # set by parallel.expert_parallel.attach() when experts are sharded over ranks
        self.last_tokens_per_expert: Optional[torch.Tensor] = None
        # aux-loss-free load balancing: a selection bias per expert and the load seen since the last update
        if cfg.moe_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(E, device=device, dtype=torch.float32), persistent=True)
            self.register_buffer("tokens_per_expert", torch.zeros(E, device=device, dtype=torch.float32), persistent=False)
        else:
            self.expert_bias = self.tokens_per_expert = None
        # routing replay: "capture" stores every pass's decision, "replay" consumes them in the same order (the
        # recompute of an activation-checkpointed block); ``routed_experts`` forces one decision from outside
        self.replay_mode: Optional[str] = None
        self._captured: list = []
        self.routed_experts: Optional[torch.Tensor] = None
        self.routing_log: Optional[list] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._routed(x)
        if self.shared_wgu is not None:
            from .decoder import gate_up_act
            shared = gemm.linear(gate_up_act(x, self.shared_wgu), self.shared_wdown)
            gate = torch.sigmoid(x.float() @ self.shared_gate.float().t())
            y = (y.float() + gate * shared.float()).to(x.dtype)
        return y

    def _routed(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        T, H = x.shape
        logits = gemm.linear(x, self.router)
        forced = self.routed_experts
        if forced is None and self.replay_mode == "replay" and self._captured:
            forced = self._captured.pop(0)
        w, idx = route_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.moe_score_func, cfg.moe_route_scale,
                            self.expert_bias, forced, cfg.moe_n_group, cfg.moe_topk_group)
        if self.replay_mode == "capture":
            self._captured.append(idx.detach())
        if self.routing_log is not None:                         # a sampler records what it routed, pass by pass
            self.routing_log.append(idx.detach())
        if self.tokens_per_expert is not None and self.training and self.replay_mode != "replay":
            self.tokens_per_expert += _expert_histogram(idx, cfg.num_experts).to(self.tokens_per_expert.dtype)
        if self.ep is not None:
            return self.ep.forward(self, x, w, idx)
        k = cfg.num_experts_per_tok
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = _expert_histogram(flat_e, cfg.num_experts)
        self.last_tokens_per_expert = counts.detach()
        src_tok = torch.div(order, k, rounding_mode="floor")
        if torch.is_grad_enabled() and padded_plan_supported(x, self.wgu):
            # training: padded expert-major rows, forward and backward as grouped GEMMs planned on the device
            plan = MoEPlan(counts.to(torch.int32), flat_e.numel(), H, self.wgu.shape[1] // 2)
            pos = plan.padded_rows(flat_e.index_select(0, order))
            x_pad = torch.zeros((plan.rows_cap, H), device=x.device, dtype=x.dtype).index_copy(
                0, pos, x.index_select(0, src_tok))
            ys = _GroupedFFNPaddedFn.apply(x_pad, self.wgu, self.wdown, plan).index_select(0, pos)
        else:
            xs = x.index_select(0, src_tok)
            ys = grouped_ffn(xs, self.wgu, self.wdown, counts)
        wflat = w.reshape(-1).index_select(0, order).to(ys.dtype)
        out = torch.zeros((T, H), device=x.device, dtype=torch.float32 if x.is_cuda else x.dtype)
        out.index_add_(0, src_tok, (ys * wflat[:, None]).to(out.dtype))
        return out.to(x.dtype)


    @torch.no_grad()
    def update_expert_bias(self, coeff: float = 1e-3, group=None) -> Optional[torch.Tensor]:
        """Moves every expert's selection bias by ``coeff`` toward the mean load (up for starved experts, down for
        crowded ones) from the token counts accumulated since the last call -- summed over ``group`` when the data
        is sharded -- and clears the counts.  Call once per optimizer step."""
        if self.expert_bias is None:
            return None
        load = self.tokens_per_expert.clone()
        if group is not False and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
            torch.distributed.all_reduce(load, group=group)
        self.expert_bias += coeff * torch.sign(load.mean() - load)
        self.expert_bias -= self.expert_bias.mean()
        self.tokens_per_expert.zero_()
        return load


class router_replay_scope:
    """Context for one pass over a block: ``capture`` on the original forward, ``replay`` on the recompute, so that
    both passes route identically and every tensor inside the checkpointed region keeps its shape even when the
    router's scores differ in the last bits (arctic_platform/model/implementations/qwen35/gpu/
    router_replay_recompute.py:1-124 patches the checkpoint machinery for the same effect)."""

    def __init__(self, block: nn.Module, mode: str):
        self.moes = [m for m in block.modules() if isinstance(m, MoEFeedForward)]
        self.mode = mode

    def __enter__(self):
        for m in self.moes:
            m.replay_mode = self.mode
        return self

    def __exit__(self, *exc):
        for m in self.moes:
            m.replay_mode = None
            if self.mode == "replay":
                m._captured.clear()
        return False
