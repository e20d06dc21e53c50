"""Gated DeltaNet linear attention (the "linear_attention" layers of the Qwen3.5 / Qwen3-Next hybrids).

Per head, with key/query dimension ``Dk``, value dimension ``Dv`` and state ``S`` of shape ``[Dk, Dv]``:

    alpha_t = exp(g_t)                       (g_t <= 0: learned decay)
    S'      = alpha_t * S_{t-1}
    S_t     = S' + beta_t * k_t (v_t - S'^T k_t)^T          (delta rule: correct the value stored under k_t)
    o_t     = S_t^T q_t / sqrt(Dk)

with L2-normalised ``q_t, k_t``.  ``gated_delta_rule_recurrent`` is that recurrence token by token (the oracle);
``gated_delta_rule_chunked`` evaluates it 64 tokens at a time: inside a chunk the corrections form a unit lower
triangular system that is solved once (forward substitution), the carried state enters through two matmuls, and the
state advances once per chunk -- the algorithm of the reference's ``torch_chunk_gated_delta_rule``
(arctic_platform/model/implementations/qwen35/models/qwen3_5_moe/modeling_qwen3_5_moe.py:73-1086).

``GatedDeltaNet`` is the layer: fused input projections, a causal depth-wise convolution (kernel 4) over q/k/v, the
rule above, a gated RMSNorm (``norm(o) * silu(z)``) and the output projection.  It runs on the packed token axis and
takes its sequence structure from the attention layout: every segment starts from the final (convolution, recurrent)
state of its prefix segment, so a prompt shared by several rollouts is processed once (prompt reuse as in
arctic_platform/rl/zorro_train/qwen_attention_patcher.py:589-752).  The state-independent parts are batched PyTorch
matmuls; the recurrence over the chunks runs as one CUDA kernel (``csrc/delta_rule.cu``) in passes that need no
gradient (scoring, prefill) and as a differentiable loop of PyTorch ops in training.  ``context_parallel_delta_rule``
is the sequence-sharded form: every rank runs its slice of a sequence and the carried state crosses the ranks as an
affine map (one small all-gather), so no rank recomputes another rank's tokens.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import gemm


def _l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def gated_delta_rule_recurrent(q, k, v, g, beta, state: Optional[torch.Tensor] = None, l2norm: bool = True
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q, k [T, H, Dk]``, ``v [T, H, Dv]``, ``g, beta [T, H]`` -> ``(o [T, H, Dv], final state [H, Dk, Dv])``."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    q, k, v, g, beta = (x.float() for x in (q, k, v, g, beta))
    if l2norm:
        q, k = _l2norm(q), _l2norm(k)
    q = q * Dk ** -0.5
    S = torch.zeros(H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float().clone()
    out = []
    for t in range(T):
        S = S * torch.exp(g[t])[:, None, None]
        pred = torch.einsum("hkv,hk->hv", S, k[t])
        S = S + torch.einsum("hk,hv->hkv", k[t] * beta[t][:, None], v[t] - pred)
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    o = torch.stack(out) if out else v.new_zeros((0, H, Dv), dtype=torch.float32)
    return o, S


def gated_delta_rule_chunked(q, k, v, g, beta, state: Optional[torch.Tensor] = None, l2norm: bool = True,
                             chunk: int = 64) -> Tuple[torch.Tensor, torch.Tensor]:
    """Same contract as the recurrent form, ``chunk`` tokens per step (differentiable)."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    if T == 0:
        S0 = torch.zeros(H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float()
        return v.new_zeros((0, H, Dv), dtype=torch.float32), S0
    q, k, v, g, beta = (x.float().transpose(0, 1) for x in (q, k, v, g, beta))          # [H, T, ...]
    if l2norm:
        q, k = _l2norm(q), _l2norm(k)
    q = q * Dk ** -0.5
    pad = (-T) % chunk
    if pad:
        q, k, v = (F.pad(x, (0, 0, 0, pad)) for x in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    N = (T + pad) // chunk
    q, k, v = (x.reshape(H, N, chunk, -1) for x in (q, k, v))
    g = g.reshape(H, N, chunk).cumsum(-1)                                                   # log decay since chunk start
    beta = beta.reshape(H, N, chunk)
    kb, vb = k * beta[..., None], v * beta[..., None]
    # decay between positions j <= i of a chunk
    diff = g[..., :, None] - g[..., None, :]
    tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
    decay = torch.where(tril, torch.exp(torch.where(tril, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    # corrections inside a chunk: (I + A) u = rhs with A strictly lower triangular -> u = (I + A)^{-1} rhs
    A = (kb @ k.transpose(-1, -2)) * decay
    A = A.masked_fill(~torch.tril(tril, -1), 0.0)
    eye = torch.eye(chunk, device=q.device, dtype=torch.float32)
    Tinv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
    u_local = Tinv @ vb                                     # corrected values if the carried state were zero
    w_state = Tinv @ (kb * torch.exp(g)[..., None])         # how the carried state enters the corrections
    S = torch.zeros(H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float()
    outs = []
    qk = (q @ k.transpose(-1, -2)) * decay                  # causal (diagonal included) intra-chunk scores
    if _scan_kernel_ok(q, chunk, Dk) and not torch.is_grad_enabled():
        # no-grad passes (scoring, prefill): the recurrence over the chunks is one kernel, the state stays on chip
        o, S = _scan_on_device(u_local, w_state, q * torch.exp(g)[..., None], qk,
                               k * torch.exp(g[..., -1:] - g)[..., None], torch.exp(g[..., -1]), S)
        return o.reshape(H, N * chunk, Dv)[:, :T].transpose(0, 1), S
    for n in range(N):
        u = u_local[:, n] - w_state[:, n] @ S               # value corrections of this chunk given the carried state
        o = (q[:, n] * torch.exp(g[:, n])[..., None]) @ S + qk[:, n] @ u
        outs.append(o)
        g_end = g[:, n, -1]
        S = S * torch.exp(g_end)[:, None, None] + (k[:, n] * torch.exp(g_end[:, None] - g[:, n])[..., None]).transpose(-1, -2) @ u
    o = torch.stack(outs, 1).reshape(H, N * chunk, Dv)[:, :T].transpose(0, 1)
    if pad:
        # padded steps have g = 0, beta = 0: they leave the state unchanged
        pass
    return o, S


def delta_rule_transition(q, k, g, beta, l2norm: bool = True, chunk: int = 64) -> torch.Tensor:
    """The linear part of the state map of a stretch of tokens: ``S_end = P S_start + C`` with ``P [H, Dk, Dk]``.
    One step is ``S <- alpha (I - beta k k^T) S + beta k v^T``; ``P`` is the ordered product of the step matrices.
    Obtained by running the rule itself on the identity (every column of ``I`` as a value column, ``v = 0``)."""
    T, H, Dk = q.shape
    eye = torch.eye(Dk, dtype=torch.float32, device=q.device).expand(H, Dk, Dk).contiguous()
    zero_v = torch.zeros((T, H, Dk), dtype=torch.float32, device=q.device)
    _, P = gated_delta_rule_chunked(q, k, zero_v, g, beta, eye, l2norm, chunk)
    return P


def context_parallel_delta_rule(q, k, v, g, beta, group, l2norm: bool = True, chunk: int = 64
                                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """One sequence cut into ``world`` consecutive slices, one per rank of ``group`` (rank order = token order).
    Every rank runs the rule on ITS slice only: first from a zero state (giving the offset ``C`` of its affine state
    map) and on the identity (giving ``P``), the ``(P, C)`` pairs are all-gathered (``world * H * Dk * (Dk + Dv)``
    floats), every rank composes the maps of the ranks before it into its true starting state, and runs its slice
    once more from there.  Three local passes instead of ``world`` redundant ones on gathered rows; differentiable
    (the all-gather is ``gather_rows_with_grad``).  Returns ``(o of the local slice, this rank's end state)`` -- the
    last rank's end state is the state after the whole sequence.  The reference passes the state between ranks
    inside the ``fla`` kernels (.../qwen3_5_moe/modeling_qwen3_5_moe.py:247-349)."""
    import torch.distributed as dist
    from ..parallel.ulysses import gather_rows_with_grad
    W, r = dist.get_world_size(group), dist.get_rank(group)
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    _, C = gated_delta_rule_chunked(q, k, v, g, beta, None, l2norm, chunk)
    P = delta_rule_transition(q, k, g, beta, l2norm, chunk)
    mine = torch.cat([P.reshape(1, -1), C.reshape(1, -1)], 1).float()
    allm = gather_rows_with_grad(mine, group)                               # [W, H*Dk*Dk + H*Dk*Dv]
    S = torch.zeros((H, Dk, Dv), dtype=torch.float32, device=q.device)
    for j in range(r):
        Pj = allm[j, :H * Dk * Dk].view(H, Dk, Dk)
        Cj = allm[j, H * Dk * Dk:].view(H, Dk, Dv)
        S = Pj @ S + Cj
    return gated_delta_rule_chunked(q, k, v, g, beta, S, l2norm, chunk)


def _scan_kernel_ok(q: torch.Tensor, chunk: int, Dk: int) -> bool:
    import os
    return (q.is_cuda and chunk == 64 and Dk % 4 == 0 and 4 <= Dk <= 256
            and os.environ.get("APB_DELTA_RULE_KERNEL", "1") != "0")


def _scan_on_device(u_local, w_state, q_dec, qk, k_dec, e_end, S0):
    """``delta_rule_scan_kernel``: all operands fp32 ``[H, N, 64, *]`` (``e_end [H, N]``, ``S0 [H, Dk, Dv]``) ->
    ``(o [H, N, 64, Dv], final state)``."""
    import ctypes as c
    from ..ops import _lib
    H, N, C, Dv = u_local.shape
    Dk = w_state.shape[-1]
    t = [x.float().contiguous() for x in (u_local, w_state, q_dec, qk, k_dec, e_end, S0)]
    out = torch.empty((H, N, C, Dv), dtype=torch.float32, device=u_local.device)
    s_out = torch.empty((H, Dk, Dv), dtype=torch.float32, device=u_local.device)
    vp, i = c.c_void_p, c.c_int
    fn = _lib.declare("apb_delta_rule_scan", [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, vp])
    _lib.check(fn(*[_lib.ptr(x) for x in t], _lib.ptr(out), _lib.ptr(s_out), H, N, Dk, Dv, _lib.stream_ptr()),
               "apb_delta_rule_scan")
    return out, s_out


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Depth-wise causal convolution along tokens.  ``x [T, C]``, ``w [C, K]``, ``state [K-1, C]`` = the last
    ``K-1`` inputs of the preceding context (zeros at a sequence start).  Returns ``(y [T, C], new state)``."""
    K = w.shape[1]
    hist = x.new_zeros((K - 1, x.shape[1])) if state is None else state.to(x.dtype)
    xx = torch.cat([hist, x], 0)                             # [T + K - 1, C]
    y = F.conv1d(xx.t()[None].float(), w[:, None, :].float(), groups=w.shape[0])[0].t()
    return y.to(x.dtype), xx[-(K - 1):]


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg, device, dtype):
        super().__init__()
        self.cfg = cfg
        H = cfg.hidden_size
        self.Hk, self.Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.Dk, self.Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.key_dim, self.value_dim = self.Hk * self.Dk, self.Hv * self.Dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        mk = lambda *s: nn.Parameter(torch.empty(*s, device=device, dtype=dtype))
        self.in_qkv = mk(self.conv_dim, H)
        self.in_z = mk(self.value_dim, H)
        self.in_b = mk(self.Hv, H)
        self.in_a = mk(self.Hv, H)
        self.conv_w = mk(self.conv_dim, cfg.linear_conv_kernel_dim)
        self.dt_bias = mk(self.Hv)
        self.A_log = mk(self.Hv)
        self.norm_w = mk(self.Dv)
        self.out_proj = mk(H, self.value_dim)
        self.chunk = 64
        # a sampler's prefill sets this to a dict; forward then leaves ``end row -> (conv state, S)`` of every
        # segment in it, the starting point of token-by-token decoding
        self.capture: Optional[Dict[int, Tuple[torch.Tensor, torch.Tensor]]] = None

    def forward(self, x: torch.Tensor, layout) -> torch.Tensor:
        """``x [T, H]`` on the packed axis -> ``[T, H]``.  Under sequence parallelism ``x`` is this rank's row shard
        and ``layout`` the (padded) global layout: the rows are gathered, the layer runs on the whole axis and the
        rank keeps its slice."""
        sp_group = getattr(self, "sp_group", None)
        if sp_group is not None and self._context_parallel_ok(x, layout):
            return self._forward_context_parallel(x, layout, sp_group)
        if sp_group is not None:
            import torch.distributed as dist
            from ..parallel.ulysses import gather_rows_with_grad
            rows = x.shape[0]
            full = self._forward_full(gather_rows_with_grad(x, sp_group), layout)
            r = dist.get_rank(sp_group)
            return full[r * rows:(r + 1) * rows]
        return self._forward_full(x, layout)

    # ------------------------------------------------------------------ sequence-sharded form
    def _context_parallel_ok(self, x: torch.Tensor, layout) -> bool:
        """Every rank can run its own rows when no segment reads another segment's state (no shared-prefix ranges:
        plain packing) and a rank holds at least the convolution's history length.  De-duplicated prompts fall back
        to the gathered form."""
        import os
        if os.environ.get("APB_LINEAR_ATTN_CP", "1") == "0" or self.capture is not None:
            return False
        segs = layout.segs
        return bool((segs[:, 3] == 0).all()) and x.shape[0] >= self.cfg.linear_conv_kernel_dim - 1

    def _forward_context_parallel(self, x: torch.Tensor, layout, group) -> torch.Tensor:
        """``x``: this rank's rows ``[lo, hi)`` of the padded packed axis.  A segment that crosses a rank boundary is
        continued by the next rank from (a) the last ``K - 1`` pre-convolution rows and (b) the recurrent state at
        the boundary; (a) travels as one small all-gather of every rank's tail rows, (b) as the all-gather of the
        affine state maps of the ranks' LAST pieces (see ``context_parallel_delta_rule``).  Which pieces start or
        end inside a rank follows from the layout, which every rank has."""
        import torch.distributed as dist
        from ..parallel.ulysses import gather_rows_with_grad
        W, r = dist.get_world_size(group), dist.get_rank(group)
        rows = x.shape[0]
        K1 = self.cfg.linear_conv_kernel_dim - 1
        Hv, Dk, Dv = self.Hv, self.Dk, self.Dv
        rep = self.Hv // self.Hk
        mixed = gemm.linear(x, self.in_qkv)
        z = gemm.linear(x, self.in_z).view(rows, Hv, Dv)
        beta = torch.sigmoid(x.float() @ self.in_b.float().t())
        g = -torch.exp(self.A_log.float()) * F.softplus(x.float() @ self.in_a.float().t() + self.dt_bias.float())

        def pieces_of(rank: int):
            lo, hi = rank * rows, (rank + 1) * rows
            out = []
            for _qs, _ql, _ps, _pl, os_, ol in layout.segs.tolist():
                a, b = max(os_, lo), min(os_ + ol, hi)
                if b > a:
                    out.append((a, b, os_ >= lo, os_ + ol <= hi, os_))       # rows, starts here, ends here, seg start
            return sorted(out)

        mine = pieces_of(r)
        lo = r * rows

        def qkv_of(a: int, b: int, conv_state):
            y, _ = causal_conv1d(mixed[a - lo:b - lo], self.conv_w, conv_state)
            y = F.silu(y)
            n = b - a
            q = y[:, :self.key_dim].reshape(n, self.Hk, Dk)
            k = y[:, self.key_dim:2 * self.key_dim].reshape(n, self.Hk, Dk)
            v = y[:, 2 * self.key_dim:].reshape(n, Hv, Dv)
            if rep > 1:
                q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
            return q, k, v

        # (a) convolution history across the boundary: everybody's last K-1 pre-convolution rows
        tails = gather_rows_with_grad(mixed[rows - K1:].reshape(1, -1).float(), group).view(W, K1, -1)
        first_state = None
        if mine and not mine[0][2]:
            prev = pieces_of(r - 1)[-1]                       # the piece this one continues
            hist = tails[r - 1].to(mixed.dtype)
            have = prev[1] - prev[0]                          # rows of the segment on the previous rank
            if have < K1:
                if not prev[2]:
                    raise NotImplementedError("a rank holds fewer rows of a sequence than the convolution reaches back")
                hist = torch.cat([hist.new_zeros((K1 - have, hist.shape[1])), hist[K1 - have:]], 0)
            first_state = hist
        # (b) state maps of every rank's last piece, when it continues on the next rank
        P = torch.zeros((Hv, Dk, Dk), dtype=torch.float32, device=x.device)
        C = torch.zeros((Hv, Dk, Dv), dtype=torch.float32, device=x.device)
        last_done = None
        if mine and not mine[-1][3]:
            a, b, starts, _e, _s = mine[-1]
            q, k, v = qkv_of(a, b, None if starts else first_state)
            sl = slice(a - lo, b - lo)
            o0, C = gated_delta_rule_chunked(q, k, v, g[sl], beta[sl], None, chunk=self.chunk)
            if starts:
                last_done = o0                                # started from a true zero state: this IS its output
            else:
                P = delta_rule_transition(q, k, g[sl], beta[sl], chunk=self.chunk)
        # (a rank whose last piece ends inside it contributes zeros; tied to `mixed` so that the gather's collective
        # backward exists in every rank's graph)
        maps = gather_rows_with_grad(torch.cat([P.reshape(1, -1), C.reshape(1, -1)], 1) + 0.0 * mixed[:1].float().sum(),
                                     group)
        S_in = None
        if mine and not mine[0][2]:
            # walk back to the rank where the sequence started, then compose forward
            j0 = r - 1
            while not pieces_of(j0)[-1][2]:
                j0 -= 1
            S_in = torch.zeros((Hv, Dk, Dv), dtype=torch.float32, device=x.device)
            for j in range(j0, r):
                Pj = maps[j, :Hv * Dk * Dk].view(Hv, Dk, Dk)
                Cj = maps[j, Hv * Dk * Dk:].view(Hv, Dk, Dv)
                S_in = Cj if j == j0 else Pj @ S_in + Cj
        out = x.new_zeros((rows, Hv, Dv), dtype=torch.float32)
        for i, (a, b, starts, ends, _s) in enumerate(mine):
            sl = slice(a - lo, b - lo)
            if i == len(mine) - 1 and last_done is not None:
                o = last_done
            else:
                q, k, v = qkv_of(a, b, None if starts else first_state)
                o, _ = gated_delta_rule_chunked(q, k, v, g[sl], beta[sl], None if starts else S_in, chunk=self.chunk)
            out = out.index_put((torch.arange(a - lo, b - lo, device=x.device),), o)
        # both all-gathers have a collective backward: tie them into every rank's graph (a rank whose rows start a
        # new sequence does not read them), so that all ranks run the same collectives in the same order
        out = out + 0.0 * (tails.sum() + maps.sum())
        return self._gated_out(out, z, x.dtype)

    def _forward_full(self, x: torch.Tensor, layout) -> torch.Tensor:
        T = x.shape[0]
        mixed = gemm.linear(x, self.in_qkv)
        z = gemm.linear(x, self.in_z).view(T, self.Hv, self.Dv)
        b = x.float() @ self.in_b.float().t()
        a = x.float() @ self.in_a.float().t()
        beta = torch.sigmoid(b)
        g = -torch.exp(self.A_log.float()) * F.softplus(a + self.dt_bias.float())
        out = x.new_zeros((T, self.Hv, self.Dv), dtype=torch.float32)
        final: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}          # end row of a key range -> states after it
        rep = self.Hv // self.Hk
        for qs, ql, ps, pl, os_, ol in layout.segs.tolist():
            if ol == 0:
                continue
            init = final.get(ps + pl) if pl > 0 else None
            if pl > 0 and init is None:
                raise ValueError("linear attention: a segment's prefix range must be an earlier segment's own range")
            conv_state, S = init if init is not None else (None, None)
            sl = slice(os_, os_ + ol)
            y, conv_new = causal_conv1d(mixed[sl], self.conv_w, conv_state)
            y = F.silu(y)
            q = y[:, :self.key_dim].reshape(ol, self.Hk, self.Dk)
            k = y[:, self.key_dim:2 * self.key_dim].reshape(ol, self.Hk, self.Dk)
            v = y[:, 2 * self.key_dim:].reshape(ol, self.Hv, self.Dv)
            if rep > 1:
                q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
            o, S_new = gated_delta_rule_chunked(q, k, v, g[sl], beta[sl], S, chunk=self.chunk)
            final[os_ + ol] = (conv_new, S_new)
            # the segment's query rows are the last ``ql`` rows of its own range
            out = out.index_put((torch.arange(qs, qs + ql, device=x.device),), o[ol - ql:])
        if self.capture is not None:
            self.capture.update(final)
        return self._gated_out(out, z, x.dtype)

    def _gated_out(self, out: torch.Tensor, z: torch.Tensor, dtype) -> torch.Tensor:
        """Gated RMSNorm ``norm(o) * w * silu(z)`` and the output projection; ``out, z [T, Hv, Dv]``."""
        T = out.shape[0]
        o = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * self.norm_w.float()
        o = (o * F.silu(z.float())).to(dtype)
        return gemm.linear(o.reshape(T, self.value_dim), self.out_proj)

    @torch.no_grad()
    def step(self, x: torch.Tensor, conv_state: torch.Tensor, S: torch.Tensor
             ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """One token for each of ``B`` independent sequences: ``x [B, H]``, ``conv_state [B, K-1, C]``,
        ``S [B, Hv, Dk, Dv]`` (fp32) -> ``(y [B, H], new conv_state, new S)``.  The same arithmetic as one step
        of :func:`gated_delta_rule_recurrent` behind the causal convolution."""
        B = x.shape[0]
        mixed = gemm.linear(x, self.in_qkv)
        z = gemm.linear(x, self.in_z).view(B, self.Hv, self.Dv)
        beta = torch.sigmoid(x.float() @ self.in_b.float().t())
        g = -torch.exp(self.A_log.float()) * F.softplus(x.float() @ self.in_a.float().t() + self.dt_bias.float())
        window = torch.cat([conv_state.to(mixed.dtype), mixed[:, None, :]], 1)              # [B, K, C]
        y = (window.float() * self.conv_w.float().t()[None]).sum(1).to(mixed.dtype)
        y = F.silu(y)
        q = y[:, :self.key_dim].reshape(B, self.Hk, self.Dk)
        k = y[:, self.key_dim:2 * self.key_dim].reshape(B, self.Hk, self.Dk)
        v = y[:, 2 * self.key_dim:].reshape(B, self.Hv, self.Dv).float()
        rep = self.Hv // self.Hk
        if rep > 1:
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
        q, k = _l2norm(q.float()) * self.Dk ** -0.5, _l2norm(k.float())
        S = S * torch.exp(g)[:, :, None, None]
        pred = torch.einsum("bhkv,bhk->bhv", S, k)
        S = S + torch.einsum("bhk,bhv->bhkv", k * beta[:, :, None], v - pred)
        o = torch.einsum("bhkv,bhk->bhv", S, q)
        return self._gated_out(o, z, x.dtype), window[:, 1:], S
