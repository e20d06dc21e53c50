"""Latent mixture of experts with non-gated relu^2 experts (the Nemotron-H style feed-forward).

Differences from the SwiGLU layer of :mod:`.moe`:

* experts are TWO projections with a squared ReLU between them, ``down(relu(up(x))^2)``, no gate;
* routed tokens are projected from the model width ``H`` to a narrower latent width ``L`` before the experts and
  back after them (``fc1 [L, H]`` / ``fc2 [H, L]``; without a latent width the experts work at ``H``), so expert
  weights and -- under expert parallelism -- the dispatched rows are ``L`` wide;
* the router scores with independent sigmoids, selects among the best groups of experts with a learned-elsewhere
  correction bias (plus the load-balancing bias when enabled) and weighs with the UNBIASED scores;
* the shared expert is non-gated too and is added without a per-token gate.

The routing weight and the route scale are applied in the latent space, before ``fc2``, as the reference does
(arctic_platform/model/implementations/qwen35/models/layers/moe.py:564-606 experts, :653-721 router, :739-938
layer).  On a GPU the projections run through the tcgen05 GEMM (one launch per expert with rows; the activation
is elementwise); the class plugs into the decoder block, activation checkpointing (routing replay) and the
load-balancing update exactly as the SwiGLU layer does."""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..ops import gemm
from .config import DecoderConfig
from .moe import MoEFeedForward, route_topk


def relu2(x: torch.Tensor) -> torch.Tensor:
    return torch.relu(x).square()


def nongated_grouped_ffn(x_sorted: torch.Tensor, wup: torch.Tensor, wdown: torch.Tensor, counts: torch.Tensor
                         ) -> torch.Tensor:
    """``y[r] = W_down[e(r)] relu(W_up[e(r)] x[r])^2`` for rows sorted by expert.  ``wup [E, I, L]``,
    ``wdown [E, L, I]``, ``counts [E]`` rows per expert."""
    outs, row = [], 0
    for e, c in enumerate(counts.tolist()):
        if c:
            xe = x_sorted[row:row + c]
            outs.append(gemm.linear(relu2(gemm.linear(xe, wup[e])), wdown[e]))
        row += c
    return torch.cat(outs) if outs else x_sorted.new_zeros((0, wdown.shape[1]))


class LatentMoEFeedForward(MoEFeedForward):
    latent = True

    def __init__(self, cfg: DecoderConfig, device, dtype):
        nn.Module.__init__(self)
        self.cfg = cfg
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        L = cfg.moe_latent_dim or H
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, device=device, dtype=dtype))
        self.router = mk(E, H)
        self.wup = mk(E, I, L)
        self.wdown = mk(E, L, I)
        if cfg.moe_latent_dim:
            self.fc1 = mk(L, H)
            self.fc2 = mk(H, L)
        else:
            self.fc1 = self.fc2 = None
        S = cfg.shared_expert_intermediate_size
        if S > 0:
            self.shared_wup = mk(S, H)
            self.shared_wdown = mk(H, S)
        else:
            self.shared_wup = self.shared_wdown = None
        # selection bias that comes with a checkpoint; it is not trained here (a buffer, as in the reference)
        self.register_buffer("e_score_correction_bias", torch.zeros(E, device=device, dtype=torch.float32))
        self.ep = None
        self.last_tokens_per_expert: Optional[torch.Tensor] = None
        if cfg.moe_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(E, device=device, dtype=torch.float32), persistent=True)
            self.register_buffer("tokens_per_expert", torch.zeros(E, device=device, dtype=torch.float32), persistent=False)
        else:
            self.expert_bias = self.tokens_per_expert = None
        self.replay_mode: Optional[str] = None
        self._captured: list = []
        self.routed_experts: Optional[torch.Tensor] = None
        self.routing_log: Optional[list] = None
        # names the SwiGLU layer's users look for
        self.shared_wgu = self.shared_gate = None
        self.wgu = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._routed(x)
        if self.shared_wup is not None:
            y = y + gemm.linear(relu2(gemm.linear(x, self.shared_wup)), self.shared_wdown)
        return y

    def _routed(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        if self.ep is not None:
            raise NotImplementedError("expert parallelism is built for the SwiGLU expert layout only")
        T, H = x.shape
        k = cfg.num_experts_per_tok
        logits = gemm.linear(x, self.router)
        forced = self.routed_experts
        if forced is None and self.replay_mode == "replay" and self._captured:
            forced = self._captured.pop(0)
        bias = self.e_score_correction_bias if self.expert_bias is None else self.e_score_correction_bias + self.expert_bias
        w, idx = route_topk(logits, k, cfg.norm_topk_prob, "sigmoid", cfg.moe_route_scale, bias, forced,
                            cfg.moe_n_group, cfg.moe_topk_group)
        if self.replay_mode == "capture":
            self._captured.append(idx.detach())
        if self.routing_log is not None:
            self.routing_log.append(idx.detach())
        if self.tokens_per_expert is not None and self.training and self.replay_mode != "replay":
            self.tokens_per_expert += torch.bincount(idx.reshape(-1), minlength=cfg.num_experts).to(self.tokens_per_expert.dtype)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=cfg.num_experts)
        self.last_tokens_per_expert = counts.detach()
        src_tok = torch.div(order, k, rounding_mode="floor")
        xs = x.index_select(0, src_tok)
        if self.fc1 is not None:
            xs = gemm.linear(xs, self.fc1)
        ys = nongated_grouped_ffn(xs, self.wup, self.wdown, counts)
        wflat = w.reshape(-1).index_select(0, order)
        ys = (ys.float() * wflat[:, None]).to(ys.dtype)
        if self.fc2 is not None:
            ys = gemm.linear(ys, self.fc2)
        out = torch.zeros((T, H), device=x.device, dtype=torch.float32 if x.is_cuda else x.dtype)
        out.index_add_(0, src_tok, ys.to(out.dtype))
        return out.to(x.dtype)
