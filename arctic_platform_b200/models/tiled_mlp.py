"""Sequence-tiled MLP: bounds the activation memory of the feed-forward sublayer for long packed batches.

The gate/up pre-activations of a dense block are ``[tokens, 2 * intermediate]`` -- for Qwen3-4B 7.6x the hidden
state -- and are what the backward of the SwiGLU needs.  With tiling the forward runs the MLP on ``shards`` row
tiles and keeps only its input; the backward re-runs one tile at a time, back-propagates it and frees it, so the
peak holds one tile's pre-activations instead of the whole batch's.  Rows are independent in an MLP, so the result
is bit-identical to the untiled computation; weight gradients accumulate tile by tile (into the engine's fp32
gradient buffer when the kernels write there, else into ``.grad``).

Same contract as the reference's TiledMLP patch (arctic_platform/model/implementations/qwen35/gpu/tiled_mlp.py:19-39,
which wraps DeepSpeed's sequence-tiled compute; ``shards="auto"`` uses its rule ceil(tokens / hidden))."""
from __future__ import annotations

import math
from typing import Callable, Sequence, Union

import torch


class _TiledMLPFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, fn, shards, *params):
        ctx.fn, ctx.shards = fn, shards
        ctx.save_for_backward(x)
        with torch.no_grad():
            return torch.cat([fn(t) for t in torch.chunk(x, shards, 0)], 0)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        row = 0
        for xs, gs in zip(torch.chunk(x, ctx.shards, 0), torch.chunk(grad_out, ctx.shards, 0)):
            xs = xs.detach().requires_grad_(True)
            with torch.enable_grad():
                out = ctx.fn(xs)
            torch.autograd.backward(out, gs)              # parameter gradients accumulate as a side effect
            dx[row:row + xs.shape[0]] = xs.grad
            row += xs.shape[0]
        return (dx, None, None) + (None,) * (len(ctx.needs_input_grad) - 3)


def resolve_shards(shards: Union[int, str, None], tokens: int, hidden: int) -> int:
    if shards in (None, 0, 1, False):
        return 1
    if shards == "auto" or shards is True:
        return max(1, math.ceil(tokens / max(1, hidden)))
    if isinstance(shards, str) and shards.startswith("chunk:"):        # tiles of a fixed number of tokens
        return max(1, math.ceil(tokens / max(1, int(shards[6:]))))
    return max(1, min(int(shards), tokens))


def tiled_mlp(x: torch.Tensor, fn: Callable[[torch.Tensor], torch.Tensor], shards: Union[int, str],
              params: Sequence[torch.Tensor]) -> torch.Tensor:
    """``fn(x)`` computed over ``shards`` row tiles of ``x [tokens, hidden]``.  ``params`` are the parameters ``fn``
    uses (listed so that autograd sees the dependency)."""
    n = resolve_shards(shards, x.shape[0], x.shape[-1])
    if n <= 1 or not torch.is_grad_enabled():
        return fn(x)
    return _TiledMLPFn.apply(x, fn, n, *params)
