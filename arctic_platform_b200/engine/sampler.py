"""Rollout engine: paged KV cache, prefix-sharing prefill, CUDA-graph decode, forest-cascade attention.

The reference delegates generation to vLLM replicas managed by ArcticInference's ``ReplicaPool``
(arctic_platform/common/ray_server.py:197-201,375-404,921-933) and only flips ``use_fca`` for
forest cascade attention (common/utils/server_models.py:123-132).  This module is a from-scratch
engine for the same contract -- ``generate(prompts, sampling_params)`` returning per-sample records
``{token_ids, finish_reason, logprobs, prompt_len}`` -- built on this package's kernels:

* prefill runs the training-side tcgen05 attention over the packed prompts; every DISTINCT prompt
  is prefilled once and its full KV pages are shared (reference counted) by all of its rollouts;
* decode is one CUDA graph per batch-size bucket: embedding, the tcgen05 GEMMs (narrow tiles for
  skinny problems), fused q/k-norm+RoPE, paged split-KV attention, SwiGLU epilogue, lm-head and a
  Gumbel-max sampling kernel; sequence lengths, positions and page tables live in device buffers
  that the graph reads, so the host only looks at finished flags every ``sync_interval`` steps;
* with ``cascade=True`` decode attention is a forest cascade (``ops/forest_attention.py``): prompts that
  start with the same tokens share a HEADER node (found at admission from the token ids, page aligned,
  prefilled and stored once), the rollouts of one prompt share the PROMPT node, and every sequence owns
  its private pages; each node is attended once per step by all sequences below it and the levels are
  merged by log-sum-exp.

Pages for a sequence's maximum length are reserved at admission, which keeps the decode loop free
of host-side allocation.
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.config import DecoderConfig
from ..models.decoder import DecoderLM
from ..ops import _lib, gemm, norm
from ..ops.attention import AttnLayout, attention_fwd_cuda
from ..utils.transfer_stats import to_device, to_host

from ..ops.forest_attention import ForestNode, forest_decode_attention, plan_forest

PAGE = 16
MIN_HEADER_PAGES = 4      # a common prefix shorter than this many pages is not worth a node of its own


_WARNED_KEYS: set = set()


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    max_tokens: int = 16
    top_p: float = 1.0
    top_k: int = -1
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False
    logprobs: Optional[int] = None
    seed: Optional[int] = None

    @staticmethod
    def from_dict(d: Optional[dict], supported: Tuple[str, ...] = ()) -> "SamplingParams":
        """``supported`` names extra keys the calling engine implements itself (they are then not reported)."""
        d = dict(d or {})
        sp = SamplingParams()
        for k in ("n", "temperature", "max_tokens", "top_p", "top_k", "ignore_eos", "logprobs", "seed"):
            if k in d and d[k] is not None:
                setattr(sp, k, d[k])
        if d.get("stop_token_ids"):
            sp.stop_token_ids = tuple(int(x) for x in d["stop_token_ids"])
        # keys of other samplers that would change the distribution if honoured: say so once instead of silently
        # sampling from a different policy than the caller believes
        for k in ("repetition_penalty", "presence_penalty", "frequency_penalty", "min_p", "min_tokens", "logit_bias",
                  "bad_words", "best_of", "use_beam_search"):
            v = d.get(k)
            neutral = {"repetition_penalty": 1.0, "best_of": sp.n}.get(k, 0)
            if k not in supported and v not in (None, False, neutral, [], {}) and k not in _WARNED_KEYS:
                _WARNED_KEYS.add(k)
                import logging
                logging.getLogger(__name__).warning("sampling parameter %s=%r is not supported and is ignored", k, v)
        return sp


class PageAllocator:
    """Reference-counted KV pages (C++ runtime, ``runtime.cpp``)."""

    def __init__(self, num_pages: int):
        self.rt = _lib.rt_lib()
        self.h = self.rt.apb_rt_pages_create(num_pages)
        self.num_pages = num_pages

    def free_count(self) -> int:
        return self.rt.apb_rt_pages_free_count(self.h)

    def alloc(self, n: int) -> Optional[np.ndarray]:
        out = np.empty(max(n, 1), dtype=np.int32)
        if n == 0:
            return out[:0]
        rc = self.rt.apb_rt_pages_alloc(self.h, n, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)))
        return out[:n] if rc == 0 else None

    def retain(self, pages: np.ndarray) -> None:
        if len(pages):
            p = np.ascontiguousarray(pages, dtype=np.int32)
            if self.rt.apb_rt_pages_retain(self.h, len(p), p.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))) != 0:
                raise RuntimeError("retain of a page that is not allocated")

    def release(self, pages: np.ndarray) -> None:
        if len(pages):
            p = np.ascontiguousarray(pages, dtype=np.int32)
            if self.rt.apb_rt_pages_release(self.h, len(p), p.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))) < 0:
                raise RuntimeError("release of a page that is not allocated")

    def __del__(self):
        try:
            self.rt.apb_rt_pages_destroy(self.h)
        except Exception:
            pass


@dataclass
class _Seq:
    req: int                     # index of the prompt in the generate() call
    sample: int                  # rollout index within the prompt
    prompt_len: int
    max_new: int
    shared_pages: np.ndarray     # full prompt pages (beyond the header) shared with the prompt's rollouts
    private_pages: np.ndarray    # prompt tail + response pages owned by this sequence
    group: int
    header_pages: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=np.int32))   # shared with other prompts
    root: int = -1               # id of the header node, -1 = none
    out: List[int] = field(default_factory=list)
    lps: List[float] = field(default_factory=list)
    finish: Optional[str] = None


_FN: Dict[str, object] = {}


def _fn(name: str):
    if not _FN:
        c = ctypes
        vp, i, ll, f, u = c.c_void_p, c.c_int, c.c_longlong, c.c_float, c.c_uint
        _FN["kvw"] = _lib.declare("apb_kv_cache_write", [vp, ll, vp, ll, vp, vp, vp, i, i, i, vp])
        _FN["dec"] = _lib.declare("apb_paged_decode_partial", [vp, vp, vp, vp, i, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp])
        _FN["merge"] = _lib.declare("apb_decode_merge", [vp, vp, vp, i, vp, vp, vp, i, i, i, vp])
        _FN["sample"] = _lib.declare("apb_sample", [vp, ll, vp, i, i, u, vp, vp, vp, vp])
        _FN["sample_f"] = _lib.declare("apb_sample_filtered", [vp, ll, vp, i, i, u, vp, vp, vp, vp, vp, vp, vp])
        _FN["qkv_post"] = _lib.declare("apb_decode_qkv_post", [vp, ll, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, f, vp])
        _FN["swiglu32"] = _lib.declare("apb_swiglu_f32in", [vp, vp, ll, ll, vp])
        _FN["norm32"] = _lib.declare("apb_rmsnorm_fwd_f32in", [vp, vp, vp, vp, vp, i, i, f, f, vp])
        _FN["begin"] = _lib.declare("apb_decode_begin", [vp, vp, vp, vp, i, vp, ll, i, i, vp, vp, i, vp])
        _FN["advance"] = _lib.declare("apb_decode_advance", [vp] * 13 + [i, vp, i, vp])
        _FN["chain"] = _lib.declare("apb_set_chained_launch", [i])
    return _FN[name]


class _TPDecode:
    """Symmetric scratch and epoch state of one tensor-parallel replica's decode loop: two fp32 partial buffers
    (``[max_batch, H]`` per rank: the local GEMM adds its split-K partials there, the row owners pull their rows
    from every rank), two bf16 activation buffers (``[max_batch, H]`` per rank, targets of the owners' normalised
    rows), the flags of the in-kernel barriers and a DEVICE epoch counter -- the kernels read ``*epoch + offset``,
    so a captured step can be replayed."""

    def __init__(self, device, group, max_batch: int, hidden: int):
        import torch.distributed as dist
        from ..parallel.symm import EpochFlags, SymmetricBuffer
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.H = hidden
        self.rows = max_batch // self.world
        self.flags = EpochFlags(device, group)
        self.acc = [SymmetricBuffer(max_batch * hidden, torch.float32, device, group) for _ in range(2)]
        self.hbuf = [SymmetricBuffer(max_batch * hidden, torch.bfloat16, device, group) for _ in range(2)]
        self.resid = torch.zeros((self.rows, hidden), device=device, dtype=torch.bfloat16)
        self.epoch = torch.ones(1, device=device, dtype=torch.int32)      # 0 is what fresh flags hold
        self.done = torch.zeros(1, device=device, dtype=torch.int32)
        self._calls = 0
        # APB_TP_DECODE=nccl: the library shape of the same step (local bf16 GEMM, NCCL all-reduce, residual + norm
        # kernel on every rank) -- the twin the decode benchmark times the fused kernels against
        self.library_twin = os.environ.get("APB_TP_DECODE", "fused") == "nccl"
        self.twin_stream: Optional[torch.Tensor] = None
        c = ctypes
        vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
        self._na = _lib.declare("apb_tp_norm_allgather",
                                [vp, i, i, vp, i, vp, vp, ll, vp, i, vp, f, vp, i, i, vp, vp])
        self._adv = _lib.declare("apb_tp_epoch_advance", [vp, i, vp])

    def begin_step(self) -> None:
        self._calls = 0

    def rs_norm_allgather(self, x: torch.Tensor, w_local: torch.Tensor, norm_w: torch.Tensor, eps: float, B: int,
                          H: int, splits: int) -> torch.Tensor:
        """``RMSNorm(residual += sum over ranks of x @ w_local^T) * norm_w`` for all ``B`` rows, on every rank."""
        k = self._calls
        self._calls += 1
        if self.library_twin:
            import torch.distributed as dist
            y = gemm.matmul_nt(x, w_local)
            dist.all_reduce(y, group=self.group)
            h, self.twin_stream = norm.rmsnorm(y, norm_w, eps, self.twin_stream)
            return h
        acc, other, hb = self.acc[k & 1], self.acc[(k + 1) & 1], self.hbuf[k & 1]
        rl = B // self.world
        s = _lib.stream_ptr()
        # this rank's partial [B, H] stays local (split-K partials meet through local red.add) ...
        gemm.gemm_raw(x, w_local, acc.tensor[:B * H].view(B, H), M=B, N=H, K=x.shape[1], epi=gemm.EPI_F32_ATOMIC,
                      splits=splits, bn=128)
        # ... and the row owners pull, sum, normalise and hand the rows to everybody; the buffer of the previous
        # call is cleared on the way (all of it: a later step may run with more rows than this one)
        _lib.check(self._na(self.flags.ptr_table(), self.rank, self.world, _lib.ptr(self.epoch), 2 * k,
                            acc.ptr_table(), _lib.ptr(other.tensor), other.tensor.numel(), _lib.ptr(self.resid), 1, _lib.ptr(norm_w),
                            float(eps), hb.ptr_table(), rl, H, _lib.ptr(self.done), s), "apb_tp_norm_allgather")
        return hb.tensor[:B * H].view(B, H)

    def end_step(self) -> None:
        if self._calls & 1:
            raise RuntimeError("a decode step must use the accumulator pair an even number of times")
        if self.library_twin:
            return
        _lib.check(self._adv(_lib.ptr(self.epoch), 2 * self._calls, _lib.stream_ptr()), "apb_tp_epoch_advance")


class SamplerEngine:
    def __init__(self, cfg: DecoderConfig, device="cuda", model: Optional[DecoderLM] = None,
                 kv_cache_tokens: int = 1 << 20, max_batch: int = 256, max_seq_len: int = 8192,
                 cascade: bool = True, sync_interval: int = 16, use_cuda_graph: bool = True, seed: int = 0,
                 eos_token_id: Optional[int] = None, prefix_on_tensor_cores: bool = True, split_k: bool = True,
                 quantization: Optional[str] = None, tp_group=None):
        self.device = torch.device(device)
        # tensor-parallel replica: this engine is ONE rank of ``tp`` and holds the heads / columns of its shard
        # (``vllm_config.tensor_parallel_size`` in the reference, arctic_platform/common/ray_server.py:375-404)
        self.tp_group = tp_group
        self.tp = 1
        self.tp_rank = 0
        self.full_cfg = cfg
        if tp_group is not None:
            import torch.distributed as dist
            self.tp = dist.get_world_size(tp_group)
            self.tp_rank = dist.get_rank(tp_group)
        if self.tp > 1:
            from ..parallel.tp_sampler import tp_config
            if cfg.is_moe:
                raise NotImplementedError("tensor-parallel replicas of the paged engine serve dense decoders")
            if max_batch % self.tp:
                raise ValueError(f"max_num_seqs={max_batch} must be a multiple of tensor_parallel_size={self.tp}")
            cfg = tp_config(cfg, self.tp)
            if model is not None and model.cfg.num_heads != cfg.num_heads:
                full, model = model, DecoderLM(cfg, self.device, torch.bfloat16)
                self.cfg, self.model = cfg, model
                from ..models.hf_io import iter_hf_tensors
                self.load_weights(iter_hf_tensors(full), notify=False)
        self.cfg = cfg
        self.model = model if model is not None else DecoderLM(cfg, self.device, torch.bfloat16)
        self.max_batch = max_batch
        self.max_seq_len = max_seq_len
        self._sm_count = (torch.cuda.get_device_properties(self.device).multi_processor_count
                          if self.device.type == "cuda" else 1)
        from ..utils import memory_budget
        memory_budget.register("sampler", self.device)
        self.cascade = cascade
        self.sync_interval = sync_interval
        self.use_cuda_graph = use_cuda_graph
        self.seed = seed
        self.eos = eos_token_id
        self.prefix_on_tensor_cores = prefix_on_tensor_cores
        self.split_k = split_k
        if quantization not in (None, "", "fp8"):
            raise ValueError(f"unsupported sampler quantization {quantization!r} (None or 'fp8')")
        # "fp8": the dense projections are served from block-scaled e4m3 copies (128 x 128 weight blocks, per-token
        # activation scales) that are rebuilt after every weight sync
        self.fp8 = quantization == "fp8" and not cfg.is_moe
        self._fp8_stale = True
        self._fp8_w: List[dict] = []
        self.num_pages = max(64, kv_cache_tokens // PAGE)
        self.max_pages = (max_seq_len + PAGE - 1) // PAGE + 1
        self._alloc_cache()
        self.pages = PageAllocator(self.num_pages)
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._graph_launches: Dict[int, int] = {}
        self._step_count = 0
        self._asleep = False
        self._alloc_state()
        self._tpd = _TPDecode(self.device, tp_group, max_batch, cfg.hidden_size) if self.tp > 1 else None
        self._sync_plan = None           # table of the one-kernel weight hand-over (parallel/weight_sync.py)

    # ------------------------------------------------------------------ memory
    def _alloc_cache(self) -> None:
        c = self.cfg
        shape = (c.num_layers, self.num_pages, c.num_kv_heads, PAGE, c.head_dim)
        # zero-filled: the unwritten tail of a last page is multiplied by probability 0 and must be finite
        self.kcache = torch.zeros(shape, device=self.device, dtype=torch.bfloat16)
        self.vcache = torch.zeros(shape, device=self.device, dtype=torch.bfloat16)
        if self.device.type == "cuda":
            from ..utils import memory_budget
            memory_budget.set_kv_resident(self.device, self.kv_bytes())

    def kv_bytes(self) -> int:
        c = self.cfg
        return 2 * c.num_layers * self.num_pages * c.num_kv_heads * PAGE * c.head_dim * 2

    def _alloc_state(self) -> None:
        B, dev, c = self.max_batch, self.device, self.cfg
        i32 = dict(device=dev, dtype=torch.int32)
        self.d_tokens = torch.zeros(B, **i32)
        self.d_pos = torch.zeros(B, **i32)
        self.d_len = torch.zeros(B, **i32)            # tokens in cache incl. the current one (0 = inactive slot)
        self.d_active = torch.zeros(B, **i32)
        self.d_max_len = torch.zeros(B, **i32)
        self.d_finished = torch.zeros(B, **i32)
        self.d_temp = torch.ones(B, device=dev, dtype=torch.float32)
        self.d_page_table = torch.zeros((B, self.max_pages), **i32)       # all pages of the sequence, in order
        self.d_priv_table = torch.zeros((B, self.max_pages), **i32)       # private pages only
        self.d_priv_len = torch.zeros(B, **i32)
        self.d_shared_tokens = torch.zeros(B, **i32)
        self.d_q_start = torch.arange(B, **i32)
        self.d_q_one = torch.ones(B, **i32)
        # prefix forest (cascade): one table row per run of consecutive slots under a shared node; a sequence sits
        # under at most two shared nodes (header, prompt), so 2 * B rows always suffice
        self.n_node_rows = 2 * B
        self.d_g_start = torch.zeros(self.n_node_rows, **i32)
        self.d_g_count = torch.zeros(self.n_node_rows, **i32)
        self.d_g_pages = torch.zeros((self.n_node_rows, self.max_pages), **i32)
        self.d_g_len = torch.zeros(self.n_node_rows, **i32)
        self.d_g_level = torch.zeros(self.n_node_rows, **i32)
        self.d_row_mask = torch.full((B,), 1, **i32)
        self.n_levels = 1            # shared levels in use: 1 = prompt nodes only, 2 = header + prompt nodes
        self.forest_stats = {"shared_tokens": 0, "covered_tokens": 0}
        self.out_cap = 0
        self.d_out_tokens = None
        self.d_out_lps = None
        self.d_out_idx = torch.zeros((B, 1), device=dev, dtype=torch.int64)   # tokens emitted so far per slot
        self.d_step = torch.zeros(1, **i32)                                   # global decode step (RNG stream)
        self.d_stop = torch.full((8,), -1, **i32)
        self.d_topk = torch.zeros(B, **i32)                       # per-slot top-k (0 = off)
        self.d_topp = torch.ones(B, device=dev, dtype=torch.float32)
        self.d_thr = torch.zeros(B, device=dev, dtype=torch.float32)
        self._filter_on = False
        self.splits = 4
        self.n_groups = B            # rows in use in the node tables (a power-of-two bucket bounds the prefix grid)
        Hq, D = c.num_heads, c.head_dim
        f32 = dict(device=dev, dtype=torch.float32)
        # partial results per source: header level, prompt level, private pass
        self.part_o = [torch.empty((B, Hq, self.splits, D), **f32) for _ in range(3)]
        self.part_ml = [torch.empty((B, Hq, self.splits, 2), **f32) for _ in range(3)]
        self.d_logits = torch.empty((B, c.vocab_size), **f32)
        # fp32 split-K accumulators of the two skinny projections (kept zero between uses by the norm kernel)
        self.acc_o = torch.zeros((B, c.hidden_size), **f32)
        self.acc_d = torch.zeros((B, c.hidden_size), **f32)
        self.acc_qkv = torch.zeros((B, c.qkv_size), **f32)
        self.acc_gu = torch.zeros((B, 2 * c.intermediate_size), **f32) if not c.is_moe else None   # split-K gate/up sums
        self.d_new_tok = torch.zeros(B, **i32)
        self.d_new_lp = torch.zeros(B, **f32)
        self.d_slots = torch.full((B,), -1, **i32)                              # cache slot of the token being fed
        self.d_x = torch.empty((B, c.hidden_size), device=dev, dtype=torch.bfloat16)   # its embedding row

    def kv_bytes(self) -> int:
        return 2 * self.kcache.numel() * 2

    # ------------------------------------------------------------------ layers (no autograd)
    @torch.no_grad()
    def _block(self, li: int, x, stream, positions, slots, attn_fn):
        c = self.cfg
        blk = self.model.blocks[li]
        if self.fp8:
            return self._block_fp8(li, x, stream, positions, slots, attn_fn)
        h, stream = norm.rmsnorm(x, blk.ln1, c.rms_norm_eps, stream)
        qkv = gemm.matmul_nt(h, blk.wqkv)
        q, k, v = norm.qknorm_rope(qkv, blk.q_norm, blk.k_norm, *self.model.rope(self.device), positions, c.num_heads,
                                   c.num_kv_heads, c.head_dim, c.rms_norm_eps)
        _lib.check(_fn("kvw")(_lib.ptr(k), k.stride(0), _lib.ptr(v), v.stride(0), _lib.ptr(slots),
                              _lib.ptr(self.kcache[li]), _lib.ptr(self.vcache[li]), k.shape[0], c.num_kv_heads,
                              c.head_dim, _lib.stream_ptr()), "kv_cache_write")
        a = attn_fn(li, q, k, v)
        o = self._tp_sum(gemm.matmul_nt(a.reshape(a.shape[0], -1), blk.wo))
        h2, stream = norm.rmsnorm(o, blk.ln2, c.rms_norm_eps, stream)
        if blk.mlp is not None:
            d = blk.mlp(h2)
        else:
            _, act = gemm.gate_up_swiglu(h2, blk.wgu, keep_gu=False)
            d = self._tp_sum(gemm.matmul_nt(act, blk.wdown))
        return d, stream

    def _tp_sum(self, t: torch.Tensor) -> torch.Tensor:
        """Prefill under tensor parallelism: the row-parallel projections' partial results are summed over the
        replica with a library all-reduce (prefill runs once per prompt; decode uses the fused kernels)."""
        if self.tp > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.tp_group)
        return t

    @torch.no_grad()
    def weights_updated(self) -> None:
        """Called after a weight sync / load: derived copies (fp8) are rebuilt before the next generation."""
        self._fp8_stale = True

    @torch.no_grad()
    def _requantize_fp8(self) -> None:
        from ..parallel.weight_sync import quantize_fp8_block128
        self._fp8_w = []
        self._graphs.clear()             # captured graphs hold pointers to the previous copies
        self._parked_graphs = None
        for blk in self.model.blocks:
            self._fp8_w.append({n: quantize_fp8_block128(getattr(blk, n).data) for n in ("wqkv", "wo", "wgu", "wdown")})
        self._fp8_stale = False

    @torch.no_grad()
    def _block_fp8(self, li: int, x, stream, positions, slots, attn_fn):
        from ..ops.fp8 import fp8_linear
        c = self.cfg
        blk = self.model.blocks[li]
        w = self._fp8_w[li]
        h, stream = norm.rmsnorm(x, blk.ln1, c.rms_norm_eps, stream)
        qkv = fp8_linear(h, *w["wqkv"])
        q, k, v = norm.qknorm_rope(qkv, blk.q_norm, blk.k_norm, *self.model.rope(self.device), positions, c.num_heads,
                                   c.num_kv_heads, c.head_dim, c.rms_norm_eps)
        _lib.check(_fn("kvw")(_lib.ptr(k), k.stride(0), _lib.ptr(v), v.stride(0), _lib.ptr(slots),
                              _lib.ptr(self.kcache[li]), _lib.ptr(self.vcache[li]), k.shape[0], c.num_kv_heads,
                              c.head_dim, _lib.stream_ptr()), "kv_cache_write")
        a = attn_fn(li, q, k, v)
        o = self._tp_sum(fp8_linear(a.reshape(a.shape[0], -1).contiguous(), *w["wo"]))
        h2, stream = norm.rmsnorm(o, blk.ln2, c.rms_norm_eps, stream)
        act = norm.swiglu(fp8_linear(h2, *w["wgu"]))
        return self._tp_sum(fp8_linear(act, *w["wdown"])), stream

    # ------------------------------------------------------------------ decode step
    @torch.no_grad()
    def _decode_attention(self, li: int, q: torch.Tensor, B: int) -> torch.Tensor:
        c = self.cfg
        scale = 1.0 / math.sqrt(c.head_dim)
        kc, vc = self.kcache[li], self.vcache[li]
        # per-sequence pass: one CTA per (sequence, kv head) already fills the GPU at rollout batch sizes, so the
        # KV range is split only when there are fewer CTAs than two waves of SMs
        seq_splits = max(1, min(self.splits, 296 // max(1, B * c.num_kv_heads)))
        if os.environ.get("APB_DECODE_SEQ_SPLITS"):               # tuning knob for A/B timing
            seq_splits = max(1, min(self.splits, int(os.environ["APB_DECODE_SEQ_SPLITS"])))
        out = torch.empty((B, c.num_heads, c.head_dim), device=self.device, dtype=torch.bfloat16)
        if self._cascade_on():
            # shared pass: as many KV splits as keep all its CTAs (nodes x KV heads x splits) within one wave of SMs
            nodes = self._group_bucket()
            node_splits = max(1, min(self.splits, self._sm_count // max(1, nodes * c.num_kv_heads)))
            return forest_decode_attention(q, kc, vc, self._forest_view(B), self.d_q_start, self.d_active,
                                           self.d_priv_table, self.d_priv_len, self.part_o, self.part_ml, node_splits,
                                           seq_splits, scale, out=out, n_nodes=nodes)
        s = _lib.stream_ptr()
        _lib.check(_fn("dec")(_lib.ptr(q), _lib.ptr(self.d_q_start), _lib.ptr(self.d_active), _lib.ptr(self.d_page_table),
                              self.max_pages, _lib.ptr(self.d_len), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(self.part_o[0]),
                              _lib.ptr(self.part_ml[0]), B, c.num_heads, c.num_kv_heads, c.head_dim, seq_splits, scale, s),
                   "paged_decode")
        o_ptrs = (ctypes.c_void_p * 4)(self.part_o[0].data_ptr(), 0, 0, 0)
        ml_ptrs = (ctypes.c_void_p * 4)(self.part_ml[0].data_ptr(), 0, 0, 0)
        sp = (ctypes.c_int * 4)(seq_splits, 0, 0, 0)
        _lib.check(_fn("merge")(o_ptrs, ml_ptrs, sp, 1, None, _lib.ptr(out), None, B, c.num_heads, c.head_dim, s),
                   "decode_merge")
        return out

    def _cascade_on(self) -> bool:
        """The shared-node pass runs on 128-row tensor-core tiles: head_dim 128 and a query-head group that divides
        128.  Other shapes decode every sequence over its whole page table."""
        c = self.cfg
        R = c.num_heads // c.num_kv_heads
        return bool(self.cascade and self.prefix_on_tensor_cores and c.head_dim == 128 and 128 % R == 0)

    def _max_rows(self) -> int:
        """Sequences per shared-node tile (their query heads of one KV head fill at most 128 rows)."""
        return max(1, 128 // (self.cfg.num_heads // self.cfg.num_kv_heads))

    def _forest_view(self, B: int):
        from ..ops.forest_attention import ForestTables
        return ForestTables(self.d_g_start, self.d_g_count, self.d_g_pages, self.d_g_len, self.d_g_level,
                            self.d_row_mask, int(self.n_groups), int(self.n_levels),
                            self.forest_stats["shared_tokens"], self.forest_stats["covered_tokens"])

    def _group_bucket(self) -> int:
        """Rows of the node tables in use, rounded up to a power of two: the grid of the shared-node pass (and the
        key of the captured graph) changes only when the count crosses a bucket."""
        n = max(1, int(self.n_groups))
        return min(self.n_node_rows, 1 << (n - 1).bit_length())

    @torch.no_grad()
    def _decode_step(self, B: int) -> None:
        """One token for slots [0, B).  Reads and updates device state only, so the whole step can be
        captured in a CUDA graph and replayed."""
        c = self.cfg
        # chained launches: every kernel of the step may start (set-up, weight prefetch) while its predecessor is
        # still running; valid here because no kernel of a decode step writes the weights
        prev_chain = _fn("chain")(1)
        try:
            positions = self.d_pos[:B]
            slots = self.d_slots[:B]
            x = self.d_x[:B]
            # one kernel: cache slot of the fed token (page-table look-up) + its embedding row
            _lib.check(_fn("begin")(_lib.ptr(self.d_tokens), _lib.ptr(self.d_pos), _lib.ptr(self.d_active),
                                    _lib.ptr(self.d_page_table), self.max_pages, _lib.ptr(self.model.embed),
                                    self.model.embed.stride(0), c.hidden_size, c.vocab_size, _lib.ptr(slots), _lib.ptr(x), B,
                                    _lib.stream_ptr()), "decode_begin")
            stream = None
            attn = lambda li, q, k, v: self._decode_attention(li, q, B)
            if self.tp > 1 and not self.fp8:
                h = self._decode_layers_tp(x, positions, slots, B)
            elif self.split_k and not c.is_moe and not self.fp8:
                h = self._decode_layers_splitk(x, positions, slots, B)
            else:
                for li in range(c.num_layers):
                    x, stream = self._block(li, x, stream, positions, slots, attn)
                h, _ = norm.rmsnorm(x, self.model.final_norm, c.rms_norm_eps, stream)
            logits = self.d_logits[:B]
            gemm.matmul_nt(h, self.model.output_weight, out=logits)
            if self._filter_on:
                _lib.check(_fn("sample_f")(_lib.ptr(logits), logits.stride(0), _lib.ptr(self.d_temp), B, c.vocab_size,
                                           ctypes.c_uint(self.seed & 0xFFFFFFFF), _lib.ptr(self.d_step),
                                           _lib.ptr(self.d_topk), _lib.ptr(self.d_topp), _lib.ptr(self.d_thr),
                                           _lib.ptr(self.d_new_tok), _lib.ptr(self.d_new_lp), _lib.stream_ptr()),
                           "sample_filtered")
            else:
                _lib.check(_fn("sample")(_lib.ptr(logits), logits.stride(0), _lib.ptr(self.d_temp), B, c.vocab_size,
                                         ctypes.c_uint(self.seed & 0xFFFFFFFF), _lib.ptr(self.d_step),
                                         _lib.ptr(self.d_new_tok), _lib.ptr(self.d_new_lp), _lib.stream_ptr()), "sample")
            # one kernel: store token + log-prob, stop / length decisions, advance positions and lengths, step counter
            _lib.check(_fn("advance")(_lib.ptr(self.d_new_tok), _lib.ptr(self.d_new_lp), _lib.ptr(self.d_active),
                                      _lib.ptr(self.d_finished), _lib.ptr(self.d_tokens), _lib.ptr(self.d_pos),
                                      _lib.ptr(self.d_len), _lib.ptr(self.d_priv_len), _lib.ptr(self.d_max_len),
                                      _lib.ptr(self.d_stop), _lib.ptr(self.d_out_idx), _lib.ptr(self.d_out_tokens),
                                      _lib.ptr(self.d_out_lps), self.out_cap, _lib.ptr(self.d_step), B,
                                      _lib.stream_ptr()), "decode_advance")
        finally:
            _fn("chain")(prev_chain)

    def _moe_graph_ok(self) -> bool:
        """A mixture-of-experts step can be captured when routing, the expert histogram and the grouped-GEMM tile
        tables are all built on the device (no expert parallelism, no group-limited routing, at most 512 experts)."""
        if os.environ.get("APB_MOE_GRAPH", "1") == "0":
            return False
        c = self.cfg
        if c.num_experts > 512 or getattr(c, "moe_n_group", 1) > 1 or getattr(c, "moe_activation", "swiglu") != "swiglu":
            return False
        return all(getattr(b.mlp, "ep", None) is None for b in self.model.blocks if b.mlp is not None)

    def _norm_f32(self, acc: torch.Tensor, w: torch.Tensor, res: torch.Tensor):
        """RMSNorm whose input is an fp32 split-K accumulator (reset to zero as it is read)."""
        T, H = acc.shape
        y = torch.empty((T, H), device=self.device, dtype=torch.bfloat16)
        stream = torch.empty((T, H), device=self.device, dtype=torch.bfloat16)
        _lib.check(_fn("norm32")(_lib.ptr(acc), _lib.ptr(res), _lib.ptr(w), _lib.ptr(y), _lib.ptr(stream), T, H,
                                 self.cfg.rms_norm_eps, 0.0, _lib.stream_ptr()), "rmsnorm_f32in")
        return y, stream

    def _gate_up_bn(self, B: int) -> int:
        """Tile width of the gate/up projection in decode.  0 lets the kernel pick the width that covers the
        columns in one wave of SMs (144-wide tiles for 19456 columns: 136 tiles, where 128-wide ones would leave
        four SMs with two tiles each and double the kernel's time)."""
        if os.environ.get("APB_GATE_UP_BN"):
            return int(os.environ["APB_GATE_UP_BN"])
        return 0

    def _decode_layers_splitk(self, x: torch.Tensor, positions, slots, B: int) -> torch.Tensor:
        """Decoder stack for one decode step.  The two projections with few output columns (o_proj, down_proj)
        run as split-K GEMMs with fp32 ``red.add`` epilogues so that every SM streams weights; the norm that
        follows reads the fp32 sums directly."""
        c = self.cfg
        H = c.hidden_size
        acc_o, acc_d = self.acc_o[:B], self.acc_d[:B]
        tiles = (H + 127) // 128
        so = max(1, min(148 // tiles, (c.q_size + 63) // 64))
        sd = max(1, min(148 // tiles, (c.intermediate_size + 63) // 64))
        qkv_tiles = (c.qkv_size + 127) // 128
        sq = max(1, min(148 // qkv_tiles, (H + 63) // 64)) if (B <= 128 and c.head_dim in (64, 128, 256)) else 1
        if os.environ.get("APB_DECODE_QKV_SPLITS"):
            sq = int(os.environ["APB_DECODE_QKV_SPLITS"])
        acc_qkv = self.acc_qkv[:B]
        sgu = int(os.environ.get("APB_DECODE_GU_SPLITS", "1"))      # >1: split-K gate/up with a separate SwiGLU pass
        stream = None
        for li in range(c.num_layers):
            blk = self.model.blocks[li]
            if li == 0:
                h, stream = norm.rmsnorm(x, blk.ln1, c.rms_norm_eps, None)
            else:
                h, stream = self._norm_f32(acc_d, blk.ln1, stream)
            if sq > 1:
                # split-K qkv into fp32 sums, then one kernel: q/k norm + RoPE, q to bf16, k and v into the cache
                gemm.gemm_raw(h, blk.wqkv, acc_qkv, M=B, N=c.qkv_size, K=H, epi=gemm.EPI_F32_ATOMIC, splits=sq, bn=128)
                q = torch.empty((B, c.num_heads, c.head_dim), device=self.device, dtype=torch.bfloat16)
                cos_t, sin_t = self.model.rope(self.device)
                _lib.check(_fn("qkv_post")(_lib.ptr(acc_qkv), acc_qkv.stride(0), _lib.ptr(blk.q_norm), _lib.ptr(blk.k_norm),
                                           _lib.ptr(cos_t), _lib.ptr(sin_t), _lib.ptr(positions), _lib.ptr(slots),
                                           _lib.ptr(q), _lib.ptr(self.kcache[li]), _lib.ptr(self.vcache[li]), B,
                                           c.num_heads, c.num_kv_heads, c.head_dim, c.rms_norm_eps, _lib.stream_ptr()),
                           "decode_qkv_post")
            else:
                qkv = gemm.matmul_nt(h, blk.wqkv)
                q, k, v = norm.qknorm_rope(qkv, blk.q_norm, blk.k_norm, *self.model.rope(self.device), positions,
                                           c.num_heads, c.num_kv_heads, c.head_dim, c.rms_norm_eps)
                _lib.check(_fn("kvw")(_lib.ptr(k), k.stride(0), _lib.ptr(v), v.stride(0), _lib.ptr(slots),
                                      _lib.ptr(self.kcache[li]), _lib.ptr(self.vcache[li]), B, c.num_kv_heads,
                                      c.head_dim, _lib.stream_ptr()), "kv_cache_write")
            a = self._decode_attention(li, q, B).reshape(B, -1)
            gemm.gemm_raw(a, blk.wo, acc_o, M=B, N=H, K=c.q_size, epi=gemm.EPI_F32_ATOMIC, splits=so, bn=128)
            h2, stream = self._norm_f32(acc_o, blk.ln2, stream)
            act = torch.empty((B, c.intermediate_size), device=self.device, dtype=torch.bfloat16)
            if sgu > 1:
                # 256-wide tiles halve the activation re-reads; two K splits restore one CTA per SM
                acc_gu = self.acc_gu[:B]
                gemm.gemm_raw(h2, blk.wgu, acc_gu, M=B, N=2 * c.intermediate_size, K=H, epi=gemm.EPI_F32_ATOMIC,
                              splits=sgu, bn=256)
                _lib.check(_fn("swiglu32")(_lib.ptr(acc_gu), _lib.ptr(act), B, c.intermediate_size, _lib.stream_ptr()),
                           "swiglu_f32in")
            else:
                gemm.gemm_raw(h2, blk.wgu, None, M=B, N=2 * c.intermediate_size, K=H, epi=gemm.EPI_SWIGLU, out2=act,
                              bn=self._gate_up_bn(B))
            gemm.gemm_raw(act, blk.wdown, acc_d, M=B, N=H, K=c.intermediate_size, epi=gemm.EPI_F32_ATOMIC, splits=sd,
                          bn=128)
        h, _ = self._norm_f32(acc_d, self.model.final_norm, stream)
        return h

    def _decode_layers_tp(self, x: torch.Tensor, positions, slots, B: int) -> torch.Tensor:
        """Decoder stack of one decode step on one rank of a tensor-parallel replica.  Column-parallel projections
        (qkv, gate/up) read the full activation from LOCAL memory; row-parallel ones (o, down) leave their partial
        result in a local fp32 buffer, and ``apb_tp_norm_allgather`` on the rank that owns a row pulls the row's
        partials from every rank (peer loads), adds the residual, applies RMSNorm and stores the normalised row into
        every rank's activation buffer -- two kernels per projection, no library collective in the loop."""
        c, t = self.cfg, self._tpd
        H, T = c.hidden_size, self.tp
        if B % T:
            raise ValueError(f"decode batch {B} is not a multiple of tensor_parallel_size {T}")
        rl = B // T
        tiles = (H + 127) // 128
        so = max(1, min(148 // tiles, (c.q_size + 63) // 64))
        sd = max(1, min(148 // tiles, (c.intermediate_size + 63) // 64))
        qkv_tiles = (c.qkv_size + 127) // 128
        sq = max(1, min(148 // qkv_tiles, (H + 63) // 64))
        gu_tiles = (2 * c.intermediate_size + 255) // 256
        sgu = max(1, min(148 // gu_tiles, 4))
        acc_qkv = self.acc_qkv[:B]
        acc_gu = self.acc_gu[:B]
        cos_t, sin_t = self.model.rope(self.device)
        t.begin_step()
        # the residual stream is carried for this rank's rows only
        t.resid[:rl].copy_(x[self.tp_rank * rl:(self.tp_rank + 1) * rl])
        t.twin_stream = x
        h, _ = norm.rmsnorm(x, self.model.blocks[0].ln1, c.rms_norm_eps, None)
        for li in range(c.num_layers):
            blk = self.model.blocks[li]
            gemm.gemm_raw(h, blk.wqkv, acc_qkv, M=B, N=c.qkv_size, K=H, epi=gemm.EPI_F32_ATOMIC, splits=sq, bn=128)
            q = torch.empty((B, c.num_heads, c.head_dim), device=self.device, dtype=torch.bfloat16)
            _lib.check(_fn("qkv_post")(_lib.ptr(acc_qkv), acc_qkv.stride(0), _lib.ptr(blk.q_norm), _lib.ptr(blk.k_norm),
                                       _lib.ptr(cos_t), _lib.ptr(sin_t), _lib.ptr(positions), _lib.ptr(slots),
                                       _lib.ptr(q), _lib.ptr(self.kcache[li]), _lib.ptr(self.vcache[li]), B,
                                       c.num_heads, c.num_kv_heads, c.head_dim, c.rms_norm_eps, _lib.stream_ptr()),
                       "decode_qkv_post")
            a = self._decode_attention(li, q, B).reshape(B, -1)
            h2 = t.rs_norm_allgather(a, blk.wo, blk.ln2, c.rms_norm_eps, B, H, so)
            act = torch.empty((B, c.intermediate_size), device=self.device, dtype=torch.bfloat16)
            if sgu > 1:
                gemm.gemm_raw(h2, blk.wgu, acc_gu, M=B, N=2 * c.intermediate_size, K=H, epi=gemm.EPI_F32_ATOMIC,
                              splits=sgu, bn=256)
                _lib.check(_fn("swiglu32")(_lib.ptr(acc_gu), _lib.ptr(act), B, c.intermediate_size, _lib.stream_ptr()),
                           "swiglu_f32in")
            else:
                gemm.gemm_raw(h2, blk.wgu, None, M=B, N=2 * c.intermediate_size, K=H, epi=gemm.EPI_SWIGLU, out2=act,
                              bn=self._gate_up_bn(B))
            nxt = self.model.blocks[li + 1].ln1 if li + 1 < c.num_layers else self.model.final_norm
            h = t.rs_norm_allgather(act, blk.wdown, nxt, c.rms_norm_eps, B, H, sd)
        t.end_step()
        return h

    def _run_steps(self, B: int, n: int) -> None:
        if not self.use_cuda_graph or (self.cfg.is_moe and not self._moe_graph_ok()):
            for _ in range(n):
                self._decode_step(B)
            return
        key = (B, self._group_bucket() if self._cascade_on() else 0, self.n_levels, self._filter_on)
        g = self._graphs.get(key)
        if g is None:
            # the first steps run eagerly (kernel attribute set-up, device binding, allocator warm-up)
            self._decode_step(B)
            n -= 1
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            before = _lib.launch_count()
            with torch.cuda.graph(g):
                self._decode_step(B)
            self._graph_launches[key] = _lib.launch_count() - before
            _lib.add_launches(-self._graph_launches[key])     # capture records, it does not launch
            self._graphs[key] = g
        for _ in range(n):
            g.replay()
        _lib.add_launches(n * self._graph_launches[key])

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sampling_params=None) -> List[dict]:
        """Generates ``n`` samples per prompt.  Returns one record per sample, prompt-major:
        ``{"token_ids", "logprobs", "finish_reason", "prompt_len", "prompt_index", "text"}``."""
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        if self._asleep:
            raise RuntimeError("sampler is asleep; call wake() first")
        if self.fp8 and self._fp8_stale:
            self._requantize_fp8()
        self._filter_on = bool((sp.top_k is not None and sp.top_k > 0) or sp.top_p < 1.0)
        self.d_topk.fill_(int(sp.top_k) if sp.top_k and sp.top_k > 0 else 0)
        self.d_topp.fill_(float(sp.top_p))
        prompts_np = [np.asarray(p, dtype=np.int64) for p in prompts]
        for p in prompts_np:
            if len(p) == 0:
                raise ValueError("empty prompt")
            if len(p) + sp.max_tokens > self.max_seq_len:
                raise ValueError(f"prompt ({len(p)}) + max_tokens ({sp.max_tokens}) exceeds max_seq_len {self.max_seq_len}")
        stops = list(sp.stop_token_ids)
        if self.eos is not None and not sp.ignore_eos:
            stops.append(self.eos)
        stops = stops[:8]
        self.d_stop.fill_(-1)
        if stops:
            self.d_stop[:len(stops)] = torch.tensor(stops, dtype=torch.int32, device=self.device)
        if self.out_cap < sp.max_tokens:
            self.out_cap = sp.max_tokens
            self.d_out_tokens = torch.zeros((self.max_batch, self.out_cap), device=self.device, dtype=torch.int32)
            self.d_out_lps = torch.zeros((self.max_batch, self.out_cap), device=self.device, dtype=torch.float32)
            self._graphs.clear()
            self._parked_graphs = None
        if sp.seed is not None:
            self.seed = int(sp.seed)
            self.d_step.zero_()            # a seeded call restarts the random stream
        results: List[Optional[dict]] = [None] * (len(prompts_np) * sp.n)
        # work queue: runs of prompts that start with the same (page-aligned) header; a run is admitted as a whole --
        # its header is prefilled and stored once, every prompt's n rollouts form one prompt node below it
        queue: List[Tuple[List[int], int]] = self._plan_runs(prompts_np) if self._cascade_on() else \
            [([r], 0) for r in range(len(prompts_np))]
        slots_free = list(range(self.max_batch))
        live: Dict[int, _Seq] = {}
        group_members: Dict[int, List[int]] = {}
        root_members: Dict[int, List[int]] = {}
        next_group = next_root = 0
        while queue or live:
            # ---- admission: as many whole runs as fit in slots and pages
            admitted: List[dict] = []
            while queue:
                idxs, hlen = queue[0]
                if len(idxs) > 1 and len(idxs) * sp.n > self.max_batch:
                    # more sequences than the engine has slots: the run is cut in two (each half keeps the header)
                    queue[0:1] = [(idxs[:len(idxs) // 2], hlen), (idxs[len(idxs) // 2:], hlen)]
                    continue
                if len(idxs) * sp.n > len(slots_free):
                    break
                n_hdr = hlen // PAGE
                per_prompt = []
                need = n_hdr
                for r in idxs:
                    P = len(prompts_np[r])
                    n_full = (P - hlen) // PAGE
                    priv_pages = (P % PAGE + sp.max_tokens + PAGE - 1) // PAGE
                    per_prompt.append((r, P, n_full, priv_pages))
                    need += n_full + sp.n * priv_pages
                if self.pages.free_count() < need:
                    if not live and not admitted and len(idxs) > 1:
                        queue[0:1] = [(idxs[:len(idxs) // 2], hlen), (idxs[len(idxs) // 2:], hlen)]
                        continue
                    break
                queue.pop(0)
                header = self.pages.alloc(n_hdr)
                rid = -1
                if n_hdr:
                    rid = next_root
                    next_root += 1
                    root_members[rid] = []
                run = {"root": rid, "header_len": hlen, "header_pages": header, "prompts": []}
                slots_free.sort()
                first_of_run = True
                for r, P, n_full, priv_pages in per_prompt:
                    shared = self.pages.alloc(n_full)
                    gid = next_group
                    next_group += 1
                    mem = []
                    for si in range(sp.n):
                        slot = slots_free.pop(0)
                        priv = self.pages.alloc(priv_pages)
                        if si > 0:
                            self.pages.retain(shared)
                        if not first_of_run:
                            self.pages.retain(header)          # every sequence below the header holds a reference
                        first_of_run = False
                        live[slot] = _Seq(req=r, sample=si, prompt_len=P, max_new=sp.max_tokens, shared_pages=shared,
                                          private_pages=priv, group=gid, header_pages=header, root=rid)
                        mem.append(slot)
                        if rid >= 0:
                            root_members[rid].append(slot)
                    group_members[gid] = mem
                    run["prompts"].append((gid, mem))
                admitted.append(run)
            if not admitted and not live:
                raise RuntimeError("KV cache too small for a single prompt group; raise kv_cache_tokens")
            if admitted:
                self._admit(admitted, prompts_np, live, sp)
            # ---- decode until the next look at the finished flags
            B = max(live) + 1 if live else 0
            bucket = next((b for b in (8, 16, 32, 64, 128, 256, 512, 1024) if b >= B), self.max_batch)
            bucket = min(bucket, self.max_batch)
            if B > 0:
                self._set_groups(group_members, root_members, live)
                self._run_steps(bucket, self.sync_interval)
            # ---- harvest
            fin = to_host(self.d_finished[:max(B, 1)]).numpy() if B else np.zeros(0, dtype=np.int32)
            done_slots = [s for s in list(live) if fin[s]]
            if done_slots:
                nout = to_host(self.d_out_idx[:B, 0]).numpy()
                toks = to_host(self.d_out_tokens[:B]).numpy()
                lps = to_host(self.d_out_lps[:B]).numpy()
                for s in done_slots:
                    sq = live.pop(s)
                    k = int(nout[s])
                    out = toks[s, :k].tolist()
                    reason = "stop" if (out and out[-1] in stops) else "length"
                    results[sq.req * sp.n + sq.sample] = {
                        "token_ids": out, "logprobs": lps[s, :k].tolist(), "finish_reason": reason,
                        "prompt_len": sq.prompt_len, "prompt_index": sq.req, "text": None}
                    self.pages.release(sq.private_pages)
                    self.pages.release(sq.shared_pages)
                    self.pages.release(sq.header_pages)
                    group_members[sq.group].remove(s)
                    if not group_members[sq.group]:
                        del group_members[sq.group]
                    if sq.root >= 0:
                        root_members[sq.root].remove(s)
                        if not root_members[sq.root]:
                            del root_members[sq.root]
                    slots_free.append(s)
                    self.d_finished[s] = 0
                    self.d_len[s] = 0
                    self.d_priv_len[s] = 0
        return results  # type: ignore[return-value]

    # ------------------------------------------------------------------ admission
    def _plan_runs(self, prompts_np: List[np.ndarray]) -> List[Tuple[List[int], int]]:
        """Prefix-tree discovery from the token ids: prompts are sorted so that common prefixes become neighbours, and
        neighbours whose common prefix covers at least ``MIN_HEADER_PAGES`` pages form a run ``(prompt indices,
        header length)``.  The header length is a multiple of the page size and leaves every prompt of the run at
        least one token of its own (the position its first sampled token is predicted from).  Prompts without such
        a neighbour are runs of one with header length 0.  Runs come back in order of their first prompt."""
        n = len(prompts_np)
        order = sorted(range(n), key=lambda i: prompts_np[i].tobytes())

        def lcp(a: np.ndarray, b: np.ndarray) -> int:
            m = min(len(a), len(b))
            neq = np.flatnonzero(a[:m] != b[:m])
            return int(neq[0]) if len(neq) else m

        def header_of(common: int, shortest: int) -> int:
            return (min(common, shortest - 1) // PAGE) * PAGE

        runs: List[Tuple[List[int], int]] = []
        cur, common, shortest = [order[0]] if n else [], 1 << 60, len(prompts_np[order[0]]) if n else 0
        for k in range(1, n):
            i, prev = order[k], order[k - 1]
            c2 = min(common, lcp(prompts_np[prev], prompts_np[i]))
            s2 = min(shortest, len(prompts_np[i]))
            if header_of(c2, s2) >= MIN_HEADER_PAGES * PAGE:
                cur.append(i)
                common, shortest = c2, s2
            else:
                runs.append((cur, header_of(common, shortest) if len(cur) > 1 else 0))
                cur, common, shortest = [i], 1 << 60, len(prompts_np[i])
        if cur:
            runs.append((cur, header_of(common, shortest) if len(cur) > 1 else 0))
        runs = [(sorted(idxs), h) for idxs, h in runs]
        runs.sort(key=lambda r: r[0][0])
        return runs

    @torch.no_grad()
    def _prefill_runs(self, runs: List[dict], prompts_np, live: Dict[int, _Seq]) -> torch.Tensor:
        """Packs the admitted runs -- every header once, then every prompt's remainder with the header as its fully
        visible prefix -- runs the model over them, fills the KV pages and returns the final-norm hidden state of
        every prompt's last token, in the order of ``runs[*]["prompts"]``."""
        toks, pos, slots, segs, last = [], [], [], [], []
        t = 0

        def put(tokens: np.ndarray, p0: int, pages: np.ndarray):
            nonlocal t
            n = len(tokens)
            toks.append(tokens)
            ar = np.arange(n)
            pos.append((p0 + ar).astype(np.int32))
            slots.append((pages[ar // PAGE] * PAGE + ar % PAGE).astype(np.int32))
            t += n

        for run in runs:
            hlen, hstart = run["header_len"], t
            first = live[run["prompts"][0][1][0]]
            if hlen:
                put(prompts_np[first.req][:hlen], 0, run["header_pages"].astype(np.int64))
                segs.append((hstart, hlen, 0, 0, hstart, hlen))
            for _gid, mem in run["prompts"]:
                s0 = live[mem[0]]
                rem = prompts_np[s0.req][hlen:]
                tail = s0.prompt_len % PAGE
                pages = s0.shared_pages if tail == 0 else np.concatenate([s0.shared_pages, s0.private_pages[:1]])
                q0 = t
                put(rem, hlen, pages.astype(np.int64))
                segs.append((q0, len(rem), hstart if hlen else 0, hlen, q0, len(rem)))
                last.append(t - 1)
        ids = to_device(torch.from_numpy(np.concatenate(toks).astype(np.int64)), self.device)
        positions = to_device(torch.from_numpy(np.concatenate(pos)), self.device)
        slot_t = to_device(torch.from_numpy(np.concatenate(slots)), self.device)
        layout = AttnLayout(np.asarray(segs, dtype=np.int32), t)
        scale = 1.0 / math.sqrt(self.cfg.head_dim)

        def attn(li, q, k, v):
            o, _ = attention_fwd_cuda(q, k, v.contiguous() if v.stride(1) != v.shape[2] else v, layout, scale,
                                      need_lse=False)
            return o

        x = torch.nn.functional.embedding(ids, self.model.embed)
        stream = None
        for li in range(self.cfg.num_layers):
            x, stream = self._block(li, x, stream, positions, slot_t, attn)
        last_t = to_device(torch.from_numpy(np.asarray(last, dtype=np.int64)), self.device)
        h, _ = norm.rmsnorm(x.index_select(0, last_t), self.model.final_norm, self.cfg.rms_norm_eps,
                            stream.index_select(0, last_t))
        return h

    @torch.no_grad()
    def _admit(self, admitted: List[dict], prompts_np, live: Dict[int, _Seq], sp: SamplingParams,
               token_budget: int = 32768) -> None:
        """Prefills each admitted header and prompt ONCE, copies a prompt's partial tail page to every rollout's
        private page, samples the first token of every rollout and initialises the slot state."""
        c = self.cfg
        # batches of whole runs under the token budget (a prompt attends to its header inside one packed batch)
        batches: List[List[dict]] = [[]]
        tok = 0
        for run in admitted:
            n_tok = run["header_len"] + sum(live[mem[0]].prompt_len - run["header_len"] for _g, mem in run["prompts"])
            if batches[-1] and tok + n_tok > token_budget:
                batches.append([])
                tok = 0
            batches[-1].append(run)
            tok += n_tok
        for runs in batches:
            batch = [pm for run in runs for pm in run["prompts"]]
            h = self._prefill_runs(runs, prompts_np, live)
            # tail page copies for rollouts 1..n-1
            src, dst = [], []
            for gid, mem in batch:
                s0 = live[mem[0]]
                if s0.prompt_len % PAGE:
                    for slot in mem[1:]:
                        src.append(int(s0.private_pages[0]))
                        dst.append(int(live[slot].private_pages[0]))
            if src:
                si = torch.tensor(src, device=self.device)
                di = torch.tensor(dst, device=self.device)
                self.kcache[:, di] = self.kcache[:, si]
                self.vcache[:, di] = self.vcache[:, si]
            # first token of every rollout
            rows = [gi for gi, (_, mem) in enumerate(batch) for _ in mem]
            slots = [slot for _, mem in batch for slot in mem]
            hrep = h.index_select(0, torch.tensor(rows, device=self.device))
            logits = gemm.matmul_nt(hrep.contiguous(), self.model.output_weight, out_dtype=torch.float32)
            n = len(slots)
            temp = torch.full((n,), float(sp.temperature), device=self.device, dtype=torch.float32)
            tok0 = torch.empty(n, device=self.device, dtype=torch.int32)
            lp0 = torch.empty(n, device=self.device, dtype=torch.float32)
            seed0 = ctypes.c_uint((self.seed * 2654435761 + 12345) & 0xFFFFFFFF)
            if self._filter_on:       # the first token obeys the same top-k / top-p cut-off as the decode steps
                topk0 = torch.full((n,), int(sp.top_k) if sp.top_k and sp.top_k > 0 else 0, device=self.device, dtype=torch.int32)
                topp0 = torch.full((n,), float(sp.top_p), device=self.device, dtype=torch.float32)
                thr0 = torch.empty(n, device=self.device, dtype=torch.float32)
                _lib.check(_fn("sample_f")(_lib.ptr(logits), logits.stride(0), _lib.ptr(temp), n, c.vocab_size, seed0,
                                           _lib.ptr(self.d_step), _lib.ptr(topk0), _lib.ptr(topp0), _lib.ptr(thr0),
                                           _lib.ptr(tok0), _lib.ptr(lp0), _lib.stream_ptr()), "sample_filtered")
            else:
                _lib.check(_fn("sample")(_lib.ptr(logits), logits.stride(0), _lib.ptr(temp), n, c.vocab_size, seed0,
                                         _lib.ptr(self.d_step), _lib.ptr(tok0), _lib.ptr(lp0), _lib.stream_ptr()), "sample")
            self.d_step += 1
            st = torch.tensor(slots, device=self.device, dtype=torch.long)
            P_t = torch.tensor([live[s].prompt_len for s in slots], device=self.device, dtype=torch.int32)
            stop_hit = (tok0[:, None] == self.d_stop[None, :]).any(1)
            fin = stop_hit | (sp.max_tokens <= 1)
            self.d_tokens[st] = tok0
            self.d_pos[st] = P_t
            self.d_len[st] = P_t + 1
            self.d_max_len[st] = P_t + int(sp.max_tokens)
            self.d_active[st] = (~fin).int()
            self.d_finished[st] = fin.int()
            self.d_temp[st] = temp
            self.d_out_tokens[st, 0] = tok0
            self.d_out_lps[st, 0] = lp0
            self.d_out_idx[st, 0] = 1
            pt = np.zeros((n, self.max_pages), dtype=np.int32)
            pv = np.zeros((n, self.max_pages), dtype=np.int32)
            plen = np.zeros(n, dtype=np.int32)
            sh = np.zeros(n, dtype=np.int32)
            for i, s in enumerate(slots):
                sq = live[s]
                allp = np.concatenate([sq.header_pages, sq.shared_pages, sq.private_pages])
                pt[i, :len(allp)] = allp
                pv[i, :len(sq.private_pages)] = sq.private_pages
                sh[i] = (len(sq.header_pages) + len(sq.shared_pages)) * PAGE
                plen[i] = sq.prompt_len - sh[i] + 1
            from ..utils import checked
            if checked.enabled():                   # host arrays: no synchronisation involved
                checked.check_page_table("page_table", pt, plen + sh - 1, self.num_pages, PAGE)
                checked.check_page_table("priv_table", pv, plen - 1, self.num_pages, PAGE)
            self.d_page_table[st] = to_device(torch.from_numpy(pt), self.device)
            self.d_priv_table[st] = to_device(torch.from_numpy(pv), self.device)
            self.d_priv_len[st] = to_device(torch.from_numpy(plen), self.device)
            self.d_shared_tokens[st] = to_device(torch.from_numpy(sh), self.device)

    def _set_groups(self, group_members: Dict[int, List[int]], root_members: Dict[int, List[int]],
                    live: Dict[int, _Seq]) -> None:
        """Node tables of the prefix forest for cascade decode: header nodes (level 0, when any is live) over all
        sequences of their prompts, prompt nodes over the prompt's rollouts; runs of consecutive slots (one
        tensor-core tile each) become table rows."""
        if not self._cascade_on():
            return
        nodes: List[ForestNode] = []
        two = bool(root_members)
        for rid, mem in root_members.items():
            sq = live[mem[0]]
            nodes.append(ForestNode(0, mem, sq.header_pages, len(sq.header_pages) * PAGE))
        for gid, mem in group_members.items():
            sq = live[mem[0]]
            nodes.append(ForestNode(1 if two else 0, mem, sq.shared_pages, len(sq.shared_pages) * PAGE))
        qs, qc, pg, ln, lv, mask, G, nl, shared, covered = plan_forest(
            nodes, self.max_batch, self.max_pages, self._max_rows(), n_levels=2 if two else 1)
        if G > self.n_node_rows:
            raise RuntimeError(f"prefix forest needs {G} table rows, the engine holds {self.n_node_rows}")
        self.n_groups, self.n_levels = G, nl
        self.forest_stats = {"shared_tokens": shared, "covered_tokens": covered}

        def fill(dst: torch.Tensor, arr: np.ndarray):
            buf = np.zeros(tuple(dst.shape), dtype=arr.dtype)
            buf[:len(arr)] = arr[:len(buf)]
            dst.copy_(to_device(torch.from_numpy(buf), self.device))

        for dst, arr in ((self.d_g_start, qs), (self.d_g_count, qc), (self.d_g_len, ln), (self.d_g_level, lv),
                         (self.d_g_pages, pg)):
            fill(dst, arr)
        self.d_row_mask.copy_(to_device(torch.from_numpy(mask), self.device))

    # ------------------------------------------------------------------ weights / sleep / wake
    @torch.no_grad()
    def load_weights(self, named_tensors, notify: bool = True) -> int:
        """Copies ``(hf_name, tensor)`` pairs (FULL tensors) into the engine's fused parameters -- a tensor-parallel
        rank keeps its slice of each; returns the count."""
        from ..models.hf_io import load_hf_tensor
        n = 0
        if self.tp > 1:
            from ..parallel.tp_sampler import tp_slice
        for name, t in named_tensors:
            if self.tp > 1:
                t = tp_slice(name, t, self.full_cfg, self.tp_rank, self.tp)
            load_hf_tensor(self.model, name, t)
            n += 1
        if notify:
            self.weights_updated()
        return n

    def weight_norm(self) -> Dict[str, float]:
        """Norm and size of the WHOLE model (a tensor-parallel rank adds the other ranks' slices; replicated tensors
        count once)."""
        sq_s = torch.zeros((), dtype=torch.float64, device=self.device)
        sq_r = torch.zeros((), dtype=torch.float64, device=self.device)
        n_s = n_r = 0
        for name, p in self.model.named_parameters():
            sharded = self.tp > 1 and name.split(".")[-1] in ("wqkv", "wgate", "wo", "wgu", "wdown")
            v = p.data.double().pow(2).sum()
            if sharded:
                sq_s, n_s = sq_s + v, n_s + p.numel()
            else:
                sq_r, n_r = sq_r + v, n_r + p.numel()
        if self.tp > 1:
            import torch.distributed as dist
            t = torch.stack([sq_s, torch.tensor(float(n_s), dtype=torch.float64, device=self.device)])
            dist.all_reduce(t, group=self.tp_group)
            sq_s, n_s = t[0], int(t[1].item())
        sq = sq_s + sq_r
        return {"norm": float(sq.sqrt().item()), "sq_sum": float(sq.item()), "num_params": n_s + n_r}

    def reset_prefix_cache(self) -> None:
        """Pages are released at the end of every ``generate`` call, so nothing outlives a weight sync."""
        return None

    def sleep(self, level: int = 1) -> None:
        """Level 1 frees the KV cache and the captured graphs -- unless the trainer that shares the GPU has shown
        that it runs with room to spare for the cache (``utils/memory_budget.py``): then cache and graphs stay and the
        next wake costs nothing.  Level 2 always frees them and also drops the weights (they come back with the next
        weight sync)."""
        keep = False
        if level < 2 and self.kcache is not None and self.device.type == "cuda":
            from ..utils import memory_budget
            keep = memory_budget.kv_may_stay(self.device, self.kv_bytes())
        if keep:
            self._asleep = True
            return
        # the captured decode graphs hold the cache's addresses: they are parked, and come back if the next cache
        # lands on the same addresses (the usual case when the blocks only went back to the shared allocator)
        if level < 2 and self.kcache is not None and self._graphs:
            self._parked_graphs = (self.kcache.data_ptr(), self.vcache.data_ptr(), self._graphs)
        else:
            self._parked_graphs = None
        self._graphs = {}
        self.kcache = self.vcache = None
        if self.device.type == "cuda":
            from ..utils import memory_budget
            memory_budget.set_kv_resident(self.device, 0)
        if level >= 2:
            for p in self.model.parameters():
                p.data = torch.empty(0, device=self.device, dtype=p.dtype)
            self._sync_plan = None            # its destination buffer went with the weights
        self._asleep = True
        from ..utils import memory_budget
        if level >= 2 or not memory_budget.shares_allocator(self.device):
            torch.cuda.empty_cache()      # engines in other processes can only get the memory through the driver

    def wake(self, tags: Optional[Sequence[str]] = None) -> None:
        tags = set(tags or ("weights", "kv_cache"))
        if "kv_cache" in tags:
            if self.kcache is None:
                self._alloc_cache()
                parked = getattr(self, "_parked_graphs", None)
                if parked is not None and parked[0] == self.kcache.data_ptr() and parked[1] == self.vcache.data_ptr():
                    self._graphs = parked[2]
                self._parked_graphs = None
            self._asleep = False
