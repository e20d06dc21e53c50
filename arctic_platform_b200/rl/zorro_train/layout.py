"""ZoRRo Train batch layout: prompt-deduplicated packing of an RL batch.

An RL batch arrives padded, ``input_ids [B, S]`` with a left-padded prompt in
``[:, :S-R]`` and a right-padded response in ``[:, S-R:]`` (verl convention, as in the
reference's ``create_dummy_batch``, arctic_platform/rl/zorro_train/tests.py:46).
Rollouts of the same prompt repeat the prompt tokens ``rollout_n`` times; ZoRRo keeps
each distinct prompt once.  The packed token axis is::

    [P_g0, R_g0_0, R_g0_1, ..., P_g1, R_g1_0, ...]

(the layout of arctic_platform/rl/zorro_train/zorro_train.py:564-610).  Everything the
model needs is produced here as flat index tables in ONE pass on the host:

* ``input_ids`` / ``positions`` of the packed axis,
* attention segments (prompt: causal over itself; response: sees its group's prompt
  fully and itself causally) for :class:`~arctic_platform_b200.ops.attention.AttnLayout`,
* ``pred_index`` -- for every valid response token, the packed row whose hidden state
  predicts it (the last prompt row for the first response token, else the previous
  response row: the reference's ``offset=-1`` extraction,
  arctic_platform/rl/zorro_train/qwen_model_patcher.py:584-609), and ``labels``,
* ``out_index`` -- where each of those tokens sits in the padded ``[B, R]`` response
  grid, in ORIGINAL sample order, so per-token outputs scatter straight back.

No tensor surgery happens inside the model and nothing here calls ``.item()`` per
segment.  ``dedup=False`` gives the ordinary one-segment-per-sample packing used as
the equivalence oracle.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional

import numpy as np
import torch

from ...ops import _lib
from ...ops.attention import AttnLayout


@dataclass
class PackedBatch:
    input_ids: torch.Tensor      # [T] int64
    positions: torch.Tensor      # [T] int32
    layout: AttnLayout
    pred_index: torch.Tensor     # [N] int64, rows of the packed hidden states
    labels: torch.Tensor         # [N] int64
    out_index: torch.Tensor      # [N] int64, flat index into a [B, R] response grid
    batch_size: int
    response_length: int
    num_groups: int
    group_of: np.ndarray         # [B] group id per sample
    total_tokens: int            # T
    full_tokens: int             # tokens a non-deduplicated packing would have
    sample_tokens: np.ndarray    # [B] valid prompt+response tokens per sample
    src_index: Optional[torch.Tensor] = None   # [T] int64: flat index into the [B, S] input grid each packed token came from

    def gather_inputs(self, grid: torch.Tensor) -> torch.Tensor:
        """Per-input-token values ``[B, S, ...]`` -> ``[T, ...]`` in packed order (a de-duplicated prompt takes the
        values of its group's first sample)."""
        if self.src_index is None:
            raise ValueError("this packed batch does not record where its tokens came from")
        flat = grid.reshape((grid.shape[0] * grid.shape[1],) + tuple(grid.shape[2:]))
        return flat[self.src_index.to(grid.device)]

    def to(self, device) -> "PackedBatch":
        from ...utils.transfer_stats import to_device
        self.input_ids = to_device(self.input_ids, device)
        self.positions = to_device(self.positions, device)
        self.pred_index = to_device(self.pred_index, device)
        self.labels = to_device(self.labels, device)
        self.out_index = to_device(self.out_index, device)
        return self

    def scatter_to_grid(self, values: torch.Tensor, fill: float = 0.0) -> torch.Tensor:
        """Per-token values ``[N]`` -> padded ``[B, R]`` response grid."""
        grid = values.new_full((self.batch_size * self.response_length,), fill)
        grid[self.out_index.to(values.device)] = values
        return grid.view(self.batch_size, self.response_length)

    def gather_from_grid(self, grid: torch.Tensor) -> torch.Tensor:
        """Padded ``[B, R]`` grid -> per-token ``[N]`` in the order of ``labels``."""
        return grid.reshape(-1)[self.out_index.to(grid.device)]

    @property
    def redundancy(self) -> float:
        return 1.0 - self.total_tokens / max(1, self.full_tokens)


def find_prompt_groups(input_ids: torch.Tensor, response_length: int) -> np.ndarray:
    """Group id per sample; samples whose padded prompt slices are identical share an id
    (ids numbered by first appearance).  Hash + memcmp in the C++ runtime instead of the
    reference's O(B^2) ``torch.equal`` loop (zorro_train.py:241-285)."""
    ids = input_ids.detach().to("cpu", torch.int64).contiguous()
    B, S = ids.shape
    P = S - response_length
    out = np.empty(B, dtype=np.int32)
    if P <= 0:
        out[:] = np.arange(B)
        return out
    arr = ids.numpy()
    rt = _lib.rt_lib()
    rt.apb_rt_group_prompts(arr.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)), B, P, S,
                            out.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)))
    return out


def build_packed_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor, response_length: int,
                       dedup: bool = True, group_of: Optional[np.ndarray] = None) -> PackedBatch:
    ids = input_ids.detach().to("cpu", torch.int64).numpy()
    mask = attention_mask.detach().to("cpu").numpy().astype(bool)
    B, S = ids.shape
    R = int(response_length)
    P = S - R
    p_mask, r_mask = mask[:, :P], mask[:, P:]
    p_len = p_mask.sum(1).astype(np.int64)
    r_len = r_mask.sum(1).astype(np.int64)
    if group_of is None:
        group_of = find_prompt_groups(input_ids, R) if dedup else np.arange(B, dtype=np.int32)
    group_of = np.asarray(group_of, dtype=np.int32)
    G = int(group_of.max()) + 1 if B else 0
    # representative (first) sample of each group and members in original order
    rep = np.full(G, -1, dtype=np.int64)
    for b in range(B - 1, -1, -1):
        rep[group_of[b]] = b
    order = np.argsort(group_of, kind="stable")          # samples grouped, original order inside a group
    g_plen = p_len[rep]
    # packed offsets
    g_resp_total = np.zeros(G, dtype=np.int64)
    np.add.at(g_resp_total, group_of, r_len)
    g_size = g_plen + g_resp_total
    g_start = np.concatenate([[0], np.cumsum(g_size)[:-1]]) if G else np.zeros(0, dtype=np.int64)
    T = int(g_size.sum())
    resp_start = np.zeros(B, dtype=np.int64)
    cursor = g_start + g_plen
    for b in order:                                       # B iterations of scalar work, no tensor ops
        g = group_of[b]
        resp_start[b] = cursor[g]
        cursor[g] += r_len[b]

    packed_ids = np.empty(T, dtype=np.int64)
    positions = np.empty(T, dtype=np.int32)
    src = np.empty(T, dtype=np.int64)
    segs: List[List[int]] = []
    for g in range(G):
        b0 = rep[g]
        pl = int(g_plen[g])
        s0 = int(g_start[g])
        if pl:
            packed_ids[s0:s0 + pl] = ids[b0, :P][p_mask[b0]]
            src[s0:s0 + pl] = b0 * S + np.nonzero(p_mask[b0])[0]
            positions[s0:s0 + pl] = np.arange(pl, dtype=np.int32)
            segs.append([s0, pl, 0, 0, s0, pl])
    for b in range(B):
        rl = int(r_len[b])
        if rl == 0:
            continue
        g = group_of[b]
        pl = int(g_plen[g])
        s0 = int(resp_start[b])
        packed_ids[s0:s0 + rl] = ids[b, P:][r_mask[b]]
        src[s0:s0 + rl] = b * S + P + np.nonzero(r_mask[b])[0]
        positions[s0:s0 + rl] = np.arange(pl, pl + rl, dtype=np.int32)
        segs.append([s0, rl, int(g_start[g]), pl, s0, rl])

    # predictor rows / labels / output slots in ORIGINAL sample order
    n_total = int(r_len.sum())
    pred = np.empty(n_total, dtype=np.int64)
    labels = np.empty(n_total, dtype=np.int64)
    out_idx = np.empty(n_total, dtype=np.int64)
    k = 0
    cols = np.arange(R, dtype=np.int64)
    for b in range(B):
        rl = int(r_len[b])
        if rl == 0:
            continue
        g = group_of[b]
        s0 = int(resp_start[b])
        last_prompt = int(g_start[g] + g_plen[g] - 1)
        pred[k] = last_prompt if g_plen[g] > 0 else s0    # no prompt: first token has no predictor (never used)
        pred[k + 1:k + rl] = np.arange(s0, s0 + rl - 1)
        labels[k:k + rl] = ids[b, P:][r_mask[b]]
        out_idx[k:k + rl] = b * R + cols[r_mask[b]]
        k += rl

    layout = AttnLayout(np.asarray(segs, dtype=np.int32).reshape(-1, 6), T)
    return PackedBatch(
        input_ids=torch.from_numpy(packed_ids), positions=torch.from_numpy(positions), layout=layout,
        pred_index=torch.from_numpy(pred), labels=torch.from_numpy(labels), out_index=torch.from_numpy(out_idx),
        batch_size=B, response_length=R, num_groups=G, group_of=group_of, total_tokens=T,
        full_tokens=int((p_len + r_len).sum()), sample_tokens=(p_len + r_len), src_index=torch.from_numpy(src))


def build_plain_packed(input_ids: torch.Tensor, attention_mask: torch.Tensor) -> PackedBatch:
    """Packs ``[B, S]`` sequences (any padding side) for next-token prediction over every valid token:
    row ``t`` predicts token ``t+1`` of the same sequence (SFT / scoring of whole sequences)."""
    ids = input_ids.detach().to("cpu", torch.int64).numpy()
    mask = attention_mask.detach().to("cpu").numpy().astype(bool)
    B, S = ids.shape
    lens = mask.sum(1).astype(np.int64)
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]]) if B else np.zeros(0, dtype=np.int64)
    T = int(lens.sum())
    packed = np.empty(T, dtype=np.int64)
    pos = np.empty(T, dtype=np.int32)
    pred, labels, out_idx, segs = [], [], [], []
    cols = np.arange(S, dtype=np.int64)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        s0 = int(starts[b])
        packed[s0:s0 + n] = ids[b][mask[b]]
        pos[s0:s0 + n] = np.arange(n, dtype=np.int32)
        segs.append([s0, n, 0, 0, s0, n])
        if n > 1:
            pred.append(np.arange(s0, s0 + n - 1))
            labels.append(packed[s0 + 1:s0 + n])
            out_idx.append(b * S + cols[mask[b]][1:])
    cat = lambda xs: np.concatenate(xs) if xs else np.zeros(0, dtype=np.int64)
    return PackedBatch(
        input_ids=torch.from_numpy(packed), positions=torch.from_numpy(pos),
        layout=AttnLayout(np.asarray(segs, dtype=np.int32).reshape(-1, 6), T),
        pred_index=torch.from_numpy(cat(pred)), labels=torch.from_numpy(cat(labels)),
        out_index=torch.from_numpy(cat(out_idx)), batch_size=B, response_length=S, num_groups=B,
        group_of=np.arange(B, dtype=np.int32), total_tokens=T, full_tokens=T, sample_tokens=lens)


def build_prepacked(input_ids: torch.Tensor, position_ids: Optional[torch.Tensor] = None,
                    cu_seqlens: Optional[torch.Tensor] = None) -> PackedBatch:
    """A batch the client packed itself: ONE row ``[1, T]`` holding several documents back to back.  Document
    boundaries come from ``cu_seqlens`` or from the places where ``position_ids`` restart at 0; attention stays
    inside a document and the last token of a document predicts nothing (it would predict the next document's
    first token).  Per-token results map back to the ``[1, T]`` grid at the column of the predicted token."""
    ids = input_ids.detach().to("cpu", torch.int64).reshape(-1).numpy()
    T = int(ids.shape[0])
    if cu_seqlens is not None:
        cu = cu_seqlens.detach().to("cpu", torch.int64).reshape(-1).numpy()
    elif position_ids is not None:
        pos_in = position_ids.detach().to("cpu", torch.int64).reshape(-1).numpy()
        starts = np.flatnonzero(pos_in == 0)
        if starts.size == 0 or starts[0] != 0:
            starts = np.concatenate([[0], starts])
        cu = np.concatenate([starts, [T]])
    else:
        cu = np.asarray([0, T], dtype=np.int64)
    if cu[0] != 0 or cu[-1] > T or np.any(np.diff(cu) < 0):
        raise ValueError(f"document boundaries {cu.tolist()} do not partition {T} tokens")
    pos = np.empty(T, dtype=np.int32)
    pred, labels, out_idx, segs = [], [], [], []
    lens = np.diff(cu)
    for s0, n in zip(cu[:-1].tolist(), lens.tolist()):
        if n == 0:
            continue
        pos[s0:s0 + n] = np.arange(n, dtype=np.int32)
        segs.append([s0, n, 0, 0, s0, n])
        if n > 1:
            pred.append(np.arange(s0, s0 + n - 1))
            labels.append(ids[s0 + 1:s0 + n])
            out_idx.append(np.arange(s0 + 1, s0 + n))
    used = int(cu[-1])
    if used < T:                                   # trailing padding: its own never-scored segment
        pos[used:] = np.arange(T - used, dtype=np.int32)
        segs.append([used, T - used, 0, 0, used, T - used])
    cat = lambda xs: np.concatenate(xs).astype(np.int64) if xs else np.zeros(0, dtype=np.int64)
    D = len(lens)
    return PackedBatch(
        input_ids=torch.from_numpy(ids.copy()), positions=torch.from_numpy(pos),
        layout=AttnLayout(np.asarray(segs, dtype=np.int32).reshape(-1, 6), T),
        pred_index=torch.from_numpy(cat(pred)), labels=torch.from_numpy(cat(labels)),
        out_index=torch.from_numpy(cat(out_idx)), batch_size=1, response_length=T, num_groups=max(D, 1),
        group_of=np.zeros(1, dtype=np.int32), total_tokens=T, full_tokens=T, sample_tokens=np.asarray([T], dtype=np.int64))
