"""Forest-cascade decode attention over a three-level KV tree, against the per-sequence paged kernel.

Default shape (a Qwen3-8B layer: 32 query / 8 KV heads, head_dim 128, bf16 KV ~ N(0,1), 16-token pages):
16 root prompts of 16384 tokens, each with 4 branches of 2048 tokens, each branch with 8 leaves of 512 tokens
= 512 decode sequences with one query token each.  The cascade reads every node once per step (roots and
branches on tensor-core tiles shared by the sequences below them, leaves per sequence) and merges the three
levels by log-sum-exp; the baseline reads every sequence's 18944-token context by itself.

    python benchmarks/bench_forest_decode.py [--roots 16 --root-len 16384 --branches 4 --branch-len 2048
                                              --leaves 8 --leaf-len 512] [--iters 20] [--no-baseline] [--check]

CUDA events after 3 warm-up launches; the KV cache (2.7 GB at the default shape) is far larger than L2, so every
launch streams it from HBM.  ``--hbm-gbs`` is the measured copy bandwidth of the machine (denominator of the
reported fraction).  ``--check`` compares both kernels with a dense fp32 oracle on a reduced tree first.
Prints one JSON line.
"""
import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.ops import _lib  # noqa: E402
from arctic_platform_b200.ops import forest_attention as fa  # noqa: E402

PAGE = fa.PAGE


def build_tree(roots, root_len, branches, branch_len, leaves, leaf_len, Hq, Hkv, D, device, seed=0):
    """KV cache with random contents plus the tables of both kernels.  Slots are numbered depth first, so the
    sequences below every node are consecutive."""
    assert root_len % PAGE == 0 and branch_len % PAGE == 0, "shared nodes hold whole pages"
    B = roots * branches * leaves
    n_root_p, n_br_p, n_leaf_p = root_len // PAGE, branch_len // PAGE, (leaf_len + PAGE - 1) // PAGE
    num_pages = roots * n_root_p + roots * branches * n_br_p + B * n_leaf_p
    g = torch.Generator(device=device).manual_seed(seed)
    kc = torch.randn((num_pages, Hkv, PAGE, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    vc = torch.randn((num_pages, Hkv, PAGE, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    q = torch.randn((B, Hq, D), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    nxt = 0

    def take(n):
        nonlocal nxt
        out = np.arange(nxt, nxt + n, dtype=np.int32)
        nxt += n
        return out

    nodes, contexts = [], [[] for _ in range(B)]
    max_pages = n_root_p + n_br_p + n_leaf_p
    full = np.zeros((B, max_pages), dtype=np.int32)
    priv = np.zeros((B, max_pages), dtype=np.int32)
    for r in range(roots):
        rp = take(n_root_p)
        r_slots = list(range(r * branches * leaves, (r + 1) * branches * leaves))
        nodes.append(fa.ForestNode(0, r_slots, rp, root_len))
        for b in range(branches):
            bp = take(n_br_p)
            b_slots = list(range((r * branches + b) * leaves, (r * branches + b + 1) * leaves))
            nodes.append(fa.ForestNode(1, b_slots, bp, branch_len))
            for s in b_slots:
                lp = take(n_leaf_p)
                allp = np.concatenate([rp, bp, lp])
                full[s, :len(allp)] = allp
                priv[s, :len(lp)] = lp
                contexts[s] = [(rp, root_len), (bp, branch_len), (lp, leaf_len)]
    Rg = Hq // Hkv
    forest = fa.build_forest_tables(nodes, B, max_pages, max(1, 128 // Rg), device)
    i32 = dict(device=device, dtype=torch.int32)
    tabs = {
        "q": q, "kc": kc, "vc": vc, "forest": forest, "contexts": contexts, "B": B, "max_pages": max_pages,
        "slot_ids": torch.arange(B, **i32), "ones": torch.ones(B, **i32),
        "priv_table": torch.from_numpy(priv).to(device), "priv_len": torch.full((B,), leaf_len, **i32),
        "full_table": torch.from_numpy(full).to(device),
        "full_len": torch.full((B,), root_len + branch_len + leaf_len, **i32),
    }
    return tabs


def run_cascade(t, splits, part_o, part_ml, out):
    return fa.forest_decode_attention(t["q"], t["kc"], t["vc"], t["forest"], t["slot_ids"], t["ones"], t["priv_table"],
                                      t["priv_len"], part_o, part_ml, splits, 1, out=out)


def run_flat(t, splits, part_o, part_ml, out):
    """Every sequence over its whole page table (the non-cascade decode path of the engine)."""
    import ctypes
    q = t["q"]
    B, Hq, D = q.shape
    Hkv = t["kc"].shape[1]
    s = _lib.stream_ptr()
    _lib.check(fa._fn("dec")(_lib.ptr(q), _lib.ptr(t["slot_ids"]), _lib.ptr(t["ones"]), _lib.ptr(t["full_table"]),
                             t["max_pages"], _lib.ptr(t["full_len"]), _lib.ptr(t["kc"]), _lib.ptr(t["vc"]),
                             _lib.ptr(part_o[0]), _lib.ptr(part_ml[0]), B, Hq, Hkv, D, splits, 1.0 / D ** 0.5, s),
               "paged_decode")
    o_ptrs = (ctypes.c_void_p * 4)(part_o[0].data_ptr(), 0, 0, 0)
    ml_ptrs = (ctypes.c_void_p * 4)(part_ml[0].data_ptr(), 0, 0, 0)
    sp = (ctypes.c_int * 4)(splits, 0, 0, 0)
    _lib.check(fa._fn("merge")(o_ptrs, ml_ptrs, sp, 1, None, _lib.ptr(out), None, B, Hq, D, s), "decode_merge")
    return out


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(iters):
        fn()
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


def scratch(B, Hq, D, splits, device, n=4):
    f32 = dict(device=device, dtype=torch.float32)
    return ([torch.empty((B, Hq, splits, D), **f32) for _ in range(n)],
            [torch.empty((B, Hq, splits, 2), **f32) for _ in range(n)])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--roots", type=int, default=16)
    ap.add_argument("--root-len", type=int, default=16384)
    ap.add_argument("--branches", type=int, default=4)
    ap.add_argument("--branch-len", type=int, default=2048)
    ap.add_argument("--leaves", type=int, default=8)
    ap.add_argument("--leaf-len", type=int, default=512)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--splits", type=int, default=4)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hbm-gbs", type=float, default=6536.0)
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda")
    Hq, Hkv, D = args.heads, args.kv_heads, 128
    res = {"bench": "forest_decode", "heads": [Hq, Hkv, D], "page": PAGE}
    if args.check:
        t = build_tree(2, 256, 2, 64, 3, 40, Hq, Hkv, D, dev, seed=1)
        po, pml = scratch(t["B"], Hq, D, args.splits, dev)
        out = torch.empty_like(t["q"])
        ref = fa.forest_decode_reference(t["q"], t["kc"], t["vc"], t["contexts"])
        e1 = (run_cascade(t, args.splits, po, pml, out).float() - ref).abs().max().item()
        e2 = (run_flat(t, args.splits, po, pml, out).float() - ref).abs().max().item()
        _lib.check_status("forest check")
        res["check_max_abs_err"] = {"cascade": e1, "flat": e2}
        assert e1 < 2e-2 and e2 < 2e-2, res
    t = build_tree(args.roots, args.root_len, args.branches, args.branch_len, args.leaves, args.leaf_len, Hq, Hkv, D, dev)
    B = t["B"]
    po, pml = scratch(B, Hq, D, args.splits, dev)
    out = torch.empty_like(t["q"])
    tok_bytes = 2 * Hkv * D * 2                       # K + V of one token, one layer
    f = t["forest"]
    shared_tok = f.shared_tokens
    priv_tok = B * args.leaf_len
    flat_tok = B * (args.root_len + args.branch_len + args.leaf_len)
    ms_c = timeit(lambda: run_cascade(t, args.splits, po, pml, out), args.iters)
    _lib.check_status("forest cascade")
    casc_bytes = (shared_tok + priv_tok) * tok_bytes
    res.update({"sequences": B, "tree": [args.roots, args.root_len, args.branches, args.branch_len, args.leaves, args.leaf_len],
                "kv_cache_gb": round(2 * t["kc"].numel() * 2 / 1e9, 2), "node_table_rows": f.n_nodes,
                "cascade_ms": round(ms_c, 4), "cascade_kv_bytes": casc_bytes,
                "cascade_gbs": round(casc_bytes / ms_c / 1e6, 1),
                "cascade_frac_of_measured_hbm": round(casc_bytes / ms_c / 1e6 / args.hbm_gbs, 3),
                "per_sequence_kv_bytes": flat_tok * tok_bytes,
                "kv_traffic_ratio": round(flat_tok / (shared_tok + priv_tok), 2)})
    if not args.no_baseline:
        ms_f = timeit(lambda: run_flat(t, args.splits, po, pml, out), max(3, args.iters // 4))
        _lib.check_status("forest flat")
        res.update({"per_sequence_ms": round(ms_f, 4), "per_sequence_gbs": round(flat_tok * tok_bytes / ms_f / 1e6, 1),
                    "speedup": round(ms_f / ms_c, 2)})
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
