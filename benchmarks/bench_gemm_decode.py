"""Skinny (decode-time) GEMM shapes of Qwen3-4B, M = batch: tile width and split-K variants of the
tcgen05 kernel against torch.matmul.  CUDA events; weights rotate through a pool larger than L2.

    python benchmarks/bench_gemm_decode.py [--batch 128]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.ops import _lib, gemm  # noqa: E402


def timeit(fn, nv, iters=30, warmup=5):
    for i in range(warmup):
        fn(i % nv)
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for i in range(iters):
        fn(i % nv)
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=128)
    args = ap.parse_args()
    M = args.batch
    shapes = [("qkv", 6144, 2560), ("o_proj", 2560, 4096), ("gate_up", 19456, 2560), ("down", 2560, 9728),
              ("lm_head", 151936, 2560)]
    for name, N, K in shapes:
        nv = max(2, int(400e6 // (N * K * 2)) + 1)
        xs = [torch.randn(M, K, device="cuda").bfloat16() for _ in range(nv)]
        ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(nv)]
        ideal_us = N * K * 2 / 6536e9 * 1e6
        row = {"shape": name, "M": M, "N": N, "K": K, "hbm_ideal_us": round(ideal_us, 1),
               "cublas_us": round(timeit(lambda i: torch.matmul(xs[i], ws[i].t()), nv), 1)}
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for bn in (64, 128, 256):
            if N < bn:
                continue
            row[f"bn{bn}_us"] = round(timeit(lambda i: gemm.gemm_raw(xs[i], ws[i], out, M=M, N=N, K=K, bn=bn), nv), 1)
        acc = torch.zeros(M, N, device="cuda", dtype=torch.float32)
        for bn, splits in ((128, 3), (128, 7), (64, 4), (256, 7), (256, 14)):
            tiles = (N + bn - 1) // bn
            if tiles * splits > 4 * 148:
                continue
            row[f"bn{bn}_split{splits}_us"] = round(
                timeit(lambda i: gemm.gemm_raw(xs[i], ws[i], acc, M=M, N=N, K=K, bn=bn, splits=splits,
                                               epi=gemm.EPI_F32_ATOMIC), nv), 1)
        _lib.check_status(name)
        print(json.dumps(row), flush=True)
        del xs, ws


if __name__ == "__main__":
    main()
