"""Times the tcgen05 GEMMs against torch.matmul (cuBLAS) on the linear-layer shapes of Qwen3-4B.

Three columns per shape: the automatic dispatch (CTA-pair kernel, 256 x 256 tiles on two SMs, for problems of at
least one wave of pairs), the one-CTA kernel forced (128 x 256 tiles), and cuBLAS.  CUDA-event timing after
warm-up, inputs rotated through a pool larger than L2 so no iteration re-reads operands from cache.  Prints one
JSON line per shape; ``--peak-tflops`` is the measured cuBLAS bf16 burst figure of the machine (the denominator of
``frac_of_measured_peak``).

    python benchmarks/bench_gemm.py [--tokens 8192] [--iters 20] [--peak-tflops 1635.6]
"""
import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
from arctic_platform_b200.ops import _lib, gemm  # noqa: E402


def timeit(fn, n_variants, iters, warmup=3):
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for i in range(iters):
        fn(i % n_variants)
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--peak-tflops", type=float, default=1635.6)
    args = ap.parse_args()
    T = args.tokens
    H, I, QKV = 2560, 9728, 6144
    shapes = [("qkv_fwd", "nt", T, QKV, H), ("o_fwd", "nt", T, H, 4096), ("gate_up_fwd", "nt", T, 2 * I, H),
              ("down_fwd", "nt", T, H, I), ("gate_up_dgrad", "nn", T, H, 2 * I), ("gate_up_wgrad", "tn", 2 * I, H, T),
              ("down_dgrad", "nn", T, I, H), ("down_wgrad", "tn", H, I, T)]
    peaks = {"bf16_tflops": args.peak_tflops}
    for name, kind, M, N, K in shapes:
        bytes_per = 2 * (M * K + N * K + M * N)
        nv = max(2, int(300e6 // bytes_per) + 1)
        if kind == "nt":
            As = [torch.randn(M, K, device="cuda").bfloat16() for _ in range(nv)]
            Bs = [torch.randn(N, K, device="cuda").bfloat16() for _ in range(nv)]
            ours = lambda i: gemm.matmul_nt(As[i], Bs[i])
            one = lambda i: gemm.matmul_nt(As[i], Bs[i], bn=256)
            ref = lambda i: torch.matmul(As[i], Bs[i].t())
        elif kind == "nn":
            As = [torch.randn(M, K, device="cuda").bfloat16() for _ in range(nv)]
            Bs = [torch.randn(K, N, device="cuda").bfloat16() for _ in range(nv)]
            ours = lambda i: gemm.matmul_nn(As[i], Bs[i])
            one = lambda i: gemm.matmul_nn(As[i], Bs[i], bn=256)
            ref = lambda i: torch.matmul(As[i], Bs[i])
        else:
            As = [torch.randn(K, M, device="cuda").bfloat16() for _ in range(nv)]
            Bs = [torch.randn(K, N, device="cuda").bfloat16() for _ in range(nv)]
            ours = lambda i: gemm.matmul_tn(As[i], Bs[i])
            one = lambda i: gemm.matmul_tn(As[i], Bs[i], bn=256)
            ref = lambda i: torch.matmul(As[i].t(), Bs[i])
        t_ours = timeit(ours, nv, args.iters)
        t_one = timeit(one, nv, args.iters)
        t_ref = timeit(ref, nv, args.iters)
        _lib.check_status(name)
        fl = 2.0 * M * N * K
        print(json.dumps({"shape": name, "kind": kind, "M": M, "N": N, "K": K,
                          "ours_ms": round(t_ours, 4), "one_cta_ms": round(t_one, 4), "cublas_ms": round(t_ref, 4),
                          "ours_tflops": round(fl / t_ours / 1e9, 1), "one_cta_tflops": round(fl / t_one / 1e9, 1),
                          "cublas_tflops": round(fl / t_ref / 1e9, 1),
                          "frac_of_measured_peak": round(fl / t_ours / 1e9 / peaks["bf16_tflops"], 3)}), flush=True)
        del As, Bs


if __name__ == "__main__":
    main()
