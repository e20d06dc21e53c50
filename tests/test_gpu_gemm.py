"""tcgen05 GEMM against a plain fp32 PyTorch product (arctic_platform_b200/csrc/gemm_tcgen05.cu)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, ref, K):
    tol = 2e-2 * (K ** 0.5) * 0.05 + 2e-2
    err = (got.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol + 8e-3 * scale, f"max err {err} (ref scale {scale})"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 256), (200, 136, 72), (1024, 2560, 2560),
                                   (4096, 6144, 2560), (77, 8, 8), (3000, 19456, 2560)])
@pytest.mark.parametrize("bn", [0, 128, 256])
def test_matmul_nt(M, N, K, bn):
    from arctic_platform_b200.ops import _lib, gemm
    a, b = _rand((M, K)), _rand((N, K))
    out = gemm.matmul_nt(a, b, bn=bn)
    _lib.check_status("gemm nt")
    _close(out, a.float() @ b.float().t(), K)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (512, 384, 320), (200, 136, 72), (2048, 2560, 9728)])
def test_matmul_nn_and_tn(M, N, K):
    from arctic_platform_b200.ops import _lib, gemm
    a, b = _rand((M, K)), _rand((K, N))
    out = gemm.matmul_nn(a, b)
    _lib.check_status("gemm nn")
    _close(out, a.float() @ b.float(), K)
    at = _rand((K, M))
    out2 = gemm.matmul_tn(at, b, out_dtype=torch.float32)
    _lib.check_status("gemm tn")
    _close(out2, at.float().t() @ b.float(), K)
    acc = torch.ones((M, N), device="cuda", dtype=torch.float32)
    gemm.matmul_tn(at, b, out=acc, accumulate=True)
    _lib.check_status("gemm tn acc")
    _close(acc, at.float().t() @ b.float() + 1.0, K)


def test_bias_fp32_and_splitk():
    from arctic_platform_b200.ops import _lib, gemm
    M, N, K = 130, 264, 1024
    a, b, bias = _rand((M, K)), _rand((N, K)), _rand((N,))
    out = gemm.matmul_nt(a, b, bias=bias)
    _lib.check_status("gemm bias")
    ref = a.float() @ b.float().t()
    _close(out, ref + bias.float(), K)
    acc = torch.zeros((M, N), device="cuda", dtype=torch.float32)
    gemm.gemm_raw(a, b, acc, M=M, N=N, K=K, epi=gemm.EPI_F32_ATOMIC, splits=4)
    _lib.check_status("gemm splitk")
    _close(acc, ref, K)


def test_swiglu_epilogue():
    from arctic_platform_b200.ops import _lib, gemm, norm
    M, K, I = 300, 256, 688
    x, w = _rand((M, K)), _rand((2 * I, K), 0.1)
    gu, act = gemm.gate_up_swiglu(x, w)
    _lib.check_status("gemm swiglu")
    ref_gu = x.float() @ w.float().t()
    _close(gu, ref_gu, K)
    ref_act = torch.nn.functional.silu(ref_gu[:, 0::2]) * ref_gu[:, 1::2]
    _close(act, ref_act, K)
    assert torch.allclose(norm.swiglu(gu).float(), norm.swiglu_ref(gu).float(), atol=2e-2, rtol=2e-2)


def test_grouped_tile_map():
    from arctic_platform_b200.ops import _lib, gemm
    E, N, K = 3, 256, 128
    counts = [130, 0, 77]
    T = sum(counts)
    x, w = _rand((T, K)), _rand((E * N, K))
    out = torch.zeros((T, N), device="cuda", dtype=torch.bfloat16)
    tiles, row = [], 0
    for e, c in enumerate(counts):
        for m0 in range(row, row + c, 128):
            for nt in range(N // 128):
                tiles.append([m0, row + c, e * N, nt])
        row += c
    tm = torch.tensor(tiles, device="cuda", dtype=torch.int32)
    gemm.gemm_raw(x, w, out, M=T, N=N, K=K, tile_map=tm, b_rows=E * N, bn=128)
    _lib.check_status("gemm grouped")
    row = 0
    for e, c in enumerate(counts):
        if c:
            ref = x[row:row + c].float() @ w[e * N:(e + 1) * N].float().t()
            _close(out[row:row + c], ref, K)
        row += c


def test_linear_autograd():
    from arctic_platform_b200.ops import _lib, gemm
    x = _rand((4, 65, 256)).requires_grad_()
    w = _rand((384, 256), 0.05).requires_grad_()
    y = gemm.linear(x, w)
    dy = _rand(y.shape)
    y.backward(dy)
    _lib.check_status("linear")
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(dy.float())
    _close(y, yr.detach(), 256)
    _close(x.grad, xr.grad, 384)
    _close(w.grad, wr.grad, 260)


@pytest.mark.parametrize("bn", [64, 128])
@pytest.mark.parametrize("epi", ["bf16", "swiglu"])
def test_two_ctas_per_sm_variant_matches_reference(bn, epi):
    """The 3-stage, two-CTAs-per-SM kernel (decode-shaped problems between one and two waves of tiles)."""
    from arctic_platform_b200.ops import _lib, gemm
    torch.manual_seed(bn)
    M, N, K = 128, 19456 if bn == 128 else 12800, 512
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    ref = a.float() @ b.float().t()
    if epi == "bf16":
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        gemm.gemm_raw(a, b, out, M=M, N=N, K=K, bn=gemm.BN_X2 + bn)
        _lib.check_status("x2 gemm")
        assert (out.float() - ref).abs().max() < 0.05
    else:
        act = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
        gemm.gemm_raw(a, b, None, M=M, N=N, K=K, epi=gemm.EPI_SWIGLU, out2=act, bn=gemm.BN_X2 + bn)
        _lib.check_status("x2 gemm swiglu")
        want = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
        assert (act.float() - want).abs().max() < 0.05
