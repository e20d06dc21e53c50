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


def _pair(a, b, out, M, N, K, a_mn=False, b_mn=False, epi=0, alpha=1.0, bias=None, out2=None):
    """Direct call of the CTA-pair kernel (any size; the automatic dispatch only sends large problems there)."""
    import ctypes as c
    from arctic_platform_b200.ops import _lib
    vp, i, ll, f = c.c_void_p, c.c_int, c.c_longlong, c.c_float
    fn = _lib.declare("apb_gemm_bf16_pair", [vp, vp, vp, i, i, i, ll, ll, ll, i, i, i, f, vp, vp, ll, vp])
    _lib.check(fn(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0),
                  out.stride(0) if out is not None else 0, int(a_mn), int(b_mn), epi, alpha, _lib.ptr(bias),
                  _lib.ptr(out2), out2.stride(0) if out2 is not None else 0, _lib.stream_ptr()), "apb_gemm_bf16_pair")


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (300, 264, 72), (1000, 2568, 1096),
                                   (4096, 2560, 2560), (77, 8, 8)])
def test_cta_pair_kernel_all_operand_layouts(M, N, K):
    """256 x 256 tiles on two SMs (tcgen05 cta_group::2): NT / NN / TN products, bf16 and fp32 outputs, accumulation,
    row / column / depth tails, against fp32 matmul."""
    from arctic_platform_b200.ops import _lib
    a, b = _rand((M, K)), _rand((N, K))
    ref = a.float() @ b.float().t()
    out = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    _pair(a, b, out, M, N, K)
    _lib.check_status("pair nt")
    _close(out, ref, K)
    bias = _rand((N,))
    _pair(a, b, out, M, N, K, bias=bias, alpha=0.5)
    _lib.check_status("pair nt bias")
    _close(out, 0.5 * ref + bias.float(), K)
    bt = b.t().contiguous()                                   # [K, N]: the data-gradient form
    out32 = torch.empty((M, N), device="cuda", dtype=torch.float32)
    _pair(a, bt, out32, M, N, K, b_mn=True, epi=1)
    _lib.check_status("pair nn")
    _close(out32, ref, K)
    if M % 8 == 0:                                            # A stored [K, M]: rows of M elements, 16-byte aligned
        at = a.t().contiguous()                               # the weight-gradient form, accumulated
        acc = torch.full((M, N), 2.0, device="cuda", dtype=torch.float32)
        _pair(at, bt, acc, M, N, K, a_mn=True, b_mn=True, epi=3)
        _lib.check_status("pair tn acc")
        _close(acc, ref + 2.0, K)


def test_cta_pair_kernel_splits_long_k_accumulation():
    """A weight-gradient shaped product (few output tiles, K = tokens) is cut along K by the kernel; the parts add
    into the fp32 accumulator."""
    from arctic_platform_b200.ops import _lib
    M, N, K = 2560, 4096, 16384                               # 160 tiles: 2.2 waves of pairs without a split
    at, bt = _rand((K, M)), _rand((K, N))
    acc = torch.full((M, N), -1.0, device="cuda", dtype=torch.float32)
    _pair(at, bt, acc, M, N, K, a_mn=True, b_mn=True, epi=3)
    _lib.check_status("pair tn split")
    _close(acc, at.float().t() @ bt.float() - 1.0, K)


def test_cta_pair_kernel_swiglu_and_many_tiles_per_pair():
    """More tiles than resident pairs (the persistent loop and both accumulator buffers are exercised) and the
    SwiGLU epilogue; also the automatic dispatch of a large product equals the one-CTA kernel's result."""
    from arctic_platform_b200.ops import _lib, gemm
    M, K, I = 2304, 512, 9728
    x, w = _rand((M, K)), _rand((2 * I, K), 0.1)
    gu = torch.empty((M, 2 * I), device="cuda", dtype=torch.bfloat16)
    act = torch.empty((M, I), device="cuda", dtype=torch.bfloat16)
    _pair(x, w, gu, M, 2 * I, K, epi=4, out2=act)
    _lib.check_status("pair swiglu")
    ref_gu = x.float() @ w.float().t()
    _close(gu, ref_gu, K)
    _close(act, torch.nn.functional.silu(ref_gu[:, 0::2]) * ref_gu[:, 1::2], K)
    auto = gemm.matmul_nt(x, w)                               # dispatch picks the pair kernel for this size
    one = gemm.matmul_nt(x, w, bn=256)                        # forced one-CTA kernel
    _lib.check_status("pair vs one")
    assert torch.equal(auto, gu)
    assert (auto.float() - one.float()).abs().max().item() <= 2e-2 * ref_gu.abs().max().item()


@pytest.mark.parametrize("bn", [144, 208])
@pytest.mark.parametrize("M,N,K", [(128, 2880, 256), (100, 1160, 200), (128, 19456, 512), (300, 424, 64)])
def test_in_between_tile_widths(M, N, K, bn):
    """144- and 208-column tiles (16-column multiples between the power-of-two widths, used to cover decode-shaped
    products in one wave of SMs): bf16 / fp32 outputs and the SwiGLU epilogue, with row, column and depth tails."""
    from arctic_platform_b200.ops import _lib, gemm
    a, b = _rand((M, K)), _rand((N, K), 0.2)
    ref = a.float() @ b.float().t()
    out = gemm.matmul_nt(a, b, bn=bn)
    _lib.check_status("gemm bn")
    _close(out, ref, K)
    out32 = torch.full((M, N), 7.0, device="cuda", dtype=torch.float32)
    gemm.matmul_nt(a, b, out=out32, bn=bn)
    _lib.check_status("gemm bn f32")
    _close(out32, ref, K)
    if N % 16 == 0:
        act = torch.empty((M, N // 2), device="cuda", dtype=torch.bfloat16)
        gemm.gemm_raw(a, b, None, M=M, N=N, K=K, epi=gemm.EPI_SWIGLU, out2=act, bn=bn)
        _lib.check_status("gemm bn swiglu")
        _close(act, torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2], K)
    auto = gemm.matmul_nt(a, b)                      # the automatic choice for one row tile may be one of these widths
    _lib.check_status("gemm auto")
    _close(auto, ref, K)
