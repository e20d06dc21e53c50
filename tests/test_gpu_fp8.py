"""Block-scaled fp8 GEMM: the tensor-core kernel against the same quantised operands multiplied in fp32, and the
end-to-end error of the fp8 linear against the bf16 product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 2560, 4096), (64, 19456, 2560), (300, 1000, 1280), (1, 768, 2048)])
def test_fp8_blockscale_gemm_matches_dequantised_reference(M, N, K):
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops.fp8 import dequant_weight, fp8_gemm, fp8_linear, quant_act_fp8
    from arctic_platform_b200.parallel.weight_sync import quantize_fp8_block128
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda").bfloat16()
    x[:, :128] *= 8.0                                                  # K blocks with different dynamic ranges
    w = (torch.randn(N, K, device="cuda") * 0.03).bfloat16()
    w[:256] *= 5.0
    wq, sw = quantize_fp8_block128(w)
    xq, sa = quant_act_fp8(x)
    # quantisation round trip stays within fp8 resolution of the block maximum
    xd = xq.float().view(M, K // 128, 128) * sa[..., None]
    assert ((xd.view(M, K) - x.float()).abs() <= 0.07 * x.float().view(M, K // 128, 128).abs().amax(-1, keepdim=True)
            .expand(M, K // 128, 128).reshape(M, K) + 1e-6).all()
    got = fp8_gemm(xq, sa, wq, sw).float()
    _lib.check_status("fp8 gemm")
    ref = xd.view(M, K) @ dequant_weight(wq, sw).t()
    scale = ref.abs().max()
    assert (got - ref).abs().max() < 0.01 * scale + 0.02, float((got - ref).abs().max())      # same operands: bf16 rounding only
    full = x.float() @ w.float().t()
    y = fp8_linear(x, wq, sw).float()
    rel = (y - full).norm() / full.norm()
    assert rel < 0.05, float(rel)                                                         # fp8 quantisation error
