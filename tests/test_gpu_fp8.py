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


def test_sampler_serves_fp8_weights():
    """Rollouts from block-scaled fp8 projections: log-probs reported by the engine stay close to the bf16 model's
    own scoring of the same tokens, before and after a weight update."""
    import dataclasses
    import numpy as np
    from arctic_platform_b200.engine.sampler import SamplerEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM, token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    cfg = dataclasses.replace(PRESETS["qwen3-tiny-d128"], intermediate_size=768, name="tiny-fp8")
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=5, std=0.05)
    eng = SamplerEngine(cfg, "cuda", model=model, kv_cache_tokens=1 << 14, max_batch=16, max_seq_len=256,
                        sync_interval=4, quantization="fp8")
    assert eng.fp8
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, cfg.vocab_size, size=n).tolist() for n in (33, 64)]
    for round_ in range(2):
        outs = eng.generate(prompts, {"n": 2, "temperature": 0.0, "max_tokens": 12})
        _lib.check_status("fp8 generate")
        P, R = 64, 12
        ids = torch.zeros((4, P + R), dtype=torch.int64)
        mask = torch.zeros_like(ids)
        for i, o in enumerate(outs):
            p = prompts[o["prompt_index"]]
            ids[i, P - len(p):P] = torch.tensor(p)
            mask[i, P - len(p):P] = 1
            ids[i, P:] = torch.tensor(o["token_ids"])
            mask[i, P:] = 1
        pb = build_packed_batch(ids, mask, R).to("cuda")
        with torch.no_grad():
            lp, _ = token_logprobs(model, pb, 1.0)
        got = torch.tensor([o["logprobs"] for o in outs]).reshape(-1)
        ref = pb.scatter_to_grid(lp).cpu().reshape(-1)
        assert (got - ref).abs().mean() < 0.2, float((got - ref).abs().mean())
        with torch.no_grad():                                         # weight update -> fp8 copies are rebuilt
            for p_ in model.parameters():
                if p_.dim() == 2:
                    p_.mul_(1.02)
        eng.weights_updated()
