"""Fused lm_head log-prob / entropy kernel against the fp32 chunked reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,H,V", [(300, 256, 32000), (129, 512, 151936), (5, 128, 1000)])
@pytest.mark.parametrize("per_row_temp", [False, True])
def test_logprob_forward_backward(N, H, V, per_row_temp):
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops.logprob import lm_head_logprobs, logprobs_entropy_ref
    torch.manual_seed(0)
    hidden = torch.randn(N, H, device="cuda").bfloat16().requires_grad_()
    weight = (torch.randn(V, H, device="cuda") * 0.05).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (N,), device="cuda")
    it = (0.5 + torch.rand(N, device="cuda")) if per_row_temp else 0.7
    lp, ent = lm_head_logprobs(hidden, weight, labels, it, with_entropy=True, bwd_chunk=128)
    g1, g2 = torch.randn(N, device="cuda"), torch.randn(N, device="cuda") * 0.1
    ((lp * g1).sum() + (ent * g2).sum()).backward()
    _lib.check_status("lmhead")
    hr, wr = hidden.detach().float().requires_grad_(), weight.detach().float().requires_grad_()
    lpr, entr = logprobs_entropy_ref(hr, wr, labels, it, True)
    ((lpr * g1).sum() + (entr * g2).sum()).backward()
    assert torch.allclose(lp, lpr.detach(), atol=3e-2, rtol=1e-2), (lp - lpr).abs().max()
    assert torch.allclose(ent, entr.detach(), atol=3e-2, rtol=1e-2), (ent - entr).abs().max()
    for got, ref, nm in ((hidden.grad, hr.grad, "dh"), (weight.grad, wr.grad, "dw")):
        err = (got.float() - ref).abs().max().item()
        sc = ref.abs().max().item()
        assert err <= 3e-2 * sc + 1e-3, f"{nm}: {err} vs scale {sc}"
