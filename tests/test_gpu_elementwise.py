"""RMSNorm / qk-norm+RoPE / SwiGLU kernels against fp32 PyTorch expressions."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("T,H", [(7, 256), (513, 2560), (64, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(T, H, with_res):
    from arctic_platform_b200.ops import _lib, norm
    x = _rand((T, H)).requires_grad_()
    res = _rand((T, H)).requires_grad_() if with_res else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    y, stream = norm.rmsnorm(x, w, 1e-6, res)
    dy, ds = _rand((T, H)), _rand((T, H))
    (y.float() * dy.float()).sum().add((stream.float() * ds.float()).sum() if with_res else 0).backward()
    _lib.check_status("rmsnorm")
    xr = x.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    xs = xr + rr if with_res else xr
    if with_res:
        xs_q = xs.detach().to(torch.bfloat16).float()
        xs = xs + (xs_q - xs).detach()
    yr = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ((yr * dy.float()).sum() + ((xs * ds.float()).sum() if with_res else 0)).backward()
    assert torch.allclose(y.float(), yr.detach(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=6e-2, rtol=3e-2)
    if with_res:
        assert torch.allclose(res.grad.float(), rr.grad, atol=6e-2, rtol=3e-2)
    rel = (w.grad.float() - wr.grad).abs().max() / (wr.grad.abs().max() + 1e-6)
    assert rel < 2e-2, rel


@pytest.mark.parametrize("D", [64, 128])
def test_qknorm_rope_fwd_bwd(D):
    from arctic_platform_b200.ops import _lib, norm
    T, Hq, Hkv = 131, 8, 2
    qkv = _rand((T, (Hq + 2 * Hkv) * D)).requires_grad_()
    wq = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_()
    wk = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_()
    cos_t, sin_t = norm.rope_tables(4096, D, 1e6, "cuda")
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    q, k, v = norm.qknorm_rope(qkv, wq, wk, cos_t, sin_t, pos, Hq, Hkv, D)
    gq, gk, gv = _rand(q.shape), _rand(k.shape), _rand(v.shape)
    ((q.float() * gq.float()).sum() + (k.float() * gk.float()).sum() + (v.float() * gv.float()).sum()).backward()
    _lib.check_status("qknorm_rope")
    qkvr = qkv.detach().float().requires_grad_()
    wqr, wkr = wq.detach().float().requires_grad_(), wk.detach().float().requires_grad_()
    q0 = qkvr[:, :Hq * D].reshape(T, Hq, D)
    k0 = qkvr[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
    v0 = qkvr[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    qr, kr = norm.qknorm_rope_ref(q0, k0, wqr, wkr, cos_t, sin_t, pos, 1e-6)
    ((qr * gq.float()).sum() + (kr * gk.float()).sum() + (v0 * gv.float()).sum()).backward()
    assert torch.allclose(q.float(), qr.detach(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(k.float(), kr.detach(), atol=3e-2, rtol=2e-2)
    assert torch.equal(v, v0.detach().to(torch.bfloat16))
    assert torch.allclose(qkv.grad.float(), qkvr.grad, atol=8e-2, rtol=3e-2)
    for g, gr in ((wq.grad, wqr.grad), (wk.grad, wkr.grad)):
        rel = (g.float() - gr).abs().max() / (gr.abs().max() + 1e-6)
        assert rel < 2e-2, rel


def test_swiglu_fwd_bwd():
    from arctic_platform_b200.ops import _lib, norm
    gu = _rand((257, 2 * 688)).requires_grad_()
    act = norm.swiglu(gu)
    d = _rand(act.shape)
    act.backward(d)
    _lib.check_status("swiglu")
    gr = gu.detach().float().requires_grad_()
    ar = torch.nn.functional.silu(gr[:, 0::2]) * gr[:, 1::2]
    ar.backward(d.float())
    assert torch.allclose(act.float(), ar.detach(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(gu.grad.float(), gr.grad, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("T,H,Dk,Dv", [(200, 4, 128, 128), (64, 2, 32, 48), (1000, 3, 64, 128)])
def test_delta_rule_scan_kernel_matches_the_token_by_token_recurrence(T, H, Dk, Dv):
    """The chunk recurrence of the gated delta rule as one kernel (no-grad passes) against the token-by-token oracle
    and against the differentiable PyTorch loop, with and without a carried-in state."""
    from arctic_platform_b200.models.linear_attention import gated_delta_rule_chunked, gated_delta_rule_recurrent
    from arctic_platform_b200.ops import _lib
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(T, H, Dk, device="cuda", generator=g)
    k = torch.randn(T, H, Dk, device="cuda", generator=g)
    v = torch.randn(T, H, Dv, device="cuda", generator=g)
    gate = -torch.rand(T, H, device="cuda", generator=g) * 0.3
    beta = torch.rand(T, H, device="cuda", generator=g)
    S0 = torch.randn(H, Dk, Dv, device="cuda", generator=g) * 0.1
    for state in (None, S0):
        want_o, want_S = gated_delta_rule_recurrent(q, k, v, gate, beta, state)
        with torch.no_grad():
            got_o, got_S = gated_delta_rule_chunked(q, k, v, gate, beta, state)            # kernel
        _lib.check_status("delta rule scan")
        with torch.enable_grad():
            loop_o, loop_S = gated_delta_rule_chunked(q, k, v, gate, beta, state)          # PyTorch loop
        for a, b in ((got_o, want_o), (got_S, want_S), (got_o, loop_o), (got_S, loop_S)):
            assert (a - b).abs().max() < 2e-3 * b.abs().max() + 1e-4
