"""tcgen05 segment attention (varlen causal + ZoRRo shared prefix) against the dense fp32 reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, scale=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _layouts():
    from arctic_platform_b200.ops.attention import AttnLayout
    varlen = AttnLayout.from_cu_seqlens([0, 1, 130, 386, 700, 1212])
    # two groups: prompt 300 with responses 70 / 130 / 1, prompt 129 with responses 256 / 40
    segs, t = [], 0
    for plen, rlens in ((300, (70, 130, 1)), (129, (256, 40))):
        p0 = t
        segs.append([p0, plen, 0, 0, p0, plen])
        t += plen
        for r in rlens:
            segs.append([t, r, p0, plen, t, r])
            t += r
    zorro = AttnLayout(np.array(segs, dtype=np.int32), t)
    return {"varlen": varlen, "zorro": zorro}


@pytest.mark.parametrize("name", ["varlen", "zorro"])
@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 128), (8, 2, 128), (2, 2, 128), (4, 2, 64)])
def test_attention_forward(name, Hq, Hkv, D):
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops.attention import attention_fwd_cuda, attention_ref
    layout = _layouts()[name]
    T = layout.total_tokens
    q, k, v = _rand((T, Hq, D)), _rand((T, Hkv, D)), _rand((T, Hkv, D))
    o, lse = attention_fwd_cuda(q, k, v, layout, D ** -0.5)
    _lib.check_status("attn fwd")
    o_ref, lse_ref = attention_ref(q, k, v, layout, D ** -0.5, return_lse=True)
    assert torch.allclose(o.float(), o_ref.float(), atol=2e-2, rtol=2e-2), (o.float() - o_ref.float()).abs().max()
    assert torch.allclose(lse, lse_ref, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("name", ["varlen", "zorro"])
@pytest.mark.parametrize("Hq,Hkv", [(4, 2), (8, 2), (2, 2)])
def test_attention_backward(name, Hq, Hkv):
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops.attention import attention_ref, segment_attention
    D = 128
    layout = _layouts()[name]
    T = layout.total_tokens
    q, k, v = (_rand((T, Hq, D)).requires_grad_(), _rand((T, Hkv, D)).requires_grad_(),
               _rand((T, Hkv, D)).requires_grad_())
    d_o = _rand((T, Hq, D))
    o = segment_attention(q, k, v, layout)
    o.backward(d_o)
    _lib.check_status("attn bwd")
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    o_ref = attention_ref(qr, kr, vr, layout)
    o_ref.backward(d_o.float())
    for got, ref, nm in ((q.grad, qr.grad, "dq"), (k.grad, kr.grad, "dk"), (v.grad, vr.grad, "dv")):
        err = (got.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= 2e-2 * scale + 2e-2, f"{nm}: err {err} scale {scale}"


def test_zorro_matches_replicated_layout():
    """Shared-prefix attention equals ordinary causal attention on [prompt || response] copies."""
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops.attention import AttnLayout, attention_fwd_cuda
    Hq, Hkv, D, P = 4, 2, 128, 333
    rl = (100, 57)
    T = P + sum(rl)
    q, k, v = _rand((T, Hq, D)), _rand((T, Hkv, D)), _rand((T, Hkv, D))
    segs, t = [[0, P, 0, 0, 0, P]], P
    for r in rl:
        segs.append([t, r, 0, P, t, r])
        t += r
    o, _ = attention_fwd_cuda(q, k, v, AttnLayout(np.array(segs, dtype=np.int32), T), D ** -0.5)
    t = P
    for r in rl:
        idx = torch.cat([torch.arange(P), torch.arange(t, t + r)]).cuda()
        o2, _ = attention_fwd_cuda(q[idx].contiguous(), k[idx].contiguous(), v[idx].contiguous(),
                                   AttnLayout.from_cu_seqlens([0, P + r]), D ** -0.5)
        assert torch.allclose(o2[P:].float(), o[t:t + r].float(), atol=1e-2, rtol=1e-2)
        t += r
    _lib.check_status("attn zorro")
