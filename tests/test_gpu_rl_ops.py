"""Fused RL-step kernels against their PyTorch twins: the token-mean GRPO objective (loss, statistics, gradient), the
mixture-of-experts routing decision, and the expert FFN whose grouped-GEMM tile tables are built on the device."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kl", [None, "low_var_kl", "kl", "mse", "abs"])
@pytest.mark.parametrize("weighted", [False, True])
def test_grpo_token_loss_matches_the_composed_torch_ops(kl, weighted):
    from arctic_platform_b200.ops import _lib, rl_ops
    from arctic_platform_b200.rl.processors.functional import agg_loss, kl_penalty, ppo_clip_token_loss
    g = torch.Generator(device="cuda").manual_seed(5)
    n = 10_007
    lp = (torch.randn(n, generator=g, device="cuda") * 0.7 - 2.0).requires_grad_(True)
    old = lp.detach() + torch.randn(n, generator=g, device="cuda") * 0.5
    old[::97] -= 30.0                                         # beyond the +-20 clamp of the log ratio
    ref = lp.detach() + torch.randn(n, generator=g, device="cuda") * 0.3
    adv = torch.randn(n, generator=g, device="cuda")
    mask = torch.rand(n, generator=g, device="cuda") > 0.2
    w = torch.rand(n, generator=g, device="cuda") + 0.5 if weighted else None
    dp, ntok, coef = 2, 12345.0, 0.01
    # twin
    lp2 = lp.detach().clone().requires_grad_(True)
    tok, d, clipped, lower = ppo_clip_token_loss(lp2, old, adv, 0.2, 0.2, 3.0)
    if w is not None:
        tok = tok * w
    want = agg_loss(tok, mask, "token-mean", dp_size=dp, batch_num_tokens=ntok)
    if kl:
        kld = kl_penalty(lp2, ref, kl)
        want = want + coef * agg_loss(kld, mask, "token-mean", dp_size=dp, batch_num_tokens=ntok)
    want.backward()
    # fused
    loss, sums = rl_ops.grpo_token_loss(lp, old, adv, mask, dp / ntok, ref_lp=ref if kl else None, kl_kind=kl,
                                        kl_coef=coef if kl else 0.0, weight=w)
    (loss * 3.0).backward()
    _lib.check_status("grpo kernel")
    assert float(loss) == pytest.approx(float(want), rel=2e-5, abs=1e-7)
    assert torch.allclose(lp.grad / 3.0, lp2.grad, rtol=2e-4, atol=1e-9)
    mf = mask.float()
    s = sums.tolist()
    assert s[0] == float(mf.sum()) and s[1] == float((clipped.float() * mf).sum()) and s[3] == float((lower.float() * mf).sum())
    assert s[2] == pytest.approx(float((-d.detach() * mf).sum()), rel=1e-4)
    assert s[4] == pytest.approx(float((tok.detach() * mf).sum()), rel=1e-4)


@pytest.mark.parametrize("E,k,score", [(128, 8, "softmax"), (64, 6, "sigmoid"), (8, 2, "softmax"), (384, 8, "softmax")])
def test_route_kernel_picks_the_same_experts_as_topk(E, k, score):
    from arctic_platform_b200.ops import _lib, rl_ops
    g = torch.Generator(device="cuda").manual_seed(E)
    T = 777
    logits = torch.randn(T, E, generator=g, device="cuda") * 2.0
    bias = torch.randn(E, generator=g, device="cuda") * 0.1
    counts = torch.zeros(E, device="cuda", dtype=torch.int32)
    idx = rl_ops.moe_route(logits, k, score, bias, counts)
    _lib.check_status("route")
    scores = torch.softmax(logits, -1) if score == "softmax" else torch.sigmoid(logits)
    want = torch.topk(scores + bias, k, dim=-1).indices
    assert torch.equal(idx.sort(-1).values, want.sort(-1).values)
    assert torch.equal(idx, want)                                            # best first, like topk
    assert torch.equal(counts.long(), torch.bincount(want.reshape(-1), minlength=E))


def test_moe_layer_forward_and_backward_with_device_built_tiles():
    """The expert FFN with tile tables written by a kernel (no copy of the expert histogram to the host in the forward)
    against the per-expert fp32 loop, values and gradients; skewed routing with empty experts."""
    import dataclasses
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.moe import MoEFeedForward, grouped_ffn
    from arctic_platform_b200.ops import _lib
    name = next((n for n in PRESETS if PRESETS[n].is_moe and PRESETS[n].moe_activation == "swiglu"
                 and not PRESETS[n].layer_types), None)
    if name is None:
        pytest.skip("no plain MoE preset")
    cfg = dataclasses.replace(PRESETS[name], hidden_size=256, moe_intermediate_size=128, num_experts=16,
                              num_experts_per_tok=4, shared_expert_intermediate_size=0)
    torch.manual_seed(0)
    moe = MoEFeedForward(cfg, "cuda", torch.bfloat16)
    for p in moe.parameters():
        p.data.normal_(0, 0.05)
    R = 700
    counts = torch.tensor([300, 0, 5, 128, 129, 0, 0, 1, 37, 0, 100, 0, 0, 0, 0, 0], device="cuda")
    x = (torch.randn(R, cfg.hidden_size, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    y = grouped_ffn(x, moe.wgu, moe.wdown, counts)
    y.float().pow(2).sum().backward()
    _lib.check_status("moe device tiles")
    xr = x.detach().float().requires_grad_(True)
    outs, row = [], 0
    for e, c in enumerate(counts.tolist()):
        gu = xr[row:row + c] @ moe.wgu[e].float().t()
        outs.append((torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ moe.wdown[e].float().t())
        row += c
    ref = torch.cat(outs)
    ref.pow(2).sum().backward()
    assert (y.float() - ref).abs().max() < 3e-2 * ref.abs().max() + 1e-3
    assert (x.grad.float() - xr.grad).abs().max() < 5e-2 * xr.grad.abs().max() + 1e-3


@pytest.mark.parametrize("tokens,experts,top_k", [(300, 16, 4), (37, 8, 2), (1024, 64, 8)])
def test_moe_layer_padded_plan_backward_matches_per_expert_fp32(tokens, experts, top_k):
    """Training path of the expert layer: padded expert-major rows, forward, data gradients and weight gradients as
    grouped GEMMs planned by a kernel (no expert count reaches the host) against an fp32 per-expert loop; skewed
    routing leaves some experts without tokens."""
    import dataclasses
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.moe import MoEFeedForward
    from arctic_platform_b200.ops import _lib
    cfg = dataclasses.replace(PRESETS["qwen3-moe-tiny"], hidden_size=256, moe_intermediate_size=192, num_experts=experts,
                              num_experts_per_tok=top_k, shared_expert_intermediate_size=0)
    torch.manual_seed(1)
    moe = MoEFeedForward(cfg, "cuda", torch.bfloat16)
    for p in moe.parameters():
        p.data.normal_(0, 0.05)
    moe.router.data[experts // 2:] -= 1.0                          # starve the upper half of the experts
    x = (torch.randn(tokens, 256, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    from arctic_platform_b200.models.moe import route_topk
    route = lambda lg, forced: route_topk(lg, top_k, cfg.norm_topk_prob, cfg.moe_score_func, cfg.moe_route_scale, None,
                                          forced, cfg.moe_n_group, cfg.moe_topk_group)
    with torch.no_grad():
        _, idx = route((x.float() @ moe.router.float().t()), None)
    moe.routed_experts = idx                                       # both sides route identically
    y = moe(x)
    (y.float() * torch.linspace(-1, 1, 256, device="cuda")).sum().backward()
    _lib.check_status("moe padded plan")
    # oracle: same routing decision, fp32 math (the routing weights carry gradient to x through the router)
    xr = x.detach().float().requires_grad_(True)
    wgu = moe.wgu.detach().float().requires_grad_(True)
    wdn = moe.wdown.detach().float().requires_grad_(True)
    w, _ = route(xr @ moe.router.detach().float().t(), idx)
    out = torch.zeros(tokens, 256, device="cuda")
    for e in range(experts):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = xr[tok] @ wgu[e].t()
        ye = (torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]) @ wdn[e].t()
        out = out.index_add(0, tok, ye * w[tok, slot, None].float())
    (out * torch.linspace(-1, 1, 256, device="cuda")).sum().backward()
    tol = lambda ref: 4e-2 * ref.abs().max() + 1e-3
    assert (y.float() - out).abs().max() < tol(out)
    assert (x.grad.float() - xr.grad).abs().max() < tol(xr.grad)
    g_gu = moe.wgu.grad_f32 if getattr(moe.wgu, "grad_f32", None) is not None else moe.wgu.grad.float()
    g_dn = moe.wdown.grad_f32 if getattr(moe.wdown, "grad_f32", None) is not None else moe.wdown.grad.float()
    assert (g_gu - wgu.grad).abs().max() < tol(wgu.grad)
    assert (g_dn - wdn.grad).abs().max() < tol(wdn.grad)
    starved = (torch.bincount(idx.reshape(-1), minlength=experts) == 0).nonzero().flatten().tolist()
    for e in starved:                                              # experts without tokens: exactly zero gradient
        assert float(g_gu[e].abs().max()) == 0.0 and float(g_dn[e].abs().max()) == 0.0
