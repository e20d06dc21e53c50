import pytest
import torch

from arctic_platform_b200.utils.action_masks import ActionMasks, masked_logprobs


def _dense_ref(hidden, weight, labels, allowed, it):
    logits = (hidden.float() @ weight.float().t()) * it
    logits = logits.masked_fill(~allowed, float("-inf"))
    lse = torch.logsumexp(logits, -1)
    lp = logits.gather(-1, labels[:, None]).squeeze(-1) - lse
    p = torch.softmax(logits, -1)
    ent = lse - (p * logits.masked_fill(~allowed, 0.0)).sum(-1)
    return lp, ent


def test_action_masks_match_dense_masking_and_gradients():
    g = torch.Generator().manual_seed(0)
    N, H, V = 9, 16, 50
    hidden = torch.randn(N, H, generator=g, requires_grad=True)
    weight = torch.randn(V, H, generator=g, requires_grad=True)
    labels = torch.randint(0, V, (N,), generator=g)
    cons = {1: ("allow", [3, 7, int(labels[1])]), 4: ("deny", [0, 1, 2, 5]), 6: ("allow", [int(labels[6])]),
            7: ("deny", [int(labels[7])])}
    masks = ActionMasks.from_constraints(N, cons)
    allowed = masks.dense_allowed(V)
    assert allowed[0].all() and allowed[1].sum() == 3 and allowed[4].sum() == V - 4
    lp, ent = masked_logprobs(hidden, weight, labels, masks, 0.7)
    ref_lp, ref_ent = _dense_ref(hidden, weight, labels, allowed, 0.7)
    fin = torch.isfinite(ref_lp)
    assert not fin[7] and lp[7] == float("-inf")                  # the label itself is denied
    assert torch.allclose(lp[fin], ref_lp[fin], atol=1e-4) and torch.allclose(ent, ref_ent, atol=1e-4)
    assert abs(float(ent[6])) < 1e-5                               # single legal token: zero entropy
    (lp[fin].sum() + 0.3 * ent.sum()).backward()
    gh, gw = hidden.grad.clone(), weight.grad.clone()
    hidden.grad = weight.grad = None
    (ref_lp[fin].sum() + 0.3 * ref_ent.sum()).backward()
    assert torch.allclose(gh, hidden.grad, atol=1e-4) and torch.allclose(gw, weight.grad, atol=1e-4)
    # validation of sampled tokens, packing and sharding
    ok = labels.clone()
    masks.validate_sampled(torch.where(torch.arange(N) == 7, (labels + 1) % V, ok))
    with pytest.raises(ValueError, match="rows \\[7\\]"):
        masks.validate_sampled(ok)
    with pytest.raises(ValueError):
        ActionMasks.from_constraints(3, {0: ("allow", [])})
    both = ActionMasks.pack([masks, masks])
    assert both.num_rows == 2 * N and torch.equal(both.dense_allowed(V), torch.cat([allowed, allowed]))
    sel = both.select(torch.tensor([4, 9 + 1, 0]))
    assert torch.equal(sel.dense_allowed(V), torch.stack([allowed[4], allowed[1], allowed[0]]))
    owned = torch.zeros(2 * N, dtype=torch.bool)
    owned[N:] = True
    assert torch.equal(both.select(owned).dense_allowed(V), allowed)


def test_activation_offload_passthrough_on_cpu():
    from arctic_platform_b200.utils.activation_offload import ActivationOffload
    x = torch.randn(64, 64, requires_grad=True)
    with ActivationOffload(min_bytes=1) as off:
        y = (x @ x).relu().sum()
    y.backward()
    assert off.stats.offloaded_tensors == 0 and off.stats.skipped_tensors > 0 and x.grad is not None


@pytest.mark.gpu
def test_activation_offload_round_trip_and_pool_reuse():
    from arctic_platform_b200.utils.activation_offload import ActivationOffload, PinnedPool
    dev = torch.device("cuda")
    torch.manual_seed(0)
    ws = [torch.randn(512, 512, device=dev, requires_grad=True) for _ in range(6)]
    x = torch.randn(1024, 512, device=dev)

    def run(ctx):
        h = x
        with ctx:
            for w in ws:
                h = torch.tanh(h @ w) * 0.5
            loss = h.square().mean()
        loss.backward()
        g = [w.grad.clone() for w in ws]
        for w in ws:
            w.grad = None
        return float(loss.detach()), g

    import contextlib
    ref_loss, ref_g = run(contextlib.nullcontext())
    off = ActivationOffload(min_bytes=1 << 16, keep_last=2, prefetch=2)
    loss, g = run(off)
    assert loss == ref_loss and all(torch.equal(a, b) for a, b in zip(g, ref_g))
    st = off.stats
    assert st.offloaded_tensors >= 6 and st.kept_tensors >= 1 and st.offloaded_bytes >= 6 * 1024 * 512 * 4
    assert st.prefetch_hits >= 1
    off.release()
    allocs = st.pool_allocations
    off2 = ActivationOffload(min_bytes=1 << 16, keep_last=2, prefetch=2, pool=off.pool)
    loss2, g2 = run(off2)
    assert loss2 == ref_loss and all(torch.equal(a, b) for a, b in zip(g2, ref_g))
    assert off2.stats.pool_allocations == 0 and off2.stats.pool_reuses >= allocs - 1   # steady state: no new pinned memory
    off2.release()
