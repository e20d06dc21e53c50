"""The reference's log-prob entry points on this build's single implementation: same numbers as a dense softmax,
gradients included."""
import pytest
import torch

from arctic_platform_b200.common.utils import tiled_logits as tl
from arctic_platform_b200.testing_utils import make_tied_lm_head_model


def _dense(h, w, y, temperature):
    logits = (h.float() @ w.float().t()) / temperature
    ls = torch.log_softmax(logits, -1)
    return ls.gather(-1, y.unsqueeze(-1)).squeeze(-1), -(ls.exp() * ls).sum(-1)


def test_chunk_rows_budget():
    assert tl.logits_chunk_rows(151936, 4.0) == (4 * 2 ** 30) // (151936 * 4)
    assert tl.logits_chunk_rows(10 ** 12, 0.001) == 1 and tl.logits_chunk_rows(1000, 1.0, bytes_per_elem=2) == 2 ** 30 // 2000


@pytest.mark.parametrize("entry", ["tiled", "chunked", "function"])
def test_entry_points_match_a_dense_softmax(entry):
    torch.manual_seed(0)
    model = make_tied_lm_head_model(16, 50)
    h = torch.randn(3, 7, 16, requires_grad=True)
    y = torch.randint(0, 50, (3, 7))
    T = 0.7
    if entry == "tiled":
        lp, ent = tl.tiled_logprobs_entropy_from_hidden(model, h, y, temperature=T)
    elif entry == "chunked":
        lp, ent = tl.chunked_logprobs_entropy_from_hidden(model, h, y, temperature=T, peak_mem_gib=1e-6)   # 1-row chunks
    else:
        lp, ent = tl.TiledLogProbEntropy.apply(h, model.output_weight, y, T, True, 1e-6)
    want_lp, want_ent = _dense(h.reshape(-1, 16), model.output_weight, y.reshape(-1), T)
    torch.testing.assert_close(lp.reshape(-1), want_lp, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ent.reshape(-1), want_ent, rtol=1e-5, atol=1e-5)
    assert lp.shape == (3, 7)
    (lp.sum() + 0.1 * ent.sum()).backward()
    h2 = h.detach().clone().requires_grad_(True)
    a, b = _dense(h2.reshape(-1, 16), model.output_weight, y.reshape(-1), T)
    (a.sum() + 0.1 * b.sum()).backward()
    torch.testing.assert_close(h.grad, h2.grad, rtol=1e-4, atol=1e-5)


def test_per_row_temperature_no_entropy_and_full_logits():
    torch.manual_seed(1)
    model = make_tied_lm_head_model(8, 20)
    h, y = torch.randn(5, 8), torch.randint(0, 20, (5,))
    temps = torch.tensor([0.5, 1.0, 2.0, 1.0, 0.25])
    lp, ent = tl.tiled_logprobs_entropy_from_hidden(model, h, y, temperature=temps, calculate_entropy=False)
    assert ent is None
    for i in range(5):
        want, _ = _dense(h[i:i + 1], model.output_weight, y[i:i + 1], float(temps[i]))
        torch.testing.assert_close(lp[i:i + 1], want, rtol=1e-5, atol=1e-5)
    logits = tl.lm_head_logits(model, h, temperature=2.0, logits_compute_in_fp32=True)
    torch.testing.assert_close(logits, (h @ model.output_weight.t()) / 2.0)
    a, b = tl.logprobs_entropy_from_flat_logits(logits, y)
    want, want_e = _dense(h, model.output_weight, y, 2.0)
    torch.testing.assert_close(a, want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(b, want_e, rtol=1e-5, atol=1e-5)
    with pytest.raises(AttributeError):
        tl.lm_head_logits(object(), h)
