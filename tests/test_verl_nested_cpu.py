"""Padding-free (nested-jagged) verl batches <-> the platform's dense wire batch."""
import pytest
import torch

from arctic_platform_b200.integrations.verl import nested as nj
from arctic_platform_b200.integrations.verl.adapter import prepare_padded_batch


def _batch():
    prompts = [[11, 12, 13], [21], [31, 32]]
    responses = [[14, 15], [22, 23, 24, 25], [33]]
    rows = [torch.tensor(p + r) for p, r in zip(prompts, responses)]
    nt = lambda xs: torch.nested.nested_tensor([torch.tensor(x) for x in xs], layout=torch.jagged)
    return {"input_ids": torch.nested.nested_tensor(rows, layout=torch.jagged), "prompts": nt(prompts),
            "responses": nt(responses)}, prompts, responses


def _loop_reference(prompts, responses, P, R, pad):
    out = []
    for p, r in zip(prompts, responses):
        out.append([pad] * (P - len(p)) + p + r + [pad] * (R - len(r)))
    return torch.tensor(out)


def test_nested_batch_becomes_left_padded_prompt_right_padded_response():
    data, prompts, responses = _batch()
    out, P, R = prepare_padded_batch(data, pad_token_id=0)
    assert (P, R) == (3, 4)
    assert torch.equal(out["input_ids"], _loop_reference(prompts, responses, 3, 4, 0))
    assert out["attention_mask"].tolist() == [[1, 1, 1, 1, 1, 0, 0], [0, 0, 1, 1, 1, 1, 1], [0, 1, 1, 1, 0, 0, 0]]
    data.update(max_prompt_len=5, max_response_len=6)
    out, P, R = prepare_padded_batch(data, pad_token_id=9)
    assert (P, R) == (5, 6) and torch.equal(out["input_ids"], _loop_reference(prompts, responses, 5, 6, 9))
    # position ids travel when asked for
    data["position_ids"] = torch.nested.nested_tensor([torch.arange(5), torch.arange(5), torch.arange(3)], layout=torch.jagged)
    out, _, _ = prepare_padded_batch(data, pad_token_id=0, drop_position_ids=False)
    assert out["position_ids"][1].tolist() == [0, 0, 0, 0, 0, 1, 2, 3, 4, 0, 0]
    with pytest.raises(ValueError, match="longer"):
        nj.nested_to_padded(data["input_ids"], torch.tensor([3, 1, 2]), torch.tensor([2, 4, 1]), 2, 4)
    with pytest.raises(ValueError, match="sum"):
        nj.nested_to_padded(data["input_ids"], torch.tensor([3, 1, 2]), torch.tensor([2, 4, 2]), 3, 4)


def test_dense_prompts_with_flat_values():
    # the other layout verl hands over: flat values next to dense (padded) prompts / responses and their mask
    prompts = torch.tensor([[0, 11, 12], [21, 22, 23]])
    responses = torch.tensor([[13, 0], [24, 25]])
    mask = torch.tensor([[0, 1, 1, 1, 0], [1, 1, 1, 1, 1]])
    flat = torch.tensor([11, 12, 13, 21, 22, 23, 24, 25])
    out, P, R = prepare_padded_batch({"input_ids": flat, "prompts": prompts, "responses": responses,
                                      "attention_mask": mask}, pad_token_id=0)
    assert (P, R) == (3, 2) and out["input_ids"].tolist() == [[0, 11, 12, 13, 0], [21, 22, 23, 24, 25]]
    assert out["attention_mask"] is mask


def test_response_grids_return_as_nested_rows_in_either_alignment():
    data, prompts, responses = _batch()
    grid = torch.tensor([[1.0, 2.0, 0, 0], [3.0, 4.0, 5.0, 6.0], [7.0, 0, 0, 0]])
    nxt = nj.make_njt(data, grid)                                     # on the predicting token
    assert [r.tolist() for r in nxt.unbind()] == [[0, 0, 1, 2, 0], [3, 4, 5, 6, 0], [0, 7, 0]]
    own = nj.make_njt(data, grid, align="response")                  # on the response token itself
    assert [r.tolist() for r in own.unbind()] == [[0, 0, 0, 1, 2], [0, 3, 4, 5, 6], [0, 0, 7]]
    assert torch.equal(nxt.offsets(), data["input_ids"].offsets())
    shifted = nj.shift_nested_left(own)
    assert torch.equal(shifted.values(), nxt.values()) and torch.equal(shifted.offsets(), nxt.offsets())
    # a full [B, P + R] grid is cut to its response part first
    full = torch.cat([torch.full((3, 3), 99.0), grid], 1)
    assert torch.equal(nj.make_njt(data, full).values(), nxt.values())
    with pytest.raises(ValueError):
        nj.response_grid_to_nested(grid[:, :2], *nj.prompt_response_lengths(data)[:2])
    with pytest.raises(ValueError):
        nj.response_grid_to_nested(grid, torch.tensor([0, 1, 2]), torch.tensor([2, 4, 1]))


def test_round_trip_matches_a_row_loop_on_random_shapes():
    g = torch.Generator().manual_seed(0)
    for _ in range(5):
        B = int(torch.randint(1, 9, (1,), generator=g))
        pl = torch.randint(1, 7, (B,), generator=g)
        rl = torch.randint(1, 9, (B,), generator=g)
        rows = [torch.randint(1, 100, (int(p + r),), generator=g) for p, r in zip(pl, rl)]
        ids = torch.nested.nested_tensor(rows, layout=torch.jagged)
        P, R = int(pl.max()), int(rl.max())
        dense = nj.nested_to_padded(ids, pl, rl, P, R, 0)
        grid = torch.rand(B, R, generator=g)
        out = nj.response_grid_to_nested(grid, pl, rl, "predict_next")
        for b, row in enumerate(rows):
            p, r = int(pl[b]), int(rl[b])
            assert torch.equal(dense[b, P - p:P + r], row) and dense[b, :P - p].sum() == 0 and dense[b, P + r:].sum() == 0
            got = out.unbind()[b]
            assert torch.equal(got[p - 1:p - 1 + r], grid[b, :r]) and got[:p - 1].sum() == 0 and got[p - 1 + r:].sum() == 0


def test_metrics_become_lists_of_floats():
    got = nj.normalize_backend_metrics({"a": 1, "b": torch.tensor(2.5), "c": torch.tensor([1.0, 2.0]), "d": [1, 2.5],
                                        "e": "text", "f": True, "g": None, "h": [1, "x"]})
    assert got == {"a": [1.0], "b": [2.5], "c": [1.0, 2.0], "d": [1.0, 2.5]}
