"""JSON batch descriptions -> forward-backward tensors (cortex_client/dss_client/batch_spec.py)."""
import pytest
import torch

from arctic_platform_b200 import wire
from cortex_client.dss_client import batch_spec as bs


class FakeTokenizer:
    """Pads on the right to ``max_length`` with id 0; one token per character."""

    def __init__(self):
        self.calls = []

    def __call__(self, texts, **kw):
        self.calls.append((list(texts), kw))
        n = kw.get("max_length") or max(len(t) for t in texts)
        ids = torch.zeros(len(texts), n, dtype=torch.long)
        mask = torch.zeros(len(texts), n, dtype=torch.long)
        for i, t in enumerate(texts):
            m = min(len(t), n)
            ids[i, :m] = torch.tensor([ord(c) for c in t[:m]])
            mask[i, :m] = 1
        return {"input_ids": ids, "attention_mask": mask}


def test_direct_ids_default_next_token_labels():
    out = bs.build_forward_backward_kwargs({"input_ids": [[5, 6, 7, 8], [1, 2, 3, 4]]})
    assert set(out) == {"input_ids", "labels"}
    assert out["labels"].tolist() == [[6, 7, 8, -100], [2, 3, 4, -100]]
    assert out["input_ids"].dtype == torch.int64 and out["input_ids"].is_contiguous()


def test_padding_is_masked_out_of_the_targets():
    spec = {"input_ids": [[5, 6, 7, 0]], "attention_mask": {"data": [[1, 1, 1, 0]]}, "include_attention_mask": True,
            "position_ids": True, "ignore_index": -1}
    out = bs.build_forward_backward_kwargs(spec)
    assert out["labels"].tolist() == [[6, 7, -1, -1]]              # the padded target and the last column
    assert out["attention_mask"].tolist() == [[1, 1, 1, 0]]
    assert out["position_ids"].tolist() == [[0, 1, 2, 3]]
    out = bs.build_forward_backward_kwargs({**spec, "mask_padding": False})
    assert out["labels"].tolist() == [[6, 7, 0, -1]]
    out = bs.build_forward_backward_kwargs({**spec, "labels": {"strategy": "input_ids", "ignore_index": -7}})
    assert out["labels"].tolist() == [[5, 6, 7, -7]]
    out = bs.build_forward_backward_kwargs({**spec, "labels": "none"})
    assert "labels" not in out


def test_attention_mask_switch_without_data_is_all_ones():
    out = bs.build_forward_backward_kwargs({"input_ids": [[1, 2, 3]], "attention_mask": True, "labels": [[2, 3, -100]]})
    assert out["attention_mask"].tolist() == [[1, 1, 1]] and out["labels"].tolist() == [[2, 3, -100]]
    out = bs.build_forward_backward_kwargs({"input_ids": [[1, 2, 3]], "attention_mask": False})
    assert "attention_mask" not in out


def test_texts_are_tokenised_and_repeated():
    tok = FakeTokenizer()
    seen = []

    def loader(spec):
        seen.append(spec)
        return tok

    out = bs.build_forward_backward_kwargs({"texts": ["ab", "cde"], "batch_size": 3, "tokenizer": {"model_name": "m"},
                                            "max_length": 4, "include_attention_mask": True}, tokenizer_loader=loader)
    assert seen == [{"model_name": "m"}]
    texts, kw = tok.calls[0]
    assert texts == ["ab", "cde", "ab"] and kw["padding"] == "max_length" and kw["max_length"] == 4 and kw["truncation"] is True
    assert out["input_ids"].shape == (3, 4)
    assert out["labels"][0].tolist() == [ord("b"), -100, -100, -100]
    assert out["labels"][1].tolist() == [ord("d"), ord("e"), -100, -100]
    assert out["attention_mask"][0].tolist() == [1, 1, 0, 0]


def test_kwargs_form_tensorises_lists_and_typed_objects():
    out = bs.build_forward_backward_kwargs({"kwargs": {"input_ids": [[1, 2]], "w": {"data": [0.5], "dtype": "bf16"},
                                                       "flag": True, "name": "x"}})
    assert out["input_ids"].dtype == torch.int64 and out["w"].dtype == torch.bfloat16
    assert out["flag"] is True and out["name"] == "x"


@pytest.mark.parametrize("spec,needle", [
    ({"input_ids": [1, 2, 3]}, "shape"),
    ({"input_ids": [[1, 2]], "attention_mask": [[1, 1, 1]]}, "attention_mask"),
    ({"input_ids": [[1, 2]], "labels": "previous_token"}, "labels"),
    ({"input_ids": [[1, 2]], "position_ids": "sinusoidal"}, "position_ids"),
    ({"input_ids": {"data": [[1]], "dtype": "complex"}}, "dtype"),
    ({"input_ids": {"dtype": "long"}}, "data"),
    ({"input_ids": [[1, 2]], "mask_padding": "yes"}, "mask_padding"),
    ({"texts": ["a"], "tokenizer": "m", "max_length": 0}, "max_length"),
    ({"texts": [], "tokenizer": "m", "max_length": 4}, "texts"),
    ({"texts": ["a"], "max_length": 4}, "tokenizer"),
    ({"kwargs": [1]}, "kwargs"),
])
def test_bad_descriptions_name_the_key(spec, needle):
    with pytest.raises(bs.BatchSpecError, match=needle):
        bs.build_forward_backward_kwargs(spec, tokenizer_loader=lambda s: FakeTokenizer())


def test_payload_is_one_frame_with_response_options():
    raw = bs.build_forward_backward_payload({"payload": {"input_ids": [[1, 2, 3]], "args": []}})
    obj = wire.loads(raw)
    assert obj["args"] == [] and obj["kwargs"]["labels"].tolist() == [[2, 3, -100]]
    assert wire.read_metadata(raw)["response_options"] == {"format": "dssst1", "delivery": "chunked"}
    assert wire.loads(bs.build_forward_backward_payload({"input_ids": [[4, 5]]}))["kwargs"]["input_ids"].tolist() == [[4, 5]]
    with pytest.raises(bs.BatchSpecError):
        bs.serialize_forward_backward_args([1], {})
    with pytest.raises(bs.BatchSpecError):
        bs.build_forward_backward_payload({"payload": {"input_ids": [[1]], "args": {"a": 1}}})
