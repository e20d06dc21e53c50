"""Checked mode on the GPU: the validators accept the tables the engines really build (no false alarms), and a table
corrupted on the host is refused before anything is launched with it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def checked_on():
    from arctic_platform_b200.utils import checked
    checked.force(True)
    yield checked
    checked.force(None)


def test_sampler_with_forest_runs_clean_in_checked_mode(checked_on):
    from arctic_platform_b200.engine.sampler import SamplerEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.ops import _lib
    cfg = PRESETS["qwen3-tiny-d128"]
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=5)
    g = torch.Generator().manual_seed(1)
    header = torch.randint(1, cfg.vocab_size, (100,), generator=g).tolist()
    prompts = [header + torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 40)]
    sp = {"n": 3, "temperature": 0.0, "max_tokens": 8, "ignore_eos": True}
    outs = {}
    for graph in (False, True):
        eng = SamplerEngine(cfg, "cuda", model=model, kv_cache_tokens=1 << 14, max_batch=16, max_seq_len=512,
                            cascade=True, use_cuda_graph=graph)
        outs[graph] = eng.generate(prompts, sp)
        _lib.check_status("checked generate")
    assert [o["token_ids"] for o in outs[False]] == [o["token_ids"] for o in outs[True]]


def test_forest_op_refuses_a_corrupted_table_before_launching(checked_on):
    from arctic_platform_b200.ops.forest_attention import ForestNode, build_forest_tables, forest_decode_attention
    from arctic_platform_b200.ops import _lib
    B, Hq, Hkv, D, num_pages, max_pages = 8, 8, 2, 128, 32, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn(num_pages, Hkv, 16, D, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(num_pages, Hkv, 16, D, device="cuda", dtype=torch.bfloat16, generator=g)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    forest = build_forest_tables([ForestNode(0, range(0, B), np.arange(0, 4, dtype=np.int32), 64)], B, max_pages, 128, "cuda")
    priv_table = torch.arange(4, 4 + B, device="cuda", dtype=torch.int32).view(B, 1).repeat(1, max_pages)
    priv_len = torch.full((B,), 9, device="cuda", dtype=torch.int32)
    start = torch.arange(B, device="cuda", dtype=torch.int32)
    active = torch.ones(B, device="cuda", dtype=torch.int32)
    splits = 2
    part_o = [torch.zeros(B, Hq, splits, D, device="cuda") for _ in range(2)]
    part_ml = [torch.zeros(B, Hq, splits, 2, device="cuda") for _ in range(2)]
    out = forest_decode_attention(q, kc, vc, forest, start, active, priv_table, priv_len, part_o, part_ml, splits, splits)
    _lib.check_status("forest checked")
    assert torch.isfinite(out.float()).all()
    before = _lib.launch_count()
    priv_table[3, 0] = num_pages + 5                                   # a page id outside the cache
    with pytest.raises(checked_on.TableError, match=r"priv_table\[3, 0\]"):
        forest_decode_attention(q, kc, vc, forest, start, active, priv_table, priv_len, part_o, part_ml, splits, splits)
    assert _lib.launch_count() == before                               # nothing ran with the bad table
    priv_table[3, 0] = 7
    forest.kv_len[0] = 16 * max_pages + 1                              # a node longer than its page list
    with pytest.raises(checked_on.TableError, match="pages"):
        forest_decode_attention(q, kc, vc, forest, start, active, priv_table, priv_len, part_o, part_ml, splits, splits)
    assert _lib.launch_count() == before
