"""Forest-cascade decode attention (shared header / prompt nodes on tensor-core tiles + per-sequence pass + merge)
against a dense fp32 oracle, and the rollout engine's prefix-tree discovery end to end."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

PAGE = 16


def _scratch(B, Hq, D, splits):
    f32 = dict(device="cuda", dtype=torch.float32)
    return ([torch.empty((B, Hq, splits, D), **f32) for _ in range(4)],
            [torch.empty((B, Hq, splits, 2), **f32) for _ in range(4)])


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (16, 8), (8, 8)])
def test_three_level_forest_matches_dense_attention(Hq, Hkv):
    """Headers shared by several prompts, prompts shared by their rollouts, private tails; one sequence without a
    header, one prompt node whose slots are not consecutive, and a header with more sequences than one tile holds."""
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.ops import forest_attention as fa
    D, splits = 128, 4
    R = Hq // Hkv
    max_rows = 128 // R
    B = max_rows + 12                      # the first header spans more sequences than one tile
    g = torch.Generator(device="cuda").manual_seed(3)
    num_pages = 400
    kc = torch.randn((num_pages, Hkv, PAGE, D), generator=g, device="cuda").to(torch.bfloat16)
    vc = torch.randn((num_pages, Hkv, PAGE, D), generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn((B, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    rng = np.random.default_rng(0)
    perm = rng.permutation(num_pages).astype(np.int32)
    nxt = [0]

    def take(n):
        out = perm[nxt[0]:nxt[0] + n]
        nxt[0] += n
        return out

    nodes, ctx = [], [[] for _ in range(B)]
    hdr_a, hdr_b = take(9), take(5)                                       # 144 and 80 tokens
    slots_a = list(range(0, max_rows + 4))
    slots_b = list(range(max_rows + 4, B - 1))                            # the last slot has no header at all
    nodes.append(fa.ForestNode(0, slots_a, hdr_a, 144))
    nodes.append(fa.ForestNode(0, slots_b, hdr_b, 80))
    for s in slots_a:
        ctx[s].append((hdr_a, 144))
    for s in slots_b:
        ctx[s].append((hdr_b, 80))
    # prompt nodes: groups of 4 slots; one group deliberately scattered
    groups = [list(range(i, min(i + 4, B))) for i in range(0, B, 4)]
    groups[1], groups[2] = [4, 5, 8, 9], [6, 7, 10, 11]
    for grp in groups:
        n_tok = int(rng.integers(1, 6)) * PAGE
        pg = take(n_tok // PAGE)
        nodes.append(fa.ForestNode(1, grp, pg, n_tok))
        for s in grp:
            ctx[s].append((pg, n_tok))
    max_pages = 16
    priv = np.zeros((B, max_pages), dtype=np.int32)
    plen = np.zeros(B, dtype=np.int32)
    for s in range(B):
        n = int(rng.integers(1, 40))
        pg = take((n + PAGE - 1) // PAGE)
        priv[s, :len(pg)] = pg
        plen[s] = n
        ctx[s].append((pg, n))
    forest = fa.build_forest_tables(nodes, B, max_pages, max_rows, "cuda")
    assert forest.n_levels == 2 and forest.n_nodes >= len(nodes) + 2       # scattered / oversized nodes take extra rows
    i32 = dict(device="cuda", dtype=torch.int32)
    po, pml = _scratch(B, Hq, D, splits)
    for buf in po + pml:
        buf.fill_(float("nan"))                                            # stale partials must never be merged
    out = fa.forest_decode_attention(q, kc, vc, forest, torch.arange(B, **i32), torch.ones(B, **i32),
                                     torch.from_numpy(priv).cuda(), torch.from_numpy(plen).cuda(), po, pml, splits, 1)
    _lib.check_status("forest")
    ref = fa.forest_decode_reference(q, kc, vc, ctx)
    assert torch.isfinite(out.float()).all()
    assert (out.float() - ref).abs().max().item() < 2e-2


def test_engine_discovers_shared_headers_and_samples_the_same_distribution():
    """Prompts that start with the same tokens are stored and attended through one header node.  Greedy generation with
    the forest equals greedy generation with plain per-sequence decoding, and the reported log-probs match a
    teacher-forced scoring pass."""
    from arctic_platform_b200.engine.sampler import SamplerEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    from arctic_platform_b200.ops import _lib
    cfg = PRESETS["qwen3-tiny-d128"]
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=5)
    g = torch.Generator().manual_seed(1)
    header = torch.randint(1, cfg.vocab_size, (100,), generator=g).tolist()      # 6 full pages in common
    prompts = [header + torch.randint(1, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 40, 7)]
    prompts.append(torch.randint(1, cfg.vocab_size, (57,), generator=g).tolist())  # shares nothing
    sp = {"n": 3, "temperature": 0.0, "max_tokens": 12, "ignore_eos": True}
    outs = {}
    for cascade in (True, False):
        eng = SamplerEngine(cfg, "cuda", model=model, kv_cache_tokens=1 << 14, max_batch=16, max_seq_len=512,
                            cascade=cascade, use_cuda_graph=False)
        if cascade:
            runs = eng._plan_runs([np.asarray(p, dtype=np.int64) for p in prompts])
            assert sorted(map(tuple, (r[0] for r in runs))) == [(0, 1, 2), (3,)]
            assert dict((tuple(r[0]), r[1]) for r in runs)[(0, 1, 2)] == 96      # page-aligned part of the 100 tokens
        outs[cascade] = eng.generate(prompts, sp)
        if cascade:
            assert eng.n_levels == 2 and eng.forest_stats["shared_tokens"] > 0
        _lib.check_status("forest engine")
    for a, b in zip(outs[True], outs[False]):
        assert a["prompt_index"] == b["prompt_index"] and a["token_ids"] == b["token_ids"]
        assert a["logprobs"] == pytest.approx(b["logprobs"], abs=5e-2)
