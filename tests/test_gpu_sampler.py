"""Rollout engine: paged decode (plain and forest-cascade) against full-sequence scoring with the same weights."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(cascade, graph, max_batch=16, **kw):
    from arctic_platform_b200.engine.sampler import SamplerEngine
    from arctic_platform_b200.models.config import PRESETS
    from arctic_platform_b200.models.decoder import DecoderLM
    cfg = PRESETS["qwen3-tiny-d128"]
    model = DecoderLM(cfg, "cuda", torch.bfloat16).init_weights(seed=5, std=0.05)
    eng = SamplerEngine(cfg, "cuda", model=model, kv_cache_tokens=1 << 14, max_batch=max_batch, max_seq_len=512,
                        cascade=cascade, sync_interval=4, use_cuda_graph=graph, **kw)
    return cfg, model, eng


@pytest.mark.parametrize("cascade,graph,kw", [
    (False, False, {"split_k": False}), (True, False, {"prefix_on_tensor_cores": False, "split_k": False}),
    (True, False, {}), (True, True, {})])
def test_generate_logprobs_match_scoring(cascade, graph, kw):
    """Greedy rollouts: every reported log-prob must equal the model's own log-prob of that token when the
    whole sequence is scored in one packed forward pass, and the token must be the arg-max there."""
    from arctic_platform_b200.models.decoder import token_logprobs
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl.zorro_train.layout import build_packed_batch
    cfg, model, eng = _engine(cascade, graph, **kw)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, cfg.vocab_size, size=n).tolist() for n in (37, 64, 5)]
    outs = eng.generate(prompts, {"n": 3, "temperature": 0.0, "max_tokens": 21})
    _lib.check_status("generate")
    assert len(outs) == 9
    P, R = 64, 21
    ids = torch.zeros((9, P + R), dtype=torch.int64)
    mask = torch.zeros_like(ids)
    for i, o in enumerate(outs):
        p = prompts[o["prompt_index"]]
        assert o["prompt_len"] == len(p) and len(o["token_ids"]) == R and o["finish_reason"] == "length"
        ids[i, P - len(p):P] = torch.tensor(p)
        mask[i, P - len(p):P] = 1
        ids[i, P:] = torch.tensor(o["token_ids"])
        mask[i, P:] = 1
    # greedy rollouts of one prompt are identical
    assert outs[0]["token_ids"] == outs[1]["token_ids"] == outs[2]["token_ids"]
    pb = build_packed_batch(ids, mask, R, dedup=True).to("cuda")
    with torch.no_grad():
        lp, _ = token_logprobs(model, pb, 1.0)
    got = torch.tensor([o["logprobs"] for o in outs]).reshape(-1)
    ref = pb.scatter_to_grid(lp).cpu().reshape(-1)
    assert (got - ref).abs().max() < 0.08, (got - ref).abs().max()
    assert (got - ref).abs().mean() < 0.01


def test_sampling_is_seeded_and_diverse():
    cfg, model, eng = _engine(True, True, max_batch=32)
    prompt = list(range(10, 60))
    a = eng.generate([prompt], {"n": 8, "temperature": 1.0, "max_tokens": 12, "seed": 7})
    b = eng.generate([prompt], {"n": 8, "temperature": 1.0, "max_tokens": 12, "seed": 7})
    assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]
    assert len({tuple(o["token_ids"]) for o in a}) > 1
    assert eng.pages.free_count() == eng.num_pages


def test_more_sequences_than_slots_and_stop_tokens():
    cfg, model, eng = _engine(True, False, max_batch=8)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(1, cfg.vocab_size, size=20 + i).tolist() for i in range(7)]
    outs = eng.generate(prompts, {"n": 4, "temperature": 0.0, "max_tokens": 9})
    assert len(outs) == 28 and all(len(o["token_ids"]) == 9 for o in outs)
    first = outs[0]["token_ids"]
    outs2 = eng.generate(prompts[:1], {"n": 1, "temperature": 0.0, "max_tokens": 9, "stop_token_ids": [first[3]]})
    assert outs2[0]["finish_reason"] == "stop" and outs2[0]["token_ids"] == first[:first.index(first[3]) + 1]


@pytest.mark.parametrize("Hq,Hkv,nq,splits", [(32, 8, 1, 1), (32, 8, 1, 3), (32, 8, 3, 2), (16, 8, 5, 1), (8, 8, 1, 2),
                                              (32, 2, 2, 1)])
def test_paged_decode_mma_kernel_matches_reference_and_scalar_kernel(Hq, Hkv, nq, splits):
    """The tensor-core (m16n8k16) paged decode pass against a dense fp32 reference and against the scalar kernel:
    ragged lengths (including an empty range), shuffled pages, query groups of several rows, KV splits."""
    import ctypes
    import math
    from arctic_platform_b200.engine.sampler import _fn
    from arctic_platform_b200.ops import _lib
    dev, D, PAGE = "cuda", 128, 16
    g = torch.Generator(device=dev).manual_seed(Hq * 100 + nq * 10 + splits)
    lens = [0, 1, 15, 16, 17, 333, 1024, 700]
    G = len(lens)
    max_pages = 80
    num_pages = G * max_pages + 7
    kc = torch.randn(num_pages, Hkv, PAGE, D, device=dev, generator=g).bfloat16()
    vc = torch.randn(num_pages, Hkv, PAGE, D, device=dev, generator=g).bfloat16()
    perm = torch.randperm(num_pages, device=dev, generator=g)[:G * max_pages].to(torch.int32).view(G, max_pages)
    Bq = G * nq
    q = torch.randn(Bq, Hq, D, device=dev, generator=g).bfloat16()
    q_start = (torch.arange(G, device=dev, dtype=torch.int32) * nq).contiguous()
    q_count = torch.full((G,), nq, device=dev, dtype=torch.int32)
    kv_len = torch.tensor(lens, device=dev, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)

    def run(scalar):
        _lib.cuda_lib().apb_decode_use_scalar(int(scalar))
        po = torch.zeros(Bq, Hq, splits, D, device=dev, dtype=torch.float32)
        pml = torch.zeros(Bq, Hq, splits, 2, device=dev, dtype=torch.float32)
        _lib.check(_fn("dec")(_lib.ptr(q), _lib.ptr(q_start), _lib.ptr(q_count), _lib.ptr(perm), max_pages,
                              _lib.ptr(kv_len), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(po), _lib.ptr(pml), G, Hq, Hkv, D,
                              splits, scale, _lib.stream_ptr()), "paged_decode")
        out = torch.empty(Bq, Hq, D, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(Bq, Hq, device=dev, dtype=torch.float32)
        o_ptrs = (ctypes.c_void_p * 4)(po.data_ptr(), 0, 0, 0)
        ml_ptrs = (ctypes.c_void_p * 4)(pml.data_ptr(), 0, 0, 0)
        sp = (ctypes.c_int * 4)(splits, 0, 0, 0)
        _lib.check(_fn("merge")(o_ptrs, ml_ptrs, sp, 1, None, _lib.ptr(out), _lib.ptr(lse), Bq, Hq, D, _lib.stream_ptr()), "merge")
        _lib.check_status("paged decode")
        return out.float(), lse

    try:
        out_mma, lse_mma = run(False)
        out_sc, lse_sc = run(True) if Hq // Hkv in (1, 2, 4, 8) and nq <= 16 else (None, None)
    finally:
        _lib.cuda_lib().apb_decode_use_scalar(0)
    R = Hq // Hkv
    for gi, L in enumerate(lens):
        if L == 0:
            continue
        n_pg = (L + PAGE - 1) // PAGE
        pg = perm[gi, :n_pg].long()
        K = kc[pg].permute(1, 0, 2, 3).reshape(Hkv, n_pg * PAGE, D)[:, :L].float()
        V = vc[pg].permute(1, 0, 2, 3).reshape(Hkv, n_pg * PAGE, D)[:, :L].float()
        for qi in range(nq):
            row = gi * nq + qi
            qq = q[row].float().view(Hkv, R, D)
            s = torch.einsum("hrd,hld->hrl", qq, K) * scale
            ref = torch.einsum("hrl,hld->hrd", torch.softmax(s, -1), V).reshape(Hq, D)
            ref_lse = torch.logsumexp(s, -1).reshape(Hq)
            assert (out_mma[row] - ref).abs().max() < 0.03, (gi, L, float((out_mma[row] - ref).abs().max()))
            assert (lse_mma[row] - ref_lse).abs().max() < 0.02
            if out_sc is not None:
                assert (out_mma[row] - out_sc[row]).abs().max() < 0.03


def test_top_k_top_p_filter_kernel_against_sorted_reference():
    """Cut-offs of the radix-select kernel equal the sort-based definition, sampled tokens stay inside the allowed
    set, and the reported log-prob is the unfiltered one."""
    import ctypes
    from arctic_platform_b200.engine.reference_sampler import filter_logits
    from arctic_platform_b200.engine.sampler import _fn
    from arctic_platform_b200.ops import _lib
    dev = "cuda"
    B, V = 12, 151936
    g = torch.Generator(device=dev).manual_seed(3)
    logits = (torch.randn(B, V, device=dev, generator=g) * 3.0).float()
    temp = torch.tensor([1.0, 0.7, 1.3, 1.0, 1.0, 0.5, 1.0, 2.0, 1.0, 1.0, 0.0, 1.0], device=dev)
    top_k = torch.tensor([50, 0, 1, 1000, 0, 20, 7, 0, 0, 3, 5, V + 5], device=dev, dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.5, 0.01, 0.95, 0.3, 0.999, 1.0, 0.2, 0.5, 1.0], device=dev)
    thr = torch.zeros(B, device=dev)
    tok = torch.zeros(B, device=dev, dtype=torch.int32)
    lp = torch.zeros(B, device=dev)
    step = torch.zeros(1, device=dev, dtype=torch.int32)
    for it in range(3):
        step.fill_(it)
        _lib.check(_fn("sample_f")(_lib.ptr(logits), logits.stride(0), _lib.ptr(temp), B, V, ctypes.c_uint(99), _lib.ptr(step),
                                   _lib.ptr(top_k), _lib.ptr(top_p), _lib.ptr(thr), _lib.ptr(tok), _lib.ptr(lp),
                                   _lib.stream_ptr()), "sample_filtered")
        _lib.check_status("sample_filtered")
        for b in range(B):
            T = float(temp[b])
            if T <= 0:
                assert int(tok[b]) == int(logits[b].argmax()) and thr[b] == float("-inf")
                continue
            z = logits[b] / T
            allowed = torch.isfinite(filter_logits(z, int(top_k[b]) if int(top_k[b]) <= V else 0, float(top_p[b])))
            got = z >= thr[b]
            # the kernel's set equals the sorted definition up to ties / rounding at the boundary of the mass threshold
            probs = torch.softmax(z, -1)
            differ = float(probs[got ^ allowed].sum())             # mass of the tokens the two definitions disagree on
            assert abs(int(got.sum()) - int(allowed.sum())) <= 1 or differ < 1e-5, (b, int(got.sum()), int(allowed.sum()), differ)
            assert bool(got[int(tok[b])])
            ref_lp = torch.log_softmax(z, -1)[int(tok[b])]
            assert abs(float(lp[b]) - float(ref_lp)) < 2e-3
    # rows without any filter keep the whole vocabulary
    assert thr[8] == float("-inf") and thr[11] == float("-inf")


def test_engine_generates_with_top_k_and_top_p():
    cfg, model, eng = _engine(True, True, max_batch=16)
    prompt = list(range(5, 40))
    greedy = eng.generate([prompt], {"n": 4, "temperature": 0.0, "max_tokens": 8})[0]["token_ids"]   # same batch shape
    k1 = eng.generate([prompt], {"n": 4, "temperature": 1.0, "max_tokens": 8, "top_k": 1, "seed": 3})
    assert all(o["token_ids"] == greedy for o in k1)               # top-1 sampling is greedy decoding
    tiny_p = eng.generate([prompt], {"n": 4, "temperature": 1.0, "max_tokens": 8, "top_p": 1e-6, "seed": 4})
    assert all(o["token_ids"] == greedy for o in tiny_p)
    free = eng.generate([prompt], {"n": 8, "temperature": 1.0, "max_tokens": 8, "top_k": 50, "top_p": 0.95, "seed": 5})
    assert len({tuple(o["token_ids"]) for o in free}) > 1
