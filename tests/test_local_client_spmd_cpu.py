"""The ``local`` protocol as an SPMD job: two processes started with only the launcher's environment (no process
group of their own), each with its own client and its half of the batch.  The first engine forms the gloo group,
the client fills in the global normalisers, and the result equals one process on the whole batch."""
import os
import socket
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from tests.test_zorro_equivalence_cpu import make_grpo_batch


def _cfg():
    from arctic_platform_b200.rl import ArcticRLClientConfig
    return ArcticRLClientConfig(comm_protocol="local", model_name="qwen3-tiny", training_gpus=1, sampling_gpus=0,
                                log_prob_gpus=0, seed=4,
                                ds_config={"zero_optimization": {"stage": 3}, "gradient_clipping": 1.0,
                                           "optimizer": {"type": "AdamW", "params": {"lr": 1e-3}}})


def _payload(sl):
    ids, mask, R = make_grpo_batch(n_prompts=4, n_samples=2, seed=2)
    B = ids.shape[0]
    g = torch.Generator().manual_seed(0)
    old = torch.randn(B, R, generator=g) * 0.01 - 2.0
    adv = torch.randn(B, 1, generator=g).expand(B, R).contiguous()
    batch = {"input_ids": ids[sl], "attention_mask": mask[sl], "response_mask": mask[sl, -R:].contiguous(),
             "old_log_probs": old[sl], "advantages": adv[sl]}
    return {"batch": batch, "meta": {"zorro_train_enable": True}}


def _rank(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import torch.distributed as dist
    from arctic_platform_b200.rl import create_arctic_rl_client
    assert not dist.is_initialized()
    client = create_arctic_rl_client(_cfg())
    assert dist.is_initialized() and client.spmd_world == world          # formed by the training engine
    B = 8
    out = client.call("fwd_bwd", _payload(slice(rank * B // world, (rank + 1) * B // world)), {"loss_fn": "verl_grpo"})
    st = client.call("step")
    wn = client.call("weight_norm")
    torch.save({"loss": out["avg_loss"], "grad_norm": st["metrics"]["grad_norm"], "norm": wn["training_norm"]},
               os.path.join(out_dir, f"r{rank}.pt"))
    client.call("shutdown")


@pytest.mark.timeout(300)
def test_two_spmd_ranks_equal_one_process():
    from arctic_platform_b200.rl import create_arctic_rl_client
    single = create_arctic_rl_client(_cfg())
    ref = single.call("fwd_bwd", _payload(slice(0, 8)), {"loss_fn": "verl_grpo"})
    ref_st = single.call("step")
    ref_norm = single.call("weight_norm")["training_norm"]
    single.call("shutdown")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_rank, args=(2, port, d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"r{r}.pt")) for r in range(2)]
    assert res[0]["grad_norm"] == pytest.approx(res[1]["grad_norm"], rel=1e-6)
    assert res[0]["grad_norm"] == pytest.approx(ref_st["metrics"]["grad_norm"], rel=1e-4)
    assert res[0]["norm"] == pytest.approx(ref_norm, rel=1e-6) and res[1]["norm"] == pytest.approx(ref_norm, rel=1e-6)
    # each rank reports the token mean of its own shard; the global figure lies between them
    lo, hi = sorted(r["loss"] for r in res)
    assert lo - 1e-6 <= ref["avg_loss"] <= hi + 1e-6


def _tp_rank(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from arctic_platform_b200.rl import create_arctic_rl_client
    cfg = _cfg().model_copy(update={"sampling_gpus": 1, "colocate": True,
                                    "vllm_config": {"max_model_len": 64, "tensor_parallel_size": 2}})
    client = create_arctic_rl_client(cfg)
    client.call("fwd_bwd", _payload(slice(rank * 4, (rank + 1) * 4)), {"loss_fn": "verl_grpo"})
    client.call("step")
    client.call("sync_weights")
    norms = client.call("weight_norm")
    # every rank of the replica passes the same prompts, as one program on two ranks does
    out = client.call("generate", [[3, 4, 5, 9], [6, 7]], {"n": 1, "max_tokens": 5, "temperature": 0.0})
    torch.save({"norms": norms, "tokens": [r["token_ids"] for r in out]}, os.path.join(out_dir, f"t{rank}.pt"))
    client.call("shutdown")


@pytest.mark.timeout(300)
def test_spmd_ranks_form_one_tensor_parallel_sampling_replica():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_tp_rank, args=(2, port, d), nprocs=2, join=True)
        res = [torch.load(os.path.join(d, f"t{r}.pt")) for r in range(2)]
    assert res[0]["tokens"] == res[1]["tokens"] and all(len(t) == 5 for t in res[0]["tokens"])
    for r in res:
        assert r["norms"]["sampling_norm"] == pytest.approx(r["norms"]["training_norm"], rel=1e-6)
        assert r["norms"]["sampling_num_params"] == r["norms"]["training_num_params"]
