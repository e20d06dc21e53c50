"""GRPO step benchmark: Qwen3-4B, colocated trainer + sampler on every GPU, synthetic data, random-init weights.

One step = sync_weights -> rollout (n samples per prompt, temperature 1.0, fixed response budget) ->
reference log-probs -> forward/backward (ZoRRo prompt-deduplicated, verl-style GRPO loss) -> AdamW.
Weak scaling: every GPU holds ``--prompts-per-gpu`` prompts x ``--samples`` rollouts (the named
configuration, 64 prompts x 16 samples on 8 GPUs, is 8 prompts per GPU).  The headline metric is
whole-job tokens/s = global (prompt + response) tokens of a step / step time, as the reference's verl
integration reports (arctic_platform/integrations/verl/README.md:100-109).

ONE timed region of ``--steps`` steps, driven through the public client API (``create_arctic_rl_client``),
bracketed by barrier + synchronize, timed with CUDA events, max over ranks.  Every step builds its batch in
pinned host memory, copies it to the device inside the engines and reads its results (tokens, log-prob grids,
loss) back:
  * ``e2e``:   CUDA-event time of the whole region (host batch building, copies and read-backs included);
  * ``value``: the device time of the engine phases inside the SAME steps (sync_weights, rollout, reference
               log-probs, forward/backward, optimizer), each bracketed by CUDA events, host batch building excluded.
Bytes copied per step are counted where the copies are issued (``utils/transfer_stats.py``).
``--wall-limit-s`` (default 830 s after process start) is a safety net for callers that end the process after a fixed
wall time: when the next timed step would end past it, all ranks stop together (never before 5 timed steps) and the
line reports the steps actually timed in ``steps`` with the request in ``steps_requested``.

    python bench.py [--gpus N --steps K --warmup W]          # N > 1 under torch.distributed.run
    python bench.py --impl reference                          # the reference's own stack, if installable
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--prompts-per-gpu", type=int, default=8)
    ap.add_argument("--samples", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--response-len", type=int, default=2048)
    ap.add_argument("--rollouts-per-microbatch", type=int, default=8,
                    help="rollouts of one prompt per training micro-batch (prompt KV is recomputed per micro-batch)")
    ap.add_argument("--prompts-per-microbatch", type=int, default=1)
    ap.add_argument("--ref-microbatch-merge", type=int, default=2,
                    help="training micro-batches scored together in one reference (no-grad) forward")
    ap.add_argument("--zero-stage", type=int, default=3,
                    help="3: bf16 parameters sharded over ranks and gathered unit by unit; 2: replicated parameters")
    ap.add_argument("--baseline-json", default=None,
                    help="file with a same-box anchor {'grpo_step_tokens_per_s_per_gpu': x, 'what': ...}; default "
                         "benchmarks/anchors_1gpu.json when present (vs_baseline = value / (x * gpus))")
    ap.add_argument("--lr", type=float, default=1e-6)
    ap.add_argument("--wall-limit-s", type=float, default=830.0,
                    help="safety net for callers that end the process after a fixed wall time: when the next timed "
                         "step would end later than this many seconds after the process started, the timed loop "
                         "stops (all ranks together, never before 5 steps) and the line reports the steps it timed "
                         "in 'steps' and the request in 'steps_requested'; 0 = no limit")
    return ap.parse_args()


def reference_arm(args) -> None:
    """The reference needs deepspeed, ray, arctic_inference and deep_ep (pyproject.toml:111-131 of the reference);
    none is installed here or in the offline wheelhouse, and its build backend (hatchling) is missing too."""
    why = "reference not installable offline: build backend hatchling and hard deps deepspeed/ray/arctic_inference/deep_ep are absent from the image and /opt/wheelhouse"
    # only an installed copy of the reference counts (this repository's own ``arctic_platform`` is an import alias of
    # the product and must never stand in for it)
    if (ROOT / "baseline" / "_ref" / "arctic_platform" / "__init__.py").is_file():
        try:
            import deepspeed  # noqa: F401
            import ray  # noqa: F401
            why = "reference is installed, but no reference runner is wired because its engines (DeepSpeed/vLLM/ArcticInference) are unavailable"
        except Exception:
            pass
    print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of this process's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                parts = [p.strip() for p in out.split(",")]
                if len(parts) >= 7:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.5)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if s[1].replace(".", "").isdigit()]
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")):
            if any(s[3 + i].lower().startswith("active") for s in self.samples):
                reasons.append(name)
        busy = sorted(sm)[len(sm) // 4:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


MIN_TIMED_STEPS = 5


def stop_for_wall_limit(done: int, age_s: float, s_per_step: float, limit_s: float) -> bool:
    """Whether the timed loop should end after ``done`` steps: the next step (3 % slack, 5 s to report and leave) would
    finish later than ``limit_s`` seconds after the process started.  Never before ``MIN_TIMED_STEPS``."""
    if limit_s <= 0 or done < MIN_TIMED_STEPS:
        return False
    return age_s + 1.03 * s_per_step + 5.0 > limit_s


def main():
    t_start = time.perf_counter()
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if args.gpus != world and rank == 0 and world > 1:
        print(f"[bench] --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)

    from arctic_platform_b200.models.config import resolve_config
    from arctic_platform_b200.ops import _lib
    from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client

    cfg = resolve_config(args.model)
    P, R, NP, NS = args.prompt_len, args.response_len, args.prompts_per_gpu, args.samples
    B = NP * NS
    kv_tokens = NP * (P + 64) + B * (R + 64) + 4096
    client_cfg = ArcticRLClientConfig(
        comm_protocol="local", model_name=args.model, training_gpus=world, sampling_gpus=world, log_prob_gpus=world,
        colocate=True, seed=1234,
        ds_config={"zero_optimization": {"stage": args.zero_stage}, "gradient_clipping": 1.0,
                   "optimizer": {"type": "AdamW", "params": {"lr": args.lr, "betas": [0.9, 0.999], "eps": 1e-8,
                                                             "weight_decay": 0.01}}},
        vllm_config={"kv_cache_tokens": kv_tokens, "max_num_seqs": max(8, B), "max_model_len": P + R + 16},
        arctic_inference_config={"zorro_inference": {"enable": True}})
    client = create_arctic_rl_client(client_cfg)

    gen = torch.Generator().manual_seed(99 + rank)
    sp = {"n": NS, "temperature": 1.0, "max_tokens": R, "ignore_eos": True}
    rpm = max(1, min(NS, args.rollouts_per_microbatch))
    ppm = max(1, min(NP, args.prompts_per_microbatch))
    n_mb = ((NS + rpm - 1) // rpm) * ((NP + ppm - 1) // ppm)
    meta = {"zorro_train_enable": True, "temperature": 1.0, "dp_size": world,
            "batch_num_tokens": float(B * R * world), "global_batch_size": float(B * world),
            "actor_config": {"loss_agg_mode": "token-mean", "use_kl_loss": True, "kl_loss_coef": 0.001,
                             "kl_loss_type": "low_var_kl", "entropy_coeff": 0.0}}

    def make_prompts():
        return [torch.randint(1, cfg.vocab_size, (P,), generator=gen).tolist() for _ in range(NP)]

    ids_host = torch.zeros((B, P + R), dtype=torch.int64).pin_memory()
    old_host = torch.zeros((B, R), dtype=torch.float32).pin_memory()

    def build_batches(prompts, results):
        """Padded RL batch on pinned host memory, split so that each micro-batch holds every prompt with a
        slice of its rollouts (the prompt is deduplicated inside a micro-batch)."""
        ids, old = ids_host.zero_(), old_host.zero_()
        prompt_t = [torch.tensor(p) for p in prompts]
        for i, r in enumerate(results):
            ids[i, :P] = prompt_t[r["prompt_index"]]
            ids[i, P:P + len(r["token_ids"])] = torch.tensor(r["token_ids"])
            old[i, :len(r["logprobs"])] = torch.tensor(r["logprobs"])
        mask = torch.ones_like(ids)
        rewards = torch.randn(NP, NS, generator=gen)
        adv = ((rewards - rewards.mean(1, keepdim=True)) / (rewards.std(1, keepdim=True) + 1e-6)).reshape(B, 1)
        full = {"input_ids": ids, "attention_mask": mask, "response_mask": mask[:, P:].contiguous(),
                "old_log_probs": old, "advantages": adv.expand(B, R).contiguous()}
        mbs = []
        for p0 in range(0, NP, ppm):
            for r0 in range(0, NS, rpm):
                rows = torch.tensor([p * NS + j for p in range(p0, min(NP, p0 + ppm))
                                     for j in range(r0, min(NS, r0 + rpm))])
                mbs.append({k: v[rows].contiguous().pin_memory() for k, v in full.items()})
        return mbs

    def ref_groups(mbs):
        """Scoring needs no activations for backward, so the reference pass runs on larger micro-batches: all the
        rollouts of a prompt together (the prompt is stored and attended once for the 16 of them)."""
        k = max(1, min(len(mbs), args.ref_microbatch_merge))
        out = []
        for i in range(0, len(mbs), k):
            part = mbs[i:i + k]
            keys = ("input_ids", "attention_mask", "response_mask")
            batch = part[0] if len(part) == 1 else {kk: torch.cat([m[kk] for m in part]).pin_memory() for kk in keys}
            out.append({"batch": {kk: batch[kk] for kk in keys}, "parts": part})
        return out

    def scatter_ref(grp, logp):
        r0 = 0
        for m in grp["parts"]:
            n = m["input_ids"].shape[0]
            m["ref_log_prob"] = logp[r0:r0 + n]
            r0 += n

    from arctic_platform_b200.utils import transfer_stats

    PHASES = ("sync_weights", "rollout", "ref_logprob", "fwd_bwd", "optimizer")
    marks = []          # per step: list of (phase, start event, end event)

    def phase(name, fn, *a, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*a, **kw)
        e1.record()
        marks[-1].append((name, e0, e1))
        return out

    def step_client():
        """One GRPO step through the public client API; inputs start in pinned host memory, results come back to
        the host (generated tokens and log-probs, reference log-prob grids, loss and gradient norm)."""
        marks.append([])
        prompts = make_prompts()
        phase("sync_weights", client.call, "sync_weights")
        results = phase("rollout", client.call, "generate", prompts, sp)
        client.call("sleep_inference", 1)
        mbs = build_batches(prompts, results)

        def ref_pass():
            for grp in ref_groups(mbs):
                ref = client.call("fwd_no_grad", {"batch": grp["batch"], "meta": dict(meta)}, reference_model=True)
                scatter_ref(grp, ref["batch"]["log_probs"])

        phase("ref_logprob", ref_pass)
        out = phase("fwd_bwd", client.call, "fwd_bwd", {"batch": mbs, "meta": dict(meta)}, {"loss_fn": "verl_grpo"})
        st = phase("optimizer", client.call, "step")
        return out["avg_loss"], float(st["metrics"]["grad_norm"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def reduce_max(vals):
        if world == 1:
            return [float(v) for v in vals]
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def process_age():
        try:
            import psutil
            return time.time() - psutil.Process().create_time()
        except Exception:
            return time.perf_counter() - t_start + 30.0      # imports happened before t_start: assume the worst

    def out_of_time(done, s_per_step):
        """True on every rank when any rank expects the next step to end after the wall limit."""
        late = stop_for_wall_limit(done, process_age(), s_per_step, args.wall_limit_s)
        if world > 1:
            t = torch.tensor([1.0 if late else 0.0], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            late = bool(t.item() > 0)
        if late and rank == 0:
            print(f"[bench] wall limit {args.wall_limit_s:.0f} s: stopping after {done} of {args.steps} timed steps",
                  file=sys.stderr, flush=True)
        return late

    if rank == 0:
        print(f"[bench] engines ready after {time.perf_counter() - t_start:.1f} s", file=sys.stderr, flush=True)
    for _ in range(args.warmup):
        step_client()
    if rank == 0:
        print(f"[bench] warm-up done after {time.perf_counter() - t_start:.1f} s", file=sys.stderr, flush=True)
    marks.clear()
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    transfer_stats.reset()
    l0 = _lib.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t_timed = time.time()
    steps_done = 0
    for _ in range(args.steps):
        loss, gnorm = step_client()
        steps_done += 1
        if steps_done < args.steps and out_of_time(steps_done, (time.time() - t_timed) / steps_done):
            break
    ev1.record()
    barrier()
    launches = _lib.launch_count() - l0
    xfer = transfer_stats.snapshot()
    sampler.stop_flag.set()
    sampler.join(timeout=3)
    _lib.check_status("bench")
    if not (loss == loss and gnorm == gnorm):
        raise SystemExit(f"bench: non-finite loss {loss} / grad norm {gnorm}")
    phase_ms = {n: 0.0 for n in PHASES}
    for step_marks in marks:
        for name, e0, e1 in step_marks:
            phase_ms[name] += e0.elapsed_time(e1)
    K = steps_done
    red = reduce_max([ev0.elapsed_time(ev1) / K, sum(phase_ms.values()) / K] + [phase_ms[n] / K for n in PHASES])
    ms_e2e, ms_dev, per_phase = red[0], red[1], red[2:]
    if rank == 0:
        tokens = B * (P + R) * world
        value = tokens / (ms_dev / 1e3)
        anchor, vs = None, None
        bj = Path(args.baseline_json) if args.baseline_json else ROOT / "benchmarks" / "anchors_1gpu.json"
        if bj.is_file():
            try:
                anchor = json.loads(bj.read_text())
                per_gpu = float(anchor["grpo_step_tokens_per_s_per_gpu"])
                vs = value / (per_gpu * world)
            except Exception:
                anchor = None
        stage_label = f"zero{args.zero_stage}-fused" if world > 1 else "single-rank fused clip+AdamW (no sharding)"
        line = {
            "metric": "grpo_step_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": K, "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": vs, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": args.model, "global_batch": B * world, "prompts": NP * world, "samples_per_prompt": NS,
                       "seq_len": P + R, "prompt_len": P, "response_len": R,
                       "parallelism": f"dp{world} {stage_label} + sampler tp1 x{world} replicas, colocated",
                       "l2_policy": "inputs larger than L2 (new random prompts and rollouts every step)",
                       "step": "sync_weights+rollout+ref_logprob+fwd_bwd+adamw", "lr": args.lr,
                       "train_microbatches": n_mb,
                       "timed_region": "one region through the client API; value = sum of CUDA-event phase times "
                                       "inside it, e2e = the whole region",
                       "vs_baseline_is": (anchor or {}).get("what") if vs is not None else None},
            "clocks": sampler.summary(),
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": xfer["h2d"] // K, "d2h_bytes_per_step": xfer["d2h"] // K},
            "phases_ms": {n: round(v, 1) for n, v in zip(PHASES, per_phase)},
            "gpu_launches": launches,
            "peak_device_memory_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1),
            "reserved_device_memory_gb": round(torch.cuda.memory_reserved(dev) / 2 ** 30, 1),
            "rollout_tokens_per_step": B * R * world,
        }
        print(json.dumps(line), flush=True)
    # leave without tearing down 100+ GB of tensors, graphs and communicators one by one: the line is out, every rank
    # has passed the closing barrier, and an unhurried interpreter exit costs seconds per process
    if world > 1:
        dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
