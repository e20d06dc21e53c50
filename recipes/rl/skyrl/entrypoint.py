"""Runs the recipe loop as the driver does under SkyRL: in this process, or as a Ray task next to the engines.

    python -m recipes.rl.skyrl.entrypoint --data train.parquet --env bird_sql_arctic --model Qwen/Qwen3-8B ...
    python -m recipes.rl.skyrl.entrypoint --as-ray-task --data ...        # needs a running Ray cluster

With ``--as-ray-task`` the loop is submitted to the cluster as a one-CPU task (the driver stays thin, the task can be
rescheduled by Ray, and a ``reconnect_config`` / ``server_state`` handed over by a previous task re-attaches to the
engines instead of starting new ones).  The task is defined in THIS module so that Ray workers import the recipe's own
code path (and with it the environment registration) rather than anything from a SkyRL checkout.
Counterpart of recipes/rl/skyrl/*/arctic_rl/entrypoint.py in the reference.
"""
from __future__ import annotations

import sys
from typing import Any, Dict, List, Optional

from . import run_loop
from .envs import register_envs


def skyrl_entrypoint(argv: List[str], reconnect_config: Optional[Dict[str, Any]] = None, server_state: Any = None) -> List[dict]:
    """The loop itself.  ``reconnect_config`` (a dumped ``ArcticRLClientConfig`` with job ids) attaches to running
    engines; ``server_state`` is an in-process / actor server state to host them in."""
    register_envs()
    args = run_loop.build_parser().parse_args(argv)
    backend = None
    if reconnect_config is not None or server_state is not None:
        from arctic_platform_b200.rl import ArcticRLClientConfig, create_arctic_rl_client
        from .arctic_backend import SkyRLArcticBackend
        backend = SkyRLArcticBackend.__new__(SkyRLArcticBackend)
        backend.zorro, backend.loss_fn, backend.kl_loss_coef = not args.no_zorro, "verl_grpo", args.kl_loss_coef
        cfg = ArcticRLClientConfig(**reconnect_config) if reconnect_config is not None else SkyRLArcticBackend.client_config(
            args.model, args.training_gpus, args.sampling_gpus, args.log_prob_gpus, lr=args.lr, zero_stage=args.zero_stage,
            zorro=not args.no_zorro, max_model_len=args.max_prompt_tokens + args.max_tokens)
        backend.client = create_arctic_rl_client(cfg, server_state) if server_state is not None else create_arctic_rl_client(cfg)
    return run_loop.run(args, backend=backend)


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    as_task = "--as-ray-task" in argv
    argv = [a for a in argv if a != "--as-ray-task"]
    if not as_task:
        skyrl_entrypoint(argv)
        return 0
    try:
        import ray
    except ImportError:
        print("--as-ray-task needs Ray; run without it to use this process", file=sys.stderr)
        return 2
    if not ray.is_initialized():
        ray.init(address="auto", ignore_reinit_error=True)
    ray.get(ray.remote(num_cpus=1)(skyrl_entrypoint).remote(argv))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
