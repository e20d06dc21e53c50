"""HTTP front end of the job server (FastAPI), speaking DSSST1 on the tensor-carrying routes.

Routes, parameters (``job_id`` as a query parameter) and response shapes are those of the reference's
server (arctic_platform/common/http_server.py:140-970): ``GET /health``, ``POST /initialize``,
``/destroy``, ``/forward-backward`` and ``/forward`` (octet-stream in and out), ``/step``,
``/empty-training-cache``, ``/save``, ``/load-checkpoint``, ``/sleep-inference``, ``/wake-inference``,
``/reset-prefix-cache``, ``/operation``, ``/sleep-training``, ``/wake-training``, ``/sleep-log-prob``,
``/wake-log-prob``, ``/generate`` (octet-stream), ``/weight-norm``, ``/weight-sync``, ``/log-probs``,
``GET /status``, ``GET /job/{job_id}``.  Error states map to 404 (unknown job), 409 (conflict) and 400.

    python -m arctic_platform_b200.common.http_server --port 7000 --training-gpus 1 --sampling-gpus 1 --colocate
"""
from __future__ import annotations

import argparse
import asyncio
from typing import Optional

from fastapi import Body, FastAPI, HTTPException, Response

from .. import wire
from .server import ArcticRLServerCore, JobError
from .utils.server_models import (GenerateRequest, JobConfig, LoadCheckpointRequest, LogProbsRequest, OperationRequest,
                                  SaveRequest, StepRequest, WeightNormRequest, WeightSyncRequest)

OCTET = "application/octet-stream"


def create_app(core: Optional[ArcticRLServerCore] = None) -> FastAPI:
    app = FastAPI(title="arctic-platform-b200")
    app.state.core = core or ArcticRLServerCore()
    lock = asyncio.Lock()          # engines are single-threaded: one request touches the GPU at a time

    async def run(fn, *args, **kwargs):
        async with lock:
            try:
                return await asyncio.get_running_loop().run_in_executor(None, lambda: fn(*args, **kwargs))
            except JobError as exc:
                raise HTTPException(exc.status, str(exc)) from exc
            except ValueError as exc:                  # the request itself is wrong (lengths, shapes, unknown names)
                raise HTTPException(400, f"{type(exc).__name__}: {exc}") from exc
            except Exception as exc:  # noqa: BLE001 - a failing engine must not take the server down
                asleep = isinstance(exc, RuntimeError) and "asleep" in str(exc)
                raise HTTPException(409 if asleep else 500, f"{type(exc).__name__}: {exc}") from exc

    def octet(obj) -> Response:
        return Response(content=wire.dumps(obj), media_type=OCTET)

    def decode(body: bytes):
        try:
            return wire.loads(body)
        except wire.WireError as exc:
            raise HTTPException(400, f"bad DSSST1 payload: {exc}") from exc

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.post("/initialize")
    async def initialize(job_config: JobConfig):
        return await run(app.state.core.initialize, job_config.model_dump())

    @app.post("/destroy")
    async def destroy(job_id: Optional[int] = None):
        return await run(app.state.core.destroy, job_id)

    @app.post("/forward-backward")
    async def forward_backward(job_id: int, body: bytes = Body(..., media_type=OCTET)):
        return octet(await run(app.state.core.forward_backward, job_id, decode(body)))

    @app.post("/forward")
    async def forward(job_id: int, body: bytes = Body(..., media_type=OCTET)):
        return octet(await run(app.state.core.forward, job_id, decode(body)))

    @app.post("/step")
    async def step(job_id: int, request: StepRequest = Body(default=StepRequest())):
        return await run(app.state.core.step, job_id, request.learning_rate)

    @app.post("/empty-training-cache")
    async def empty_training_cache(job_id: int):
        return await run(app.state.core.empty_training_cache, job_id)

    @app.post("/save")
    async def save(job_id: int, request: SaveRequest = Body(default=SaveRequest())):
        return await run(app.state.core.save, job_id, request.path, request.step, request.export_hf,
                         request.save_total_limit)

    @app.post("/load-checkpoint")
    async def load_checkpoint(job_id: int, request: LoadCheckpointRequest = Body(default=LoadCheckpointRequest())):
        return await run(app.state.core.load_checkpoint, job_id, request.path, request.step)

    @app.post("/sleep-inference")
    async def sleep_inference(job_id: int, level: int = 1):
        return await run(app.state.core.sleep_inference, job_id, level)

    @app.post("/wake-inference")
    async def wake_inference(job_id: int, tags: Optional[list] = Body(default=None)):
        return await run(app.state.core.wake_inference, job_id, tags)

    @app.post("/reset-prefix-cache")
    async def reset_prefix_cache(job_id: int):
        return await run(app.state.core.reset_prefix_cache, job_id)

    @app.post("/operation")
    async def operation(request: OperationRequest):
        return await run(app.state.core.operation, request.operation_type, request.sub_job_id, request.payload)

    @app.post("/sleep-training")
    async def sleep_training(job_id: int, mode: str = "all"):
        return await run(app.state.core.sleep_training, job_id, mode)

    @app.post("/wake-training")
    async def wake_training(job_id: int):
        return await run(app.state.core.wake_training, job_id)

    @app.post("/sleep-log-prob")
    async def sleep_log_prob(job_id: int):
        return await run(app.state.core.sleep_training, job_id, "all")

    @app.post("/wake-log-prob")
    async def wake_log_prob(job_id: int):
        return await run(app.state.core.wake_training, job_id)

    @app.post("/generate")
    async def generate(job_id: int, body: bytes = Body(..., media_type=OCTET)):
        req = GenerateRequest(**decode(body))
        return octet(await run(app.state.core.generate, job_id, req.prompts, req.sampling_params, req.routing_key,
                               req.strict))

    @app.post("/weight-norm")
    async def weight_norm(request: WeightNormRequest):
        return await run(app.state.core.weight_norm, request.training_job_id, request.sampling_job_id)

    @app.post("/weight-sync")
    async def weight_sync(request: WeightSyncRequest):
        return await run(app.state.core.weight_sync, request.source_sub_job_id, request.target_sub_job_ids,
                         request.cuda_ipc, request.low_memory)

    @app.post("/log-probs")
    async def log_probs(job_id: int, request: LogProbsRequest):
        return await run(app.state.core.log_probs, job_id, request.prompts, request.completions, request.top_k)

    @app.post("/heartbeat")
    async def heartbeat(job_id: int):
        await run(app.state.core.heartbeat, job_id)
        return {"status": "ok"}

    @app.post("/recover")
    async def recover(job_id: int, request: LoadCheckpointRequest = Body(default=LoadCheckpointRequest())):
        return await run(app.state.core.recover, job_id, request.path, request.step)

    @app.get("/job/{job_id}/workers")
    async def job_workers(job_id: int):
        try:
            return app.state.core.check_workers(job_id)
        except JobError as exc:
            raise HTTPException(exc.status, str(exc)) from exc

    @app.get("/status")
    async def status():
        return app.state.core.status()

    @app.get("/job/{job_id}")
    async def job(job_id: int):
        try:
            return app.state.core.get_job_status(job_id)
        except JobError as exc:
            raise HTTPException(exc.status, str(exc)) from exc

    return app


def build_arg_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="B200 RL job server")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", "-p", type=int, default=7000)
    ap.add_argument("--training-gpus", type=int, default=0)
    ap.add_argument("--sampling-gpus", type=int, default=0)
    ap.add_argument("--log-prob-gpus", type=int, default=0)
    ap.add_argument("--log-prob-engine", choices=["vllm", "deepspeed"], default="deepspeed")
    ap.add_argument("--colocate", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-ray-auto-attach", action="store_true")
    ap.add_argument("--worker-watchdog-seconds", type=float, default=10.0,
                    help="period of the background liveness check of the rank processes (0 = off)")
    return ap


def main(argv=None) -> None:
    import uvicorn
    args = build_arg_parser().parse_args(argv)
    from .ray_cluster import init_ray_cluster
    cluster = init_ray_cluster(auto_attach=not args.no_ray_auto_attach)     # {"ray": False} without Ray: local ranks
    if args.verbose:
        print(f"[server] cluster: {cluster}", flush=True)
    core = ArcticRLServerCore(training_gpus=args.training_gpus, sampling_gpus=args.sampling_gpus,
                              log_prob_gpus=args.log_prob_gpus, colocate=args.colocate,
                              log_prob_engine=args.log_prob_engine)
    if args.worker_watchdog_seconds > 0:
        core.start_worker_watchdog(args.worker_watchdog_seconds)
    uvicorn.run(create_app(core), host=args.host, port=args.port, log_level="info" if args.verbose else "warning")


if __name__ == "__main__":
    main()
