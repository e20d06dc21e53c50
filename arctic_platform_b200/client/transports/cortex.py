"""Cortex (SnowAPI) transport: submit -> request id -> poll, with chunked DSSST1 bodies and retries.

The remote service takes every op as a POST that returns a ``request_id``; results are fetched by polling
an events endpoint with a cursor until a terminal event arrives, large results come back as
``result_chunk`` events that are reassembled with ``wire.decode_byte_chunks``; large request bodies are
cut into chunk frames that share a ``chunk_group_id`` (a failed upload restarts the whole group).
Transient HTTP failures are retried with exponential back-off and jitter up to ``max_retries``; auth is a
programmatic access token.  Contract of arctic_platform/client/transports/cortex.py:178-523; exercised
against a fake HTTP session in the tests (there is no network here).
"""
from __future__ import annotations

import base64
import random
import time
import uuid
from typing import Any, Dict, List, Optional

from ... import wire
from ..config import ArcticRLClientConfig, CortexConfig
from ..transport import JobHandles, Request, Transport

TRANSIENT = {408, 425, 429, 500, 502, 503, 504}
MAX_CHUNK_BYTES = 8 * 1024 * 1024


MAX_GROUP_REPLAYS = 2


class CortexError(RuntimeError):
    def __init__(self, message: str, status: Optional[int] = None, detail: Optional[dict] = None):
        super().__init__(message)
        self.status = status
        self.detail = detail or {}


class ChunkGroupError(CortexError):
    """The service refused a chunked upload for a reason that concerns the whole group (``detail["code"]``):
    the group kept getting lost after the bounded replays, its identity was reused for other contents, or it was
    closed with chunks missing."""


class CortexTransport(Transport):
    def __init__(self, config: ArcticRLClientConfig, session=None, sleep=time.sleep):
        if not isinstance(config.backend, CortexConfig):
            raise TypeError("CortexTransport needs backend.type == 'remote'")
        self.config = config
        self.backend: CortexConfig = config.backend
        if session is None:
            import requests
            session = requests.Session()
        self.session = session
        self._sleep = sleep
        self.jobs = JobHandles.from_config(config)
        self.job_id: Optional[str] = None
        if self.backend.base_url:
            self.base = self.backend.base_url.rstrip("/")
            self.headers: Dict[str, str] = {}
        else:
            self.base = (f"https://{self.backend.host}/api/v2/databases/{self.backend.database}/schemas/"
                         f"{self.backend.schema_}/{self.backend.endpoint}")
            self.headers = {"Authorization": f"Bearer {self.backend.resolve_pat()}",
                            "X-Snowflake-Authorization-Token-Type": "PROGRAMMATIC_ACCESS_TOKEN"}

    # -- HTTP with retries ----------------------------------------------------------------------------
    def _http(self, method: str, path: str, **kw):
        delay = 0.5
        last: Any = None
        extra_headers = kw.pop("headers", {})        # popped once: a retry must carry the same headers
        for attempt in range(self.backend.max_retries + 1):
            try:
                resp = self.session.request(method, self.base + path, headers={**self.headers, **extra_headers},
                                            timeout=self.config.request_timeout, **kw)
                if resp.status_code < 400:
                    return resp
                try:
                    detail = resp.json()
                except Exception:
                    detail = None
                detail = detail if isinstance(detail, dict) else {"body": detail}
                # a verdict on the chunk group is final for this attempt whatever the status code says
                verdict = wire.find_chunk_group_error(detail) if kw.get("data") is not None else None
                if resp.status_code not in TRANSIENT or verdict is not None:
                    raise CortexError(f"{method} {path} -> {resp.status_code}: {getattr(resp, 'text', '')[:200]}",
                                      resp.status_code, detail)
                last = CortexError(f"{method} {path} -> {resp.status_code}", resp.status_code)
            except CortexError:
                raise
            except Exception as exc:      # connection errors are transient
                last = exc
            if attempt < self.backend.max_retries:
                self._sleep(delay * (0.5 + random.random()))
                delay = min(delay * 2, 30.0)
        raise CortexError(f"{method} {path} failed after {self.backend.max_retries + 1} attempts: {last}")

    # -- lifecycle --------------------------------------------------------------------------------------
    def initialize(self) -> JobHandles:
        if self.jobs.any_set:
            self.job_id = str(self.jobs.training or self.jobs.sampling or self.jobs.log_prob).split(":")[0]
            return self.jobs
        resp = self._http("POST", "/jobs", json=self.config.to_cortex()).json()
        self.job_id = str(resp["job_id"])
        for sub in resp.get("sub_jobs", []):
            self.jobs.set(sub["sub_job_type"], f"{self.job_id}:{sub['sub_job_id']}")
        deadline = time.time() + self.config.job_ready_timeout
        while True:
            st = self._http("GET", f"/jobs/{self.job_id}").json().get("status")
            if st == "RUNNING":
                return self.jobs
            if st in ("FAILED", "CANCELLED") or time.time() > deadline:
                raise CortexError(f"job {self.job_id} is {st}")
            self._sleep(2.0)

    # -- one op -----------------------------------------------------------------------------------------
    def _submit(self, request: Request) -> str:
        sub = str(request.job_id).split(":")[-1] if request.job_id is not None else None
        path = f"/jobs/{self.job_id}/{request.op}"
        params = {"sub_job_id": sub} if sub else None
        if not request.binary:
            return self._http("POST", path, params=params, json=request.body).json()["request_id"]
        frame = wire.dumps(request.body)
        for attempt in range(MAX_GROUP_REPLAYS + 1):
            # every attempt is a new group identity: the service may still hold fragments of the lost one
            chunks = wire.encode_byte_chunks(frame, kind="request", operation=request.op, max_bytes=MAX_CHUNK_BYTES,
                                             chunk_group_id=str(uuid.uuid4()))
            try:
                rid = None
                for c in chunks:
                    rid = self._http("POST", path, params=params, data=c,
                                     headers={"Content-Type": "application/octet-stream"}).json().get("request_id", rid)
            except CortexError as exc:
                verdict = wire.find_chunk_group_error(exc.detail)
                if verdict is None:
                    raise                                         # not about the group: replaying cannot help
                if verdict["code"] in wire.CHUNK_GROUP_RESTART_CODES and attempt < MAX_GROUP_REPLAYS:
                    continue
                raise ChunkGroupError(f"{request.op}: {verdict.get('message') or verdict['code']}", exc.status, verdict) from exc
            if rid is None:
                raise CortexError("server did not return a request_id")
            return rid
        raise AssertionError("unreachable")

    def _poll(self, request_id: str) -> dict:
        cursor = 0
        chunks: List[bytes] = []
        deadline = time.time() + self.config.request_timeout
        while time.time() < deadline:
            events = self._http("GET", f"/requests/{request_id}/events", params={"cursor": cursor}).json()
            for ev in events.get("events", []):
                cursor = max(cursor, int(ev.get("seq", cursor)) + 1)
                kind = ev.get("type")
                if kind == "result_chunk":
                    chunks.append(base64.b64decode(ev["data"]))
                elif kind == "result":
                    if chunks:
                        return wire.decode_result_chunks(chunks)
                    data = ev.get("data")
                    return wire.loads(base64.b64decode(data)) if isinstance(data, str) else (data or {})
                elif kind == "error":
                    raise CortexError(f"request {request_id} failed: {ev.get('message')}")
            if not events.get("events"):
                self._sleep(0.5)
        raise CortexError(f"request {request_id} timed out")

    def call(self, request: Request) -> dict:
        return self._poll(self._submit(request))

    async def acall(self, request: Request) -> dict:
        import asyncio
        return await asyncio.get_running_loop().run_in_executor(None, self.call, request)

    def shutdown(self) -> None:
        if self.job_id is not None:
            try:
                self._http("DELETE", f"/jobs/{self.job_id}")
            except CortexError:
                pass
            self.job_id = None
