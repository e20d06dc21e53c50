"""In-memory stand-in for the hosted training service's REST surface (used by the client tests).

Implements ``/jobs`` CRUD, ``/jobs/{id}/{op}`` (JSON or chunked octet bodies -> request id), ``/requests/{id}/events``
polling with optional result chunking, ``/jobs/{id}/logs`` and ``/capacity``.  Failure injection: ``fail_next``
queues HTTP status codes returned before the real handler runs; ``restart_chunk_groups`` makes the first chunk
upload of a group answer 409 ``chunk_group_restart``."""
import base64
import json
import re
from typing import Any, Dict, List

from arctic_platform_b200 import wire


class FakeResponse:
    def __init__(self, status: int = 200, body: Any = None):
        self.status_code = status
        self._body = body if body is not None else {}
        self.text = json.dumps(self._body, default=str)

    def json(self):
        return self._body


class FakeServiceSession:
    def __init__(self, ready_after: int = 1, chunk_results_over: int = 0):
        self.jobs: Dict[str, dict] = {}
        self.requests: Dict[str, List[dict]] = {}
        self.calls: List[tuple] = []
        self.fail_next: List[int] = []
        self.restart_chunk_groups = 0
        self.chunk_group_reply = None          # (status, body) answered once to the next chunk upload
        self.ready_after = ready_after
        self.chunk_results_over = chunk_results_over
        self._groups: Dict[str, List[bytes]] = {}
        self._n = 0
        self.logs = [{"ts": f"t{i}", "level": "INFO", "message": f"line {i}"} for i in range(5)]
        self.events = [{"ts": f"e{i}", "kind": "ZONE_READY" if i else "SCHEDULED"} for i in range(3)]
        self.checkpoints = [{"checkpoint_id": "c1", "step": 10}, {"checkpoint_id": "c2", "step": 20}]

    # the one entry point requests.Session exposes that the clients use
    def request(self, method: str, url: str, headers=None, timeout=None, params=None, json=None, data=None):
        path = re.sub(r"^https?://[^/]+", "", url)
        path = path[path.index("/jobs"):] if "/jobs" in path else path[path.index("/requests"):] if "/requests" in path \
            else path[path.rindex("/"):]
        self.calls.append((method, path, dict(params or {}), dict(headers or {})))
        if self.fail_next:
            return FakeResponse(self.fail_next.pop(0), {"error": "injected"})
        return self._route(method, path, params or {}, json, data)

    def _new_id(self, prefix: str) -> str:
        self._n += 1
        return f"{prefix}{self._n}"

    def _route(self, method, path, params, body, data):
        if path == "/capacity":
            return FakeResponse(200, {"free_gpus": 8})
        if path == "/jobs" and method == "POST":
            jid = self._new_id("j")
            subs = [{"sub_job_type": s["sub_job_type"], "sub_job_id": f"s{i}"} for i, s in enumerate(body.get("sub_jobs", []))]
            self.jobs[jid] = {"job_id": jid, "status": "PENDING", "polls": 0, "sub_jobs": subs, "body": body}
            return FakeResponse(200, {"job_id": jid, "sub_jobs": subs})
        if path == "/jobs" and method == "GET":
            st = params.get("status")
            return FakeResponse(200, {"jobs": [j for j in self.jobs.values() if not st or j["status"] == st]})
        m = re.fullmatch(r"/jobs/([^/]+)", path)
        if m:
            job = self.jobs.get(m.group(1))
            if job is None:
                return FakeResponse(404, {"error": "no such job"})
            if method == "DELETE":
                job["status"] = "CANCELLED"
                return FakeResponse(200, {})
            job["polls"] += 1
            if job["status"] == "PENDING" and job["polls"] >= self.ready_after:
                job["status"] = "RUNNING"
            return FakeResponse(200, {k: v for k, v in job.items() if k != "body"})
        m = re.fullmatch(r"/jobs/([^/]+)/logs", path)
        if m:
            return FakeResponse(200, {"logs": self.logs[int(params.get("cursor", 0)):]})
        m = re.fullmatch(r"/jobs/([^/]+)/requests/([^/]+)", path)
        if m:
            evs = self.requests.get(m.group(2))
            if evs is None:
                return FakeResponse(404, {"error": "no such request"})
            cur = int(params.get("cursor") or 0)
            page = [e for e in evs if e["seq"] >= cur][:2]
            nxt = (page[-1]["seq"] + 1) if page else cur
            done = nxt >= len(evs)
            failed = any(e["type"] == "error" for e in evs[:nxt])
            out = {"status": "error" if failed else ("done" if done else "in-progress"), "events": page,
                   "next_cursor": str(nxt)}
            if failed:
                out["message"] = next(e["message"] for e in evs if e["type"] == "error")
            elif done:
                last = evs[-1]
                if "data" in last:
                    out["result"] = last["data"]
            return FakeResponse(200, out)
        m = re.fullmatch(r"/jobs/([^/]+)/checkpoints", path)
        if m and method == "GET":
            return FakeResponse(200, {"checkpoints": list(self.checkpoints)})
        m = re.fullmatch(r"/jobs/([^/]+)/checkpoints/([^/:]+)(:export)?", path)
        if m:
            cid = m.group(2)
            if not any(c["checkpoint_id"] == cid for c in self.checkpoints):
                return FakeResponse(404, {"error": "no such checkpoint"})
            if method == "DELETE":
                self.checkpoints = [c for c in self.checkpoints if c["checkpoint_id"] != cid]
                return FakeResponse(200, {})
            return FakeResponse(200, {"checkpoint_id": cid, "status": "EXPORTING"})
        m = re.fullmatch(r"/jobs/([^/]+)/experiment-run", path)
        if m:
            return FakeResponse(200, {"experiment_name": "exp", "experiment_run_name": f"run-{m.group(1)}"})
        m = re.fullmatch(r"/jobs/([^/]+)/([a-z_\-]+)", path)
        if m and method == "POST":
            jid, op = m.groups()
            if jid not in self.jobs:
                return FakeResponse(404, {"error": "no such job"})
            if data is not None:
                hdr = wire.read_byte_chunk_metadata(data)
                gid = hdr["chunk_group_id"] if hdr else self._new_id("g")
                if self.chunk_group_reply is not None:
                    status, reply = self.chunk_group_reply
                    self.chunk_group_reply = None
                    return FakeResponse(status, reply)
                if self.restart_chunk_groups > 0:
                    self.restart_chunk_groups -= 1
                    self._groups.pop(gid, None)
                    return FakeResponse(409, {"error": "chunk_group_restart"})
                self._groups.setdefault(gid, []).append(data)
                total = int(hdr["total_chunks"]) if hdr else 1
                if len(self._groups[gid]) < total:
                    return FakeResponse(200, {})
                frame = wire.decode_byte_chunks(self._groups.pop(gid), kind="request")
                body = wire.loads(frame)
            rid = self._new_id("r")
            self.requests[rid] = self._events_for(op, body or {}, params)
            return FakeResponse(200, {"request_id": rid})
        m = re.fullmatch(r"/requests/([^/]+)/events", path)
        if m:
            evs = self.requests.get(m.group(1))
            if evs is None:
                return FakeResponse(404, {"error": "no such request"})
            cur = int(params.get("cursor", 0))
            return FakeResponse(200, {"events": [e for e in evs if e["seq"] >= cur][:2]})
        return FakeResponse(404, {"error": f"no route {method} {path}"})

    def _result(self, op: str, body: dict, params: dict) -> dict:
        if op in ("forward-backward", "forward_backward"):
            n = int(body["batch"]["input_ids"].shape[0])
            return {"avg_loss": 0.25, "metrics": {"actor/pg_loss": 0.25, "n": n}, "sub_job_id": params.get("sub_job_id")}
        if op == "forward":
            import torch
            ids = body["batch"]["input_ids"]
            return {"batch": {"log_probs": torch.zeros(ids.shape[0], 3)}, "sub_job_id": params.get("sub_job_id")}
        if op == "generate":
            n = int((body.get("sampling_params") or {}).get("n", 1))
            return {"results": [{"token_ids": [1, 2], "prompt_index": i, "finish_reason": "length"}
                                for i in range(len(body["prompts"])) for _ in range(n)]}
        if op == "step":
            return {"metrics": {"grad_norm": 1.5, "last_lr": body.get("learning_rate") or 1e-6}}
        if op == "fail":
            raise RuntimeError("engine exploded")
        if op in ("tail-logs", "zmd-events"):
            feed, key, cap = (self.logs, "entries", "max_lines") if op == "tail-logs" else (self.events, "events", "max_events")
            cur = int(body.get("cursor") or 0)
            page = feed[cur:cur + int(body.get(cap) or 2)]
            return {key: page, "next_cursor": str(cur + len(page)), "eof": cur + len(page) >= len(feed)}
        return {"status": "ok", "op": op, "body": {k: v for k, v in body.items() if not hasattr(v, "shape")}}

    def _events_for(self, op, body, params) -> List[dict]:
        try:
            res = self._result(op, body, params)
        except RuntimeError as exc:
            return [{"seq": 0, "type": "progress"}, {"seq": 1, "type": "error", "message": str(exc)}]
        frame = wire.dumps(res)
        evs = [{"seq": 0, "type": "progress"}]
        if self.chunk_results_over and len(frame) > self.chunk_results_over:
            for c in wire.encode_byte_chunks(frame, kind="result", operation=op, max_bytes=self.chunk_results_over):
                evs.append({"seq": len(evs), "type": "result_chunk", "data": base64.b64encode(c).decode()})
            evs.append({"seq": len(evs), "type": "result"})
        else:
            evs.append({"seq": len(evs), "type": "result", "data": base64.b64encode(frame).decode()})
        return evs
