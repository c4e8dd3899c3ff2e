"""HTTP routes of the training service (``/v1/...``).

    GET  /v1/info                              service identity
    GET  /v1/hardware                          node inventory + admission state
    POST /v1/training/describe                 resolve settings, preview workers (no reservation)
    GET  /v1/components?kind=                  registered model / objective / optimizer / policy components
    POST /v1/artifacts                         begin a resumable upload
    PUT  /v1/artifacts/{id}/chunks/{offset}    upload a chunk
    POST /v1/artifacts/{id}/complete           seal (sha256 checked)
    GET  /v1/artifacts/{id}                    download (Range supported), DELETE removes
    POST /v1/runs/{session}                    create a run (202 while preparing)
    GET  /v1/runs/{session}/{run}              run info
    GET  .../progress?after=N                  preparation / startup log lines
    GET  .../checkpoints                       names saved by this run
    POST .../checkpoints/{name}/artifact       pack a checkpoint into a downloadable artifact
    GET|POST .../plans , POST .../plans/report plan names, summaries, HTML plan report
    GET  .../nsys?rank=                        Nsight capture status and report path
    POST .../writers/{writer_id}               attach as writer (fences earlier writers)
    POST .../requests                          register an operation request (idempotent by digest)
    PUT  .../requests/{id}/input               input payload (429 = back-pressure, retry)
    GET  .../requests/{id}?wait=completed&timeout=S   status / long poll
    GET|POST .../metrics , POST .../report     metric pages, caller metrics, run report
    POST /v1/nodes/{join,heartbeat,poll,receipt,leave,reconcile}   node-daemon membership (node credential)

Reference: packages/engine/src/shadowspill/server/http.py:448-520 and routes/*.py.
"""
from __future__ import annotations

import hashlib
import json
import re
import urllib.parse
from dataclasses import asdict
from http.server import BaseHTTPRequestHandler

from . import reference_protocol as refproto
from ..orchestration.nodes import AdmissionError
from ..training.controller import Rejected

MAX_BODY = 1 << 31


class HTTPError(Exception):
    def __init__(self, status: int, message: str):
        self.status, self.message = status, message


def make_handler(server):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *args):  # quiet
            pass

        # ------------------------------------------------------------------ plumbing
        def _body(self) -> bytes:
            n = int(self.headers.get("Content-Length") or 0)
            if n > MAX_BODY:
                raise HTTPError(413, "body too large")
            return self.rfile.read(n) if n else b""

        def _json(self) -> dict:
            raw = self._body()
            try:
                return json.loads(raw) if raw else {}
            except json.JSONDecodeError:
                raise HTTPError(400, "body is not JSON") from None

        def _send(self, status: int, payload, content_type: str = "application/json", headers=None):
            if content_type == "application/json" and refproto.wants_control(self.headers):
                # the reference client accepts only its own envelope: errors become service.error
                # records, routes without a translated record say so by name
                content_type = refproto.CONTROL_MEDIA_TYPE
                if status >= 400:
                    payload = refproto.service_error(status, (payload or {}).get("error", ""))
                elif not isinstance(payload, bytes):
                    status = 501
                    payload = refproto.service_error(501, f"{self.command} {self.path.split('?')[0]}: this server "
                                                          "has no reference-protocol record for this route")
            data = payload if isinstance(payload, bytes) else json.dumps(payload).encode()
            self.send_response(status)
            self.send_header("Content-Type", content_type)
            self.send_header("Content-Length", str(len(data)))
            for k, v in (headers or {}).items():
                self.send_header(k, v)
            self.end_headers()
            self.wfile.write(data)

        def _auth(self, node: bool = False) -> None:
            want = server.node_token if node else server.token
            if not want:
                return
            got = self.headers.get("Authorization", "")
            if got != f"Bearer {want}":
                raise HTTPError(401, "missing or wrong bearer token")

        def _serve(self, method: str) -> None:
            try:
                url = urllib.parse.urlparse(self.path)
                q = {k: v[0] for k, v in urllib.parse.parse_qs(url.query).items()}
                parts = [p for p in url.path.split("/") if p]
                if len(parts) < 2 or parts[0] != "v1":
                    raise HTTPError(404, "unknown path")
                self._auth(node=parts[1] == "nodes")
                self._dispatch(method, parts[1:], q)
            except HTTPError as exc:
                self._send(exc.status, {"error": exc.message})
            except Rejected as exc:
                self._send(409, {"error": str(exc)})
            except AdmissionError as exc:
                self._send(503, {"error": str(exc)})
            except BlockingIOError as exc:
                self._send(429, {"error": str(exc), "backpressure": True})
            except (KeyError, FileNotFoundError) as exc:
                self._send(404, {"error": str(exc)})
            except (ValueError, TypeError) as exc:
                self._send(400, {"error": f"{type(exc).__name__}: {exc}"})
            except Exception as exc:  # noqa: BLE001
                self._send(500, {"error": f"{type(exc).__name__}: {exc}"})

        def do_GET(self): self._serve("GET")
        def do_POST(self): self._serve("POST")
        def do_PUT(self): self._serve("PUT")
        def do_DELETE(self): self._serve("DELETE")

        # ------------------------------------------------------------------ routes
        def _dispatch(self, method: str, p: list[str], q: dict) -> None:
            head = p[0]
            control = refproto.wants_control(self.headers)
            if control and head == "info" and method == "GET":
                return self._send(200, refproto.service_info(server.incarnation, "local"),
                                  refproto.CONTROL_MEDIA_TYPE)
            if control and head == "hardware" and method == "GET":
                return self._send(200, refproto.hardware_inventory(server.hardware, server.admission.snapshot()),
                                  refproto.CONTROL_MEDIA_TYPE)
            if head == "info" and method == "GET":
                return self._send(200, {"service": "shadowspill-b200", "incarnation": server.incarnation,
                                        "owner": "local", "api": 1})
            if head == "hardware" and method == "GET":
                return self._send(200, {"nodes": [dict(server.hardware, node="local",
                                                       admission=server.admission.snapshot())],
                                        "members": server.membership.live()})
            if head == "training" and p[1:] == ["describe"] and method == "POST":
                return self._send(200, server.describe(self._json()))
            if head == "components" and method == "GET":
                return self._send(200, {"components": server.registry.list(q.get("kind"))})
            if head == "artifacts":
                return self._artifacts(method, p[1:], q)
            if head == "nodes" and method == "POST":
                return self._nodes(p[1], self._json())
            if head == "runs":
                return self._runs(method, p[1:], q)
            raise HTTPError(404, "unknown route")

        def _nodes(self, action: str, body: dict) -> None:
            m = server.membership
            if action == "join":
                return self._send(200, {"incarnation": m.join(body["node_id"], body.get("info"))})
            if action == "heartbeat":
                ok = m.heartbeat(body["node_id"], body["incarnation"])
                return self._send(200 if ok else 410, {"ok": ok})
            if action == "leave":
                return self._send(200, {"ok": m.leave(body["node_id"], body["incarnation"])})
            if action == "poll":
                cmds = m.poll(body["node_id"], body["incarnation"])
                return self._send(200 if cmds is not None else 410,
                                  {"commands": cmds or [], "ok": cmds is not None})
            if action == "receipt":
                ok = m.receipt(body["node_id"], body["incarnation"], body["command"], body.get("outcome"))
                return self._send(200 if ok else 404, {"ok": ok})
            if action == "reconcile":
                return self._send(200, {"fenced": m.reconcile(), "live": m.live()})
            raise HTTPError(404, "unknown node action")

        def _artifacts(self, method: str, p: list[str], q: dict) -> None:
            store = server.root / "artifacts"
            store.mkdir(exist_ok=True)
            if method == "POST" and not p:
                body = self._json()
                aid = hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()[:16]
                server.artifacts.setdefault(aid, {"size": int(body.get("size", 0)),
                                                  "sha256": body.get("sha256", ""), "complete": False})
                (store / f"{aid}.part").touch()
                have = (store / f"{aid}.part").stat().st_size
                return self._send(200, {"artifact": aid, "received": have})
            aid = p[0]
            meta = server.artifacts.get(aid)
            if meta is None and not (store / aid).exists():
                raise HTTPError(404, "unknown artifact")
            if method == "PUT" and len(p) == 3 and p[1] == "chunks":
                off = int(p[2])
                part = store / f"{aid}.part"
                if off != part.stat().st_size:
                    return self._send(409, {"error": "chunk offset mismatch", "received": part.stat().st_size})
                with open(part, "ab") as f:
                    f.write(self._body())
                return self._send(200, {"received": part.stat().st_size})
            if method == "POST" and p[1:] == ["complete"]:
                part = store / f"{aid}.part"
                digest = hashlib.sha256(part.read_bytes()).hexdigest()
                if meta["sha256"] and digest != meta["sha256"]:
                    raise HTTPError(422, "artifact digest mismatch")
                part.rename(store / aid)
                meta["complete"] = True
                return self._send(200, {"artifact": aid, "sha256": digest})
            if method == "GET":
                target = store / aid
                size = target.stat().st_size
                rng = self.headers.get("Range")
                if rng:
                    m = re.match(r"bytes=(\d+)-(\d*)", rng)
                    if not m:
                        raise HTTPError(400, "bad Range header")
                    lo = int(m.group(1))
                    hi = min(int(m.group(2)) if m.group(2) else size - 1, size - 1)
                    if lo >= size:
                        return self._send(416, {"error": "range starts past the end", "size": size})
                    with open(target, "rb") as f:      # only the requested window is read
                        f.seek(lo)
                        data = f.read(hi - lo + 1)
                    return self._send(206, data, "application/octet-stream",
                                      {"Content-Range": f"bytes {lo}-{hi}/{size}"})
                data = target.read_bytes()
                return self._send(200, data, "application/octet-stream",
                                  {"ETag": hashlib.sha256(data).hexdigest()})
            if method == "DELETE":
                (store / aid).unlink(missing_ok=True)
                server.artifacts.pop(aid, None)
                return self._send(200, {"deleted": aid})
            raise HTTPError(404, "unknown artifact route")

        def _runs(self, method: str, p: list[str], q: dict) -> None:
            if len(p) == 1 and method == "POST":
                live = server.create_run(p[0], self._json())
                return self._send(202, live.info())
            if len(p) < 2:
                raise HTTPError(404, "unknown run route")
            live = server.get_run(p[0], p[1])
            rest = p[2:]
            if not rest and method == "GET":
                return self._send(200 if live.state != "preparing" else 202, live.info())
            if len(rest) == 3 and rest[0] == "checkpoints" and rest[2] == "artifact" and method == "POST":
                try:
                    return self._send(200, server.checkpoint_artifact(p[0], rest[1]))
                except FileNotFoundError as exc:
                    raise HTTPError(404, str(exc)) from None
            if len(rest) == 3 and rest[0] == "checkpoints" and rest[2] == "manifest" and method == "GET":
                try:
                    return self._send(200, server.checkpoint_manifests(p[0], rest[1]))
                except FileNotFoundError as exc:
                    raise HTTPError(404, str(exc)) from None
            if rest == ["checkpoints"] and method == "GET":
                return self._send(200, {"checkpoints": sorted(live.checkpoints)})
            if rest == ["progress"]:
                after = int(q.get("after", 0))
                return self._send(200, {"lines": live.progress[after:], "next": len(live.progress)})
            if rest == ["plans"]:
                if method == "POST":
                    body = self._json()
                    live.plan_names[body["name"]] = body.get("plan", "step")
                    return self._send(200, {"plans": live.plan_names})
                if "name" in q:                       # the plan a name was given to
                    op = live.plan_names.get(q["name"])
                    if op is None:
                        raise HTTPError(404, f"no plan named {q['name']!r}")
                    summary = live.plan_summary if op == "step" else live.operation_plans.get(op)
                    if summary is None:
                        raise HTTPError(404, f"plan {q['name']!r} names operation {op!r}, which this run did not plan")
                    return self._send(200, {"name": q["name"], "operation": op, "plan": summary})
                page = int(q.get("page", 0))
                rows = [{"operation": "step", **live.plan_summary}]
                rows += [{"operation": op, **summary} for op, summary in sorted(live.operation_plans.items())]
                return self._send(200, {"plans": rows[page * 32:(page + 1) * 32], "names": live.plan_names})
            if rest == ["plans", "artifact"] and method == "POST":
                try:
                    return self._send(200, server.bundle_artifact(p[0], p[1]))
                except FileNotFoundError as exc:
                    raise HTTPError(404, str(exc)) from None
            if rest == ["plans", "report"] and method == "POST":
                return self._send(200, {"summary": live.plan_summary,
                                        "note": "workers write full HTML reports with write_report"})
            if rest == ["nsys"]:
                from ..orchestration import capture
                wanted = capture.NsysOptions.from_json((live.body.get("execution") or {}).get("nsys"))
                return self._send(200, capture.status(live.dir / "logs", int(q.get("rank", 0)), wanted))
            if len(rest) == 2 and rest[0] == "writers" and method == "POST":
                self._require_ready(live)
                live.controller.attach_writer(rest[1])
                return self._send(200, {"writer": rest[1]})
            if rest == ["requests"] and method == "POST":
                self._require_ready(live)
                res = live.controller.register(self._json())
                return self._send(200, asdict(res))
            if len(rest) == 3 and rest[0] == "requests" and rest[2] == "input" and method == "PUT":
                self._require_ready(live)
                live.controller.receive(rest[1], self._body())
                return self._send(200, {"received": True})
            if len(rest) == 2 and rest[0] == "requests" and method == "GET":
                self._require_ready(live)
                timeout = float(q.get("timeout", 0)) if q.get("wait") == "completed" else 0.0
                return self._send(200, asdict(live.controller.wait(rest[1], min(timeout, 120.0))))
            if rest == ["metrics"]:
                if method == "POST":
                    row = dict(self._json(), source="caller", position=len(live.metrics) + 1)
                    live.metrics.append(row)
                    return self._send(200, {"count": len(live.metrics), "record": row})
                # journal positions count from 1; a page covers (after, through]
                after, limit = int(q.get("after", 0)), int(q.get("limit", 1000))
                end = len(live.metrics)
                through = min(end, int(q["through"])) if "through" in q else end
                if after < 0 or limit < 1 or through < after:
                    raise HTTPError(400, "metric cursor exceeds its snapshot")
                stop = min(through, after + limit)
                return self._send(200, {"metrics": live.metrics[after:stop], "next": stop,
                                        "after": after, "through": through,
                                        "next_cursor": stop if stop < through else None})
            if rest == ["report"] and method == "POST":
                return self._send(200, {"run": live.info(), "metrics": live.metrics[-1000:],
                                        "receipts": live.journal.records("receipt")[-1000:]})
            raise HTTPError(404, "unknown run route")

        @staticmethod
        def _require_ready(live) -> None:
            if live.controller is None:
                raise HTTPError(409, f"run is {live.state}")

    return Handler
