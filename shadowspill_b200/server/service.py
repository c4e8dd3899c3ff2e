"""Training service: HTTP endpoint, run creation, live runs, durable records.

``Server(service_root).serve()`` listens on loopback (or a given address),
authenticates with a bearer token when one is configured, creates runs in
background threads (resolve settings -> admission lease -> worker group ->
controller), and answers the REST surface a ``ServiceClient`` speaks. All heavy
work happens in worker processes; this process never touches a GPU beyond
inventory. Reference: packages/engine/src/shadowspill/server/{service.py:33,334,
http.py:179,373-520, jobs.py, live.py, routes/*.py}.
"""
from __future__ import annotations

import json
import os
import re
import threading
import time
import traceback
import urllib.parse
import uuid
from dataclasses import asdict
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from pathlib import Path
from typing import Any

from ..client.protocol import OperationResult, decode_microbatches, encode_microbatches
from ..orchestration.nodes import AdmissionError, Membership, NodeAdmission, device_inventory
from ..training.components import default_registry, resolve_training
from ..training.controller import Rejected, RunController
from ..training.group import WorkerFailure, WorkerGroup
from .journal import Journal

GIB = 1 << 30
_NAME = re.compile(r"^[A-Za-z0-9._-]+$")


def safe_name(name: Any, what: str) -> str:
    """A client-supplied name that becomes one path component under the service root."""
    if not isinstance(name, str) or not _NAME.match(name) or name in (".", ".."):
        raise ValueError(f"{what} name {name!r} is not allowed: use letters, digits, '.', '_' and '-'")
    return name


class LiveRun:
    """One run: its workers, controller, journal and observations."""

    def __init__(self, server: "Server", session: str, run: str, body: dict[str, Any]):
        self.server, self.session, self.run, self.body = server, session, run, body
        self.dir = server.root / "runs" / session / run
        self.dir.mkdir(parents=True, exist_ok=True)
        self.journal = Journal(self.dir / "journal")
        self.state, self.error = "preparing", ""
        self.progress: list[str] = []
        self.metrics: list[dict[str, Any]] = []
        self.group: WorkerGroup | None = None
        self.controller: RunController | None = None
        self.resolved = None
        self.lease: str | None = None
        self.plan_summary: dict[str, Any] = {}
        self.operation_plans: dict[str, dict[str, Any]] = {}     # further operations' plans
        self.plan_names: dict[str, str] = {}
        self.checkpoints: dict[str, str] = {}
        self.thread = threading.Thread(target=self._create, name=f"create-{run}", daemon=True)
        self.thread.start()

    def log(self, msg: str) -> None:
        stamp = time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
        self.progress.append(f"{stamp} [run={self.run} +{time.monotonic() - self.server.t0:.1f}s] {msg}")

    def _create(self) -> None:
        try:
            self.journal.append("created", {"session": self.session, "run": self.run})
            self.log("resolving settings")
            weights = (self.body.get("model") or {}).get("weights") or {}
            if weights.get("source") == "artifact":
                # an uploaded TAR of a Hugging Face directory: unpack once, then it is a checkpoint path
                where = self.server.unpack_artifact(weights["location"])
                self.body["model"]["weights"] = dict(weights, source="checkpoint", location=str(where))
                self.log(f"weights artifact {weights['location']} unpacked")
            self.resolved = resolve_training(self.body, self.server.registry, self.server.hardware)
            r = self.resolved
            host_bytes = int(r.budgets["spill_gib"] * GIB) * r.workers
            gpus = r.workers if r.setups[0]["device"] == "cuda" else 0
            self.lease, devices = self.server.admission.lease(gpus, host_bytes)
            for setup, dev in zip(r.setups, devices or [0] * r.workers):
                setup["device_index"] = dev
            # prepared bundle: written by this run's rank 0, or reused from the run named in
            # "plans" (same session) when its identity matches these settings
            source = self.body.get("plans")
            bundle_dir = (self.server.root / "runs" / self.session / str(source)) if source else self.dir
            r.setups[0]["bundle"] = str(bundle_dir / "training.ssp")
            imported = self.body.get("plans_artifact")
            if imported and not source:
                # a bundle exported from another run or service (PlansHandle.export): unpack it here;
                # the worker reuses it only if its identity matches these settings, else prepares anew
                self.server.unpack_bundle(str(imported), Path(r.setups[0]["bundle"]))
                self.log(f"prepared bundle taken from artifact {imported}")
            if (self.body.get("preparation") or {}).get("separate_processes") and not source \
                    and not Path(r.setups[0]["bundle"]).exists():
                # build, profile, communicate and plan as four fresh processes; the worker then opens
                # the bundle and carries nothing of them (training/phases.py)
                from ..training.phases import prepare_job, setup_from_json
                self.log("preparing in separate processes: build, profile, communicate, plan")
                made = prepare_job(setup_from_json(r.setups[0]), self.dir / "preparation", log=self.log)
                import shutil
                shutil.copyfile(made, r.setups[0]["bundle"])
            ckpt = self.body.get("checkpoint")
            if ckpt:
                ckpt = self.server.resolve_checkpoint(self.session, ckpt)
            self.log(f"starting {r.workers} worker(s): build, profile, plan")
            self.group = WorkerGroup(r.setups, self.dir / "logs", checkpoint=ckpt,
                                     on_progress=self.log)
            self.plan_summary = self.group.ready_info[0].get("plan_summary", {})
            self.operation_plans = self.group.ready_info[0].get("operation_plans", {})
            self.journal.append("ready", {"workers": r.workers, "plan": self.plan_summary})
            if self.body.get("prepare_only"):
                self.group.stop()
                self.group = None
                self.server.admission.release(self.lease)
                self.state = "prepared"
                return
            self.controller = RunController(self._execute, self.journal,
                                            idle_timeout=float(self.body.get("execution", {})
                                                               .get("idle_timeout_seconds", 0) or 0))
            # a run restored from a checkpoint continues that checkpoint's update count
            self.controller.state.b.completed_updates = int(
                self.group.ready_info[0].get("completed_updates", 0))
            self.state = "ready"
            self.log("ready")
        except Exception as exc:  # noqa: BLE001
            self.error = f"{type(exc).__name__}: {exc}"
            self.state = "failed"
            self.log("failed: " + self.error)
            self.journal.append("failed", {"error": self.error, "traceback": traceback.format_exc()[-2000:]})
            self.release()

    def _execute(self, req: dict[str, Any], payload: bytes | None) -> dict[str, Any]:
        op, args = req["operation"], dict(req.get("arguments", {}))
        payloads = None
        if payload is not None:
            from ..training.inputs import InputError, route, validate_microbatches
            mbs = decode_microbatches(payload)
            w, per = self.resolved.workers, self.resolved.geometry["microbatches"]
            try:
                validate_microbatches(mbs, self.resolved.geometry)      # authoritative, before any worker
            except InputError as exc:
                raise WorkerFailure(f"batch rejected: {exc}", "not_started") from None
            payloads = [encode_microbatches(part) for part in route(mbs, w, per)]
        if op in ("save", "export"):
            name = args.get("name") or uuid.uuid4().hex[:8]
            try:
                args["directory"] = str(self.server.checkpoint_directory(self.session, name))
            except ValueError as exc:           # refused before any worker hears of it
                raise WorkerFailure(str(exc), "not_started") from None
            self.checkpoints[name] = args["directory"]
            self.journal.append("checkpoint", {"name": name, "directory": args["directory"]})
            op_worker = "save"
        elif op == "restore":
            try:
                args["directory"] = self.server.resolve_checkpoint(self.session, args["name"])
            except (ValueError, FileNotFoundError) as exc:
                raise WorkerFailure(str(exc), "not_started") from None
            op_worker = "restore"
        elif op == "plan_report":
            args["directory"] = str(self.dir / "plan_report")
            op_worker = op
        elif op == "step" and args.get("runtime_trace"):
            if not (self.body.get("execution") or {}).get("runtime_trace"):
                raise WorkerFailure("a traced step needs Execution(runtime_trace=True) at creation", "not_started")
            args["trace_directory"] = str(self.dir / f"trace_{req['request_id']}")
            op_worker = op
        else:
            op_worker = op
        t0 = time.perf_counter()
        replies = self.group.execute(req["request_id"], op_worker, args, payloads)
        out: dict[str, Any] = {"execution_seconds": max(r.get("execution_seconds", 0.0) for r in replies)}
        losses = [r["loss"] for r in replies if r.get("loss") is not None]
        if losses:
            out["loss"] = float(sum(losses))          # objectives sum; weights already carry 1/N
        out["metrics"] = {"wall_seconds": time.perf_counter() - t0,
                          **{k: v for k, v in (replies[0].get("metrics") or {}).items()}}
        out["outputs"] = replies[0].get("outputs", {})
        if op == "forward":
            # microbatches were routed to the workers in order: their outputs concatenate the same way
            per = [a for r in replies for a in (r.get("outputs") or {}).get("per_microbatch", [])]
            if per:
                out["outputs"] = {"per_microbatch": per}
        if op in ("save", "export"):
            out["outputs"] = {"checkpoint": args.get("name"), "directory": args["directory"]}
        if op == "step" and args.get("trace_directory"):
            out["outputs"] = dict(out.get("outputs") or {},
                                  trace=self.server.pack_directory(Path(args["trace_directory"]), "trace"))
        if op == "plan_report":
            # index.html, occupancy.html, tasks.csv, transfers.csv, timeline.*: one downloadable archive
            out["outputs"] = self.server.pack_directory(Path(args["directory"]), "plan_report")
        # the metric journal: one record per finished request of any operation, in completion order
        self.metrics.append({"position": len(self.metrics) + 1, "source": "service", "operation": op,
                             "request_id": req["request_id"], "update": replies[0].get("completed_updates"),
                             "loss": out.get("loss"), "execution_seconds": out["execution_seconds"],
                             "values": {k: v for k, v in out["metrics"].items() if isinstance(v, (int, float))}})
        if op == "close":
            self.state = "closed"
            self.journal.append("closed", {})
            threading.Thread(target=self.release, daemon=True).start()
        return out

    def release(self) -> None:
        if self.group is not None:
            try:
                self.group.stop()
            except Exception:  # noqa: BLE001
                pass
            self.group = None
        if self.lease:
            self.server.admission.release(self.lease)
            self.lease = None

    def info(self) -> dict[str, Any]:
        geo = self.resolved.geometry if self.resolved else {}
        return {"session": self.session, "run": self.run, "state": self.state, "error": self.error,
                "workers": self.resolved.workers if self.resolved else 0, "geometry": geo,
                "plan_summary": self.plan_summary, "operation_plans": self.operation_plans,
                "provenance": self.resolved.provenance if self.resolved else {},
                "budgets": self.resolved.budgets if self.resolved else {},
                "state_valid": (self.controller.boundary()["valid"] if self.controller else True),
                "boundary": self.controller.boundary() if self.controller else {}}


class RecoveredRun:
    """What the journal of a run says after the service process that owned it has gone: read-only.

    The run's own journal is replayed record by record (``created``, ``ready``, ``receipt``,
    ``checkpoint``, ``failed``, ``closed``); a run that was neither closed nor failed is
    ``interrupted``: its workers died with the old process, so it accepts no requests, but its
    status, loss history, receipts and checkpoints stay readable, and a new run can start from its
    last checkpoint. Reference: packages/engine/src/shadowspill/server/storage.py:178."""
    controller = None
    group = None

    def __init__(self, server: "Server", session: str, run: str):
        self.server, self.session, self.run = server, session, run
        self.dir = server.root / "runs" / session / run
        self.journal = Journal(self.dir / "journal")
        self.body: dict[str, Any] = {}
        self.state, self.error = "preparing", ""
        self.progress: list[str] = []
        self.metrics: list[dict[str, Any]] = []
        self.checkpoints: dict[str, str] = {}
        self.plan_summary: dict[str, Any] = {}
        self.operation_plans: dict[str, dict[str, Any]] = {}
        self.plan_names: dict[str, str] = {}
        self.completed_updates = 0
        workers = 0
        for rec in self.journal.records():
            kind, data = rec["kind"], rec["data"]
            if kind == "ready":
                self.state, workers = "ready", int(data.get("workers", 0))
                self.plan_summary = dict(data.get("plan") or {})
            elif kind == "receipt":
                if data.get("completed_updates") is not None:
                    self.completed_updates = max(self.completed_updates, int(data["completed_updates"]))
                if data.get("operation") in ("step", "optim_step") and data.get("loss") is not None \
                        and data.get("state") == "completed":
                    self.metrics.append({"update": data.get("completed_updates"), "loss": data["loss"],
                                         "execution_seconds": data.get("execution_seconds")})
            elif kind == "checkpoint":
                self.checkpoints[data["name"]] = data["directory"]
            elif kind == "failed":
                self.state, self.error = "failed", str(data.get("error", ""))
            elif kind == "closed":
                self.state = "closed"
        self.workers = workers
        if self.state in ("preparing", "ready"):
            last = next(reversed(self.checkpoints), None)
            self.error = ("the service restarted while this run was live; "
                          + (f"its last checkpoint is {last!r}" if last else "it had saved no checkpoint")
                          + f" ({self.completed_updates} completed updates)")
            self.state = "interrupted"
            self.journal.append("interrupted", {"reason": "service restart",
                                                "completed_updates": self.completed_updates})

    def info(self) -> dict[str, Any]:
        return {"session": self.session, "run": self.run, "state": self.state, "error": self.error,
                "workers": self.workers, "geometry": {}, "plan_summary": self.plan_summary, "provenance": {},
                "budgets": {}, "state_valid": False, "recovered": True,
                "boundary": {"completed_updates": self.completed_updates, "valid": False}}

    def release(self) -> None:
        """Nothing to release: the workers and the admission lease died with the old process."""


class Server:
    def __init__(self, service_root: str | Path, model_root: str | Path | None = None,
                 host: str = "127.0.0.1", port: int = 0, token: str | None = None, extensions=None):
        self.root = Path(service_root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.model_root = Path(model_root) if model_root else None
        self.host, self.port = host, port
        self.token = token if token is not None else os.environ.get("SHADOWSPILL_TOKEN", "")
        self.node_token = os.environ.get("SHADOWSPILL_NODE_TOKEN", self.token)
        self.registry = default_registry()
        from ..training.extensions import load_extensions
        self.extensions = load_extensions(self.registry, extensions)     # SHADOWSPILL_EXTENSIONS by default
        self.hardware = device_inventory()
        self.admission = NodeAdmission(self.hardware["gpus"], int(self.hardware["host_total_gib"] * GIB))
        self.membership = Membership()
        self.journal = Journal(self.root / "journal")
        self.runs: dict[tuple[str, str], LiveRun] = {}
        self.artifacts: dict[str, dict[str, Any]] = {}
        self.incarnation = uuid.uuid4().hex
        self.t0 = time.monotonic()
        self.httpd: ThreadingHTTPServer | None = None
        self._thread: threading.Thread | None = None
        # recovery: every run the service journal names is rebuilt from its own journal; those
        # that were live when the previous incarnation stopped come back as "interrupted"
        closed = {r["data"].get("run") for r in self.journal.records("run_closed")}
        for rec in self.journal.records("run"):
            session, run = rec["data"].get("session"), rec["data"]["run"]
            if not session or not (self.root / "runs" / session / run / "journal").is_dir():
                continue
            try:
                recovered = RecoveredRun(self, session, run)
            except Exception as exc:  # noqa: BLE001  (a damaged run journal must not stop the service)
                self.journal.append("recovery_failed", {"run": run, "error": f"{type(exc).__name__}: {exc}"})
                continue
            self.runs[(session, run)] = recovered
            if run not in closed:
                self.journal.append("run_closed", {"run": run, "reason": "service restart",
                                                   "state": recovered.state})
        self.journal.append("started", {"incarnation": self.incarnation})

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "Server":
        from .http import make_handler
        if not self.token and self.host not in ("127.0.0.1", "localhost", "::1"):
            raise ValueError("a service that listens beyond loopback needs a bearer token "
                             "(token=... or SHADOWSPILL_TOKEN)")
        self.httpd = ThreadingHTTPServer((self.host, self.port), make_handler(self))
        self.httpd.daemon_threads = True
        self.port = self.httpd.server_address[1]
        self._thread = threading.Thread(target=self.httpd.serve_forever, name="http", daemon=True)
        self._thread.start()
        return self

    def serve(self) -> None:
        self.start()
        try:
            while True:
                time.sleep(3600)
        except KeyboardInterrupt:
            pass
        finally:
            self.close()

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def close(self) -> None:
        for run in list(self.runs.values()):
            if run.controller:
                run.controller.stop()
            run.release()
        if self.httpd:
            self.httpd.shutdown()
            self.httpd.server_close()
            self.httpd = None

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ helpers used by routes
    def create_run(self, session: str, body: dict[str, Any]) -> LiveRun:
        safe_name(session, "session")
        run = uuid.uuid4().hex[:10]
        live = LiveRun(self, session, run, body)
        self.runs[(session, run)] = live
        self.journal.append("run", {"session": session, "run": run})
        return live

    def get_run(self, session: str, run: str) -> LiveRun:
        try:
            return self.runs[(session, run)]
        except KeyError:
            raise KeyError(f"no run {session}/{run}") from None

    def checkpoint_directory(self, session: str, name: str) -> Path:
        """``<root>/checkpoints/<session>/<name>`` for names made of letters, digits, ``.``,
        ``_`` and ``-`` only. Anything else (a separator, ``..``, an absolute path) is refused,
        so a client can neither write nor read outside its own session's checkpoints."""
        base = (self.root / "checkpoints" / safe_name(session, "session")).resolve()
        path = (base / safe_name(name, "checkpoint")).resolve()
        if not path.is_relative_to(base):
            raise ValueError(f"checkpoint name {name!r} leaves the session's directory")
        return path

    def resolve_checkpoint(self, session: str, name: str) -> str:
        path = self.checkpoint_directory(session, name)
        if not path.exists():
            raise FileNotFoundError(f"no checkpoint {name!r} in session {session!r}")
        return str(path)

    def checkpoint_manifests(self, session: str, name: str) -> dict[str, Any]:
        """The manifests of a saved checkpoint (one archive per writing rank) without any tensor
        bytes: what was saved, in which dtype and geometry, at which update."""
        from ..checkpoint.archive import read_manifest
        from ..checkpoint.load import checkpoint_files
        files = checkpoint_files(self.resolve_checkpoint(session, name))
        out = []
        for f in files:
            m = read_manifest(f)
            out.append({"file": f.name, "bytes": f.stat().st_size, "metadata": m.get("metadata", {}),
                        "tensors": len(m.get("tensors", m.get("entries", []))),
                        "names": sorted(e.get("name", "") for e in m.get("tensors", m.get("entries", [])))[:2000]})
        return {"checkpoint": name, "files": out}

    def unpack_artifact(self, artifact: str) -> Path:
        """Extracts an uploaded, sealed TAR artifact under the artifact store and returns the
        directory that holds its ``*.safetensors`` files."""
        import tarfile
        src = self.root / "artifacts" / safe_name(artifact, "artifact")
        if not src.exists():
            raise FileNotFoundError(f"no sealed artifact {artifact!r}")
        dst = self.root / "artifacts" / f"{artifact}.d"
        if not dst.exists():
            tmp = self.root / "artifacts" / f".unpack-{uuid.uuid4().hex}"
            with tarfile.open(src) as tar:
                tar.extractall(tmp, filter="data")        # refuses links and paths outside tmp
            tmp.replace(dst)
        found = sorted(dst.rglob("*.safetensors"))
        if not found:
            raise FileNotFoundError(f"artifact {artifact!r} holds no .safetensors file")
        return found[0].parent

    def checkpoint_artifact(self, session: str, name: str) -> dict[str, Any]:
        """Packs a saved checkpoint (or exported weights) directory into one artifact that the
        client can download with byte ranges; returns its handle. The archive is an
        uncompressed TAR with members in sorted order, so the same checkpoint always gives
        the same bytes and digest."""
        return dict(self.pack_directory(Path(self.resolve_checkpoint(session, name)), name), checkpoint=name)

    def bundle_artifact(self, session: str, run: str) -> dict[str, Any]:
        """The prepared bundle of a run (plans, profiles, calibration: ``training.ssp``) as one
        sealed artifact that another run, or another service, can start from."""
        import shutil
        import tempfile
        bundle = self.root / "runs" / session / run / "training.ssp"
        if not bundle.exists():
            raise FileNotFoundError(f"run {run} has no prepared bundle")
        with tempfile.TemporaryDirectory(dir=self.root) as tmp:
            shutil.copyfile(bundle, Path(tmp) / "training.ssp")
            return dict(self.pack_directory(Path(tmp), "plans"), run=run)

    def unpack_bundle(self, artifact: str, target: Path) -> None:
        import tarfile
        meta = self.artifacts.get(artifact)
        if not meta or not meta.get("complete"):
            raise ValueError(f"artifact {artifact} is unknown or still uploading")
        with tarfile.open(self.root / "artifacts" / artifact) as tar:
            member = next((m for m in tar.getmembers() if m.isfile() and Path(m.name).name == "training.ssp"), None)
            if member is None:
                raise ValueError(f"artifact {artifact} holds no prepared bundle")
            target.parent.mkdir(parents=True, exist_ok=True)
            with tar.extractfile(member) as src, open(target, "wb") as dst:
                import shutil
                shutil.copyfileobj(src, dst)

    def pack_directory(self, directory: Path, name: str) -> dict[str, Any]:
        """``directory`` as one sealed artifact (deterministic TAR under ``name/``); its handle."""
        import hashlib
        import tarfile
        store = self.root / "artifacts"
        store.mkdir(exist_ok=True)
        tmp = store / f".pack-{uuid.uuid4().hex}"
        with tarfile.open(tmp, "w", format=tarfile.PAX_FORMAT) as tar:
            for f in sorted(p for p in directory.rglob("*") if p.is_file()):
                info = tar.gettarinfo(str(f), arcname=str(Path(name) / f.relative_to(directory)))
                info.mtime, info.uid, info.gid, info.uname, info.gname = 0, 0, 0, "", ""
                with open(f, "rb") as fh:
                    tar.addfile(info, fh)
        h = hashlib.sha256()
        with open(tmp, "rb") as fh:
            for block in iter(lambda: fh.read(1 << 20), b""):
                h.update(block)
        digest = h.hexdigest()
        aid = digest[:16]
        tmp.replace(store / aid)
        size = (store / aid).stat().st_size
        self.artifacts[aid] = {"size": size, "sha256": digest, "complete": True}
        return {"artifact": aid, "size": size, "sha256": digest}

    def describe(self, body: dict[str, Any]) -> dict[str, Any]:
        r = resolve_training(body, self.registry, self.hardware)
        params = r.cfg.parameter_count()
        return {"workers": r.workers, "geometry": r.geometry, "budgets": r.budgets,
                "provenance": r.provenance, "parameters": params,
                "state_bytes_per_worker": params * 2 * 3 // r.workers,
                "components": self.registry.list()}
