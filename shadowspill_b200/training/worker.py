"""Worker process: one rank of a run.

Started by the service as ``python -m shadowspill_b200.training.worker
--control-fd R,W``. It receives a ``launch`` frame with the resolved setup, opens
a ``TrainingSession`` (build, profile, plan, executor), reports ``ready`` and then
serves two-phase commands: a ``call`` is *staged* (inputs decoded and validated,
reply ``ready``) and runs only when the matching ``control`` frame says
``execute``; ``abort`` drops it with the state untouched. A reply names the
effect on training state: ``not_started``, ``completed`` or ``unknown`` (a
failure after execution began), and an unknown effect is never retried.
Reference: packages/engine/src/shadowspill/training/worker/{bootstrap.py:28,111,
loop.py:71-181, protocol.py}.
"""
from __future__ import annotations

import os as _os

# task workspaces come from the caching allocator under a hard cap: expandable segments keep
# fragmentation from turning a fitting plan into an allocation failure
_os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import argparse
import os
import sys
import time
import traceback

from .channel import Channel, ChannelClosed


def _to_host_batches(payload: bytes):
    from ..client.protocol import decode_microbatches
    from ..data.synthetic import HostMicrobatch
    return [HostMicrobatch(m.tokens, m.targets, m.weights, m.positions, m.cu_seqlens, m.max_seqlen,
                           dict(getattr(m, "extras", None) or {}))
            for m in decode_microbatches(payload)]


def serve(chan: Channel) -> int:
    header, _ = chan.recv()
    if header.get("type") != "launch":
        chan.send({"type": "failed", "error": "expected a launch frame"})
        return 2
    rank, world = int(header["rank"]), int(header["world_size"])
    log = lambda msg: chan.send({"type": "progress", "rank": rank, "message": msg})
    session = None
    window = None
    try:
        import torch
        setup_json = header["setup"]
        if world > 1:
            import torch.distributed as dist
            os.environ.update(MASTER_ADDR=header["master_addr"], MASTER_PORT=str(header["master_port"]),
                              RANK=str(rank), WORLD_SIZE=str(world))
            cuda = setup_json["device"] == "cuda"
            if cuda:
                torch.cuda.set_device(setup_json["device_index"])
            dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        from ..models.config import DecoderConfig
        from ..planning.plan import SearchOptions
        from .session import TrainingSession, TrainingSetup
        kw = dict(setup_json)
        from ..orchestration import capture
        nsys = capture.NsysOptions.from_json(kw.pop("nsys", None))
        if nsys is not None and capture.available(nsys):
            barrier = (lambda: dist.barrier()) if world > 1 else None
            window = capture.StepWindow(nsys, barrier=barrier)
        if isinstance(kw.get("model"), dict):
            kw["model"] = DecoderConfig.from_json(kw["model"])
        kw["search"] = SearchOptions(**kw.get("search", {}))
        for k in ("walks", "recompute_shares", "operations"):
            if k in kw:
                kw[k] = tuple(kw[k])
        kw["search"].strategies = tuple(kw["search"].strategies)
        kw["search"].fetch_rules = tuple(kw["search"].fetch_rules)
        session = TrainingSession(TrainingSetup(**kw), log=log)
        if header.get("checkpoint"):
            session.restore(header["checkpoint"])
        from dataclasses import asdict
        chan.send({"type": "ready", "rank": rank, "plan_summary": asdict(session.plan.summary),
                   "operation_plans": {op: asdict(pl.summary)
                                       for op, (pl, _) in getattr(session, "extra_plans", {}).items()},
                   "slots": session.slots, "timings": session.timings,
                   "completed_updates": session.executor.completed_updates,
                   "operations": session.executor.operations()})
    except Exception as exc:  # noqa: BLE001
        chan.send({"type": "failed", "rank": rank, "error": f"{type(exc).__name__}: {exc}",
                   "traceback": traceback.format_exc()})
        return 1
    staged = None
    while True:
        try:
            header, payload = chan.recv()
        except ChannelClosed:
            break
        kind = header.get("type")
        if kind == "call":
            try:
                op = header["operation"]
                batch = _to_host_batches(payload) if payload else None
                if op in ("step", "forward_backward", "forward") and batch is None:
                    raise ValueError(f"{op} needs an input batch")
                staged = (header, batch)
                chan.send({"type": "reply", "state": "ready", "request_id": header["request_id"]})
            except Exception as exc:  # noqa: BLE001
                staged = None
                chan.send({"type": "reply", "state": "failed", "effect": "not_started",
                           "request_id": header.get("request_id"), "error": f"{type(exc).__name__}: {exc}"})
        elif kind == "control":
            if staged is None or header.get("request_id") != staged[0]["request_id"]:
                chan.send({"type": "reply", "state": "failed", "effect": "not_started",
                           "request_id": header.get("request_id"), "error": "nothing staged"})
                continue
            call, batch = staged
            staged = None
            if header.get("action") != "execute":
                chan.send({"type": "reply", "state": "aborted", "effect": "not_started",
                           "request_id": call["request_id"]})
                continue
            started = False
            t0 = time.perf_counter()
            try:
                op, args = call["operation"], call.get("arguments", {})
                out = {"loss": None, "metrics": {}, "outputs": {}}
                if args.get("lr") is not None:
                    session.executor.hyper.lr = float(args["lr"])
                if op in ("step", "forward_backward", "forward", "optim_step"):
                    if op in ("optim_step", "step"):
                        session.executor.hyper.grad_scale = float(args.get("grad_scale") or 1.0)
                    started = True
                    if window is not None and op != "optim_step":
                        window.before_step()
                    if op == "step" and args.get("runtime_trace") and args.get("trace_directory"):
                        # per-task device clocks + the runtime's trace ring -> runtime.html etc.
                        res, _ = session.traced_step(batch, f"{args['trace_directory']}/rank{rank}")
                    else:
                        res = session.run(op, batch)
                    if window is not None and op != "optim_step":
                        window.after_step()
                    out["loss"] = res.loss if op != "optim_step" else None
                    if op == "forward" and res.outputs:
                        from ..client.protocol import encode_array
                        out["outputs"] = {"per_microbatch": [encode_array(a) for a in res.outputs]}
                    out["metrics"] = {"tokens": res.tokens, "device_seconds": res.device_seconds,
                                      **{k: float(v) for k, v in (res.metrics or {}).items()}}
                elif op == "discard":
                    session.executor.discard_gradients()
                elif op == "save":
                    started = True
                    path = session.save(args["directory"], args.get("metadata"))
                    out["outputs"] = {"path": str(path)}
                elif op == "plan_report":
                    if rank == 0:          # one plan for the whole job: rank 0 renders it
                        session.write_plan_report(args["directory"])
                    out["outputs"] = {"path": args["directory"]}
                elif op == "restore":
                    started = True
                    out["outputs"] = {"metadata": session.restore(args["directory"])}
                elif op == "close":
                    chan.send({"type": "reply", "state": "completed", "effect": "completed",
                               "request_id": call["request_id"], "completed_updates":
                               session.executor.completed_updates, "execution_seconds": 0.0})
                    break
                else:
                    raise ValueError(f"unknown operation {op!r}")
                chan.send({"type": "reply", "state": "completed", "effect": "completed",
                           "request_id": call["request_id"],
                           "completed_updates": session.executor.completed_updates,
                           "execution_seconds": time.perf_counter() - t0, **out})
            except Exception as exc:  # noqa: BLE001
                chan.send({"type": "reply", "state": "failed",
                           "effect": "unknown" if started else "not_started",
                           "request_id": call["request_id"], "error": f"{type(exc).__name__}: {exc}",
                           "traceback": traceback.format_exc()})
        elif kind == "shutdown":
            break
    try:
        if session is not None:
            session.close()
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        pass
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--control-fd", required=True, help="READ,WRITE file descriptors")
    a = ap.parse_args(argv)
    r, w = (int(x) for x in a.control_fd.split(","))
    return serve(Channel(r, w))


if __name__ == "__main__":
    sys.exit(main())
