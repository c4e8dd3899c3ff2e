"""Qualification gates: ``python -m shadowspill_b200.qualification.gates [suite] [numerical] [twin] [performance] [determinism]``.

suite        the repository's tests for this machine, in child processes

numerical    planned bf16 execution on the GPU (fp32 on CPU) against an independent resident
             trainer on the same data: 5 updates of 2 heterogeneous microbatches, a checkpoint
             saved at update 3 and replayed, tolerances weights rel-L2 <= 2.5 %, cosine >= 0.999,
             sign agreement >= 99 %, near-zero weights within 2*lr; moments rel-L2 <= 5 %.
performance  build -> profile -> plan -> execute; median measured step against the simulated step
             (within 10 %) and, when a floor is recorded for this hardware and configuration,
             at least 95 % of it.

Each gate prints one JSON record and the process exits non-zero if a gate fails. The gate
definitions follow the reference's (qualification/numerical/README.md:199-213,
qualification/performance/README.md:69-100).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import tempfile

import torch

from ..data.synthetic import make_batch, to_device
from ..execution.resident import ResidentTrainer
from ..planning.plan import SearchOptions
from ..training.session import TrainingSession, TrainingSetup


def compare_tensors(a: torch.Tensor, b: torch.Tensor, lr: float, updates: int = 0) -> dict[str, float]:
    """``updates`` > 0: elements the reference left within ``2*lr*updates`` of zero (weights that
    start at zero, such as zero-centered norm gains, move by at most ``lr`` per update) are judged
    by their absolute difference only; the relative measures are taken over the rest."""
    a, b = a.detach().float().reshape(-1).cpu(), b.detach().float().reshape(-1).cpu()
    if updates > 0:
        keep = b.abs() > 2 * lr * updates
        near = float((a[~keep] - b[~keep]).abs().max()) if (~keep).any() else 0.0
        if not keep.any():
            return {"rel_l2": 0.0, "cosine": 1.0, "sign_agreement": 1.0, "near_zero_abs": near}
        a2, b2 = a[keep], b[keep]
        return {"rel_l2": float((a2 - b2).norm() / (b2.norm() + 1e-12)),
                "cosine": float(torch.dot(a2, b2) / (a2.norm() * b2.norm() + 1e-12)),
                "sign_agreement": float((torch.sign(a2) == torch.sign(b2)).float().mean()),
                "near_zero_abs": near}
    rel = float((a - b).norm() / (b.norm() + 1e-12))
    cos = float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))
    big = b.abs() > 2 * lr
    sign = float((torch.sign(a[big]) == torch.sign(b[big])).float().mean()) if big.any() else 1.0
    near = float((a[~big] - b[~big]).abs().max()) if (~big).any() else 0.0
    return {"rel_l2": rel, "cosine": cos, "sign_agreement": sign, "near_zero_abs": near}


def numerical_gate(model: str = "llama3-tiny", device: str = "cpu", updates: int = 5,
                   lr: float = 1e-3) -> dict:
    cpu = device == "cpu"
    T, n_mb = (256, 2) if cpu else (2048, 2)
    setup = TrainingSetup(model=model, device_gib=0.53 if cpu else 8.0, spill_gib=0.25 if cpu else 16.0,
                          tokens_per_step=T * n_mb, microbatch_tokens=T, lr=lr, seed=7, device=device,
                          dtype="float32" if cpu else "bfloat16", stochastic_rounding=False,
                          profile=not cpu, calibrate=not cpu,
                          search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=2))
    session = TrainingSession(setup)
    cfg = session.cfg
    if not cpu:
        # the independent trainer shares this process: lift the session's allocator cap
        torch.cuda.set_per_process_memory_fraction(1.0, setup.device_index)
    ref = ResidentTrainer(cfg, device=device if cpu else "cuda", dtype=session.dtype, seed=7, lr=lr,
                          stochastic_rounding=False)
    # same starting point: the planned run's initial weights (its on-device initialisation
    # draws from another generator than the resident trainer's)
    start = session.executor.state_dict()
    for k, v in ref.state_dict().items():
        v.copy_(start[k].to(v.device))
    del start
    batches = [make_batch(i, vocab=cfg.vocab_size, tokens_per_step=T * n_mb, microbatch_tokens=T,
                          median=60 if cpu else 300, min_len=8, max_len=T // 2, slots=session.slots)
               for i in range(updates)]
    losses, failures = [], []
    with tempfile.TemporaryDirectory() as ckpt:
        for i, b in enumerate(batches):
            got = session.step(b).loss
            want = ref.step([to_device(m, ref.device) for m in b])
            losses.append((got, want))
            if abs(got - want) > (1e-5 if cpu else 2e-2) * max(1.0, abs(want)):
                failures.append(f"loss at update {i + 1}: {got} vs {want}")
            if i == 2:
                session.save(ckpt)
        final = session.executor.state_dict()
        # replay from the checkpoint: updates 4.. must reproduce the same state
        session.restore(ckpt)
        for b in batches[3:]:
            session.step(b)
        replay = session.executor.state_dict()
    worst = {"rel_l2": 0.0, "cosine": 1.0, "sign_agreement": 1.0, "near_zero_abs": 0.0}
    moments, moments_at, moments_embed = 0.0, "", 0.0
    for k, v in ref.state_dict().items():
        m = compare_tensors(final[k], v, lr)
        worst = {"rel_l2": max(worst["rel_l2"], m["rel_l2"]), "cosine": min(worst["cosine"], m["cosine"]),
                 "sign_agreement": min(worst["sign_agreement"], m["sign_agreement"]),
                 "near_zero_abs": max(worst["near_zero_abs"], m["near_zero_abs"])}
    for si, st in enumerate(ref.stages):
        for p in st.params:
            if p.trainable:
                key = f"exp_avg.{st.name}.{p.name}"
                if key in final:
                    rel = compare_tensors(final[key], ref.M[si][p.name], lr)["rel_l2"]
                    if st.kind == "embedding":
                        moments_embed = rel      # its gradient is summed with bf16 atomics (order varies)
                    elif rel > moments:
                        moments, moments_at = rel, key
    replay_diff = max(float((replay[k].float() - final[k].float()).abs().max()) for k in final)
    if worst["rel_l2"] > 0.025 or worst["cosine"] < 0.999 or worst["sign_agreement"] < 0.99:
        failures.append(f"weights outside tolerance: {worst}")
    # a near-zero weight can move by lr per update in either direction
    if worst["near_zero_abs"] > 2 * lr * updates + 1e-7:
        failures.append(f"near-zero weights differ by {worst['near_zero_abs']}")
    if moments > 0.05:
        failures.append(f"first moments rel-L2 {moments} at {moments_at}")
    if moments_embed > 0.10:
        failures.append(f"embedding first moment rel-L2 {moments_embed}")
    # on the GPU a few reductions use atomics, so a replay agrees to rounding, not bit for bit
    if replay_diff > (0.0 if cpu else 2 * lr):
        failures.append(f"checkpoint replay differs by {replay_diff}")
    session.close()
    return {"gate": "numerical", "model": model, "device": device, "updates": updates,
            "weights": worst, "moments_rel_l2": moments, "moments_worst_tensor": moments_at,
            "embedding_moment_rel_l2": moments_embed, "replay_max_abs": replay_diff,
            "losses": losses, "passed": not failures, "failures": failures}


def twin_config(family: str):
    """Small shapes of a family whose head widths the sm_100a attention and DeltaNet kernels take."""
    from dataclasses import replace
    from ..models.config import preset
    if family == "llama3":
        return replace(preset("llama3-tiny"), n_layers=3, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512)
    if family == "qwen35":
        return replace(preset("qwen35-numerical"), n_layers=4, d_model=512, d_ff=1024, n_heads=4, n_kv_heads=2,
                       head_dim=128, dn_qk_heads=2, dn_v_heads=4, vocab_size=2048)
    if family == "olmoe":
        return replace(preset("olmoe-tiny"), n_layers=3, d_model=256, n_heads=4, n_kv_heads=4, head_dim=64)
    raise ValueError(f"no twin configuration for family {family!r}")


def torch_twin_gate(cfg, device: str = "cuda", updates: int = 5, microbatches: int = 2, tokens: int = 1024,
                    lr: float = 3e-4, frontend: str = "stages") -> dict:
    """Planned execution in the model dtype (bf16 on a GPU) against an independent fp32 PyTorch
    model (``models/torch_reference.py``: plain tensor code, no kernel of this package) trained by
    ``torch.optim.AdamW`` on the same data from the same starting weights: ``updates`` updates of
    ``microbatches`` heterogeneous microbatches, forced to spill, at the reference gate's learning
    rate of 3e-4 (tools/planning/cases/full_model.py:24). Tolerances as in the reference's
    numerical gate (qualification/numerical/README.md:199-213): weights rel-L2 <= 2.5 %, cosine >=
    0.999, sign agreement >= 99 %, near-zero weights within 2*lr per update."""
    from ..communication.info import CommunicationInfo
    from ..execution.executor import Executor, Hyperparameters
    from ..frontend.capture import BatchGeometry, StepDataOrdering, build_step
    from ..models import torch_reference as twin
    from ..planning.plan import MemoryBudgets, PlanningError, plan_program
    cpu = device == "cpu"
    dtype = torch.float32 if cpu else torch.bfloat16
    slots = tokens // 32 + 1
    geo = BatchGeometry(microbatch_tokens=tokens, n_microbatches=microbatches, slots=slots, mean_seqlen=tokens / 4)
    from ..frontend.graph_stage import supports
    graph = frontend == "graph" and supports(cfg)
    sel = {i: ("save" if i % 2 else "save_attention") for i in range(1, cfg.n_layers + 1)} if graph else {}
    prog, desc = build_step(cfg, geo, StepDataOrdering(), dtype=dtype, selection=sel,
                            frontend="graph" if graph else "stages")
    total = sum(o.bytes for o in prog.objects)
    ws = max(t.workspace_bytes for t in prog.tasks)
    plan = None
    for pct in range(50, 101, 10):
        try:
            plan = plan_program(prog, MemoryBudgets(4 * ws + total * pct // 100, 4 << 30, headroom_bytes=0),
                                CommunicationInfo(), SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=2))
            break
        except PlanningError:
            continue
    if plan is None:
        raise PlanningError("no budget planned")
    hyper = Hyperparameters(lr=lr, beta2=0.95, weight_decay=0.0)
    ex = Executor(plan, desc, device=device, seed=11, hyper=hyper, stochastic_rounding=False)
    ex.initialize(on_device=False)
    dev = torch.device(device)
    params = {k: v.to(dev, torch.float32).clone().requires_grad_(True)
              for k, v in ex.state_dict().items() if not k.startswith("exp_avg")}
    opt = torch.optim.AdamW(list(params.values()), lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    losses, failures = [], []
    for step in range(updates):
        host = make_batch(100 + step, vocab=cfg.vocab_size, tokens_per_step=tokens * microbatches,
                          microbatch_tokens=tokens, median=tokens / 5, min_len=16, max_len=tokens, slots=slots)
        got = ex.run(host).loss
        opt.zero_grad()
        want = 0.0
        for m in host:
            loss = twin.model_loss(cfg, params, to_device(m, dev))
            loss.backward()
            want += float(loss)
        opt.step()
        losses.append((got, want))
        if abs(got - want) > (1e-5 if cpu else 2e-2) * max(1.0, abs(want)):
            failures.append(f"loss at update {step + 1}: {got} vs {want}")
    state = ex.state_dict()
    worst = {"rel_l2": 0.0, "cosine": 1.0, "sign_agreement": 1.0, "near_zero_abs": 0.0}
    at = {}
    for k, v in params.items():
        m = compare_tensors(state[k], v, lr, updates)
        for name, better in (("rel_l2", max), ("cosine", min), ("sign_agreement", min), ("near_zero_abs", max)):
            new = better(worst[name], m[name])
            if new != worst[name]:
                worst[name], at[name] = new, k
    if worst["rel_l2"] > 0.025 or worst["cosine"] < 0.999 or worst["sign_agreement"] < 0.99:
        failures.append(f"weights outside tolerance: {worst} at {at}")
    if worst["near_zero_abs"] > 2 * lr * updates + 1e-7:
        failures.append(f"near-zero weights differ by {worst['near_zero_abs']} at {at.get('near_zero_abs')}")
    fetched = plan.summary.fetch_bytes
    ex.close()
    per_tensor = {k: compare_tensors(state[k], v, lr, updates)["rel_l2"] for k, v in params.items()}
    worst5 = dict(sorted(per_tensor.items(), key=lambda kv: -kv[1])[:5])
    return {"gate": "torch_twin", "family": cfg.family, "worst_tensors": worst5, "device": device, "updates": updates,
            "frontend": "graph" if graph else "stages", "fetch_bytes": fetched, "weights": worst,
            "worst_at": at, "losses": losses, "passed": not failures, "failures": failures}


# Recorded floors, tokens/s: (device name fragment, model, device GiB, spill GiB, tokens per step).
# Each is a few per cent under the slowest measured run of that configuration on that hardware (boxes
# differ in the clock they sustain under the power cap), so that a pass means "no regression", not luck.
# The reference records its floors the same way per GPU model (qualification/performance/README.md:69-100:
# 3,423 / 3,027 / 13,907 tokens/s for these three models on one RTX 5090).
FLOORS: dict[tuple, float] = {
    ("B200", "llama3-8b", 24.0, 128.0, 65536): 15_800.0,          # measured 16,289 .. 16,667
    ("B200", "qwen35-9b", 24.0, 128.0, 65536): 12_500.0,          # measured 13,127
    ("B200", "olmoe-7b-a1b", 24.0, 128.0, 65536): 45_000.0,       # measured 46,553 .. 48,005
}


def recorded_floor(device_name: str, model: str, device_gib: float, spill_gib: float, tokens: int) -> float | None:
    for (fragment, m, d, s, t), floor in FLOORS.items():
        if fragment in device_name and (m, float(d), float(s), int(t)) == (model, float(device_gib), float(spill_gib), int(tokens)):
            return floor
    return None


def performance_gate(model: str = "llama3-8b", device_gib: float = 24.0, spill_gib: float = 128.0,
                     tokens: int = 65536, microbatch: int = 8192, groups: int = 3, updates: int = 4,
                     floor: float | None = None) -> dict:
    if floor is None and torch.cuda.is_available():
        floor = recorded_floor(torch.cuda.get_device_name(0), model, device_gib, spill_gib, tokens)
    setup = TrainingSetup(model=model, device_gib=device_gib, spill_gib=spill_gib, tokens_per_step=tokens,
                          microbatch_tokens=microbatch, lr=1e-5, seed=1,
                          candidate_selections=("100", "0:save_attention"))
    session = TrainingSession(setup)
    cfg = session.cfg
    cycles = []
    for gidx in range(groups):
        times = []
        for u in range(updates):
            b = make_batch(100 * gidx + u, vocab=cfg.vocab_size, tokens_per_step=tokens,
                           microbatch_tokens=microbatch, max_len=min(8192, microbatch), median=1200.0,
                           slots=session.slots)
            times.append(session.step(b).device_seconds)
        cycles.append(statistics.median(times[1:]))      # the first update of a group warms up
    measured = statistics.median(cycles)
    simulated = session.plan.summary.duration_seconds
    tps = tokens / measured
    failures = []
    if abs(measured - simulated) > 0.10 * simulated:
        failures.append(f"measured {measured:.3f} s vs simulated {simulated:.3f} s: outside 10 %")
    if floor is not None and tps < 0.95 * floor:
        failures.append(f"{tps:.0f} tokens/s is under 95 % of the floor {floor:.0f}")
    session.close()
    return {"gate": "performance", "model": model, "measured_seconds": measured,
            "simulated_seconds": simulated, "tokens_per_second": tps, "floor": floor,
            "group_cycles": cycles, "passed": not failures, "failures": failures}


def suite_gate(device: str = "cpu", extra: tuple[str, ...] = ()) -> dict:
    """The repository's test suite as a gate: the CPU tests always, the GPU tests too when the
    gates run on a GPU. One child process per marker expression; the record keeps pytest's last
    line and the exit status. (The reference's gate launcher runs its suite before the numerical
    and performance gates the same way: qualification/gates/.)"""
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parents[2]
    runs = []
    for marker in (["not gpu"] + (["gpu"] if device == "cuda" else [])):
        cmd = [sys.executable, "-m", "pytest", str(root / "tests"), "-q", "-m", marker, *extra]
        proc = subprocess.run(cmd, capture_output=True, text=True, cwd=root)
        tail = [ln for ln in proc.stdout.splitlines() if ln.strip()][-1:] or [""]
        runs.append({"marker": marker, "exit": proc.returncode, "summary": tail[0]})
    return {"gate": "suite", "passed": all(r["exit"] == 0 for r in runs), "runs": runs}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m shadowspill_b200.qualification.gates")
    ap.add_argument("gates", nargs="*", default=["numerical"],
                    choices=["suite", "numerical", "performance", "twin", "determinism"],
                    help="run in the order given; suite = the test suite for this machine (CPU tests, plus the "
                         "GPU tests where a GPU is present); determinism = the bitwise divergence probe")
    ap.add_argument("--frontend", default="stages", choices=["stages", "graph"])
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--model", default=None)
    ap.add_argument("--floor", type=float, default=None, help="recorded tokens/s floor for this box")
    a = ap.parse_args(argv)
    ok = True
    for gate in a.gates:
        if gate == "suite":
            rec = suite_gate(a.device)
        elif gate == "determinism":
            from .nondeterminism import probe
            found = probe(a.model or "llama3-tiny", a.device, updates=3, frontend=a.frontend)
            rec = dict(found, gate="determinism", passed=found["diverged_at"] is None)
        elif gate == "twin":
            rec = torch_twin_gate(twin_config(a.model or "llama3"), a.device, frontend=a.frontend,
                                  tokens=256 if a.device == "cpu" else 1024)
        elif gate == "numerical":
            default = "llama3-tiny" if a.device == "cpu" else "llama3-1b"
            rec = numerical_gate(a.model or default, a.device)
        else:
            rec = performance_gate(a.model or "llama3-8b", floor=a.floor)
        print(json.dumps(rec), flush=True)
        ok &= rec["passed"]
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
