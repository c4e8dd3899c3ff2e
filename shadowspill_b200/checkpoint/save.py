"""``save_checkpoint``: stream an executor's persistent state into per-rank archives.

Every persistent tensor is read from its home in the pinned spill pool (nothing
is gathered onto a device). A rank writes only the region it owns: the whole
tensor when storage is whole, its slice when storage is sharded. Restore binds
to the *state identity* (names, geometry, owned regions), not to the plan, so a
run with another plan, budget or microbatch geometry can resume from it.

Manifest entries follow the reference's geometry record
(packages/engine/src/shadowspill/checkpoint/tensors.py:11-31): ``dtype`` is
``str(torch.dtype)`` (``"torch.bfloat16"``), ``region_offset`` /
``region_elements`` appear only when the rank stores part of the storage, and
``additional_programs`` maps operation names to program digests
(checkpoint/save.py:263-291). With ``frozen_state_id`` the parameters no admitted
plan can change (a frozen LoRA base) are left out and listed in
``omitted_parameters`` (checkpoint/frozen.py:35-79); ``weights`` picks which copy of
a weight held in two precisions is written, the other is listed in
``derived_tensors`` and rebuilt on load (checkpoint/load.py:289). Generator states
travel in ``metadata["random_streams"]`` (checkpoint/random_streams.py:55).
"""
from __future__ import annotations

import base64
import hashlib
import json
import random
import sys
from pathlib import Path
from typing import Any

import numpy as np
import torch

from .archive import FORMAT, VERSION, ArchiveWriter

_NP = {torch.bfloat16: np.uint16, torch.float32: np.float32, torch.float16: np.float16,
       torch.int64: np.int64, torch.int32: np.int32}
# dtype spellings accepted on load: the reference's ``str(torch.dtype)`` and the bare name
TORCH_DTYPES = {str(dt): dt for dt in _NP}
TORCH_DTYPES.update({str(dt).removeprefix("torch."): dt for dt in _NP})


def entry_region(entry: dict[str, Any]) -> tuple[int, int]:
    """``(first element, elements)`` of the storage a manifest entry holds. Reads the
    optional ``region_offset`` / ``region_elements`` keys, the whole storage when they
    are absent, and the ``region: [lo, n]`` pair of archives written by earlier builds."""
    if "region" in entry:
        lo, n = entry["region"]
        return int(lo), int(n)
    if "region_elements" in entry:
        return int(entry.get("region_offset", 0)), int(entry["region_elements"])
    return 0, int(entry["storage_elements"])


def _geometry(name: str, shape, dtype: torch.dtype, numel: int, lo: int, hi: int) -> dict[str, Any]:
    e = {"name": name, "shape": list(shape), "dtype": str(dtype),
         "stride": _contiguous_stride(shape), "storage_offset": 0, "storage_elements": numel}
    if lo != 0 or hi - lo != numel:
        e["region_offset"], e["region_elements"] = lo, hi - lo
    return e


def state_entries(executor, omit_frozen: bool = False, weights: str = "compute") -> list[dict[str, Any]]:
    """Geometry of every persistent tensor as this rank stores it. ``omit_frozen``
    drops parameters that own no gradient (no plan can change them); ``weights``
    = ``"master"`` drops the compute-precision copy of every weight that has an fp32
    master, ``"compute"`` drops the master (it is rebuilt from the other on load)."""
    world, rank = executor.world, executor.rank
    has_master = {st.name for st in executor.stages if f"{st.name}.master" in executor._obj}
    out = []
    for st in executor.stages:
        for kind, prefix in (("weights", ""), ("exp_avg", "exp_avg."), ("exp_avg_sq", "exp_avg_sq."),
                             ("master", "master.")):
            if f"{st.name}.{kind}" not in executor._obj:
                continue
            for p in st.params:
                if kind != "weights" and not p.trainable:
                    continue          # frozen parameters own no moments and no master copy
                if omit_frozen and not p.trainable:
                    continue
                if st.name in has_master and p.trainable and (
                        (kind == "weights" and weights == "master")
                        or (kind == "master" and weights == "compute")):
                    continue
                dt = p.dtype or (torch.float32 if kind == "master" else executor.desc.dtype)
                numel, shape = p.numel, p.shape
                if p.expert_sharded:
                    # this rank's experts are rows [expert_lo, expert_lo + local) of the whole bank
                    shape = tuple(p.global_shape)
                    row = p.numel // p.shape[0]
                    numel = row * shape[0]
                    lo, hi = p.expert_lo * row, p.expert_lo * row + p.numel
                else:
                    lo, hi = st.owned_span(p, executor.desc.dtype, world, rank)
                out.append(_geometry(f"{prefix}{st.name}.{p.name}", shape, dt, numel, lo, hi))
    return out


def omitted_parameters(executor) -> list[str]:
    """Names of the parameters a checkpoint with a ``frozen_state_id`` leaves out."""
    return sorted(f"{st.name}.{p.name}" for st in executor.stages for p in st.params
                  if not p.trainable)


def derived_tensors(executor, weights: str) -> list[str]:
    """Names left out because the other precision of the same weight is saved."""
    out = []
    for st in executor.stages:
        if f"{st.name}.master" not in executor._obj:
            continue
        for p in st.params:
            if p.trainable:
                out.append(f"{st.name}.{p.name}" if weights == "master" else f"master.{st.name}.{p.name}")
    return sorted(out)


def _contiguous_stride(shape) -> list[int]:
    stride, acc = [], 1
    for d in reversed(shape):
        stride.append(acc)
        acc *= d
    return list(reversed(stride))


def state_identity(entries: list[dict[str, Any]], world: int) -> str:
    """Digest of names and geometry, independent of which rank owns what."""
    ident = [[e["name"], list(e["shape"]), str(TORCH_DTYPES[e["dtype"]])] for e in entries]
    return hashlib.sha256(json.dumps([ident, world], sort_keys=True).encode()).hexdigest()


# ---------------------------------------------------------------- generator states
def _streams(logical_rank: int, accelerator: bool) -> dict[str, str]:
    reps = {"python": "python.random@3", "numpy": "numpy.MT19937@1",
            "torch": "torch.cpu@" + torch.__version__}
    if accelerator:
        reps["accelerator"] = "torch.cuda@" + torch.__version__
    return reps


def capture_random_streams(logical_rank: int, accelerator: bool = False) -> list[dict[str, Any]]:
    """The worker's default generator states as small JSON records: identity
    ``("rng", "worker.default", (rank, "training", name))``, a representation tag
    naming the generator and its version, and the state as JSON text (integers for
    the Python and NumPy generators, base64 of the state bytes for torch's)."""
    out = []
    for name, rep in _streams(logical_rank, accelerator).items():
        if name == "python":
            version, words, gauss = random.getstate()
            state = [version, list(words), gauss]
        elif name == "numpy":
            kind, keys, pos, has_gauss, cached = np.random.get_state()
            state = [kind, [int(k) for k in keys], int(pos), int(has_gauss), float(cached)]
        elif name == "torch":
            state = base64.b64encode(torch.get_rng_state().numpy().tobytes()).decode()
        else:
            state = base64.b64encode(torch.cuda.get_rng_state().numpy().tobytes()).decode()
        out.append({"identity": {"role": "rng", "name": "worker.default",
                                 "component_path": [str(logical_rank), "training", name]},
                    "representation": rep, "rank": logical_rank, "payload": json.dumps(state)})
    return out


def restore_random_streams(records: list[dict[str, Any]], logical_rank: int) -> list[str]:
    """Puts back every stream saved for ``logical_rank`` whose representation tag matches
    the running generator; returns the names restored. A stream with another tag (a
    different torch version, say) is left alone: its state would not mean the same."""
    reps = _streams(logical_rank, torch.cuda.is_available())
    done = []
    for r in records:
        path = r.get("identity", {}).get("component_path", [])
        if len(path) != 3 or path[0] != str(logical_rank) or path[1] != "training":
            continue
        name = path[2]
        if reps.get(name) != r.get("representation"):
            continue
        state = json.loads(r["payload"])
        if name == "python":
            random.setstate((state[0], tuple(state[1]), state[2]))
        elif name == "numpy":
            np.random.set_state((state[0], np.asarray(state[1], dtype=np.uint32), state[2],
                                 state[3], state[4]))
        else:
            raw = torch.frombuffer(bytearray(base64.b64decode(state)), dtype=torch.uint8)
            (torch.set_rng_state if name == "torch" else torch.cuda.set_rng_state)(raw)
        done.append(name)
    return done


def save_checkpoint(executor, directory: str | Path, *, metadata: dict[str, Any] | None = None,
                    weights: str = "master", frozen_state_id: str | None = None,
                    random_streams: bool = True) -> Path:
    """Writes ``<directory>/rank<r>.tar`` for this rank and returns its path.

    ``frozen_state_id`` names a frozen base the caller keeps elsewhere: parameters that
    own no gradient are then left out of the archive, and loading needs the same id.
    ``weights``: ``"master"`` (the reference's default) or ``"compute"``, which copy of a
    weight with an fp32 master is written; without master copies the two are the same."""
    if metadata is not None and len(json.dumps(metadata)) > (16 << 20):
        raise ValueError("checkpoint metadata is limited to 16 MiB of JSON")
    if frozen_state_id is not None and (not isinstance(frozen_state_id, str) or not frozen_state_id.strip()):
        raise ValueError("frozen_state_id must be a nonempty string")
    if weights not in ("compute", "master"):
        raise ValueError("weights must be 'compute' or 'master'")
    directory = Path(directory)
    if getattr(executor, "replicas", 1) > 1 and executor.global_rank >= executor.world:
        # replicas hold identical state: the first replica's ranks write the checkpoint
        return directory / f"rank{executor.rank}.tar"
    omit = frozen_state_id is not None
    entries = state_entries(executor, omit, weights)
    writer = ArchiveWriter(directory / f"rank{executor.rank}.tar")
    try:
        # streamed: with state homed in a file pool each object is read from the file when its
        # first tensor comes up and dropped again, so one object is in host memory at a time
        by_name = {e["name"]: e for e in entries}
        for name, t in executor.named_tensors(writable=False):
            e = by_name.pop(name, None)
            if e is None:
                continue
            lo, n = entry_region(e)
            flat = t.reshape(-1)[:n] if executor.world > 1 else t.reshape(-1)
            arr = flat.view(torch.uint8).numpy() if flat.numel() else np.zeros(0, np.uint8)
            writer.add_tensor(e, arr)
            release = getattr(executor, "release_mirrors", None)
            if release is not None:
                release()
        if by_name:
            raise KeyError(f"state tensors without a home: {sorted(by_name)[:3]}")
        saved_metadata = dict(metadata or {}, completed_updates=executor.completed_updates,
                              logical_ranks=executor.world)
        if random_streams:
            saved_metadata["random_streams"] = capture_random_streams(
                executor.rank, bool(getattr(executor, "cuda", False)))
        extra = {op: b["program"].digest() for op, b in getattr(executor, "_bound", {}).items()
                 if b["program"] is not executor.program}
        manifest = {
            "format": FORMAT, "version": VERSION, "byteorder": sys.byteorder,
            "state": state_identity(entries, executor.world),
            "program": executor.program.digest(), "logical_rank": executor.rank,
            "additional_programs": extra, "metadata": saved_metadata,
            "frozen_state_id": frozen_state_id,
            "omitted_parameters": omitted_parameters(executor) if omit else [],
            "weights": weights, "derived_tensors": derived_tensors(executor, weights),
            "gathered_tensors": [], "retained_weight_copies": [],
        }
        return writer.finish(manifest)
    except BaseException:
        writer.abort()
        raise
