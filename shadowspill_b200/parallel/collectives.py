"""Data-parallel collectives behind one interface, two arms.

``PeerCollectives``  the product path on NVLink/NVSwitch: the executor's device
                     pool is one symmetric allocation mapped into every rank, so
                     an object at pool offset X on this rank is at ``base[r] + X``
                     on rank r, and the hand-written kernels in
                     ``peer_collectives.cu`` reach it with plain loads/stores:
                     pull all-gather, reduce-scatter fused with sharded AdamW,
                     flag barriers with bounded waits.
``DistCollectives``  the library arm (``torch.distributed``: NCCL on GPUs, gloo on
                     CPU). It is the baseline the fused path is measured against
                     and the functional stand-in for multi-rank tests on CPU.

Both run on the compute stream as plan tasks, in the same order on every rank.
Reference for what is being replaced: the NCCL calls in
packages/engine/csrc/adapter/pytorch/storage/sharded.cpp:87,94,118 and
packages/engine/src/shadowspill/communication/operations.py:9-26.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import functional as F

_c = _lib
_lib.register("ss_peer_barrier", [_c.c_p, _c.c_int, _c.c_int, C.c_uint, _c.c_p, _c.c_p])
_lib.register("ss_peer_barrier_timed", [_c.c_p, _c.c_int, _c.c_int, C.c_uint, _c.c_ull, _c.c_p, _c.c_p])
_lib.register("ss_peer_allgather", [_c.c_p, _c.c_p, _c.c_ll, _c.c_ll, _c.c_int, _c.c_int, _c.c_p])
_lib.register("ss_rs_adamw", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_ll, _c.c_int, _c.c_int,
                              _c.c_f, _c.c_f, _c.c_f, _c.c_f, _c.c_f, _c.c_int, _c.c_f, _c.c_ull,
                              _c.c_ull, _c.c_int, _c.c_int, _c.c_p])
_lib.register("ss_rs_adamw_acc", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_ll, _c.c_int, _c.c_int,
                                  _c.c_f, _c.c_f, _c.c_f, _c.c_f, _c.c_f, _c.c_int, _c.c_f, _c.c_ull,
                                  _c.c_ull, _c.c_int, _c.c_int, _c.c_p])
_lib.register("ss_rs_accumulate", [_c.c_p, _c.c_p, _c.c_ll, _c.c_ll, _c.c_int, _c.c_int, _c.c_int, _c.c_p])
_lib.register("ss_rs_adamw_nvls", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_ll, _c.c_int,
                                   _c.c_f, _c.c_f, _c.c_f, _c.c_f, _c.c_f, _c.c_int, _c.c_f, _c.c_ull,
                                   _c.c_ull, _c.c_int, _c.c_int, _c.c_p])
_lib.register("ss_peer_allreduce_f32", [_c.c_p, _c.c_p, _c.c_ll, _c.c_int, _c.c_p])


def shard_numel(numel: int, world: int) -> int:
    """Elements per rank: equal padded shards, a multiple of 8 elements so that
    every shard starts on a 16-byte boundary for 2-byte types."""
    per = -(-numel // world)
    return -(-per // 8) * 8


class DistCollectives:
    """torch.distributed arm (NCCL / gloo)."""
    name = "dist"

    def __init__(self, group=None, ranks_per_replica: int | None = None):
        """With ``ranks_per_replica`` smaller than the job, weights are gathered inside this
        rank's replica group and gradients are summed over every rank of the job."""
        self.group = group
        total = dist.get_world_size(group) if dist.is_initialized() else 1
        global_rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = ranks_per_replica or total
        self.rank = global_rank % self.world
        self.shard_group = group
        if self.world != total:
            for r in range(total // self.world):       # every rank creates every subgroup, same order
                g = dist.new_group(list(range(r * self.world, (r + 1) * self.world)))
                if r == global_rank // self.world:
                    self.shard_group = g

    def barrier_begin(self) -> None:
        pass

    def barrier_end(self) -> None:
        pass

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        """``full`` (numel elements) <- concatenation of every rank's ``shard``."""
        n, per = full.numel(), shard.numel()
        if self.world == 1:
            full.view(-1)[:n].copy_(shard.view(-1)[:n])
            return
        parts = [torch.empty_like(shard.view(-1)) for _ in range(self.world)]
        dist.all_gather(parts, shard.view(-1).contiguous(), group=self.shard_group)
        flat = full.view(-1)
        for k, part in enumerate(parts):
            lo = k * per
            if lo < n:
                flat[lo:min(n, lo + per)].copy_(part[:min(n, lo + per) - lo])

    def reduce_scatter_update(self, rule: str, grad: torch.Tensor, p, m, v, *, whole: bool = False,
                              acc: torch.Tensor | None = None, **hyper) -> None:
        """The unfused form for update rules other than AdamW: sum ``grad`` over every rank with
        the library all-reduce (on a copy: this rank's gradient buffer stays as peers expect it),
        then apply ``rule`` to the slice of (p, m, v) this rank owns. ``acc``: this rank's fp32
        sum of earlier groups' gradients over that slice, added first."""
        from ..ops import reference
        n, per = grad.numel(), p.numel()
        g = grad.view(-1).clone()
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(g, group=self.group)
        lo = 0 if whole else self._owned_rank() * per
        hi = min(n, lo + per)
        if hi <= lo:
            return
        cnt = hi - lo
        owned = g[lo:hi] if acc is None else g[lo:hi].float() + acc.view(-1)[:cnt]
        reference.update_rule_(rule, p.view(-1)[:cnt], owned, m.view(-1)[:cnt], v.view(-1)[:cnt], **hyper)

    def _owned_rank(self) -> int:
        return self.rank

    def reduce_scatter_adamw(self, grad: torch.Tensor, p, m, v, *, offset: int, whole: bool = False,
                             acc: torch.Tensor | None = None, **adam) -> None:
        """Sum ``grad`` over ranks; update this rank's owned slice of (p, m, v). ``whole``: the
        tensor is stored whole on every rank, which all apply the same update to all of it.
        ``acc``: this rank's fp32 sum of earlier groups' gradients over the slice, added first."""
        n, per = grad.numel(), p.numel()
        g = grad.view(-1).clone()
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(g, group=self.group)          # over every rank, replicas included
        lo = 0 if whole else self.rank * per
        hi = min(n, lo + per)
        if hi <= lo:
            return
        cnt = hi - lo
        owned = g[lo:hi] if acc is None else g[lo:hi].float() + acc.view(-1)[:cnt]
        F.adamw_(p.view(-1)[:cnt], owned, m.view(-1)[:cnt], v.view(-1)[:cnt],
                 offset=offset + lo, **adam)

    def reduce_scatter_accumulate(self, grad: torch.Tensor, acc: torch.Tensor, *, first: bool,
                                  whole: bool = False) -> None:
        """``acc`` (fp32, this rank's owned slice) = (0 if ``first`` else ``acc``) + the sum of
        ``grad`` over every rank: one group's gradient folded into the running sum."""
        n, per = grad.numel(), acc.numel()
        g = grad.view(-1).clone()
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(g, group=self.group)
        lo = 0 if whole else self.rank * per
        hi = min(n, lo + per)
        if hi <= lo:
            return
        cnt = hi - lo
        dst = acc.view(-1)[:cnt]
        if first:
            dst.copy_(g[lo:hi])
        else:
            dst.add_(g[lo:hi].float())


class PeerCollectives:
    """Own kernels over the symmetric device pool."""
    name = "peer"

    def __init__(self, pool: torch.Tensor, group=None, ranks_per_replica: int | None = None):
        """``ranks_per_replica``: size of the shard group (default: every rank). With replicas
        the pool is still symmetric over the whole job: gathers read the ranks of this replica,
        the fused update reads every rank's gradient."""
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group or dist.group.WORLD
        self.total = dist.get_world_size(self.group)
        self.global_rank = dist.get_rank(self.group)
        self.shard_world = ranks_per_replica or self.total
        self.shard_rank = self.global_rank % self.shard_world
        self.replica_base = self.global_rank - self.shard_rank
        self.world, self.rank = self.total, self.global_rank      # barrier and peer tables span the job
        self.pool = pool
        _keep_multicast_unbound()
        self.handle = symm_mem.rendezvous(pool, self.group.group_name)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        self.local_base = pool.data_ptr()
        # NVSwitch multicast view of the pool (0 when the fabric or the driver has none). Without
        # SS_NVLS=1 no multicast object may exist at all (see _keep_multicast_unbound): the
        # in-switch reduction is opted into by jobs that do not expect rank loss.
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if not nvls_requested() and mc != 0:
            raise RuntimeError("the symmetric pool was bound to an NVSwitch multicast object although "
                               "SS_NVLS is not set; refusing to run with rank-loss handling invalid")
        self.mc_base = mc if nvls_requested() else 0
        if self.bases[self.rank] != self.local_base:
            raise RuntimeError("symmetric pool base does not match the local tensor")
        self.flags = symm_mem.empty(64, dtype=torch.int32, device=pool.device)
        self.flags.zero_()
        self.flag_handle = symm_mem.rendezvous(self.flags, self.group.group_name)
        self.flag_ptrs = (C.c_void_p * self.world)(*[int(p) for p in self.flag_handle.buffer_ptrs])
        self.epoch = 0
        self.flags2, self.flag2_ptrs, self.epoch2 = None, None, 0
        # how long a flag wait lasts before the kernel gives up with status 5 (0 = 2 s); a job
        # that wants to notice a lost rank quickly sets SS_PEER_WAIT_MS
        import os
        self.wait_ns = int(float(os.environ.get("SS_PEER_WAIT_MS", "0")) * 1e6)
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def _peers(self, t: torch.Tensor):
        off = t.data_ptr() - self.local_base
        if off < 0 or off + t.numel() * t.element_size() > self.pool.numel():
            raise ValueError("tensor is not inside the symmetric pool")
        return (C.c_void_p * self.world)(*[b + off for b in self.bases])

    def _barrier(self) -> None:
        self.epoch += 1
        _lib.check(_lib.lib().ss_peer_barrier_timed(self.flag_ptrs, self.rank, self.world, self.epoch,
                                                    int(self.wait_ns),
                                                    _lib.status_word(self.pool.device).data_ptr(),
                                                    _lib.stream_ptr()), "ss_peer_barrier")

    barrier_begin = _barrier
    barrier_end = _barrier

    def barrier_compute(self) -> None:
        """A barrier on a second set of flag words, for the compute stream: barriers on two streams
        must not share an epoch counter, or one stream's later barrier could satisfy the other's
        earlier one."""
        if self.flags2 is None:
            import torch.distributed._symmetric_memory as symm_mem
            self.flags2 = symm_mem.empty(64, dtype=torch.int32, device=self.pool.device)
            self.flags2.zero_()
            handle = symm_mem.rendezvous(self.flags2, self.group.group_name)
            self.flag2_ptrs = (C.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])
            self._flag2_handle = handle
            torch.cuda.synchronize()
            dist.barrier(self.group)
        self.epoch2 += 1
        _lib.check(_lib.lib().ss_peer_barrier_timed(self.flag2_ptrs, self.rank, self.world, self.epoch2,
                                                    int(self.wait_ns),
                                                    _lib.status_word(self.pool.device).data_ptr(),
                                                    _lib.stream_ptr()), "ss_peer_barrier")

    def register_fused_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        """Leaves the gather of ``full`` (a 2-D weight in the pool) to the first GEMM that reads it:
        the kernel pulls every rank's ``shard`` over NVLink while it computes."""
        base = self.replica_base
        peers = self._peers(shard)
        ptrs = [int(peers[base + k]) for k in range(self.shard_world)]
        flat = full.view(-1)
        F.register_gather(F.PendingGather(full, ptrs, shard.numel(), self.shard_world, self.shard_rank,
                                          lambda: self.all_gather(shard, flat)))

    def all_gather(self, shard: torch.Tensor, full: torch.Tensor) -> None:
        peers = self._peers(shard)
        if self.shard_world != self.total:       # this replica's ranks only
            peers = (C.c_void_p * self.shard_world)(
                *[peers[self.replica_base + j] for j in range(self.shard_world)])
        _lib.check(_lib.lib().ss_peer_allgather(
            peers, full.data_ptr(), shard.numel() * shard.element_size(),
            full.numel() * full.element_size(), self.shard_rank, self.shard_world, _lib.stream_ptr()),
            "ss_peer_allgather")

    def reduce_scatter_update(self, rule: str, grad: torch.Tensor, p, m, v, *, whole: bool = False,
                              acc: torch.Tensor | None = None, **hyper) -> None:
        """The unfused form for update rules other than AdamW: sum ``grad`` over every rank with
        the library all-reduce (on a copy: this rank's gradient buffer stays as peers expect it),
        then apply ``rule`` to the slice of (p, m, v) this rank owns. ``acc``: this rank's fp32
        sum of earlier groups' gradients over that slice, added first."""
        from ..ops import reference
        n, per = grad.numel(), p.numel()
        g = grad.view(-1).clone()
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(g, group=self.group)
        lo = 0 if whole else self._owned_rank() * per
        hi = min(n, lo + per)
        if hi <= lo:
            return
        cnt = hi - lo
        owned = g[lo:hi] if acc is None else g[lo:hi].float() + acc.view(-1)[:cnt]
        reference.update_rule_(rule, p.view(-1)[:cnt], owned, m.view(-1)[:cnt], v.view(-1)[:cnt], **hyper)

    def _owned_rank(self) -> int:
        return self.shard_rank

    def reduce_scatter_adamw(self, grad: torch.Tensor, p, m, v, *, offset: int, lr, beta1, beta2,
                             eps, weight_decay, step, grad_scale, seed, stochastic_param,
                             stochastic_state, whole: bool = False, acc: torch.Tensor | None = None) -> None:
        n, per = grad.numel(), p.numel()
        # the slice this rank owns inside its replica; a tensor stored whole is updated whole by
        # every rank (same summed gradient, same counter-based rounding: identical results)
        lo = 0 if whole else self.shard_rank * per
        hi = min(n, lo + per)
        if hi <= lo:
            return
        if acc is not None:
            _lib.check(_lib.lib().ss_rs_adamw_acc(
                self._peers(grad), acc.data_ptr(), p.data_ptr(), m.data_ptr(), v.data_ptr(), lo, hi,
                self.world, int(grad.dtype == torch.float32), lr, beta1, beta2, eps, weight_decay, step,
                grad_scale, seed, offset, int(stochastic_param), int(stochastic_state),
                _lib.stream_ptr()), "ss_rs_adamw_acc")
            return
        if self.mc_base and grad.dtype == torch.bfloat16:
            off = grad.data_ptr() - self.local_base
            _lib.check(_lib.lib().ss_rs_adamw_nvls(
                self._peers(grad), self.mc_base + off, p.data_ptr(), m.data_ptr(), v.data_ptr(), lo, hi,
                self.world, lr, beta1, beta2, eps, weight_decay, step, grad_scale, seed, offset,
                int(stochastic_param), int(stochastic_state), _lib.stream_ptr()), "ss_rs_adamw_nvls")
            return
        _lib.check(_lib.lib().ss_rs_adamw(
            self._peers(grad), p.data_ptr(), m.data_ptr(), v.data_ptr(), lo, hi, self.world,
            int(grad.dtype == torch.float32), lr, beta1, beta2, eps, weight_decay, step,
            grad_scale, seed, offset, int(stochastic_param), int(stochastic_state),
            _lib.stream_ptr()), "ss_rs_adamw")

    def reduce_scatter_accumulate(self, grad: torch.Tensor, acc: torch.Tensor, *, first: bool,
                                  whole: bool = False) -> None:
        """One group's gradient, summed over every rank's buffer with peer loads, folded into this
        rank's fp32 running sum of its owned slice."""
        n, per = grad.numel(), acc.numel()
        lo = 0 if whole else self.shard_rank * per
        hi = min(n, lo + per)
        if hi <= lo:
            return
        if acc.dtype != torch.float32:
            raise ValueError("the gradient sum is kept in fp32")
        _lib.check(_lib.lib().ss_rs_accumulate(
            self._peers(grad), acc.data_ptr(), lo, hi, self.world, int(grad.dtype == torch.float32),
            int(first), _lib.stream_ptr()), "ss_rs_accumulate")


def nvls_requested() -> bool:
    """``SS_NVLS=1`` opts a job into NVSwitch multicast (in-switch gradient sums)."""
    import os
    return os.environ.get("SS_NVLS", "0") == "1"


def _keep_multicast_unbound() -> None:
    """Unless the job asked for NVSwitch multicast, tell the symmetric-memory allocator not to
    create a multicast object at rendezvous. A rank that dies while its memory is bound to one
    can raise NVLink faults on its peers' GPUs, so rank-loss handling (a worker that crashes or
    is killed) is only valid with the binding off. Must run before the first rendezvous."""
    import os
    if not nvls_requested():
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"


def allocate_symmetric_pool(nbytes: int, device: torch.device) -> torch.Tensor:
    import torch.distributed._symmetric_memory as symm_mem
    _keep_multicast_unbound()
    return symm_mem.empty(int(nbytes), dtype=torch.uint8, device=device)


def collective_sequence_digest(program) -> str:
    """SHA-256 over the ordered collective work of a program: every task that runs a
    collective (gathers, sharded optimizer updates, expert-parallel layers) with the sizes
    of the objects it touches. Ranks whose digests differ would deadlock or corrupt data."""
    import hashlib
    h = hashlib.sha256()
    for t in program.tasks:
        if t.kind == "collective" or t.variant == "adamw_dp" or ":ep" in (t.profile_key or ""):
            sizes = ",".join(str(program.objects[u.object].bytes) for u in t.uses)
            h.update(f"{t.name}|{t.kind}|{t.variant}|{sizes};".encode())
    return h.hexdigest()


def check_collective_order(programs: dict[str, object], group=None) -> None:
    """Every rank must be about to run the same collectives in the same order for each
    operation's plan: compared before any collective is issued (reference:
    packages/engine/src/shadowspill/execution/distributed/sequence.py:42-78)."""
    world = dist.get_world_size(group)
    mine = {op: collective_sequence_digest(p) for op, p in sorted(programs.items())}
    everyone: list = [None] * world
    dist.all_gather_object(everyone, mine, group=group)
    for r, other in enumerate(everyone):
        if other != mine:
            bad = sorted(op for op in set(mine) | set(other) if mine.get(op) != other.get(op))
            raise RuntimeError(f"collective sequence of {bad} differs between rank "
                               f"{dist.get_rank(group)} and rank {r}; refusing to execute")


def backend_identity() -> dict:
    """What the collective calibration is valid for: library versions and the NCCL_* environment."""
    import os
    out = {"torch": torch.__version__, "backend": dist.get_backend() if dist.is_initialized() else "",
           "env": {k: v for k, v in sorted(os.environ.items()) if k.startswith("NCCL_")}}
    try:
        out["nccl"] = ".".join(str(x) for x in torch.cuda.nccl.version())
    except Exception:  # noqa: BLE001
        out["nccl"] = ""
    return out
