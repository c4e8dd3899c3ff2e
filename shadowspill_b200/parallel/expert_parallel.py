"""Expert parallelism: routed experts whose banks are split over the ranks of a
group, with dispatch and combine done by this framework's own kernels over
NVLink peer memory instead of a library all-to-all.

Data flow of one layer on rank ``r`` (``T`` local tokens, ``k`` slots, experts
``[r*E/R, (r+1)*E/R)`` local):

  route (local)  ->  hidden rows and routing weights copied into the symmetric
  workspace  ->  routing ids all-gathered (metadata, a few hundred KB)  ->
  flag barrier  ->  ``ss_ep_layout``: rows of MY experts from ALL ranks' ids  ->
  ``ss_ep_pull``: each row reads its token from the owning rank (dispatch and
  the permutation into expert order in one pass over NVLink)  ->  grouped
  tcgen05 GEMM (gate/up)  ->  SwiGLU  ->  grouped tcgen05 GEMM (down) whose
  epilogue stores every output row straight into the owning rank's staging
  slot (combine transfer inside the GEMM, overlapped tile by tile with the
  MMAs)  ->  flag barrier  ->  local weighted sum over the k slots.

The backward pass is the same machine run the other way: ``w * dout`` rows are
pulled, the data-gradient GEMM of the gate/up bank scatters ``dx`` rows back.
Every wait is bounded (the flag barrier reports through the status word).

Reference behaviour: packages/workloads/src/shadowspill_workloads/models/shared/
expert_parallel/routing.py:6-28 (route, experts, counts and probability sums) and
the ownership rules in packages/workloads/src/shadowspill_workloads/components/
expert_parallel.py:74-140 (experts divided evenly, 2..128 ranks, top_k <= 32).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import functional as F
from ..ops import moe as moe_ops
from .collectives import PeerCollectives, allocate_symmetric_pool

_c = _lib
_lib.register("ss_ep_layout", [_c.c_p, _c.c_ll, _c.c_int, _c.c_int, _c.c_p, _c.c_p, _c.c_p, _c.c_int,
                               _c.c_p, _c.c_p, _c.c_p])
_lib.register("ss_ep_pull", [_c.c_p, _c.c_ll, _c.c_p, _c.c_int, _c.c_p, _c.c_int, _c.c_int, _c.c_int,
                             _c.c_int, _c.c_p, _c.c_ll, _c.c_p])
_lib.register("ss_ep_row_dst", [_c.c_p, _c.c_int, _c.c_p, _c.c_int, _c.c_int, _c.c_ll, _c.c_p, _c.c_p])
_lib.register("ss_gemm_grouped_scatter_bf16", [_c.c_p, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int,
                                               _c.c_int, _c.c_ll, _c.c_ll, _c.c_int, _c.c_p, _c.c_int,
                                               _c.c_p, _c.c_p])


def _align(n: int, a: int = 256) -> int:
    return -(-n // a) * a


class _RowLayout:
    """What ``grouped_linear`` / ``grouped_wgrad`` need to know about sorted rows."""

    def __init__(self, rows, tile_expert, offsets, row_src, row_dst):
        self.rows, self.tile_expert, self.offsets = rows, tile_expert, offsets
        self.row_src, self.row_dst = row_src, row_dst


class ExpertParallelGroup:
    """Symmetric workspace, peer address tables and the flag barrier of one group.
    One instance serves every layer of a model (the calls are ordered on the
    compute stream and fenced by the barriers)."""

    def __init__(self, max_tokens: int, top_k: int, d_model: int, n_experts: int, group=None,
                 device: torch.device | None = None):
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if not 2 <= self.world <= 128:
            raise ValueError("expert parallelism needs 2 to 128 ranks")
        if n_experts % self.world:
            raise ValueError("n_experts must be divisible by the number of ranks")
        if not 1 <= top_k <= 32:
            raise ValueError("top_k must be between 1 and 32")
        if d_model % 8:
            raise ValueError("d_model must be a multiple of 8")
        self.T, self.k, self.D, self.E = max_tokens, top_k, d_model, n_experts
        self.e_local = n_experts // self.world
        self.e_lo = self.rank * self.e_local
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        x_bytes = _align(max_tokens * d_model * 2)
        w_bytes = _align(max_tokens * top_k * 4)
        s_bytes = _align(max_tokens * top_k * d_model * 2)
        self.pool = allocate_symmetric_pool(x_bytes + w_bytes + s_bytes, self.device)
        self.peer = PeerCollectives(self.pool, self.group)
        self.x = self.pool[:max_tokens * d_model * 2].view(torch.bfloat16).view(max_tokens, d_model)
        self.w = self.pool[x_bytes:x_bytes + max_tokens * top_k * 4].view(torch.float32)
        self.stage = (self.pool[x_bytes + w_bytes:x_bytes + w_bytes + max_tokens * top_k * d_model * 2]
                      .view(torch.bfloat16).view(max_tokens * top_k, d_model))
        self.x_peers = self.peer._peers(self.x)
        self.w_peers = self.peer._peers(self.w)
        self.stage_peers = self.peer._peers(self.stage)
        self._arange = torch.arange(max_tokens * top_k, dtype=torch.int32, device=self.device)
        # worst case: every assignment of every rank lands here
        self.max_tiles = -(-(self.world * max_tokens * top_k + self.e_local * 127) // 128)
        # > 1 cuts the rows into chunks whose pulls overlap the previous chunk's GEMMs; measured
        # on 2 B200s the pull (0.24 ms of 1.0 ms) is too short to repay the smaller GEMMs
        self.pipeline_chunks = 1
        self.side = torch.cuda.Stream(device=self.device)

    # ------------------------------------------------------------------ pieces
    def barrier(self) -> None:
        self.peer._barrier()

    def publish(self, rows: torch.Tensor, weights: torch.Tensor) -> None:
        """Puts this rank's token rows and routing weights where peers can read them."""
        T = rows.shape[0]
        self.x[:T].copy_(rows)
        self.w[:T * self.k].copy_(weights.reshape(-1))

    def layout(self, ids: torch.Tensor) -> _RowLayout:
        """Rows of this rank's experts among the assignments of all ranks. Every rank
        must pass ids of the same shape ``[T, k]`` with ``T == max_tokens``."""
        T, k = ids.shape
        if T != self.T or k != self.k:
            raise ValueError("ids must be [max_tokens, top_k] on every rank")
        dev = self.device
        gids = torch.empty((self.world * T, k), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(gids, ids.contiguous(), group=self.group)
        counts = torch.empty(self.e_local, dtype=torch.int32, device=dev)
        offsets = torch.empty(self.e_local + 1, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(self.max_tiles, dtype=torch.int32, device=dev)
        cursor = torch.empty(self.e_local, dtype=torch.int32, device=dev)
        row_src = torch.empty(self.max_tiles * 128, dtype=torch.int32, device=dev)
        _lib.check(_lib.lib().ss_ep_layout(gids.data_ptr(), gids.numel(), self.e_lo, self.e_local,
                                           counts.data_ptr(), offsets.data_ptr(),
                                           tile_expert.data_ptr(), self.max_tiles, cursor.data_ptr(),
                                           row_src.data_ptr(), _lib.stream_ptr()), "ss_ep_layout")
        host_off = offsets.tolist()             # one host read: sizes the buffers, cuts the chunks
        rows = int(host_off[-1])
        row_dst = torch.empty(max(rows, 1), dtype=torch.int64, device=dev)
        _lib.check(_lib.lib().ss_ep_row_dst(self.stage_peers, self.world, row_src.data_ptr(), rows,
                                            T * k, self.D * 2, row_dst.data_ptr(), _lib.stream_ptr()),
                   "ss_ep_row_dst")
        lay = _RowLayout(rows, tile_expert[:max(rows // 128, 1)], offsets, row_src, row_dst)
        lay.chunks = self._chunks(host_off)
        return lay

    def _chunks(self, host_off: list[int]) -> list[tuple[int, int]]:
        """Row ranges ``[r0, r1)`` on expert boundaries, about equal in rows: the unit in which
        the pull of one range overlaps the GEMMs of the previous one."""
        rows = host_off[-1]
        if rows == 0:
            return []
        want = max(1, min(self.pipeline_chunks, self.e_local))
        target = rows / want
        cuts, out = [0], []
        for e in range(1, self.e_local):
            if host_off[e] - cuts[-1] >= target and rows - host_off[e] > 0:
                cuts.append(host_off[e])
        cuts.append(rows)
        for a, b in zip(cuts[:-1], cuts[1:]):
            if b > a:
                out.append((a, b))
        return out

    def pull(self, lay: _RowLayout, scaled: bool, out: torch.Tensor | None = None,
             r0: int = 0, r1: int | None = None) -> torch.Tensor:
        """Dispatch: the published rows of all ranks that belong to local experts, in
        expert order (scaled by the publisher's routing weight when ``scaled``); rows
        ``[r0, r1)`` only when given. Runs on the current stream."""
        r1 = lay.rows if r1 is None else r1
        if out is None:
            out = torch.empty((lay.rows, self.D), dtype=torch.bfloat16, device=self.device)
        if r1 > r0:
            _lib.check(_lib.lib().ss_ep_pull(
                self.x_peers, self.D, self.w_peers if scaled else None, self.world,
                lay.row_src[r0:].data_ptr(), r1 - r0, self.T * self.k, self.k, self.D,
                out[r0:].data_ptr(), self.D, _lib.stream_ptr()), "ss_ep_pull")
        return out

    def pull_pipelined(self, lay: _RowLayout, scaled: bool):
        """Starts the pull of every chunk on the side stream and yields, chunk by chunk,
        ``(r0, r1, rows tensor)`` once that chunk has landed: the caller's GEMMs on chunk
        ``i`` run while chunk ``i+1`` is still crossing NVLink."""
        out = torch.empty((lay.rows, self.D), dtype=torch.bfloat16, device=self.device)
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)
        events = []
        with torch.cuda.stream(self.side):
            for r0, r1 in lay.chunks:
                self.pull(lay, scaled, out, r0, r1)
                ev = torch.cuda.Event()
                ev.record(self.side)
                events.append(ev)
        out.record_stream(self.side)
        for (r0, r1), ev in zip(lay.chunks, events):
            main.wait_event(ev)
            yield r0, r1, out

    def scatter_linear(self, x_sorted: torch.Tensor, bank: torch.Tensor, lay: _RowLayout,
                       transpose: bool, r0: int = 0, r1: int | None = None) -> None:
        """Grouped GEMM whose output rows go straight to their owners' staging slots
        (rows ``[r0, r1)`` of the layout; ``x_sorted`` holds exactly those rows)."""
        r1 = lay.rows if r1 is None else r1
        if r1 <= r0:
            return
        N = bank.shape[2] if transpose else bank.shape[1]
        if N != self.D:
            raise ValueError("scattered rows must have the model width")
        _lib.check(_lib.lib().ss_gemm_grouped_scatter_bf16(
            x_sorted.data_ptr(), bank.data_ptr(), lay.row_dst[r0:].data_ptr(), r1 - r0, N,
            x_sorted.shape[1], bank.shape[0], x_sorted.stride(0), bank.stride(1), int(transpose),
            lay.tile_expert[r0 // 128:].data_ptr(), 0, _lib.status_word(self.device).data_ptr(),
            _lib.stream_ptr()), "ss_gemm_grouped_scatter_bf16")

    def range_layout(self, lay: _RowLayout, r0: int, r1: int) -> _RowLayout:
        """The layout restricted to rows ``[r0, r1)`` (an expert boundary on both sides)."""
        return _RowLayout(r1 - r0, lay.tile_expert[r0 // 128:r1 // 128], lay.offsets,
                          lay.row_src[r0:r1], lay.row_dst[r0:r1])

    def reduce_slots(self, T: int, weights: torch.Tensor | None, dots_with: torch.Tensor | None = None,
                     source: torch.Tensor | None = None, only_dots: bool = False):
        """``out[t] = sum_j w[t,j] * stage[t*k+j]`` (unit weights when ``None``) and/or the
        dot products ``<dots_with[t], stage[t*k+j]>``."""
        src = self.stage if source is None else source
        out = None if only_dots else torch.empty((T, self.D), dtype=torch.bfloat16, device=self.device)
        dots = (torch.empty((T, self.k), dtype=torch.float32, device=self.device)
                if dots_with is not None else None)
        _lib.check(_lib.lib().ss_moe_combine(
            src.data_ptr(), src.stride(0), self._arange.data_ptr(),
            None if weights is None else weights.data_ptr(),
            None if out is None else out.data_ptr(), 0 if out is None else out.stride(0),
            T, self.k, self.D, 0,
            None if dots_with is None else dots_with.data_ptr(),
            0 if dots_with is None else dots_with.stride(0),
            None if dots is None else dots.data_ptr(), _lib.stream_ptr()), "ss_moe_combine")
        return out, dots


class _EPExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, logits, w13, w2, ep: ExpertParallelGroup, renormalize, sink):
        T = h.shape[0]
        ids, wts, _ = moe_ops.route(logits, ep.k, renormalize)
        ep.publish(h, wts)
        lay = ep.layout(ids)
        ep.barrier()                               # every rank's rows are published
        xs = h.new_empty((0, ep.D))
        gu = h.new_empty((lay.rows, w13.shape[1]))
        for r0, r1, xs in ep.pull_pipelined(lay, scaled=False):
            sub = ep.range_layout(lay, r0, r1)
            moe_ops.grouped_linear(xs[r0:r1], w13, sub, out=gu[r0:r1])
            ep.scatter_linear(F.swiglu_fwd(gu[r0:r1]), w2, lay, False, r0, r1)
        ep.barrier()                               # every expert row has landed in its slot
        out, _ = ep.reduce_slots(T, wts)
        ctx.save_for_backward(logits, ids, wts, xs, gu, w13, w2, ep.stage[:T * ep.k].clone())
        ctx.lay, ctx.ep, ctx.sink, ctx.renormalize = lay, ep, sink, renormalize
        return out

    @staticmethod
    def backward(ctx, dout):
        logits, ids, wts, xs, gu, w13, w2, slots = ctx.saved_tensors
        lay, ep, sink = ctx.lay, ctx.ep, ctx.sink
        T = dout.shape[0]
        dout = dout.contiguous()
        _, dwts = ep.reduce_slots(T, None, dots_with=dout, source=slots, only_dots=True)
        ep.publish(dout, wts)
        ep.barrier()
        have_sink = sink is not None and sink.G is not None
        if lay.rows:
            # data gradients chunk by chunk under the pull; the bank gradients contract over
            # all rows of an expert and run once at the end
            dgu = torch.empty_like(gu)
            dys = None
            for r0, r1, dys in ep.pull_pipelined(lay, scaled=True):   # w * dout per assignment
                sub = ep.range_layout(lay, r0, r1)
                dhm = moe_ops.grouped_linear(dys[r0:r1], w2, sub, transpose=True)
                dgu[r0:r1] = F.swiglu_bwd(gu[r0:r1], dhm)
                ep.scatter_linear(dgu[r0:r1], w13, lay, True, r0, r1)
            if have_sink:
                moe_ops.grouped_wgrad(dys, F.swiglu_fwd(gu), lay, sink.G["w2"], sink.accumulate("w2"))
                moe_ops.grouped_wgrad(dgu, xs, lay, sink.G["w13"], sink.accumulate("w13"))
        elif have_sink:
            for name in ("w2", "w13"):
                if not sink.accumulate(name):
                    sink.G[name].zero_()
        ep.barrier()
        dh, _ = ep.reduce_slots(T, None)
        with torch.enable_grad():
            l = logits.detach().requires_grad_(True)
            moe_ops._weights_from_logits(l, ids.long(), ctx.renormalize).backward(dwts)
        return dh, l.grad, None, None, None, None, None


def experts(h, logits, w13_local, w2_local, ep: ExpertParallelGroup, renormalize: bool, sink=None):
    """Routed experts with the banks split over ``ep``'s ranks. ``h`` [T,D] bf16 and
    ``logits`` fp32 [T,E] are this rank's tokens; ``w13_local`` [E/R, 2F, D] and
    ``w2_local`` [E/R, D, F] are this rank's slice of the banks. Bank gradients go to
    ``sink.G['w13'|'w2']`` (already summed over every rank's tokens, so they need no
    reduction); returns this rank's output rows [T, D]."""
    if h.shape[0] != ep.T:
        raise ValueError("every rank must pass max_tokens rows (pad the batch)")
    return _EPExperts.apply(h.contiguous(), logits.contiguous(), w13_local, w2_local, ep,
                            renormalize, sink)
