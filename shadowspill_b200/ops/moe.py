"""Routed-expert layer on the sm_100a kernels: router top-k, expert-sorted token
layout with 128-row-aligned segments, grouped tcgen05 GEMMs over the expert
banks, and a deterministic weighted combine; forward and backward.

``experts`` is the differentiable entry point used by the mixture layers on CUDA.
Bank weight gradients are written by grouped weight-gradient GEMMs directly into
the stage's gradient buffers (experts that received no tokens get zeros).
The math is the reference's routed-expert layer
(packages/workloads/src/shadowspill_workloads/models/shared/qwen_moe/experts.py:31-72).
"""
from __future__ import annotations

import torch

from . import _lib
from . import functional as F

_c = _lib
_lib.register("ss_moe_route", [_c.c_p, _c.c_ll, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_p,
                               _c.c_p, _c.c_p, _c.c_p])
_lib.register("ss_moe_layout", [_c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int, _c.c_p, _c.c_p,
                                _c.c_int, _c.c_p, _c.c_p, _c.c_p])
_lib.register("ss_moe_gather", [_c.c_p, _c.c_ll, _c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_int,
                                _c.c_int, _c.c_int, _c.c_p])
_lib.register("ss_moe_combine", [_c.c_p, _c.c_ll, _c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_int,
                                 _c.c_int, _c.c_int, _c.c_int, _c.c_p, _c.c_ll, _c.c_p, _c.c_p])
_lib.register("ss_gemm_grouped_bf16", [_c.c_p, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int,
                                       _c.c_int, _c.c_int, _c.c_int, _c.c_ll, _c.c_ll, _c.c_ll,
                                       _c.c_int, _c.c_int, _c.c_int, _c.c_p, _c.c_p, _c.c_int,
                                       _c.c_p, _c.c_p])


def route(logits: torch.Tensor, k: int, renormalize: bool):
    """fp32 logits [T,E] -> (ids int32 [T,k], weights fp32 [T,k], counts int32 [E])."""
    T, E = logits.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    counts = torch.empty(E, dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib().ss_moe_route(logits.data_ptr(), logits.stride(0), T, E, k,
                                       int(renormalize), ids.data_ptr(), wts.data_ptr(),
                                       counts.data_ptr(), _lib.stream_ptr()), "ss_moe_route")
    return ids, wts, counts


class Layout:
    """Expert-sorted row layout of one routing decision."""

    def __init__(self, ids: torch.Tensor, counts: torch.Tensor):
        T, k = ids.shape
        E = counts.numel()
        dev = ids.device
        self.T, self.k, self.E = T, k, E
        self.rows = -(-(T * k + E * 127) // 128) * 128      # worst-case padded rows
        self.tiles = self.rows // 128
        self.offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
        self.tile_expert = torch.empty(self.tiles, dtype=torch.int32, device=dev)
        self.dest = torch.empty(T * k, dtype=torch.int32, device=dev)
        cursor = torch.empty(E, dtype=torch.int32, device=dev)
        _lib.check(_lib.lib().ss_moe_layout(counts.data_ptr(), ids.data_ptr(), T, E, k,
                                            self.offsets.data_ptr(), self.tile_expert.data_ptr(),
                                            self.tiles, cursor.data_ptr(), self.dest.data_ptr(),
                                            _lib.stream_ptr()), "ss_moe_layout")

    def gather(self, x: torch.Tensor, weights: torch.Tensor | None = None) -> torch.Tensor:
        """Token rows -> zero-padded expert-sorted rows (scaled by ``weights`` when given)."""
        out = torch.zeros((self.rows, x.shape[1]), dtype=x.dtype, device=x.device)
        _lib.check(_lib.lib().ss_moe_gather(x.data_ptr(), x.stride(0), self.dest.data_ptr(),
                                            None if weights is None else weights.data_ptr(),
                                            out.data_ptr(), out.stride(0), self.T, self.k,
                                            x.shape[1], _lib.stream_ptr()), "ss_moe_gather")
        return out

    def combine(self, y: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor | None = None,
                accumulate: bool = False, dots_with: torch.Tensor | None = None,
                only_dots: bool = False):
        """Expert-sorted rows -> token rows; optionally the per-assignment dot products
        ``<dots_with[t], y[dest[t,j]]>`` (``only_dots`` skips the row output)."""
        D = y.shape[1]
        if only_dots:
            res = None
        else:
            res = out if out is not None else torch.empty((self.T, D), dtype=y.dtype, device=y.device)
        dots = (torch.empty((self.T, self.k), dtype=torch.float32, device=y.device)
                if dots_with is not None else None)
        _lib.check(_lib.lib().ss_moe_combine(
            y.data_ptr(), y.stride(0), self.dest.data_ptr(),
            None if weights is None else weights.data_ptr(),
            None if res is None else res.data_ptr(), 0 if res is None else res.stride(0),
            self.T, self.k, D, int(accumulate),
            None if dots_with is None else dots_with.data_ptr(),
            0 if dots_with is None else dots_with.stride(0),
            None if dots is None else dots.data_ptr(), _lib.stream_ptr()), "ss_moe_combine")
        return (res, dots) if dots_with is not None else res


def grouped_linear(x_sorted: torch.Tensor, bank: torch.Tensor, lay: Layout, transpose: bool = False,
                   out: torch.Tensor | None = None):
    """``y[r] = x[r] @ bank[e(r)]^T`` (or ``@ bank[e(r)]`` when ``transpose``) over sorted rows."""
    E = bank.shape[0]
    K = x_sorted.shape[1]
    N = bank.shape[2] if transpose else bank.shape[1]
    if out is None:
        out = torch.empty((lay.rows, N), dtype=x_sorted.dtype, device=x_sorted.device)
    _lib.check(_lib.lib().ss_gemm_grouped_bf16(
        x_sorted.data_ptr(), bank.data_ptr(), out.data_ptr(), 1, lay.rows, 0, N, K, E,
        x_sorted.stride(0), bank.stride(1), out.stride(0), int(transpose), 0, 0,
        lay.tile_expert.data_ptr(), None, 0, _lib.status_word(x_sorted.device).data_ptr(),
        _lib.stream_ptr()), "ss_gemm_grouped_bf16")
    return out


def grouped_wgrad(dy_sorted: torch.Tensor, x_sorted: torch.Tensor, lay: Layout, out: torch.Tensor,
                  accumulate: bool) -> None:
    """``out[e] (+)= dy[rows_e]^T @ x[rows_e]`` for every expert of a bank gradient [E, M, N]."""
    E, M, N = out.shape
    _lib.check(_lib.lib().ss_gemm_grouped_bf16(
        dy_sorted.data_ptr(), x_sorted.data_ptr(), out.data_ptr(), 2, lay.rows, M, N, 0, E,
        dy_sorted.stride(0), x_sorted.stride(0), out.stride(1), 1, int(out.dtype == torch.float32),
        int(accumulate), None, lay.offsets.data_ptr(), 0,
        _lib.status_word(out.device).data_ptr(), _lib.stream_ptr()), "ss_gemm_grouped_bf16")


def _weights_from_logits(logits, ids, renormalize):
    if renormalize:
        return torch.softmax(logits.gather(1, ids), dim=-1)
    return torch.softmax(logits, dim=-1).gather(1, ids)


class _Experts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, logits, w13, w2, k, renormalize, sink):
        ids, wts, counts = route(logits, k, renormalize)
        lay = Layout(ids, counts)
        xs = lay.gather(h)
        gu = grouped_linear(xs, w13, lay)
        ys = grouped_linear(F.swiglu_fwd(gu), w2, lay)
        out = lay.combine(ys, wts)
        ctx.save_for_backward(logits, ids, wts, xs, gu, w13, w2)
        ctx.lay, ctx.sink, ctx.renormalize = lay, sink, renormalize
        return out

    @staticmethod
    def backward(ctx, dout):
        logits, ids, wts, xs, gu, w13, w2 = ctx.saved_tensors
        lay, sink = ctx.lay, ctx.sink
        dout = dout.contiguous()
        hm = F.swiglu_fwd(gu)
        ys = grouped_linear(hm, w2, lay)
        _, dwts = lay.combine(ys, None, dots_with=dout, only_dots=True)
        del ys
        dys = lay.gather(dout, wts)                      # w * dout at every assignment
        if sink is not None and sink.wants("w2"):            # a frozen bank has no gradient buffer
            grouped_wgrad(dys, hm, lay, sink.G["w2"], sink.accumulate("w2"))
        dhm = grouped_linear(dys, w2, lay, transpose=True)
        del dys, hm
        dgu = F.swiglu_bwd(gu, dhm)
        del dhm
        if sink is not None and sink.wants("w13"):
            grouped_wgrad(dgu, xs, lay, sink.G["w13"], sink.accumulate("w13"))
        dxs = grouped_linear(dgu, w13, lay, transpose=True)
        dh = lay.combine(dxs, None)
        with torch.enable_grad():
            l = logits.detach().requires_grad_(True)
            _weights_from_logits(l, ids.long(), ctx.renormalize).backward(dwts)
        return dh, l.grad, None, None, None, None, None


def experts(h, logits, w13, w2, k: int, renormalize: bool, sink):
    """Routed experts on CUDA. ``h`` [T,D] bf16, ``logits`` fp32 [T,E], banks [E,2F,D] / [E,D,F]."""
    return _Experts.apply(h.contiguous(), logits.contiguous(), w13, w2, k, renormalize, sink)
