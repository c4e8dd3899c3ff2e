"""Gated DeltaNet chunked rule on the tcgen05 kernels of ``ops/csrc/deltanet_chunk.cu``.

Forward is two launches after a tiny sequence-id kernel: ``ss_dn_prep`` (per chunk and pair of
V heads: K K^T, Q K^T, the 64x64 triangular inverse, W^T, U0^T) and ``ss_dn_fwd`` (per V head, the
state walk over chunks with S^T resident in TMEM). Backward recomputes both with their saves
switched on, then runs the reverse state walk, the per-chunk products and the gradient of the
chunk-local algebra. Nothing but the inputs is kept between forward and backward.

Reference math: packages/workloads/src/shadowspill_workloads/models/qwen35/implementations/
pytorch/delta_rule/reference.py:8-41 (forward) and :43-132 (backward).
"""
from __future__ import annotations

import torch

from . import _lib

_c = _lib
_P = _c.c_p
_lib.register("ss_dn_seq_ids", [_P, _c.c_int, _c.c_int, _P, _P])
_lib.register("ss_dn_prep", [_P] * 16 + [_c.c_int] * 3 + [_c.c_f, _P, _P])
_lib.register("ss_dn_fwd", [_P] * 9 + [_c.c_int] * 3 + [_P, _P])
_lib.register("ss_dn_bwd_state", [_P] * 8 + [_c.c_int] * 3 + [_P, _P])
_lib.register("ss_dn_bwd_chunk", [_P] * 10 + [_c.c_int] * 3 + [_P, _P])
_lib.register("ss_dn_bwd_prep", [_P] * 21 + [_c.c_int] * 3 + [_c.c_f, _P, _P])

CHUNK, WIDTH = 64, 128


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, chunk: int = CHUNK) -> bool:
    """Do these operands run on the kernels (bf16 on a GPU, 128-wide heads, 64-token chunks)?"""
    return (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16 and chunk == CHUNK
            and q.shape[-1] == WIDTH and v.shape[-1] == WIDTH and v.shape[1] % q.shape[1] == 0)


class _Geometry:
    def __init__(self, T: int, H: int, Hk: int):
        self.T, self.H, self.Hk = T, H, Hk
        self.n = -(-T // CHUNK)
        self.rep = H // Hk
        self.P = (self.rep + 1) // 2
        self.NP = Hk * self.P


def _ptr(t):
    return None if t is None else t.data_ptr()


class _Buffers:
    """Per-call operands of the chunk kernels. ``backward`` adds what only a backward pass reads."""

    def __init__(self, geo: _Geometry, dev, backward: bool):
        n, NP, H = geo.n, geo.NP, geo.H
        # a pair slot without a second head is never written: keep it defined
        make = torch.zeros if geo.rep % 2 else torch.empty
        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.sid = torch.empty(n * CHUNK, dtype=torch.int32, device=dev)
        self.WTp, self.U0Tp = make((n, NP, 128, 128), **bf), make((n, NP, 128, 128), **bf)
        self.QG, self.KD = torch.empty((n, H, 64, 128), **bf), torch.empty((n, H, 64, 128), **bf)
        self.MQ = make((n, NP, 128, 64), **bf)
        self.gam, self.gc = torch.empty((n, H, 64), **f32), torch.empty((n, H), **f32)
        self.TMT = self.XW = self.XU = self.ST = self.UTp = None
        if backward:
            self.TMT, self.XW, self.XU = (make((n, NP, 128, 64), **bf) for _ in range(3))
            self.ST, self.dSpT = torch.empty((n, H, 128, 128), **bf), torch.empty((n, H, 128, 128), **bf)
            self.UTp, self.dUTp = make((n, NP, 128, 128), **bf), make((n, NP, 128, 128), **bf)
            self.dKdTp, self.dQgTp, self.dWTp = (make((n, NP, 128, 128), **bf) for _ in range(3))
            self.dMQ = make((n, NP, 128, 64), **bf)
            self.dgc = torch.empty((n, H), **f32)


# A backward task that recomputes its forward pass runs the rule's forward twice on the same
# operands: once for the layer's output, once inside the rule's own backward, which needs the
# chunk intermediates. Inside ``keeping_intermediates()`` the first run keeps them and the second
# is skipped. The scope is one task, so nothing outlives it and a pointer reused by other data in
# a later task can never match.
_scope = {"on": False, "key": None, "value": None}


class keeping_intermediates:
    def __enter__(self):
        _scope.update(on=True, key=None, value=None)
        return self

    def __exit__(self, *exc):
        _scope.update(on=False, key=None, value=None)
        return False


def _operand_key(q, k, v, beta, g, cu_seqlens):
    return tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in (q, k, v, beta, g, cu_seqlens))


def _forward(q, k, v, beta, g, cu_seqlens, backward: bool):
    T, Hk, _ = q.shape
    H = v.shape[1]
    geo = _Geometry(T, H, Hk)
    B = _Buffers(geo, q.device, backward)
    L, st, status = _lib.lib(), _lib.stream_ptr(), _lib.status_word(q.device).data_ptr()
    _lib.check(L.ss_dn_seq_ids(cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, T, B.sid.data_ptr(), st),
               "ss_dn_seq_ids")
    scale = WIDTH ** -0.5
    _lib.check(L.ss_dn_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), g.data_ptr(),
                            B.sid.data_ptr(), B.WTp.data_ptr(), B.U0Tp.data_ptr(), B.QG.data_ptr(),
                            B.KD.data_ptr(), B.MQ.data_ptr(), _ptr(B.TMT), _ptr(B.XW), _ptr(B.XU),
                            B.gam.data_ptr(), B.gc.data_ptr(), T, H, Hk, scale, status, st), "ss_dn_prep")
    out = torch.empty((T, H, WIDTH), dtype=torch.bfloat16, device=q.device)
    _lib.check(L.ss_dn_fwd(B.WTp.data_ptr(), B.U0Tp.data_ptr(), B.QG.data_ptr(), B.KD.data_ptr(),
                           B.MQ.data_ptr(), B.gc.data_ptr(), out.data_ptr(), _ptr(B.ST), _ptr(B.UTp),
                           T, H, Hk, status, st), "ss_dn_fwd")
    return out, B, geo


def forward_keeping(q, k, v, beta, g, cu_seqlens, raw_key=None):
    """The forward pass on prepared operands; inside ``keeping_intermediates()`` with its saves on,
    kept for a backward pass in the same scope that names the same operands, either as the caller
    passed them (``raw_key``) or prepared."""
    if not _scope["on"] or _head_groups > 1:       # head groups are about holding less, not more
        return _forward(q, k, v, beta, g, cu_seqlens, backward=False)[0]
    out, B, geo = _forward(q, k, v, beta, g, cu_seqlens, backward=True)
    _scope["key"] = {raw_key, _operand_key(q, k, v, beta, g, cu_seqlens)}
    _scope["value"] = (B, geo, (q, k, v, beta, g))
    return out


def _operands(q, k, v, beta, g):
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    return q, k, v, beta.float().contiguous(), g.float().contiguous()


# Head-group chunks: the rule is independent per key head (and the value heads that share it), so
# a call can run in groups of key heads one after another; the chunk intermediates (about 1 GB for
# 8,192 tokens of 16/32 heads with the backward saves) then exist for one group at a time.
# (packages/workloads/src/shadowspill_workloads/policies/text/chunking.py:22,
# ``linear_attention_head_chunks``.)
_head_groups = 1


def set_head_groups(groups: int) -> None:
    """Run every call in ``groups`` groups of key heads (1 = all heads at once)."""
    global _head_groups
    if groups < 1:
        raise ValueError("head groups must be at least 1")
    _head_groups = int(groups)


def _groups(Hk: int) -> list[tuple[int, int]]:
    g = _head_groups
    if g <= 1 or Hk % g:
        return [(0, Hk)]
    per = Hk // g
    return [(a, a + per) for a in range(0, Hk, per)]


class _GatedDeltaRule(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, beta, g, cu_seqlens):
        raw = _operand_key(q, k, v, beta, g, cu_seqlens)
        q, k, v, bf, gf = _operands(q, k, v, beta, g)
        out = forward_keeping(q, k, v, bf, gf, cu_seqlens, raw)
        ctx.save_for_backward(q, k, v, bf, gf, cu_seqlens)
        ctx.scalar_dtypes = (beta.dtype, g.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, bf, gf, cu_seqlens = ctx.saved_tensors
        dq, dk, dv, dbeta, dg = backward(q, k, v, bf, gf, cu_seqlens, dout)
        return dq, dk, dv, dbeta.to(ctx.scalar_dtypes[0]), dg.to(ctx.scalar_dtypes[1]), None


def backward(q, k, v, beta, g, cu_seqlens, dout):
    """Gradients of :func:`gated_delta_rule` for ``dout`` [T,H,128] (bf16): ``(dq, dk, dv, dbeta,
    dg)`` with dbeta, dg in fp32. The forward pass is recomputed with its saves switched on."""
    spans = _groups(q.shape[1])
    if len(spans) > 1:
        rep = v.shape[1] // q.shape[1]
        parts = [_backward_all(q[:, a:b], k[:, a:b], v[:, a * rep:b * rep], beta[:, a * rep:b * rep],
                               g[:, a * rep:b * rep], cu_seqlens, dout[:, a * rep:b * rep]) for a, b in spans]
        return tuple(torch.cat([p[i] for p in parts], dim=1) for i in range(5))
    return _backward_all(q, k, v, beta, g, cu_seqlens, dout)


def _backward_all(q, k, v, beta, g, cu_seqlens, dout):
    dout = dout.to(torch.bfloat16).contiguous()
    if _scope["on"] and _scope["key"] and _operand_key(q, k, v, beta, g, cu_seqlens) in _scope["key"]:
        B, geo, (q, k, v, beta, g) = _scope["value"]     # the forward pass of this task kept them
        _scope["key"] = _scope["value"] = None
    else:
        q, k, v, beta, g = _operands(q, k, v, beta, g)
        _, B, geo = _forward(q, k, v, beta, g, cu_seqlens, backward=True)
    T, H, Hk = geo.T, geo.H, geo.Hk
    L, st, status = _lib.lib(), _lib.stream_ptr(), _lib.status_word(q.device).data_ptr()
    _lib.check(L.ss_dn_bwd_state(dout.data_ptr(), B.MQ.data_ptr(), B.KD.data_ptr(), B.QG.data_ptr(),
                                 B.WTp.data_ptr(), B.gc.data_ptr(), B.dSpT.data_ptr(), B.dUTp.data_ptr(),
                                 T, H, Hk, status, st), "ss_dn_bwd_state")
    _lib.check(L.ss_dn_bwd_chunk(B.dSpT.data_ptr(), B.ST.data_ptr(), B.UTp.data_ptr(), B.dUTp.data_ptr(),
                                 dout.data_ptr(), B.dKdTp.data_ptr(), B.dQgTp.data_ptr(),
                                 B.dWTp.data_ptr(), B.dMQ.data_ptr(), B.dgc.data_ptr(), T, H, Hk, status,
                                 st), "ss_dn_bwd_chunk")
    dev = q.device
    dq = torch.empty((T, geo.NP, WIDTH), dtype=torch.bfloat16, device=dev)
    dk = torch.empty_like(dq)
    dv = torch.empty((T, H, WIDTH), dtype=torch.bfloat16, device=dev)
    dbeta = torch.empty((T, H), dtype=torch.float32, device=dev)
    dg = torch.empty_like(dbeta)
    _lib.check(L.ss_dn_bwd_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(),
                                B.sid.data_ptr(), B.gam.data_ptr(), B.gc.data_ptr(), B.dgc.data_ptr(),
                                B.dWTp.data_ptr(), B.dUTp.data_ptr(), B.TMT.data_ptr(), B.XW.data_ptr(),
                                B.XU.data_ptr(), B.dKdTp.data_ptr(), B.dQgTp.data_ptr(), B.dMQ.data_ptr(),
                                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dbeta.data_ptr(),
                                dg.data_ptr(), T, H, Hk, WIDTH ** -0.5, status, st), "ss_dn_bwd_prep")
    if geo.P > 1:      # several pairs of V heads share one QK head: add their contributions
        dq = dq.view(T, Hk, geo.P, WIDTH).float().sum(2).to(torch.bfloat16)
        dk = dk.view(T, Hk, geo.P, WIDTH).float().sum(2).to(torch.bfloat16)
    return dq.view(T, Hk, WIDTH), dk.view(T, Hk, WIDTH), dv, dbeta, dg


def gated_delta_rule(q, k, v, beta, g, cu_seqlens):
    """q, k [T,Hk,128] bf16 (L2-normalised), v [T,H,128] bf16, beta, g [T,H] (g = log decay <= 0),
    ``cu_seqlens`` int32 on the device. Returns [T,H,128] bf16; differentiable in q, k, v, beta, g."""
    spans = _groups(q.shape[1])
    if len(spans) > 1:
        rep = v.shape[1] // q.shape[1]
        return torch.cat([_GatedDeltaRule.apply(q[:, a:b], k[:, a:b], v[:, a * rep:b * rep], beta[:, a * rep:b * rep],
                                                g[:, a * rep:b * rep], cu_seqlens) for a, b in spans], dim=1)
    return _GatedDeltaRule.apply(q, k, v, beta, g, cu_seqlens)
