"""Tensor-level entry points of the op library.

CUDA tensors go to the hand-written sm_100a kernels in ``libss_kernels.so``;
CPU tensors go to the plain-PyTorch definitions in :mod:`.reference`, which are
also the numerical oracles of the kernel tests. There is no third path: a CUDA
tensor with the library missing raises.
"""
from __future__ import annotations

import math

import os

import torch

from . import _lib, reference

_BF16 = torch.bfloat16


# SS_KERNELS=library is the comparison arm: the same planner, runtime and model code, but every op
# runs on vendor libraries and eager PyTorch (cuBLAS GEMMs, flash-attn, elementwise tensor
# operations) instead of this repository's kernels. It exists to be timed against, never as a
# fallback: nothing selects it but the variable.
_LIBRARY = os.environ.get("SS_KERNELS", "native") == "library"


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and not _LIBRARY


def _gemm_library(a, b, a_mn, b_mn, out, accumulate, alpha, out_dtype):
    """cuBLAS arm of ``gemm`` (bf16 operands, fp32 accumulation inside the library)."""
    am = a.t() if a_mn else a
    bm = b if b_mn else b.t()
    if out is None:
        res = torch.mm(am, bm)
        return (res if alpha == 1.0 else res * alpha).to(out_dtype)
    if out.dtype == am.dtype and out.is_contiguous():
        return torch.addmm(out, am, bm, beta=1.0 if accumulate else 0.0, alpha=alpha, out=out)
    res = torch.mm(am, bm).to(out.dtype)
    if alpha != 1.0:
        res = res * alpha
    return out.add_(res) if accumulate else out.copy_(res)


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------------ GEMM
# plain GEMMs run on the CTA-pair kernel; SS_GEMM_PAIR=0 selects the single-CTA kernel
_PAIR_GEMM = os.environ.get("SS_GEMM_PAIR", "1") == "1"


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, accumulate: bool = False, alpha: float = 1.0,
         out_dtype: torch.dtype | None = None, bn: int = 0) -> torch.Tensor:
    """``C[M,N] (+)= alpha * op(A) @ op(B)`` with bf16 operands, fp32 accumulation.

    ``a_mn``: A is stored ``[K, M]`` (else ``[M, K]``); ``b_mn``: B is stored
    ``[K, N]`` (else ``[N, K]``). ``accumulate`` adds the existing ``out``.
    """
    M = a.shape[1] if a_mn else a.shape[0]
    K = a.shape[0] if a_mn else a.shape[1]
    N = b.shape[1] if b_mn else b.shape[0]
    Kb = b.shape[0] if b_mn else b.shape[1]
    if K != Kb:
        raise ValueError(f"contraction mismatch: {tuple(a.shape)} vs {tuple(b.shape)}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an existing output")
        out_dtype = out_dtype or a.dtype
    elif out.shape != (M, N):
        raise ValueError(f"output shape {tuple(out.shape)} != {(M, N)}")
    if a.is_cuda and _LIBRARY:
        return _gemm_library(a, b, a_mn, b_mn, out, accumulate, alpha, out_dtype or a.dtype)
    if not _cuda(a):
        return reference.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=accumulate,
                              alpha=alpha, out_dtype=out_dtype or a.dtype)
    if a.dtype != _BF16 or b.dtype != _BF16:
        raise TypeError("gemm operands must be bfloat16 on CUDA")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm operands must have unit inner stride")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.stride(-1) != 1 or out.dtype not in (_BF16, torch.float32):
        raise ValueError("gemm output must be bf16/fp32 with unit inner stride")
    if N % 8 or a.stride(0) % 8 or b.stride(0) % 8 or out.stride(0) % (4 if out.dtype == torch.float32 else 8):
        # TMA moves 16-byte pieces: say which size breaks that instead of returning the kernel's code
        raise ValueError(f"gemm on the GPU needs N and the row strides in multiples of 8 elements "
                         f"(N={N}, strides {a.stride(0)}, {b.stride(0)}, {out.stride(0)}); pad the operand")
    if _PAIR_GEMM and bn == 0 and M >= 256 and N >= 128:
        # CTA-pair kernel (tcgen05 cta_group::2): 256x256 tiles, half the shared-memory
        # traffic per FLOP of the single-CTA kernel
        rc = _lib.lib().ss_gemm2_bf16(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
            out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate),
            float(alpha), 0, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "ss_gemm2_bf16")
        return out
    rc = _lib.lib().ss_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0),
        out.stride(0), int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate),
        float(alpha), int(bn), 0, _lib.status_word(a.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "ss_gemm_bf16")
    return out


# ------------------------------------------------------------------------ gather fused into the GEMM
class PendingGather:
    """A sharded weight whose all-gather has not happened yet: the first GEMM that consumes the
    full-weight buffer pulls the shards from the peers itself (``ss_gemm2_gather_bf16``)."""

    def __init__(self, full: torch.Tensor, shard_ptrs, per: int, world: int, rank: int, fallback):
        self.full, self.shard_ptrs, self.per, self.world, self.rank = full, shard_ptrs, per, world, rank
        self.fallback = fallback          # gathers with the stand-alone kernel instead


_pending_gathers: dict[int, PendingGather] = {}
fused_gather_launches = 0


def register_gather(info: PendingGather) -> None:
    _pending_gathers[info.full.data_ptr()] = info


def flush_gathers(ptrs=None) -> int:
    """Runs the stand-alone gather for every registered weight no GEMM consumed (all of them, or
    those whose buffers start at ``ptrs``). Returns how many there were."""
    keys = [k for k in list(_pending_gathers) if ptrs is None or k in ptrs]
    for k in keys:
        _pending_gathers.pop(k).fallback()
    return len(keys)


def _gemm_gather(x: torch.Tensor, info: PendingGather, out, accumulate: bool):
    global fused_gather_launches
    w = info.full
    N, K = w.shape
    M = x.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    counters = torch.zeros(-(-N // 256), dtype=torch.int32, device=x.device)
    import ctypes
    ptrs = (ctypes.c_void_p * info.world)(*info.shard_ptrs)
    rc = _lib.lib().ss_gemm2_gather_bf16(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0), out.stride(0),
        int(out.dtype == torch.float32), int(accumulate), 1.0, ptrs, info.per, info.world, info.rank,
        counters.data_ptr(), 0, 0, _lib.status_word(x.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "ss_gemm2_gather_bf16")
    fused_gather_launches += 1
    return out


def linear_fwd(x, w, out=None, accumulate=False):
    """``y[T,N] (+)= x[T,K] @ w[N,K]^T``. A weight registered by ``register_gather`` is gathered
    from its shards by this GEMM itself."""
    if _pending_gathers:
        info = _pending_gathers.pop(w.data_ptr(), None)
        if info is not None:
            fits = (_cuda(x) and x.dtype == _BF16 and w.dim() == 2 and w.is_contiguous() and x.stride(-1) == 1
                    and x.shape[0] >= 256 and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0
                    and (out is None or out.stride(-1) == 1))
            if fits:
                return _gemm_gather(x, info, out, accumulate)
            info.fallback()
    return gemm(x, w, out=out, accumulate=accumulate)


def linear_dgrad(dy, w, out=None, accumulate=False):
    """``dx[T,K] (+)= dy[T,N] @ w[N,K]``"""
    return gemm(dy, w, b_mn=True, out=out, accumulate=accumulate)


def linear_wgrad(dy, x, out=None, accumulate=False, out_dtype=None):
    """``dw[N,K] (+)= dy[T,N]^T @ x[T,K]`` -- the in-place gradient accumulation
    (reference: shadowspill::accumulate_matmul_)."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=accumulate, out_dtype=out_dtype)


# ------------------------------------------------------------------------ norms
def rmsnorm_fwd(x, w, eps=1e-5, zero_centered=False, delta=None, out=None, rstd=None):
    """``x += delta`` (optional, in place) then RMSNorm. Returns ``(y, rstd)``."""
    if not _cuda(x):
        y, rs = reference.rmsnorm_fwd(x, w, eps, zero_centered, delta)
        if out is not None:
            y = out.copy_(y)
        if rstd is not None:
            rs = rstd.copy_(rs)
        return y, rs
    T, D = x.shape
    y = torch.empty_like(x) if out is None else out
    rs = torch.empty(T, dtype=torch.float32, device=x.device) if rstd is None else rstd
    rc = _lib.lib().ss_rmsnorm_fwd(x.data_ptr(), _ptr(delta), w.data_ptr(), y.data_ptr(),
                                   rs.data_ptr(), T, D, float(eps), int(zero_centered),
                                   _lib.stream_ptr())
    _lib.check(rc, "ss_rmsnorm_fwd")
    return y, rs


def rmsnorm_bwd(x, w, gy, rstd, dw, zero_centered=False, dx=None, accumulate=False):
    """Returns ``dx`` (added into ``dx`` when ``accumulate``); ``dw`` (fp32) is
    accumulated in place."""
    if not _cuda(x):
        dxr, dwr = reference.rmsnorm_bwd(x, w, gy, rstd, zero_centered)
        if dw is not None:
            dw.add_(dwr.to(dw.dtype))
        if dx is None:
            return dxr.to(x.dtype)
        dx.copy_(((dx.float() if accumulate else 0) + dxr).to(dx.dtype))
        return dx
    T, D = x.shape
    if dx is None:
        if accumulate:
            raise ValueError("accumulate needs dx")
        dx = torch.empty_like(x)
    if dw is not None and dw.dtype != torch.float32:
        raise TypeError("rmsnorm dw accumulator must be fp32")
    rc = _lib.lib().ss_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), gy.data_ptr(), rstd.data_ptr(),
                                   dx.data_ptr(), _ptr(dw), T, D, int(zero_centered),
                                   int(accumulate), _lib.stream_ptr())
    _lib.check(rc, "ss_rmsnorm_bwd")
    return dx


# ------------------------------------------------------------------------ rotary
def rope_(buf, positions, *, col0, heads, dh, rot=None, theta=10000.0, inverse=False):
    """In-place rotary on ``heads`` heads of width ``dh`` starting at column ``col0``
    of the 2-D buffer ``buf``; ``inverse`` applies the backward rotation."""
    rot = dh if rot is None else rot
    if not _cuda(buf):
        return reference.rope_(buf, positions, col0, heads, dh, rot, theta, inverse)
    if positions.dtype != torch.int32:
        raise TypeError("positions must be int32")
    rc = _lib.lib().ss_rope(buf.data_ptr(), positions.data_ptr(), buf.shape[0], buf.stride(0),
                            col0, heads, dh, rot, float(theta), int(inverse), _lib.stream_ptr())
    _lib.check(rc, "ss_rope")
    return buf


# ------------------------------------------------------------------------ SwiGLU
def swiglu_fwd(gu, out=None):
    if not _cuda(gu):
        res = reference.swiglu_fwd(gu)
        return res if out is None else out.copy_(res)
    T, F2 = gu.shape
    h = torch.empty((T, F2 // 2), dtype=gu.dtype, device=gu.device) if out is None else out
    _lib.check(_lib.lib().ss_swiglu_fwd(gu.data_ptr(), h.data_ptr(), T, F2 // 2,
                                        _lib.stream_ptr()), "ss_swiglu_fwd")
    return h


def swiglu_bwd(gu, dh, out=None):
    if not _cuda(gu):
        res = reference.swiglu_bwd(gu, dh)
        return res if out is None else out.copy_(res)
    T, F2 = gu.shape
    dgu = torch.empty_like(gu) if out is None else out
    _lib.check(_lib.lib().ss_swiglu_bwd(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), T, F2 // 2,
                                        _lib.stream_ptr()), "ss_swiglu_bwd")
    return dgu


# ------------------------------------------------------------------------ embedding
def embedding_fwd(ids, W, out=None):
    if not _cuda(W):
        res = reference.embedding_fwd(ids, W)
        return res if out is None else out.copy_(res)
    T = ids.numel()
    V, D = W.shape
    o = torch.empty((T, D), dtype=W.dtype, device=W.device) if out is None else out
    _lib.check(_lib.lib().ss_embedding_fwd(ids.data_ptr(), W.data_ptr(), o.data_ptr(), T, D, V,
                                           _lib.stream_ptr()), "ss_embedding_fwd")
    return o


def embedding_bwd(ids, g, dW):
    """``dW[ids[t]] += g[t]`` (dW fp32 or bf16)."""
    if not _cuda(g):
        return reference.embedding_bwd(ids, g, dW)
    T = ids.numel()
    V, D = dW.shape
    _lib.check(_lib.lib().ss_embedding_bwd(ids.data_ptr(), g.data_ptr(), dW.data_ptr(), T, D, V,
                                           int(dW.dtype == torch.float32), _lib.stream_ptr()),
               "ss_embedding_bwd")
    return dW


# ------------------------------------------------------------------------ cross-entropy block
def cross_entropy_(logits, targets, weights, loss_sum, *, grad_scale=1.0, write_grad=True,
                   lse=None):
    """Adds the weighted loss of a logits block into ``loss_sum`` (fp32[1]) and
    rewrites ``logits`` with its gradient. Masked rows carry weight 0."""
    if not _cuda(logits):
        loss, _ = reference.cross_entropy_(logits, targets, weights, grad_scale, write_grad)
        loss_sum.add_(loss)
        return loss_sum
    R, V = logits.shape
    _lib.check(_lib.lib().ss_cross_entropy(logits.data_ptr(), targets.data_ptr(), _ptr(weights),
                                           loss_sum.data_ptr(), _ptr(lse), R, V, logits.stride(0),
                                           float(grad_scale), int(write_grad), _lib.stream_ptr()),
               "ss_cross_entropy")
    return loss_sum


def clipped_policy_(logits, targets, weights, old_logp, advantage, loss_sum, *, clip=0.2,
                    ref_logp=None, ref_beta=0.0, grad_scale=1.0, write_grad=True, logp=None):
    """Clipped policy objective on a logits block: adds the weighted loss into
    ``loss_sum`` and rewrites ``logits`` with its gradient; ``logp`` (fp32[R]) receives
    the target log-probabilities."""
    if not _cuda(logits):
        loss, lp = reference.clipped_policy_(logits, targets, weights, old_logp, advantage, clip,
                                             ref_logp, ref_beta, grad_scale, write_grad)
        loss_sum.add_(loss)
        if logp is not None:
            logp.copy_(lp)
        return loss_sum
    R, V = logits.shape
    _lib.check(_lib.lib().ss_token_objective(
        logits.data_ptr(), targets.data_ptr(), _ptr(weights), loss_sum.data_ptr(), _ptr(logp), R, V,
        logits.stride(0), float(grad_scale), int(write_grad), 1, old_logp.data_ptr(),
        advantage.data_ptr(), float(clip), _ptr(ref_logp), float(ref_beta), _lib.stream_ptr()),
        "ss_token_objective")
    return loss_sum


def target_logprobs_(logits, targets, logp):
    """log p(target) per row of a logits block into ``logp`` (fp32[R]); logits unchanged."""
    if not _cuda(logits):
        lf = logits.float()
        V = logits.shape[-1]
        picked = lf.gather(1, targets.clamp(0, V - 1)[:, None])[:, 0]
        logp.copy_(picked - torch.logsumexp(lf, dim=-1))
        return logp
    R, V = logits.shape
    scratch = torch.zeros(1, dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().ss_token_objective(
        logits.data_ptr(), targets.data_ptr(), None, scratch.data_ptr(), logp.data_ptr(), R, V,
        logits.stride(0), 1.0, 0, 0, None, None, 0.0, None, 0.0, _lib.stream_ptr()),
        "ss_token_objective")
    return logp


# ------------------------------------------------------------------------ AdamW
def adamw_(p, g, m, v, *, lr, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1,
           grad_scale=1.0, seed=0, offset=0, stochastic_param=True, stochastic_state=True):
    """Fused AdamW on flat tensors. bf16 parameters/moments use stochastic
    rounding driven by a counter RNG keyed on (seed, step, global element index),
    so a shard updated alone produces the same bits as the whole tensor."""
    if not _cuda(p):
        return reference.adamw_(p, g, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                                weight_decay=weight_decay, step=step, grad_scale=grad_scale)
    n = p.numel()
    L = _lib.lib()
    if p.dtype == torch.float32:
        _lib.check(L.ss_adamw_f32(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n,
                                  lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                                  _lib.stream_ptr()), "ss_adamw_f32")
        return
    _lib.check(L.ss_adamw_sr(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n,
                             int(g.dtype == torch.float32), lr, beta1, beta2, eps, weight_decay,
                             step, grad_scale, seed, offset, int(stochastic_param),
                             int(stochastic_state), _lib.stream_ptr()), "ss_adamw_sr")


def sumsq(x, partials, out, accumulate=False):
    """Sum of squares into ``out`` (fp32[1]) using caller-owned ``partials`` (fp32[256])."""
    if not _cuda(x):
        val = x.float().square().sum()
        out.copy_(out + val if accumulate else val.reshape(1))
        return out
    _lib.check(_lib.lib().ss_sumsq(x.data_ptr(), x.numel(), partials.data_ptr(), out.data_ptr(),
                                   int(accumulate), _lib.stream_ptr()), "ss_sumsq")
    return out


# ------------------------------------------------------------------------ attention
def attention_varlen(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None, lse=None):
    """Packed causal GQA forward. Returns ``(out, lse)``; ``lse`` is fp32 ``[Hq, T]``."""
    if not q.is_cuda:
        o, l = reference.attention_varlen(q, k, v, cu_seqlens, scale)
        if out is not None:
            o = out.copy_(o)
        if lse is not None:
            l = lse.copy_(l)
        return o, l
    from . import attention
    return attention.forward(q, k, v, cu_seqlens, max_seqlen, scale, out=out, lse=lse)


def attention_varlen_bwd(q, k, v, out, lse, dout, cu_seqlens, max_seqlen, scale=None):
    if not q.is_cuda:
        return reference.attention_varlen_bwd(q, k, v, out, lse, dout, cu_seqlens, scale)
    from . import attention
    return attention.backward(q, k, v, out, lse, dout, cu_seqlens, max_seqlen, scale)


def default_scale(dh: int) -> float:
    return 1.0 / math.sqrt(dh)
