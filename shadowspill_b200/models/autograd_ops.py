"""``torch.autograd.Function`` wrappers over the op library.

Stages whose backward pass is derived by autograd (hybrid and mixture layers) are
written with these functions, so the math still runs on the hand-written kernels
on CUDA and on the plain-PyTorch definitions on CPU. ``Linear`` writes its weight
gradient straight into the stage's gradient buffer (created or accumulated),
which is the reference's gradient-destination rewriting
(packages/engine/src/shadowspill/pytorch/capture/gradients/destinations.py) done
at the op level: autograd never materialises a ``.grad`` tensor for a matrix.
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from ..ops import functional as F


class GradSink:
    """Where parameter gradients of one stage execution go."""

    def __init__(self, G: dict[str, torch.Tensor] | None, first: bool):
        self.G, self.first = G, first
        self.written: set[str] = set()

    def accumulate(self, name: str) -> bool:
        """False exactly once per name when this execution creates the gradient."""
        acc = not self.first or name in self.written
        self.written.add(name)
        return acc

    def wants(self, name: str) -> bool:
        """False for frozen parameters: their gradient buffer does not exist."""
        return self.G is not None and name in self.G

    def add_vector(self, name: str, g: torch.Tensor) -> None:
        if not self.wants(name):
            return
        dst = self.G[name]
        if self.accumulate(name):
            dst.add_(g.to(dst.dtype).reshape(dst.shape))
        else:
            dst.copy_(g.to(dst.dtype).reshape(dst.shape))


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, sink, name, index):
        ctx.save_for_backward(x, w)
        ctx.sink, ctx.name, ctx.index = sink, name, index
        return F.linear_fwd(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        sink = ctx.sink
        if sink is not None and sink.wants(ctx.name):
            dst = sink.G[ctx.name]
            key = ctx.name
            if ctx.index is not None:
                dst, key = dst[ctx.index], f"{ctx.name}[{ctx.index}]"
            F.linear_wgrad(dy, x, out=dst, accumulate=sink.accumulate(key))
        dx = F.linear_dgrad(dy, w) if ctx.needs_input_grad[0] else None
        return dx, None, None, None, None


def linear(x: torch.Tensor, w: torch.Tensor, sink: GradSink | None, name: str,
           index: int | None = None) -> torch.Tensor:
    """``x[T,K] @ w[N,K]^T``; the weight gradient lands in ``sink.G[name]`` (or in its
    slice ``[index]`` for one expert of a bank)."""
    return _Linear.apply(x, w, sink, name, index)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, zero_centered, sink, name):
        y, rstd = F.rmsnorm_fwd(x, w, eps, zero_centered)
        ctx.save_for_backward(x, w, rstd)
        ctx.zc, ctx.sink, ctx.name = zero_centered, sink, name
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, rstd = ctx.saved_tensors
        dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        dx = F.rmsnorm_bwd(x, w, gy.contiguous(), rstd, dw, ctx.zc)
        if ctx.sink is not None and ctx.sink.G is not None:
            ctx.sink.add_vector(ctx.name, dw)
        return dx, None, None, None, None, None


def rmsnorm(x, w, eps, zero_centered, sink, name):
    """Row RMSNorm over the last dimension of a 2-D tensor."""
    return _RMSNorm.apply(x, w, eps, zero_centered, sink, name)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, heads, dh, rot, theta):
        ctx.save_for_backward(positions)
        ctx.args = (heads, dh, rot, theta)
        out = x.clone()
        F.rope_(out, positions, col0=0, heads=heads, dh=dh, rot=rot, theta=theta)
        return out

    @staticmethod
    def backward(ctx, g):
        (positions,) = ctx.saved_tensors
        heads, dh, rot, theta = ctx.args
        g = g.clone()
        F.rope_(g, positions, col0=0, heads=heads, dh=dh, rot=rot, theta=theta, inverse=True)
        return g, None, None, None, None, None


def rope(x, positions, heads, dh, rot, theta):
    """Half-split rotary over the first ``rot`` channels of each head of ``x`` [T, heads*dh]."""
    return _Rope.apply(x, positions, heads, dh, rot, theta)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen):
        out, lse = F.attention_varlen(q, k, v, cu_seqlens, max_seqlen)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens)
        ctx.max_seqlen = max_seqlen
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        dq, dk, dv = F.attention_varlen_bwd(q, k, v, out, lse, dout.contiguous(), cu, ctx.max_seqlen)
        return dq, dk, dv, None, None


def attention(q, k, v, cu_seqlens, max_seqlen):
    return _Attention.apply(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, max_seqlen)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return F.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        (gu,) = ctx.saved_tensors
        return F.swiglu_bwd(gu, dh.contiguous())


def swiglu(gu):
    """``silu(gate) * up`` for ``gu = [gate | up]`` along the last dimension."""
    return _SwiGLU.apply(gu)


def lora_linear(x, w, a, b, scale: float, sink: GradSink | None, name: str):
    """``x w^T + scale * (x a^T) b^T`` with factor gradients under ``<name>_lora_a/_b``;
    the base gradient is skipped when ``sink`` has no buffer for ``name`` (frozen base)."""
    y = linear(x, w, sink, name)
    low = linear(linear(x, a, sink, f"{name}_lora_a"), b, sink, f"{name}_lora_b")
    return y + low * scale


# ---------------------------------------------------------------------------- grouped (expert) ops
class _GroupedLinear(torch.autograd.Function):
    """Rows sorted by expert times that expert's matrix, differentiable on both sides."""

    @staticmethod
    def forward(ctx, xs, bank, lay, sink, name):
        from ..ops import moe as moe_ops
        ctx.save_for_backward(xs, bank)
        ctx.lay, ctx.sink, ctx.name = lay, sink, name
        return moe_ops.grouped_linear(xs, bank, lay)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import moe as moe_ops
        xs, bank = ctx.saved_tensors
        dy = dy.contiguous()
        sink = ctx.sink
        if sink is not None and sink.wants(ctx.name):
            moe_ops.grouped_wgrad(dy, xs, ctx.lay, sink.G[ctx.name], sink.accumulate(ctx.name))
        dx = moe_ops.grouped_linear(dy, bank, ctx.lay, transpose=True) if ctx.needs_input_grad[0] else None
        return dx, None, None, None, None


def grouped_linear(xs, bank, lay, sink, name):
    return _GroupedLinear.apply(xs, bank, lay, sink, name)


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, lay):
        ctx.lay = lay
        return lay.gather(x)

    @staticmethod
    def backward(ctx, dxs):
        return ctx.lay.combine(dxs.contiguous(), None), None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ys, wts, lay):
        ctx.save_for_backward(ys, wts)
        ctx.lay = lay
        return lay.combine(ys, wts)

    @staticmethod
    def backward(ctx, dout):
        ys, wts = ctx.saved_tensors
        dout = dout.contiguous()
        _, dwts = ctx.lay.combine(ys, None, dots_with=dout, only_dots=True)
        return ctx.lay.gather(dout, wts), dwts, None


def expert_gather(x, lay):
    """Token rows -> expert-sorted padded rows."""
    return _Gather.apply(x, lay)


def expert_combine(ys, wts, lay):
    """Expert-sorted rows -> token rows, weighted by the routing weights (differentiable
    in both)."""
    return _Combine.apply(ys, wts, lay)
