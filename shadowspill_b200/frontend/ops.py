"""The op library as ``torch.library`` custom operators (namespace ``ss``).

Every operator here is a functional wrapper over :mod:`shadowspill_b200.ops.functional`
(hand-written sm_100a kernels on CUDA tensors, the plain-PyTorch definitions on CPU)
with a fake (shape) implementation and an autograd rule, so that ``torch.export`` and
AOTAutograd see the model as a graph of opaque stage operators whose backward pass is
again made of ``ss`` operators. That is how the reference treats its provider
operators (docs/integrations/mlops.md:1-21; packages/engine/src/shadowspill/pytorch/
capture/export.py:126): the graph frontend never looks inside them.

Backward operators that produce a parameter gradient (``ss::gemm`` in its
weight-gradient form, ``ss::rmsnorm_bwd``, ``ss::embedding_bwd``, ``ss::head_loss``) have
an ``*_into`` twin in :mod:`.graph_pairs` that writes into the stage's gradient buffer
in place; the gradient-destination pass swaps them in
(packages/engine/src/shadowspill/pytorch/capture/gradients/destinations.py).
"""
from __future__ import annotations

import torch
from torch.library import custom_op

from ..ops import functional as F

Tensor = torch.Tensor


def _c(t: Tensor) -> Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


_pool = None


def _autograd_elsewhere(fn, inputs: tuple[Tensor, ...], grad_out: Tensor) -> tuple[Tensor, ...]:
    """Gradients of ``fn(*inputs)`` by ``torch.autograd``, for operators whose backward pass has no
    kernel of its own on this device (the CPU forms of the sequence-mixer pieces). The body of a
    custom operator runs below the autograd dispatch keys, where nothing records a graph; that
    exclusion is thread-local, so the differentiation runs on a helper thread."""
    global _pool
    if _pool is None:
        from concurrent.futures import ThreadPoolExecutor
        _pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="ss-autograd")
    stream = torch.cuda.current_stream() if grad_out.is_cuda else None

    def work():
        # device and stream are thread-local too: carry the caller's over
        import contextlib
        ctx = contextlib.ExitStack()
        if stream is not None:
            ctx.enter_context(torch.cuda.device(grad_out.device))
            ctx.enter_context(torch.cuda.stream(stream))
        with ctx, torch.enable_grad():
            leaves = [t.detach().requires_grad_(True) for t in inputs]
            y = fn(*leaves)
            return tuple(g.contiguous() for g in torch.autograd.grad(y, leaves, grad_out.to(y.dtype)))
    return _pool.submit(work).result()


# ------------------------------------------------------------------------ GEMM / linear
@custom_op("ss::gemm", mutates_args=())
def gemm(a: Tensor, b: Tensor, a_mn: bool, b_mn: bool) -> Tensor:
    return F.gemm(_c(a), _c(b), a_mn=a_mn, b_mn=b_mn)


@gemm.register_fake
def _(a, b, a_mn, b_mn):
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    return a.new_empty((M, N))


@custom_op("ss::linear", mutates_args=())
def linear(x: Tensor, w: Tensor) -> Tensor:
    return F.linear_fwd(_c(x), w)


@linear.register_fake
def _(x, w):
    return x.new_empty((x.shape[0], w.shape[0]))


def _linear_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _linear_bwd(ctx, gy):
    x, w = ctx.saved_tensors
    dx = torch.ops.ss.gemm(gy, w, False, True) if ctx.needs_input_grad[0] else None
    dw = torch.ops.ss.gemm(gy, x, True, True) if ctx.needs_input_grad[1] else None
    return dx, dw


linear.register_autograd(_linear_bwd, setup_context=_linear_setup)


# ------------------------------------------------------------------------ RMSNorm
@custom_op("ss::rmsnorm", mutates_args=())
def rmsnorm(x: Tensor, w: Tensor, eps: float, zero_centered: bool) -> tuple[Tensor, Tensor]:
    y, rstd = F.rmsnorm_fwd(x.contiguous(), w, eps, zero_centered)
    return y, rstd


@rmsnorm.register_fake
def _(x, w, eps, zero_centered):
    return torch.empty_like(x, memory_format=torch.contiguous_format), x.new_empty((x.shape[0],),
                                                                                 dtype=torch.float32)


@custom_op("ss::rmsnorm_bwd", mutates_args=())
def rmsnorm_bwd(x: Tensor, w: Tensor, gy: Tensor, rstd: Tensor, zero_centered: bool) -> tuple[Tensor, Tensor]:
    dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
    dx = F.rmsnorm_bwd(x.contiguous(), w, gy.contiguous(), rstd, dw, zero_centered)
    return dx, dw


@rmsnorm_bwd.register_fake
def _(x, w, gy, rstd, zero_centered):
    return torch.empty_like(x, memory_format=torch.contiguous_format), w.new_empty(w.shape, dtype=torch.float32)


def _rmsnorm_setup(ctx, inputs, output):
    x, w, _, zc = inputs
    ctx.save_for_backward(x, w, output[1])
    ctx.zc = zc


def _rmsnorm_bwd(ctx, gy, _grstd):
    x, w, rstd = ctx.saved_tensors
    dx, dw = torch.ops.ss.rmsnorm_bwd(x, w, gy, rstd, ctx.zc)
    return dx, dw, None, None


rmsnorm.register_autograd(_rmsnorm_bwd, setup_context=_rmsnorm_setup)


# ------------------------------------------------------------------------ rotary
@custom_op("ss::rope", mutates_args=())
def rope(x: Tensor, positions: Tensor, heads: int, dh: int, rot: int, theta: float,
         inverse: bool) -> Tensor:
    out = x.contiguous().clone()
    F.rope_(out, positions, col0=0, heads=heads, dh=dh, rot=rot, theta=theta, inverse=inverse)
    return out


@rope.register_fake
def _(x, positions, heads, dh, rot, theta, inverse):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


def _rope_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[1])
    ctx.args = inputs[2:]


def _rope_bwd(ctx, g):
    heads, dh, rot, theta, inverse = ctx.args
    (positions,) = ctx.saved_tensors
    return torch.ops.ss.rope(g, positions, heads, dh, rot, theta, not inverse), None, None, None, None, None, None


rope.register_autograd(_rope_bwd, setup_context=_rope_setup)


# ------------------------------------------------------------------------ SwiGLU
@custom_op("ss::swiglu", mutates_args=())
def swiglu(gu: Tensor) -> Tensor:
    return F.swiglu_fwd(gu.contiguous())


@swiglu.register_fake
def _(gu):
    return gu.new_empty((gu.shape[0], gu.shape[1] // 2))


@custom_op("ss::swiglu_bwd", mutates_args=())
def swiglu_bwd(gu: Tensor, gh: Tensor) -> Tensor:
    return F.swiglu_bwd(gu.contiguous(), gh.contiguous())


@swiglu_bwd.register_fake
def _(gu, gh):
    return torch.empty_like(gu, memory_format=torch.contiguous_format)


def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])


def _swiglu_bwd(ctx, gh):
    return torch.ops.ss.swiglu_bwd(ctx.saved_tensors[0], gh)


swiglu.register_autograd(_swiglu_bwd, setup_context=_swiglu_setup)


# ------------------------------------------------------------------------ attention
@custom_op("ss::attention", mutates_args=())
def attention(q: Tensor, k: Tensor, v: Tensor, cu_seqlens: Tensor, max_seqlen: int) -> tuple[Tensor, Tensor]:
    out, lse = F.attention_varlen(q, k, v, cu_seqlens, max_seqlen)
    return out, lse


@attention.register_fake
def _(q, k, v, cu_seqlens, max_seqlen):
    return q.new_empty(q.shape), q.new_empty((q.shape[1], q.shape[0]), dtype=torch.float32)


@custom_op("ss::attention_bwd", mutates_args=())
def attention_bwd(q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, dout: Tensor,
                  cu_seqlens: Tensor, max_seqlen: int) -> tuple[Tensor, Tensor, Tensor]:
    dq, dk, dv = F.attention_varlen_bwd(q, k, v, out, lse, dout.contiguous(), cu_seqlens, max_seqlen)
    return dq, dk, dv


@attention_bwd.register_fake
def _(q, k, v, out, lse, dout, cu_seqlens, max_seqlen):
    return q.new_empty(q.shape), k.new_empty(k.shape), v.new_empty(v.shape)


def _attention_setup(ctx, inputs, output):
    q, k, v, cu, ms = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1], cu)
    ctx.max_seqlen = ms


def _attention_bwd(ctx, dout, _dlse):
    q, k, v, out, lse, cu = ctx.saved_tensors
    dq, dk, dv = torch.ops.ss.attention_bwd(q, k, v, out, lse, dout, cu, ctx.max_seqlen)
    return dq, dk, dv, None, None


attention.register_autograd(_attention_bwd, setup_context=_attention_setup)


# ------------------------------------------------------------------------ embedding
@custom_op("ss::embedding", mutates_args=())
def embedding(ids: Tensor, W: Tensor) -> Tensor:
    return F.embedding_fwd(ids, W)


@embedding.register_fake
def _(ids, W):
    return W.new_empty((ids.numel(), W.shape[1]))


@custom_op("ss::embedding_bwd", mutates_args=())
def embedding_bwd(ids: Tensor, g: Tensor, rows: int) -> Tensor:
    dW = torch.zeros((rows, g.shape[1]), dtype=g.dtype, device=g.device)
    F.embedding_bwd(ids, g.contiguous(), dW)
    return dW


@embedding_bwd.register_fake
def _(ids, g, rows):
    return g.new_empty((rows, g.shape[1]))


def _embedding_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])
    ctx.rows = inputs[1].shape[0]


def _embedding_bwd(ctx, g):
    return None, torch.ops.ss.embedding_bwd(ctx.saved_tensors[0], g, ctx.rows)


embedding.register_autograd(_embedding_bwd, setup_context=_embedding_setup)


# ------------------------------------------------------------------------ head + loss
def head_loss_run(h: Tensor, W: Tensor, targets: Tensor, weights: Tensor, block_rows: int,
                  dW: Tensor | None, accumulate: bool, train: bool = True):
    """Masked weighted cross entropy of ``h @ W^T`` in row blocks: the ``[T, V]`` logits never
    exist at once. Returns ``(loss fp32[1], dh)``; the head-weight gradient is written (or added)
    into ``dW`` block by block. Shared by the operator below and its in-place twin."""
    T = h.shape[0]
    loss = torch.zeros(1, dtype=torch.float32, device=h.device)
    dh = torch.empty_like(h) if train else None
    acc = accumulate
    for r0 in range(0, T, block_rows):
        r1 = min(T, r0 + block_rows)
        logits = F.linear_fwd(h[r0:r1], W)
        F.cross_entropy_(logits, targets[r0:r1], weights[r0:r1], loss, write_grad=train)
        if train:
            if dW is not None:
                F.linear_wgrad(logits, h[r0:r1], out=dW, accumulate=acc)
                acc = True
            F.linear_dgrad(logits, W, out=dh[r0:r1])
        del logits
    return loss, dh


@custom_op("ss::head_loss", mutates_args=())
def head_loss(h: Tensor, W: Tensor, targets: Tensor, weights: Tensor, block_rows: int) -> tuple[Tensor, Tensor, Tensor]:
    dW = torch.empty_like(W)
    loss, dh = head_loss_run(h.contiguous(), W, targets, weights, block_rows, dW, False)
    return loss, dh, dW


@head_loss.register_fake
def _(h, W, targets, weights, block_rows):
    return h.new_empty((1,), dtype=torch.float32), torch.empty_like(h), torch.empty_like(W)


@custom_op("ss::head_eval", mutates_args=())
def head_eval(h: Tensor, W: Tensor, targets: Tensor, weights: Tensor, block_rows: int) -> Tensor:
    return head_loss_run(h.contiguous(), W, targets, weights, block_rows, None, False, train=False)[0]


@head_eval.register_fake
def _(h, W, targets, weights, block_rows):
    return h.new_empty((1,), dtype=torch.float32)


def _head_setup(ctx, inputs, output):
    ctx.save_for_backward(output[1], output[2])


def _head_bwd(ctx, gl, _gdh, _gdw):
    dh, dW = ctx.saved_tensors
    # the loss is a weighted SUM: its upstream gradient is a scalar (1 in a training step)
    return dh * gl.to(dh.dtype), dW * gl.to(dW.dtype), None, None, None


head_loss.register_autograd(_head_bwd, setup_context=_head_setup)


# ------------------------------------------------------------------------ DeltaNet pieces
@custom_op("ss::conv_silu", mutates_args=())
def conv_silu(x: Tensor, w: Tensor, positions: Tensor, cu_seqlens: Tensor) -> Tensor:
    from ..ops import sequence as seq
    with torch.no_grad():
        bounds = None if x.is_cuda else cu_seqlens.tolist()
        return seq.causal_conv_silu(x, w, bounds, positions).contiguous()


@conv_silu.register_fake
def _(x, w, positions, cu_seqlens):
    return x.new_empty(x.shape)


@custom_op("ss::conv_silu_bwd", mutates_args=())
def conv_silu_bwd(x: Tensor, w: Tensor, positions: Tensor, cu_seqlens: Tensor, gy: Tensor) -> tuple[Tensor, Tensor]:
    from ..ops import sequence as seq
    bounds = None if x.is_cuda else cu_seqlens.tolist()
    return _autograd_elsewhere(lambda a, b: seq.causal_conv_silu(a, b, bounds, positions), (x, w), gy)


@conv_silu_bwd.register_fake
def _(x, w, positions, cu_seqlens, gy):
    return x.new_empty(x.shape), w.new_empty(w.shape)


def _conv_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _conv_bwd(ctx, gy):
    x, w, pos, cu = ctx.saved_tensors
    dx, dw = torch.ops.ss.conv_silu_bwd(x, w, pos, cu, gy)
    return dx, dw, None, None


conv_silu.register_autograd(_conv_bwd, setup_context=_conv_setup)


@custom_op("ss::l2norm", mutates_args=())
def l2norm(x: Tensor, eps: float) -> Tensor:
    from ..ops import sequence as seq
    with torch.no_grad():
        return seq.l2_normalize(x.contiguous(), eps)


@l2norm.register_fake
def _(x, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@custom_op("ss::l2norm_bwd", mutates_args=())
def l2norm_bwd(x: Tensor, gy: Tensor, eps: float) -> Tensor:
    from ..ops import sequence as seq
    return _autograd_elsewhere(lambda a: seq.l2_normalize(a, eps), (x.contiguous(),), gy.contiguous())[0]


@l2norm_bwd.register_fake
def _(x, gy, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


def _l2_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0])
    ctx.eps = inputs[1]


def _l2_bwd(ctx, gy):
    return torch.ops.ss.l2norm_bwd(ctx.saved_tensors[0], gy, ctx.eps), None


l2norm.register_autograd(_l2_bwd, setup_context=_l2_setup)


@custom_op("ss::gated_rmsnorm", mutates_args=())
def gated_rmsnorm(x: Tensor, gate: Tensor, w: Tensor, eps: float, zero_centered: bool) -> Tensor:
    from ..ops import sequence as seq
    with torch.no_grad():
        return seq.gated_rmsnorm(x.contiguous(), gate.contiguous(), w, eps, zero_centered)


@gated_rmsnorm.register_fake
def _(x, gate, w, eps, zero_centered):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@custom_op("ss::gated_rmsnorm_bwd", mutates_args=())
def gated_rmsnorm_bwd(x: Tensor, gate: Tensor, w: Tensor, gy: Tensor, eps: float,
                      zero_centered: bool) -> tuple[Tensor, Tensor, Tensor]:
    from ..ops import sequence as seq
    return _autograd_elsewhere(lambda a, b, c: seq.gated_rmsnorm(a, b, c, eps, zero_centered),
                               (x.contiguous(), gate.contiguous(), w), gy.contiguous())


@gated_rmsnorm_bwd.register_fake
def _(x, gate, w, gy, eps, zero_centered):
    return (torch.empty_like(x, memory_format=torch.contiguous_format),
            torch.empty_like(gate, memory_format=torch.contiguous_format), torch.empty_like(w))


def _grms_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:3])
    ctx.args = inputs[3:]


def _grms_bwd(ctx, gy):
    x, gate, w = ctx.saved_tensors
    dx, dg, dw = torch.ops.ss.gated_rmsnorm_bwd(x, gate, w, gy, *ctx.args)
    return dx, dg, dw, None, None


gated_rmsnorm.register_autograd(_grms_bwd, setup_context=_grms_setup)


@custom_op("ss::gated_delta_rule", mutates_args=())
def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, g: Tensor, cu_seqlens: Tensor,
                     chunk: int) -> Tensor:
    from ..ops import sequence as seq
    with torch.no_grad():
        bounds = None if q.is_cuda else cu_seqlens.tolist()
        return seq.gated_delta_rule_chunked(q, k, v, beta, g, bounds, chunk, cu_seqlens).contiguous()


@gated_delta_rule.register_fake
def _(q, k, v, beta, g, cu_seqlens, chunk):
    return v.new_empty(v.shape)


@custom_op("ss::gated_delta_rule_bwd", mutates_args=())
def gated_delta_rule_bwd(q: Tensor, k: Tensor, v: Tensor, beta: Tensor, g: Tensor, cu_seqlens: Tensor,
                         chunk: int, dout: Tensor) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    from ..ops import delta_rule, sequence as seq
    if delta_rule.supported(q, k, v, chunk):
        dq, dk, dv, db, dg = delta_rule.backward(q, k, v, beta, g, cu_seqlens, dout)
        return dq, dk, dv, db.to(beta.dtype), dg.to(g.dtype)
    bounds = None if q.is_cuda else cu_seqlens.tolist()
    return _autograd_elsewhere(lambda *a: seq._gated_delta_rule_torch(*a, bounds, chunk, cu_seqlens),
                               (q, k, v, beta, g), dout)


@gated_delta_rule_bwd.register_fake
def _(q, k, v, beta, g, cu_seqlens, chunk, dout):
    return tuple(t.new_empty(t.shape) for t in (q, k, v, beta, g))


def _gdr_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:6])
    ctx.chunk = inputs[6]


def _gdr_bwd(ctx, dout):
    q, k, v, beta, g, cu = ctx.saved_tensors
    return (*torch.ops.ss.gated_delta_rule_bwd(q, k, v, beta, g, cu, ctx.chunk, dout), None, None)


gated_delta_rule.register_autograd(_gdr_bwd, setup_context=_gdr_setup)

# Operators whose outputs are cheap to recompute from their inputs relative to reading them back:
# the retention policy never keeps these unless a rule names them.
# ------------------------------------------------------------------------ routed experts
def _moe_torch(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, k: int, renorm: bool) -> Tensor:
    """Top-k routed SwiGLU experts as plain tensor operations (the CPU form, and the definition)."""
    if renorm:
        vals, ids = torch.topk(logits, k, dim=-1)
        wts = torch.softmax(vals, dim=-1)
    else:
        wts, ids = torch.topk(torch.softmax(logits, dim=-1), k, dim=-1)
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=w13.shape[0]).tolist()
    tok = order // k
    w_sorted = wts.reshape(-1)[order].to(h.dtype)
    out = torch.zeros_like(h)
    pos = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        rows = tok[pos:pos + n]
        x = h.index_select(0, rows)
        gu = x @ w13[e].t()
        f = gu.shape[1] // 2
        act = (torch.nn.functional.silu(gu[:, :f].float()).to(h.dtype) * gu[:, f:])
        out = out.index_add(0, rows, (act @ w2[e].t()) * w_sorted[pos:pos + n, None])
        pos += n
    return out


@custom_op("ss::moe_experts", mutates_args=())
def moe_experts(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, k: int, renorm: bool) -> Tensor:
    if h.is_cuda and F._cuda(h):
        from ..ops import moe as moe_ops
        with torch.no_grad():
            return moe_ops.experts(_c(h), _c(logits), w13, w2, k, renorm, None)
    with torch.no_grad():
        return _moe_torch(h, logits, w13, w2, k, renorm)


@moe_experts.register_fake
def _(h, logits, w13, w2, k, renorm):
    return torch.empty_like(h, memory_format=torch.contiguous_format)


def moe_bwd_run(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, gy: Tensor, k: int, renorm: bool,
                dst13: Tensor | None, dst2: Tensor | None, first: bool):
    """Gradients of the routed experts. The bank gradients are created in (``first``) or added to
    ``dst13`` / ``dst2`` when given, else returned as new tensors."""
    own = dst13 is None
    if own:
        dst13, dst2 = torch.zeros_like(w13), torch.zeros_like(w2)
    elif first:
        dst13.zero_(); dst2.zero_()                      # experts without rows still get a defined gradient
    if h.is_cuda and F._cuda(h):
        from ..models.autograd_ops import GradSink
        from ..ops import moe as moe_ops
        sink = GradSink({"w13": dst13, "w2": dst2}, False)
        dh, dlogits = _autograd_elsewhere(lambda a, b: moe_ops.experts(a, b, w13, w2, k, renorm, sink),
                                          (_c(h), _c(logits)), _c(gy))
    else:
        dh, dlogits, d13, d2 = _autograd_elsewhere(lambda a, b, c, d: _moe_torch(a, b, c, d, k, renorm),
                                                   (h, logits, w13, w2), gy)
        dst13.add_(d13.to(dst13.dtype)); dst2.add_(d2.to(dst2.dtype))
    return (dh, dlogits, dst13, dst2) if own else (dh, dlogits)


@custom_op("ss::moe_experts_bwd", mutates_args=())
def moe_experts_bwd(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, gy: Tensor, k: int,
                    renorm: bool) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    return moe_bwd_run(h, logits, w13, w2, gy, k, renorm, None, None, True)


@moe_experts_bwd.register_fake
def _(h, logits, w13, w2, gy, k, renorm):
    return (torch.empty_like(h, memory_format=torch.contiguous_format),
            torch.empty_like(logits, memory_format=torch.contiguous_format),
            torch.empty_like(w13), torch.empty_like(w2))


@custom_op("ss::moe_experts_bwd_frozen", mutates_args=())
def moe_experts_bwd_frozen(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, gy: Tensor, k: int,
                           renorm: bool) -> tuple[Tensor, Tensor]:
    """Backward of the routed experts when the banks are frozen: the gradients of the rows and of
    the router logits only; no bank-sized gradient is computed or allocated."""
    if h.is_cuda and F._cuda(h):
        from ..models.autograd_ops import GradSink
        from ..ops import moe as moe_ops
        sink = GradSink(None, False)         # no buffers: the bank gradients are skipped
        return _autograd_elsewhere(lambda a, b: moe_ops.experts(a, b, w13, w2, k, renorm, sink),
                                   (_c(h), _c(logits)), _c(gy))
    return _autograd_elsewhere(lambda a, b: _moe_torch(a, b, w13, w2, k, renorm), (h, logits), gy)


@moe_experts_bwd_frozen.register_fake
def _(h, logits, w13, w2, gy, k, renorm):
    return (torch.empty_like(h, memory_format=torch.contiguous_format),
            torch.empty_like(logits, memory_format=torch.contiguous_format))


def _moe_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:4])
    ctx.k, ctx.renorm = inputs[4], inputs[5]


def _moe_bwd(ctx, gy):
    h, logits, w13, w2 = ctx.saved_tensors
    if not (ctx.needs_input_grad[2] or ctx.needs_input_grad[3]):
        dh, dl = torch.ops.ss.moe_experts_bwd_frozen(h, logits, w13, w2, gy, ctx.k, ctx.renorm)
        return dh, dl, None, None, None, None
    dh, dl, d13, d2 = torch.ops.ss.moe_experts_bwd(h, logits, w13, w2, gy, ctx.k, ctx.renorm)
    return dh, dl, d13, d2, None, None


moe_experts.register_autograd(_moe_bwd, setup_context=_moe_setup)


# ------------------------------------------------------------------------ routed experts with adapters
def _moe_lora_torch(h, logits, w13, w2, a13, b13, a2, b2, k: int, renorm: bool, scale: float) -> Tensor:
    """``_moe_torch`` with per-expert low-rank factors on both banks (the definition; CPU form)."""
    if renorm:
        vals, ids = torch.topk(logits, k, dim=-1)
        wts = torch.softmax(vals, dim=-1)
    else:
        wts, ids = torch.topk(torch.softmax(logits, dim=-1), k, dim=-1)
    flat = ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=w13.shape[0]).tolist()
    tok = order // k
    w_sorted = wts.reshape(-1)[order].to(h.dtype)
    out = torch.zeros_like(h)
    pos = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        rows = tok[pos:pos + n]
        x = h.index_select(0, rows)
        gu = x @ w13[e].t() + ((x @ a13[e].t()) @ b13[e].t()) * scale
        f = gu.shape[1] // 2
        act = (torch.nn.functional.silu(gu[:, :f].float()).to(h.dtype) * gu[:, f:])
        y = act @ w2[e].t() + ((act @ a2[e].t()) @ b2[e].t()) * scale
        out = out.index_add(0, rows, y * w_sorted[pos:pos + n, None])
        pos += n
    return out


def _moe_lora_cuda(h, logits, w13, w2, a13, b13, a2, b2, k: int, renorm: bool, scale: float, sink):
    """The same on the grouped tcgen05 GEMMs: gather into expert order, grouped linear per bank
    plus the two thin grouped products of its factors, combine. ``sink`` receives the factor
    gradients (names ``a13`` / ``b13`` / ``a2`` / ``b2``) when this runs under autograd."""
    from ..models import autograd_ops as A
    from ..ops import moe as moe_ops
    ids, _, counts = moe_ops.route(logits.detach(), k, renorm)
    wts = moe_ops._weights_from_logits(logits, ids.long(), renorm)
    lay = moe_ops.Layout(ids, counts)
    xs = A.expert_gather(h, lay)

    def bank(x, w, a, b, an, bn):
        low = A.grouped_linear(A.grouped_linear(x, a, lay, sink, an), b, lay, sink, bn)
        return A.grouped_linear(x, w, lay, None, "") + low * scale
    ys = bank(A.swiglu(bank(xs, w13, a13, b13, "a13", "b13")), w2, a2, b2, "a2", "b2")
    return A.expert_combine(ys, wts.float().contiguous(), lay)


@custom_op("ss::moe_experts_lora", mutates_args=())
def moe_experts_lora(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, a13: Tensor, b13: Tensor,
                     a2: Tensor, b2: Tensor, k: int, renorm: bool, scale: float) -> Tensor:
    with torch.no_grad():
        if h.is_cuda and F._cuda(h):
            return _moe_lora_cuda(_c(h), _c(logits), w13, w2, a13, b13, a2, b2, k, renorm, scale, None)
        return _moe_lora_torch(h, logits, w13, w2, a13, b13, a2, b2, k, renorm, scale)


@moe_experts_lora.register_fake
def _(h, logits, w13, w2, a13, b13, a2, b2, k, renorm, scale):
    return torch.empty_like(h, memory_format=torch.contiguous_format)


@custom_op("ss::moe_experts_lora_bwd", mutates_args=())
def moe_experts_lora_bwd(h: Tensor, logits: Tensor, w13: Tensor, w2: Tensor, a13: Tensor, b13: Tensor,
                         a2: Tensor, b2: Tensor, gy: Tensor, k: int, renorm: bool, scale: float
                         ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Gradients of rows, router logits and the four factor banks; the frozen banks get none."""
    if h.is_cuda and F._cuda(h):
        from ..models.autograd_ops import GradSink
        G = {"a13": torch.zeros_like(a13), "b13": torch.zeros_like(b13),
             "a2": torch.zeros_like(a2), "b2": torch.zeros_like(b2)}     # experts without rows: zero
        sink = GradSink(G, False)
        dh, dl = _autograd_elsewhere(
            lambda x, l: _moe_lora_cuda(x, l, w13, w2, a13, b13, a2, b2, k, renorm, scale, sink),
            (_c(h), _c(logits)), _c(gy))
        return dh, dl, G["a13"], G["b13"], G["a2"], G["b2"]
    return _autograd_elsewhere(
        lambda x, l, p, q, r, s: _moe_lora_torch(x, l, w13, w2, p, q, r, s, k, renorm, scale),
        (h, logits, a13, b13, a2, b2), gy)


@moe_experts_lora_bwd.register_fake
def _(h, logits, w13, w2, a13, b13, a2, b2, gy, k, renorm, scale):
    return (torch.empty_like(h, memory_format=torch.contiguous_format),
            torch.empty_like(logits, memory_format=torch.contiguous_format),
            torch.empty_like(a13), torch.empty_like(b13), torch.empty_like(a2), torch.empty_like(b2))


def _moe_lora_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:8])
    ctx.k, ctx.renorm, ctx.scale = inputs[8], inputs[9], inputs[10]


def _moe_lora_bwd(ctx, gy):
    if ctx.needs_input_grad[2] or ctx.needs_input_grad[3]:
        raise NotImplementedError("ss::moe_experts_lora trains the factors of frozen banks only")
    grads = torch.ops.ss.moe_experts_lora_bwd(*ctx.saved_tensors, gy, ctx.k, ctx.renorm, ctx.scale)
    return grads[0], grads[1], None, None, grads[2], grads[3], grads[4], grads[5], None, None, None


moe_experts_lora.register_autograd(_moe_lora_bwd, setup_context=_moe_lora_setup)


# ------------------------------------------------------------------------ sparse latent attention (GLM)
def _sequence_start(cu_seqlens: Tensor, T: int) -> Tensor:
    """For every token row, the first row of its sequence (``cu_seqlens`` may be padded with T)."""
    rows = torch.arange(T, device=cu_seqlens.device)
    seq = torch.searchsorted(cu_seqlens.to(torch.int64), rows, right=True) - 1
    return cu_seqlens.to(torch.int64)[seq.clamp_min(0)]


@custom_op("ss::index_topk", mutates_args=())
def index_topk(q: Tensor, key: Tensor, head_weights: Tensor, cu_seqlens: Tensor, top_k: int) -> Tensor:
    """The sparse-attention indexer's selection: for query row ``t`` the ``top_k`` rows ``s <= t``
    of its own sequence with the largest score ``sum_h w[t, h] * relu(q[t, h] . key[s])`` (bf16
    operands, fp32 accumulation), as global row numbers in decreasing score order; ``-1`` where a
    query has fewer than ``top_k`` predecessors. Integer output: nothing is differentiated.
    Reference: the indexer of packages/workloads/src/shadowspill_workloads/models/glm53/
    implementations/mlops/attention.py:49-89 (``pooled_topk`` with pool size one).
    Evaluated in blocks of query rows so that the score matrix stays small."""
    T, K = q.shape[0], int(top_k)
    start = _sequence_start(cu_seqlens, T)
    out = torch.full((T, K), -1, dtype=torch.int32, device=q.device)
    cols = torch.arange(T, device=q.device)
    block = 1024
    kf = key.float()
    for lo in range(0, T, block):
        hi = min(T, lo + block)
        dots = torch.einsum("thd,sd->ths", q[lo:hi].float(), kf[:hi])
        score = (torch.relu(dots) * head_weights[lo:hi].float()[:, :, None]).sum(1)          # [b, hi]
        rows = torch.arange(lo, hi, device=q.device)[:, None]
        ok = (cols[None, :hi] <= rows) & (cols[None, :hi] >= start[lo:hi, None])
        score = score.masked_fill(~ok, float("-inf"))
        k = min(K, hi)
        vals, idx = torch.topk(score, k, dim=1)
        out[lo:hi, :k] = torch.where(torch.isfinite(vals), idx, torch.full_like(idx, -1)).to(torch.int32)
    return out


@index_topk.register_fake
def _(q, key, head_weights, cu_seqlens, top_k):
    return torch.empty((q.shape[0], int(top_k)), dtype=torch.int32, device=q.device)


def _sparse_latent_torch(q_latent: Tensor, latent: Tensor, indices: Tensor, q_rope: Tensor, k_rope: Tensor,
                         scale: float) -> Tensor:
    """Definition, in blocks of query rows: logits over the picked rows from the latent part and the
    rotary part, softmax over the picks, output = the picked latents weighted (the latent is key and
    value at once; the per-head value projection is applied by the caller)."""
    T = q_latent.shape[0]
    outs = []
    block = 512
    safe = indices.clamp_min(0).long()
    for lo in range(0, T, block):
        hi = min(T, lo + block)
        idx = safe[lo:hi]                                        # [b, K]
        keys, rope = latent[idx], k_rope[idx]                    # [b, K, L], [b, K, R]
        logits = (torch.einsum("bhl,bkl->bhk", q_latent[lo:hi].float(), keys.float())
                  + torch.einsum("bhr,bkr->bhk", q_rope[lo:hi].float(), rope.float())) * scale
        logits = logits.masked_fill((indices[lo:hi] < 0)[:, None, :], float("-inf"))
        p = torch.softmax(logits, dim=-1)
        outs.append(torch.einsum("bhk,bkl->bhl", p, keys.float()).to(q_latent.dtype))
    return torch.cat(outs, 0)


@custom_op("ss::sparse_latent_attention", mutates_args=())
def sparse_latent_attention(q_latent: Tensor, latent: Tensor, indices: Tensor, q_rope: Tensor, k_rope: Tensor,
                            scale: float) -> Tensor:
    """Attention of every query over the rows its indexer picked, in the compressed latent space
    (tensor-operation form on every device; no hand-written kernel yet). Reference:
    ``mlops.sparse_latent_attention`` as called in .../glm53/implementations/mlops/attention.py:150."""
    with torch.no_grad():
        return _sparse_latent_torch(q_latent, latent, indices, q_rope, k_rope, scale)


@sparse_latent_attention.register_fake
def _(q_latent, latent, indices, q_rope, k_rope, scale):
    return torch.empty_like(q_latent, memory_format=torch.contiguous_format)


@custom_op("ss::sparse_latent_attention_bwd", mutates_args=())
def sparse_latent_attention_bwd(q_latent: Tensor, latent: Tensor, indices: Tensor, q_rope: Tensor, k_rope: Tensor,
                                gy: Tensor, scale: float) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    return _autograd_elsewhere(lambda a, b, c, d: _sparse_latent_torch(a, b, indices, c, d, scale),
                               (q_latent, latent, q_rope, k_rope), gy)


@sparse_latent_attention_bwd.register_fake
def _(q_latent, latent, indices, q_rope, k_rope, gy, scale):
    c = torch.contiguous_format
    return (torch.empty_like(q_latent, memory_format=c), torch.empty_like(latent, memory_format=c),
            torch.empty_like(q_rope, memory_format=c), torch.empty_like(k_rope, memory_format=c))


def _sla_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:5])
    ctx.scale = inputs[5]


def _sla_bwd(ctx, gy):
    q_latent, latent, indices, q_rope, k_rope = ctx.saved_tensors
    dq, dl, dqr, dkr = torch.ops.ss.sparse_latent_attention_bwd(q_latent, latent, indices, q_rope, k_rope, gy, ctx.scale)
    return dq, dl, None, dqr, dkr, None


sparse_latent_attention.register_autograd(_sla_bwd, setup_context=_sla_setup)


# ------------------------------------------------------------------------ routed experts, routing given
def _moe_routed_torch(h: Tensor, ids: Tensor, wts: Tensor, w13: Tensor, w2: Tensor) -> Tensor:
    """Top-k SwiGLU experts with the routing decided outside (``ids`` [T, k], ``wts`` [T, k]): the
    form for routers that are not a softmax (sigmoid scores with a selection-only bias)."""
    k = ids.shape[1]
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=w13.shape[0]).tolist()
    tok = order // k
    w_sorted = wts.reshape(-1)[order].to(h.dtype)
    out = torch.zeros_like(h)
    pos = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        rows = tok[pos:pos + n]
        x = h.index_select(0, rows)
        gu = x @ w13[e].t()
        f = gu.shape[1] // 2
        act = (torch.nn.functional.silu(gu[:, :f].float()).to(h.dtype) * gu[:, f:])
        out = out.index_add(0, rows, (act @ w2[e].t()) * w_sorted[pos:pos + n, None])
        pos += n
    return out


def _moe_routed_cuda(h, ids, wts, w13, w2, sink):
    from ..models import autograd_ops as A
    from ..ops import moe as moe_ops
    counts = torch.bincount(ids.reshape(-1).long(), minlength=w13.shape[0]).to(torch.int32)
    lay = moe_ops.Layout(ids.to(torch.int32).contiguous(), counts)
    xs = A.expert_gather(h, lay)
    ys = A.grouped_linear(A.swiglu(A.grouped_linear(xs, w13, lay, sink, "w13")), w2, lay, sink, "w2")
    return A.expert_combine(ys, wts.float().contiguous(), lay)


@custom_op("ss::moe_experts_routed", mutates_args=())
def moe_experts_routed(h: Tensor, ids: Tensor, wts: Tensor, w13: Tensor, w2: Tensor) -> Tensor:
    with torch.no_grad():
        if h.is_cuda and F._cuda(h):
            return _moe_routed_cuda(_c(h), ids, wts, w13, w2, None)
        return _moe_routed_torch(h, ids, wts, w13, w2)


@moe_experts_routed.register_fake
def _(h, ids, wts, w13, w2):
    return torch.empty_like(h, memory_format=torch.contiguous_format)


@custom_op("ss::moe_experts_routed_bwd", mutates_args=())
def moe_experts_routed_bwd(h: Tensor, ids: Tensor, wts: Tensor, w13: Tensor, w2: Tensor, gy: Tensor,
                           banks: bool) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    """Gradients of rows, routing weights and (``banks``) both expert banks; without ``banks`` the
    last two results are empty and no bank-sized tensor is touched."""
    if h.is_cuda and F._cuda(h):
        from ..models.autograd_ops import GradSink
        G = {"w13": torch.zeros_like(w13), "w2": torch.zeros_like(w2)} if banks else {}
        sink = GradSink(G, False)
        dh, dw = _autograd_elsewhere(lambda a, b: _moe_routed_cuda(a, ids, b, w13, w2, sink), (_c(h), _c(wts)), _c(gy))
        return dh, dw, G.get("w13", h.new_empty(0)), G.get("w2", h.new_empty(0))
    if banks:
        return _autograd_elsewhere(lambda a, b, c, d: _moe_routed_torch(a, ids, b, c, d), (h, wts, w13, w2), gy)
    dh, dw = _autograd_elsewhere(lambda a, b: _moe_routed_torch(a, ids, b, w13, w2), (h, wts), gy)
    return dh, dw, h.new_empty(0), h.new_empty(0)


@moe_experts_routed_bwd.register_fake
def _(h, ids, wts, w13, w2, gy, banks):
    c = torch.contiguous_format
    return (torch.empty_like(h, memory_format=c), torch.empty_like(wts, memory_format=c),
            torch.empty_like(w13) if banks else h.new_empty(0), torch.empty_like(w2) if banks else h.new_empty(0))


def _moe_routed_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:5])


def _moe_routed_bwd(ctx, gy):
    h, ids, wts, w13, w2 = ctx.saved_tensors
    banks = bool(ctx.needs_input_grad[3] or ctx.needs_input_grad[4])
    dh, dw, d13, d2 = torch.ops.ss.moe_experts_routed_bwd(h, ids, wts, w13, w2, gy, banks)
    return dh, None, dw, (d13 if banks else None), (d2 if banks else None)


moe_experts_routed.register_autograd(_moe_routed_bwd, setup_context=_moe_routed_setup)


# ------------------------------------------------------------------------ routed experts, routing given, adapters
def _moe_routed_lora_torch(h, ids, wts, w13, w2, a13, b13, a2, b2, scale: float) -> Tensor:
    """``_moe_routed_torch`` with per-expert low-rank factors on both (frozen) banks."""
    k = ids.shape[1]
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=w13.shape[0]).tolist()
    tok = order // k
    w_sorted = wts.reshape(-1)[order].to(h.dtype)
    out = torch.zeros_like(h)
    pos = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        rows = tok[pos:pos + n]
        x = h.index_select(0, rows)
        gu = x @ w13[e].t() + ((x @ a13[e].t()) @ b13[e].t()) * scale
        f = gu.shape[1] // 2
        act = (torch.nn.functional.silu(gu[:, :f].float()).to(h.dtype) * gu[:, f:])
        y = act @ w2[e].t() + ((act @ a2[e].t()) @ b2[e].t()) * scale
        out = out.index_add(0, rows, y * w_sorted[pos:pos + n, None])
        pos += n
    return out


def _moe_routed_lora_cuda(h, ids, wts, w13, w2, a13, b13, a2, b2, scale: float, sink):
    from ..models import autograd_ops as A
    from ..ops import moe as moe_ops
    counts = torch.bincount(ids.reshape(-1).long(), minlength=w13.shape[0]).to(torch.int32)
    lay = moe_ops.Layout(ids.to(torch.int32).contiguous(), counts)
    xs = A.expert_gather(h, lay)

    def bank(x, w, a, b, an, bn):
        low = A.grouped_linear(A.grouped_linear(x, a, lay, sink, an), b, lay, sink, bn)
        return A.grouped_linear(x, w, lay, None, "") + low * scale
    ys = bank(A.swiglu(bank(xs, w13, a13, b13, "a13", "b13")), w2, a2, b2, "a2", "b2")
    return A.expert_combine(ys, wts.float().contiguous(), lay)


@custom_op("ss::moe_experts_routed_lora", mutates_args=())
def moe_experts_routed_lora(h: Tensor, ids: Tensor, wts: Tensor, w13: Tensor, w2: Tensor, a13: Tensor,
                            b13: Tensor, a2: Tensor, b2: Tensor, scale: float) -> Tensor:
    with torch.no_grad():
        if h.is_cuda and F._cuda(h):
            return _moe_routed_lora_cuda(_c(h), ids, wts, w13, w2, a13, b13, a2, b2, scale, None)
        return _moe_routed_lora_torch(h, ids, wts, w13, w2, a13, b13, a2, b2, scale)


@moe_experts_routed_lora.register_fake
def _(h, ids, wts, w13, w2, a13, b13, a2, b2, scale):
    return torch.empty_like(h, memory_format=torch.contiguous_format)


@custom_op("ss::moe_experts_routed_lora_bwd", mutates_args=())
def moe_experts_routed_lora_bwd(h: Tensor, ids: Tensor, wts: Tensor, w13: Tensor, w2: Tensor, a13: Tensor,
                                b13: Tensor, a2: Tensor, b2: Tensor, gy: Tensor, scale: float
                                ) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """Gradients of rows, routing weights and the four factor banks; the frozen banks get none."""
    if h.is_cuda and F._cuda(h):
        from ..models.autograd_ops import GradSink
        G = {"a13": torch.zeros_like(a13), "b13": torch.zeros_like(b13),
             "a2": torch.zeros_like(a2), "b2": torch.zeros_like(b2)}
        sink = GradSink(G, False)
        dh, dw = _autograd_elsewhere(
            lambda x, w: _moe_routed_lora_cuda(x, ids, w, w13, w2, a13, b13, a2, b2, scale, sink),
            (_c(h), _c(wts)), _c(gy))
        return dh, dw, G["a13"], G["b13"], G["a2"], G["b2"]
    return _autograd_elsewhere(
        lambda x, w, p, q, r, s: _moe_routed_lora_torch(x, ids, w, w13, w2, p, q, r, s, scale),
        (h, wts, a13, b13, a2, b2), gy)


@moe_experts_routed_lora_bwd.register_fake
def _(h, ids, wts, w13, w2, a13, b13, a2, b2, gy, scale):
    c = torch.contiguous_format
    return (torch.empty_like(h, memory_format=c), torch.empty_like(wts, memory_format=c),
            torch.empty_like(a13), torch.empty_like(b13), torch.empty_like(a2), torch.empty_like(b2))


def _moe_routed_lora_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs[:9])
    ctx.scale = inputs[9]


def _moe_routed_lora_bwd(ctx, gy):
    if ctx.needs_input_grad[3] or ctx.needs_input_grad[4]:
        raise NotImplementedError("ss::moe_experts_routed_lora trains the factors of frozen banks only")
    g = torch.ops.ss.moe_experts_routed_lora_bwd(*ctx.saved_tensors, gy, ctx.scale)
    return g[0], None, g[1], None, None, g[2], g[3], g[4], g[5], None


moe_experts_routed_lora.register_autograd(_moe_routed_lora_bwd, setup_context=_moe_routed_lora_setup)


MEMORY_BOUND = ("ss.rmsnorm", "ss.rope", "ss.swiglu", "ss.l2norm", "ss.conv_silu", "ss.gated_rmsnorm",
                "ss.embedding")
# Operators dominated by tensor-core work: keeping their outputs saves real time.
COMPUTE_BOUND = ("ss.linear", "ss.gemm", "ss.attention", "ss.gated_delta_rule", "ss.head_loss", "ss.moe_experts",
                 "ss.moe_experts_lora", "ss.sparse_latent_attention", "ss.moe_experts_routed", "ss.index_topk",
                 "ss.moe_experts_routed_lora")
