"""Sequence-mixer ops of the hybrid (Gated DeltaNet) layers.

The memory-bound pieces (causal convolution + SiLU, L2 normalisation, gated RMSNorm)
run as hand-written sm_100a kernels with explicit backward kernels on bf16 CUDA
tensors (``ops/csrc/deltanet.cu``) and as the plain PyTorch definitions below
otherwise; the chunked delta rule itself is differentiable PyTorch.

``gated_delta_rule_chunked`` evaluates the gated delta rule in chunks of 64 tokens
(the WY / UT-transform form): inside a chunk everything is dense matrix algebra,
and only the ``[dk, dv]`` state is carried from chunk to chunk. With
``a_t = exp(g_t)`` and ``G_t`` the running product of ``a`` inside the chunk,

    A[t,i] = beta_t (G_t/G_i) (k_t . k_i)  for i < t          (strictly lower)
    T      = (I + A)^-1
    U      = T (beta V) - T (beta G K) S_in                    (the "new values")
    O      = (G Q) S_in + tril((G_t/G_i) Q K^T) U
    S_out  = G_C S_in + ((G_C/G) K)^T U

which equals the token recurrence in :func:`..reference.gated_delta_rule`
(the reference's definition: packages/workloads/src/shadowspill_workloads/models/
qwen35/implementations/pytorch/delta_rule/reference.py:8-41). Sequences of a packed
batch are independent: the state starts at zero at every boundary.
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF

from . import _lib

_c = _lib
_lib.register("ss_conv_silu_fwd", [_c.c_p, _c.c_ll, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int, _c.c_p,
                                   _c.c_ll, _c.c_p])
_lib.register("ss_conv_silu_bwd", [_c.c_p, _c.c_ll, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int, _c.c_p,
                                   _c.c_ll, _c.c_p, _c.c_p, _c.c_ll, _c.c_p, _c.c_p])
_lib.register("ss_l2norm_fwd", [_c.c_p, _c.c_p, _c.c_ll, _c.c_int, _c.c_f, _c.c_p])
_lib.register("ss_l2norm_bwd", [_c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_int, _c.c_f, _c.c_p])
_lib.register("ss_gated_rmsnorm_fwd", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_ll, _c.c_int, _c.c_f, _c.c_int,
                                       _c.c_p])
_lib.register("ss_gated_rmsnorm_bwd", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_ll,
                                       _c.c_int, _c.c_f, _c.c_int, _c.c_p])


class tf32_matmul:
    """Context: fp32 matrix products on the tensor cores in TF32 (10-bit mantissa, fp32
    accumulate). The chunked delta rule's batched products, and their autograd backward,
    run under it; its operands come from bf16 activations, so nothing finer is lost."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


def _native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        x = x.contiguous()
        y = torch.empty_like(x)
        W = x.shape[-1]
        _lib.check(_lib.lib().ss_l2norm_fwd(x.data_ptr(), y.data_ptr(), x.numel() // W, W, eps,
                                            _lib.stream_ptr()), "ss_l2norm_fwd")
        ctx.save_for_backward(x)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        W = x.shape[-1]
        _lib.check(_lib.lib().ss_l2norm_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel() // W, W,
                                            ctx.eps, _lib.stream_ptr()), "ss_l2norm_bwd")
        return dx, None


class _ConvSiLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, positions):
        T, C = x.shape
        w = w.contiguous()
        y = torch.empty((T, C), dtype=x.dtype, device=x.device)
        _lib.check(_lib.lib().ss_conv_silu_fwd(x.data_ptr(), x.stride(0), w.data_ptr(),
                                               positions.data_ptr(), T, C, w.shape[1], y.data_ptr(),
                                               y.stride(0), _lib.stream_ptr()), "ss_conv_silu_fwd")
        ctx.save_for_backward(x, w, positions)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, positions = ctx.saved_tensors
        T, C = x.shape
        dy = dy.contiguous()
        dpre = torch.empty((T, C), dtype=torch.float32, device=x.device)
        dx = torch.empty((T, C), dtype=x.dtype, device=x.device)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        _lib.check(_lib.lib().ss_conv_silu_bwd(x.data_ptr(), x.stride(0), w.data_ptr(),
                                               positions.data_ptr(), T, C, w.shape[1], dy.data_ptr(),
                                               dy.stride(0), dpre.data_ptr(), dx.data_ptr(), dx.stride(0),
                                               dw.data_ptr(), _lib.stream_ptr()), "ss_conv_silu_bwd")
        return dx, dw.to(w.dtype), None


class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, w, eps, zero_centered):
        x, gate, w = x.contiguous(), gate.contiguous(), w.contiguous()
        y = torch.empty_like(x)
        W = x.shape[-1]
        _lib.check(_lib.lib().ss_gated_rmsnorm_fwd(x.data_ptr(), gate.data_ptr(), w.data_ptr(),
                                                   y.data_ptr(), x.numel() // W, W, eps,
                                                   int(zero_centered), _lib.stream_ptr()),
                   "ss_gated_rmsnorm_fwd")
        ctx.save_for_backward(x, gate, w)
        ctx.args = (eps, zero_centered)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gate, w = ctx.saved_tensors
        eps, zc = ctx.args
        dy = dy.contiguous()
        dx, dgate = torch.empty_like(x), torch.empty_like(gate)
        dw = torch.zeros(w.shape, dtype=torch.float32, device=x.device)
        W = x.shape[-1]
        _lib.check(_lib.lib().ss_gated_rmsnorm_bwd(x.data_ptr(), gate.data_ptr(), w.data_ptr(),
                                                   dy.data_ptr(), dx.data_ptr(), dgate.data_ptr(),
                                                   dw.data_ptr(), x.numel() // W, W, eps, int(zc),
                                                   _lib.stream_ptr()), "ss_gated_rmsnorm_bwd")
        return dx, dgate, dw.to(w.dtype), None, None


def l2_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if _native(x) and x.shape[-1] % 2 == 0:
        return _L2Norm.apply(x, eps)
    xf = x.float()
    return (xf * torch.rsqrt(xf.square().sum(-1, keepdim=True) + eps)).to(x.dtype)


def causal_conv_silu(x: torch.Tensor, w: torch.Tensor, bounds: list[int],
                     positions: torch.Tensor | None = None) -> torch.Tensor:
    """Depthwise causal conv1d (kernel ``w.shape[1]``) + SiLU; ``x`` [T,C], ``w`` [C,K].
    The window never crosses a sequence boundary (``bounds`` = cu_seqlens as a list;
    ``positions`` = index of each token in its sequence, which the CUDA kernel uses)."""
    T, C = x.shape
    if (_native(x) and positions is not None and C % 8 == 0 and x.stride(0) % 8 == 0
            and x.stride(1) == 1 and w.shape[1] <= 8 and w.dtype == x.dtype):
        return _ConvSiLU.apply(x, w, positions)
    K = w.shape[1]
    xf = x.float()
    # shifted copies: y[t] = sum_j w[:, K-1-j] * x[t-j], with x[t-j] zero before the sequence start
    pos = torch.zeros(T, dtype=torch.long, device=x.device)
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e > s:
            pos[s:e] = torch.arange(e - s, device=x.device)
    y = torch.zeros_like(xf)
    wf = w.float()
    for j in range(K):
        shifted = torch.roll(xf, shifts=j, dims=0) if j else xf
        valid = (pos >= j).to(xf.dtype)[:, None]
        y = y + shifted * valid * wf[:, K - 1 - j][None, :]
    return TF.silu(y).to(x.dtype)


class _LinearScan(torch.autograd.Function):
    """``S_{c+1} = A_c S_c + B_c`` over the chunk axis, ``S_0 = 0``; returns the state entering
    every chunk. The matrices are given TRANSPOSED (``At[c] = A_c^T``, [n,H,dk,dk]), ``B``
    [n,H,dk,dv], fp32: the kernel multiplies by the transpose of what it is handed, so the
    forward pass reads ``At`` as stored and the adjoint recurrence reads ``A`` as stored.
    Backward: ``lam_c = dS_c + A_c^T lam_{c+1}``, ``dB_c = lam_{c+1}``, ``dA_c = lam_{c+1} S_c^T``."""

    @staticmethod
    def run(M, B, reverse: bool):
        """``X_{c+1} = M_c^T X_c + B_c``; out[c] = X entering step c (walking down when reverse)."""
        n, H, dk, dv = B.shape
        out = torch.empty_like(B)
        if M.is_cuda and dv % 32 == 0 and dk % 4 == 0 and dk <= 128:
            _lib.check(_lib.lib().ss_linear_scan(M.data_ptr(), B.data_ptr(), out.data_ptr(), n, H, dk, dv,
                                                 int(reverse), _lib.stream_ptr()), "ss_linear_scan")
            return out
        X = B.new_zeros(H, dk, dv)
        for s in range(n):
            c = n - 1 - s if reverse else s
            out[c] = X
            X = M[c].transpose(-1, -2) @ X + B[c]
        return out

    @staticmethod
    def forward(ctx, At, B):
        At, B = At.contiguous(), B.contiguous()
        S = _LinearScan.run(At, B, False)
        ctx.save_for_backward(At, S)
        return S

    @staticmethod
    def backward(ctx, dS):
        At, S = ctx.saved_tensors
        A = At.transpose(-1, -2).contiguous()
        lam = _LinearScan.run(A, dS.contiguous(), True)           # gradient reaching S_{c+1}
        return S @ lam.transpose(-1, -2), lam                      # d(A^T) = (lam S^T)^T


_lib.register("ss_linear_scan", [_c.c_p, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                 _c.c_p])


def gated_delta_rule_chunked(q, k, v, beta, g, bounds: list[int] | None, chunk: int = 64,
                             cu_seqlens: torch.Tensor | None = None) -> torch.Tensor:
    """q,k [T,Hk,dk] (L2-normalised), v [T,Hv,dv], beta,g [T,Hv] (g = log decay <= 0).
    QK heads are repeat-interleaved to the V heads. Returns [T,Hv,dv] in ``v.dtype``.

    bf16 CUDA tensors with 128-wide heads and 64-token chunks run on the hand-written tcgen05
    kernels of ``ops/csrc/deltanet_chunk.cu`` (forward and backward); everything else (CPU, fp32,
    other head widths) evaluates the same algebra with PyTorch tensor operations."""
    from . import delta_rule
    if delta_rule.supported(q, k, v, chunk) and cu_seqlens is not None:
        return delta_rule.gated_delta_rule(q, k, v, beta, g, cu_seqlens)
    return _gated_delta_rule_torch(q, k, v, beta, g, bounds, chunk, cu_seqlens)


def _gated_delta_rule_torch(q, k, v, beta, g, bounds: list[int] | None, chunk: int = 64,
                            cu_seqlens: torch.Tensor | None = None) -> torch.Tensor:
    """The chunked gated delta rule as PyTorch tensor operations (CPU path and oracle).

    The packed stream is cut into chunks of ``chunk`` tokens regardless of where sequences
    begin; sequence boundaries act through masks (no decay path and no state carry across a
    boundary), so the work and the memory are the same for every packing and there is no
    loop over sequences. Sequence ids come from ``cu_seqlens`` on the device (no host read)
    or from ``bounds``."""
    T, Hk, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    rep = H // Hk
    C = chunk
    n = -(-T // C)
    pad = n * C - T
    dev = q.device
    pos = torch.arange(T, device=dev)
    if cu_seqlens is not None:
        sid = torch.bucketize(pos, cu_seqlens[1:].to(torch.long), right=True)
    else:
        sid = torch.bucketize(pos, torch.tensor(list(bounds[1:]), device=dev, dtype=torch.long), right=True)
    scale = dk ** -0.5                              # folded into the query-side products below
    grow = lambda t: (t if rep == 1 else t[:, :, None, :].expand(T, Hk, rep, dk).reshape(T, H, dk))
    qf, kf = grow(q).float(), grow(k).float()
    vf, bf, gf = v.float(), beta.float(), g.float()
    if pad:
        zp = lambda t: TF.pad(t, (0, 0) * (t.dim() - 1) + (0, pad))
        qf, kf, vf, bf, gf = zp(qf), zp(kf), zp(vf), zp(bf), zp(gf)
        sid = torch.cat([sid, sid.new_full((pad,), int(2 ** 31 - 1))])    # padding is its own sequence
    rs = lambda t: t.reshape(n, C, H, -1).permute(0, 2, 1, 3).contiguous()   # [n,H,C,*], one copy each
    qc, kc, vc = rs(qf), rs(kf), rs(vf)
    bc = bf.reshape(n, C, H).permute(0, 2, 1)                           # [n,H,C]
    gam = gf.reshape(n, C, H).permute(0, 2, 1).cumsum(-1)               # log of the running decay
    sidc = sid.reshape(n, C)
    same = sidc[:, :, None] == sidc[:, None, :]                         # [n,C,C]
    prev_last = torch.cat([sidc.new_full((1,), -1), sidc[:-1, -1]])
    first_seg = (sidc == prev_last[:, None])                            # continues the previous chunk
    last_seg = (sidc == sidc[:, -1:])                                   # same sequence as the chunk's end
    lower = torch.ones(C, C, device=dev, dtype=torch.bool).tril()
    valid = (same & lower)[:, None]                                     # [n,1,C,C]
    diff = gam[..., :, None] - gam[..., None, :]
    ratio = torch.exp(diff.masked_fill(~valid, float("-inf")))          # G_t/G_i inside one sequence
    strict = ~torch.eye(C, device=dev, dtype=torch.bool)
    tf32 = torch.backends.cuda.matmul.allow_tf32
    # the batched products run on the tensor cores in TF32 (10-bit mantissa, fp32 accumulate:
    # finer than the bf16 operands they come from); the triangular system stays in fp32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        A = bc[..., :, None] * ratio * (kc @ kc.transpose(-1, -2)) * strict
        eye = torch.eye(C, device=dev, dtype=qf.dtype).expand(n, H, C, C)
        torch.backends.cuda.matmul.allow_tf32 = False
        Tm = torch.linalg.solve_triangular(eye + A, eye, upper=False)
        torch.backends.cuda.matmul.allow_tf32 = True
        Gt = torch.exp(gam) * first_seg[:, None, :]                     # decay from the carried state
        W = Tm @ (bc[..., None] * Gt[..., None] * kc)                   # [n,H,C,dk]
        U0 = Tm @ (bc[..., None] * vc)                                  # [n,H,C,dv]
        M = (ratio * scale) * (qc @ kc.transpose(-1, -2))
        Qg = (Gt * scale)[..., None] * qc
        Gc = torch.exp(gam[..., -1]) * first_seg[:, -1][:, None]        # [n,H]
        Kd = (torch.exp(gam[..., -1:] - gam) * last_seg[:, None, :])[..., None] * kc
        KdT = Kd.transpose(-1, -2)
        # S_next = (Gc I - Kd^T W) S + Kd^T U0; the scan takes the matrix transposed
        AmatT = Gc[..., None, None] * torch.eye(dk, device=dev, dtype=qf.dtype) - W.transpose(-1, -2) @ Kd
        Bmat = KdT @ U0
        S = _LinearScan.apply(AmatT, Bmat)                              # state entering each chunk
        U = U0 - W @ S
        out = Qg @ S + M @ U
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
    out = out.permute(0, 2, 1, 3).reshape(n * C, H, dv)
    return out[:T].to(v.dtype)


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, eps: float,
                  zero_centered: bool = False) -> torch.Tensor:
    """RMSNorm over the last dimension followed by a SiLU gate (reference:
    models/shared/decoder.py GatedRMSNorm)."""
    if _native(x) and gate.dtype == x.dtype and w.dtype == x.dtype and x.shape[-1] % 2 == 0:
        return _GatedRMSNorm.apply(x, gate, w, eps, zero_centered)
    xf = x.float()
    r = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    scale = (1.0 + w.float()) if zero_centered else w.float()
    return (xf * r * scale * TF.silu(gate.float())).to(x.dtype)
