"""Packed variable-length causal attention on CUDA.

``forward``/``backward`` use the hand-written tcgen05 kernels of
``libss_kernels.so`` when the library exports them (``ss_attn_fwd``,
``ss_attn_bwd``). ``IMPLEMENTATION`` names the path taken so that benchmarks and
tests can state which arm they measured; the library arm (flash-attn) exists
only as the comparison baseline and is selected explicitly with
``SS_ATTENTION=library``.

Semantics: packed causal GQA with per-sequence boundaries, the contract of the
reference's ``mlops.flash_attention(q, k, v, cu_seqlens, max_seqlen)`` call
(packages/workloads/src/shadowspill_workloads/models/llama3/implementations/mlops.py:67).
"""
from __future__ import annotations

import math
import os

import torch

from . import _lib

_c = _lib
_lib.register("ss_attn_fwd", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_int, _c.c_int,
                              _c.c_int, _c.c_int, _c.c_int, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_ll,
                              _c.c_f, _c.c_p, _c.c_p])
_lib.register("ss_attn_bwd_g", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p,
                                _c.c_p, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                _c.c_int, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_ll,
                                _c.c_f, _c.c_p, _c.c_p])
_lib.register("ss_attn_bwd", [_c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p, _c.c_p,
                              _c.c_p, _c.c_p, _c.c_p, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                              _c.c_int, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_ll, _c.c_f, _c.c_p,
                              _c.c_p])


def _native_available(symbol: str) -> bool:
    try:
        handle = _lib.lib()
    except _lib.KernelLibraryMissing:
        return False
    return hasattr(handle, symbol)


def implementation(symbol: str = "ss_attn_fwd") -> str:
    want = os.environ.get("SS_ATTENTION", "native")
    if want == "native":
        if not _native_available(symbol):
            raise RuntimeError(f"{symbol} is not in libss_kernels.so; rebuild, or set "
                               "SS_ATTENTION=library for the baseline arm")
        return "native"
    return "library"


def _row_stride(t: torch.Tensor) -> int:
    if t.stride(2) != 1 or t.stride(1) != t.shape[2]:
        raise ValueError("attention operands must be [T, H, dh] with contiguous heads")
    return t.stride(0)


def forward(q, k, v, cu_seqlens, max_seqlen, scale=None, out=None, lse=None):
    T, Hq, dh = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    if implementation() == "library":
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward
        res = _flash_attn_varlen_forward(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                         0.0, scale, causal=True)
        o, l = res[0], res[1]
        if out is not None:
            out.copy_(o)
            o = out
        if lse is not None:
            l = lse.copy_(l)
        return o, l
    o = torch.empty((T, Hq, dh), dtype=q.dtype, device=q.device) if out is None else out
    if lse is None:
        lse = torch.empty((Hq, T), dtype=torch.float32, device=q.device)
    nseq = cu_seqlens.numel() - 1
    rc = _lib.lib().ss_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                lse.data_ptr(), cu_seqlens.data_ptr(), nseq, T, Hq, Hkv, dh,
                                _row_stride(q), _row_stride(k), _row_stride(v), _row_stride(o),
                                float(scale), _lib.status_word(q.device).data_ptr(),
                                _lib.stream_ptr())
    _lib.check(rc, "ss_attn_fwd")
    return o, lse


def backward(q, k, v, out, lse, dout, cu_seqlens, max_seqlen, scale=None, dq=None, dk=None,
             dv=None):
    T, Hq, dh = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(dh)
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty(k.shape, dtype=k.dtype, device=k.device) if dk is None else dk
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device) if dv is None else dv
    if implementation("ss_attn_bwd") == "library":
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward
        dqc = dq if dq.is_contiguous() else torch.empty_like(q)
        dkc = dk if dk.is_contiguous() else torch.empty_like(k)
        dvc = dv if dv.is_contiguous() else torch.empty_like(v)
        _flash_attn_varlen_backward(dout.contiguous(), q, k, v, out, lse, dqc, dkc, dvc,
                                    cu_seqlens, cu_seqlens, max_seqlen, max_seqlen, 0.0, scale,
                                    True, -1, -1, 0.0, None, False)
        for dst, src in ((dq, dqc), (dk, dkc), (dv, dvc)):
            if dst is not src:
                dst.copy_(src)
        return dq, dk, dv
    nseq = cu_seqlens.numel() - 1
    if not out.is_contiguous():
        raise ValueError("attention output must be contiguous [T, Hq, dh]")
    delta = torch.empty((Hq, T), dtype=torch.float32, device=q.device)   # kernel scratch
    rc = _lib.lib().ss_attn_bwd_g(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                  lse.data_ptr(), dout.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                  dv.data_ptr(), cu_seqlens.data_ptr(), delta.data_ptr(), nseq, T,
                                  Hq, Hkv, dh,
                                  _row_stride(q), _row_stride(k), _row_stride(v), _row_stride(dout),
                                  _row_stride(dq), _row_stride(dk), _row_stride(dv),
                                  float(scale), _lib.status_word(q.device).data_ptr(),
                                  _lib.stream_ptr())
    _lib.check(rc, "ss_attn_bwd")
    return dq, dk, dv
