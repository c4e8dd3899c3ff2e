"""The allocation-free attention-backward entry point, through its exported C symbol.

Some users of the kernel library cannot allocate device memory around a call: a
fixed-layout memory plan has no spare bytes for an unplanned buffer, an
allocation in the middle of a pipeline would synchronise the device, and an
embedding runtime that owns all device memory may hand foreign code no
allocator. ``ss_attn_bwd_noalloc`` serves them by keeping the kernel's scratch in
a fixed array inside the library. This test calls it exactly as such a caller
would (ctypes, raw pointers, no wrapper) and checks it against the ordinary
entry point, twice in a row, because consecutive calls share the scratch array
and the second must not be disturbed by what the first left behind.

This file is collected last on purpose, so a run that stops at the first failure
has already exercised everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

_ARGS = [C.c_void_p] * 10 + [C.c_int] * 5 + [C.c_longlong] * 4 + [C.c_float, C.c_void_p, C.c_void_p]


def _symbol():
    from shadowspill_b200.ops import _lib
    lib = _lib.lib()
    fn = lib.ss_attn_bwd_noalloc
    fn.argtypes = _ARGS
    fn.restype = C.c_int
    lib.ss_attn_bwd_noalloc_max_elements.restype = C.c_longlong
    return lib, fn


def _case(T, lens, Hq, Hkv, dh, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda h, s=0.8: (torch.randn(T, h, dh, generator=g) * s).to(torch.bfloat16).cuda()
    q, k, v, dout = mk(Hq), mk(Hkv), mk(Hkv, 1.0), mk(Hq, 0.5)
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    return q, k, v, dout, torch.tensor(cu, dtype=torch.int32, device="cuda")


def test_noalloc_matches_allocating_entry_point_on_two_calls():
    from shadowspill_b200.ops import _lib, attention
    lib, fn = _symbol()
    assert lib.ss_attn_bwd_noalloc_max_elements() == 2 * 1024 * 1024
    status = _lib.status_word()
    # two different problems back to back: the second reuses the array the first dirtied
    for seed, (T, lens, Hq, Hkv, dh) in enumerate([(640, [100, 37, 300, 203], 4, 2, 128),
                                                   (512, [130, 382], 8, 2, 128)]):
        q, k, v, dout, cu = _case(T, lens, Hq, Hkv, dh, seed)
        scale = dh ** -0.5
        out, lse = attention.forward(q, k, v, cu, max(lens), scale)
        want = attention.backward(q, k, v, out, lse, dout, cu, max(lens), scale)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        torch.cuda.synchronize()
        # the driver's own count of free device bytes sees a cudaMalloc made inside the
        # library, which torch's allocator statistics would not
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr(),
                cu.numel() - 1, T, Hq, Hkv, dh, Hq * dh, Hkv * dh, Hkv * dh, Hq * dh,
                C.c_float(scale), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if seed > 0:      # the first call may still load the kernels' code onto the device
            assert torch.cuda.mem_get_info()[0] == free_before
        _lib.check_status()
        for got, ref in zip((dq, dk, dv), want):
            rel = float((got.float() - ref.float()).norm() / (ref.float().norm() + 1e-12))
            assert rel < 2e-2


def test_noalloc_refuses_problems_beyond_its_array():
    lib, fn = _symbol()
    limit = lib.ss_attn_bwd_noalloc_max_elements()
    T, Hq = 4096, limit // 4096 + 1
    rc = fn(None, None, None, None, None, None, None, None, None, None, 1, T, Hq, 1, 128,
            Hq * 128, 128, 128, Hq * 128, C.c_float(1.0), None, None)
    assert rc == -3     # SS_ATTN_NOALLOC_TOO_LARGE: nothing was launched
    # bad head counts: the allocating entry point's own answer
    rc = fn(None, None, None, None, None, None, None, None, None, None, 1, 128, 0, 1, 128,
            0, 128, 128, 0, C.c_float(1.0), None, None)
    assert rc == -2


def test_noalloc_refuses_operands_that_are_not_on_the_current_device():
    lib, fn = _symbol()
    host = torch.zeros(128 * 128, dtype=torch.bfloat16)          # not device memory at all
    rc = fn(host.data_ptr(), host.data_ptr(), host.data_ptr(), host.data_ptr(), None,
            host.data_ptr(), host.data_ptr(), host.data_ptr(), host.data_ptr(), None, 1, 128, 1, 1,
            128, 128, 128, 128, 128, C.c_float(1.0), None, None)
    assert rc == -4     # SS_ATTN_NOALLOC_BAD_DEVICE: refused before any launch
