"""Kernel micro-benchmarks with roofline fractions.

    python -m shadowspill_b200.ops.microbench gemm --m 8192 --n 8192 --k 8192
    python -m shadowspill_b200.ops.microbench attention --tokens 16384 --seqlen 4096
    python -m shadowspill_b200.ops.microbench deltanet --tokens 8192 --seqlen 2048 --compare
    python -m shadowspill_b200.ops.microbench all --json out.json

Each case is timed with CUDA events on the launching stream after warm-up, with
an L2 flush (a write larger than L2) between timed iterations. Fractions are
relative to the measured peaks in ``MEASURED_PEAKS.json`` at the repository root
when that file exists ("of measured"), else to 6.65 TB/s and 1.59 PFLOP/s ("of
fallback"). ``--iters 1 --warmup 0`` gives the short run used under a profiler.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from . import _lib, attention
from . import functional as F

ROOT = Path(__file__).resolve().parents[2]


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "kind": "of measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "kind": "of fallback"}


_flush = None


def flush_l2() -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def timed(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters * 1e-3


def report(name: str, seconds: float, flops: float = 0.0, nbytes: float = 0.0, **extra) -> dict:
    pk = peaks()
    row = {"case": name, "ms": round(seconds * 1e3, 4)}
    if flops:
        row["tflops"] = round(flops / seconds / 1e12, 1)
        row["frac_compute"] = round(flops / seconds / 1e12 / pk["tflops"], 3)
    if nbytes:
        row["gbs"] = round(nbytes / seconds / 1e9, 1)
        row["frac_hbm"] = round(nbytes / seconds / 1e9 / pk["hbm_gbs"], 3)
    row["peaks"] = pk["kind"]
    row.update(extra)
    print(json.dumps(row), flush=True)
    return row


def bench_gemm(a) -> list[dict]:
    M, N, K = a.m, a.n, a.k
    out = []
    layouts = {"nt": (False, False), "nn": (False, True), "tn": (True, True)}
    for name in ([a.layout] if a.layout != "all" else layouts):
        a_mn, b_mn = layouts[name]
        A = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
        B = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
        C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        s = timed(lambda: F.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=C, accumulate=a.accumulate),
                  a.iters, a.warmup)
        out.append(report(f"gemm_{name}_{M}x{N}x{K}", s, 2.0 * M * N * K,
                          2.0 * (M * K + N * K + M * N)))
    return out


def _attn_inputs(T, seqlen, Hq, Hkv, dh):
    q = torch.randn(T, Hq, dh, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(T, Hkv, dh, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, Hkv, dh, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, T + 1, seqlen, dtype=torch.int32, device="cuda")
    return q, k, v, cu


def bench_attention(a) -> list[dict]:
    T, L, Hq, Hkv, dh = a.tokens, a.seqlen, a.heads, a.kv_heads, a.head_dim
    q, k, v, cu = _attn_inputs(T, L, Hq, Hkv, dh)
    fl = 4.0 * T * (L / 2.0) * Hq * dh          # causal: half of the score matrix
    out = []
    s = timed(lambda: attention.forward(q, k, v, cu, L), a.iters, a.warmup)
    out.append(report(f"attn_fwd_T{T}_L{L}_H{Hq}/{Hkv}_d{dh}", s, fl))
    o, lse = attention.forward(q, k, v, cu, L)
    do = torch.randn_like(q)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    s = timed(lambda: attention.backward(q, k, v, o, lse, do, cu, L, dq=dq, dk=dk, dv=dv),
              a.iters, a.warmup)
    out.append(report(f"attn_bwd_T{T}_L{L}_H{Hq}/{Hkv}_d{dh}", s, 2.5 * fl))
    if a.compare:
        # the library arm at the same shape (flash-attn's kernels through the same entry points)
        import os
        before = os.environ.get("SS_ATTENTION")
        os.environ["SS_ATTENTION"] = "library"
        try:
            s = timed(lambda: attention.forward(q, k, v, cu, L), a.iters, a.warmup)
            out.append(report(f"library_attn_fwd_T{T}_L{L}_H{Hq}/{Hkv}_d{dh}", s, fl))
            o2, lse2 = attention.forward(q, k, v, cu, L)
            s = timed(lambda: attention.backward(q, k, v, o2, lse2, do, cu, L, dq=dq, dk=dk, dv=dv),
                      a.iters, a.warmup)
            out.append(report(f"library_attn_bwd_T{T}_L{L}_H{Hq}/{Hkv}_d{dh}", s, 2.5 * fl))
        finally:
            if before is None:
                os.environ.pop("SS_ATTENTION", None)
            else:
                os.environ["SS_ATTENTION"] = before
    return out


def bench_elementwise(a) -> list[dict]:
    T, D, Fw, V = a.tokens, a.d_model, a.d_ff, a.vocab
    out = []
    x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    y, rstd = torch.empty_like(x), torch.empty(T, device="cuda")
    s = timed(lambda: F.rmsnorm_fwd(x, w, out=y, rstd=rstd), a.iters, a.warmup)
    out.append(report(f"rmsnorm_fwd_{T}x{D}", s, nbytes=4.0 * T * D))
    dw, dx = torch.zeros(D, device="cuda"), torch.empty_like(x)
    s = timed(lambda: F.rmsnorm_bwd(x, w, y, rstd, dw, dx=dx), a.iters, a.warmup)
    out.append(report(f"rmsnorm_bwd_{T}x{D}", s, nbytes=6.0 * T * D))
    gu = torch.randn(T, 2 * Fw, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(T, Fw, device="cuda", dtype=torch.bfloat16)
    s = timed(lambda: F.swiglu_fwd(gu, out=h), a.iters, a.warmup)
    out.append(report(f"swiglu_fwd_{T}x{Fw}", s, nbytes=6.0 * T * Fw))
    dgu = torch.empty_like(gu)
    s = timed(lambda: F.swiglu_bwd(gu, h, out=dgu), a.iters, a.warmup)
    out.append(report(f"swiglu_bwd_{T}x{Fw}", s, nbytes=10.0 * T * Fw))
    n = D * Fw
    p = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    g, m, vv = torch.randn_like(p), torch.zeros_like(p), torch.zeros_like(p)
    s = timed(lambda: F.adamw_(p, g, m, vv, lr=1e-4, step=2), a.iters, a.warmup)
    out.append(report(f"adamw_sr_{n}", s, nbytes=14.0 * n))
    R = min(T, 2048)
    logits = torch.randn(R, V, device="cuda", dtype=torch.bfloat16)
    tgt = torch.randint(0, V, (R,), device="cuda")
    loss = torch.zeros(1, device="cuda")
    s = timed(lambda: F.cross_entropy_(logits, tgt, None, loss), a.iters, a.warmup)
    out.append(report(f"cross_entropy_{R}x{V}", s, nbytes=6.0 * R * V))
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    qkv = torch.randn(T, 6144, device="cuda", dtype=torch.bfloat16)
    s = timed(lambda: F.rope_(qkv, pos, col0=0, heads=40, dh=128, theta=5e5), a.iters, a.warmup)
    out.append(report(f"rope_{T}x40x128", s, nbytes=4.0 * T * 40 * 128))
    return out


def bench_deltanet(a) -> list[dict]:
    """Gated delta rule, 16 QK / 32 V heads of width 128: forward and forward+backward of the
    chunk kernels, each kernel on its own, and the PyTorch tensor-operation form beside them."""
    from . import delta_rule as dr, sequence as seq
    T, L, Hk, H = a.tokens, a.seqlen, 16, 32
    nrm = lambda x: (x / x.norm(dim=-1, keepdim=True)).bfloat16()
    q, k = nrm(torch.randn(T, Hk, 128, device="cuda")), nrm(torch.randn(T, Hk, 128, device="cuda"))
    v = torch.randn(T, H, 128, device="cuda", dtype=torch.bfloat16)
    beta = torch.sigmoid(torch.randn(T, H, device="cuda"))
    g = -torch.nn.functional.softplus(torch.randn(T, H, device="cuda")) * 0.3
    cu = torch.arange(0, T + 1, L, dtype=torch.int32, device="cuda")
    dout = torch.randn_like(v)
    n = -(-T // 64)
    # products per chunk and V head (multiply-adds x 2): see the kernel file's header
    fwd_fl = n * H * 2.0 * (2 * 64 * 64 * 128 / 2 + 2 * 64 * 64 * 128 + 3 * 64 * 128 * 128 + 64 * 64 * 128)
    out = []
    s = timed(lambda: dr._forward(q, k, v, beta, g, cu, False), a.iters, a.warmup)
    out.append(report(f"deltanet_fwd_T{T}_L{L}", s, fwd_fl))
    s = timed(lambda: dr.backward(q, k, v, beta, g, cu, dout), a.iters, a.warmup)
    out.append(report(f"deltanet_recompute+bwd_T{T}_L{L}", s, 3.5 * fwd_fl))
    _, B, geo = dr._forward(q, k, v, beta, g, cu, True)
    L_, st, status = _lib.lib(), _lib.stream_ptr(), _lib.status_word().data_ptr()
    o = torch.empty_like(v)
    cases = {
        "prep": lambda: L_.ss_dn_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), g.data_ptr(),
                                      B.sid.data_ptr(), B.WTp.data_ptr(), B.U0Tp.data_ptr(), B.QG.data_ptr(),
                                      B.KD.data_ptr(), B.MQ.data_ptr(), B.TMT.data_ptr(), B.XW.data_ptr(),
                                      B.XU.data_ptr(), B.gam.data_ptr(), B.gc.data_ptr(), T, H, Hk,
                                      128 ** -0.5, status, st),
        "state_walk": lambda: L_.ss_dn_fwd(B.WTp.data_ptr(), B.U0Tp.data_ptr(), B.QG.data_ptr(), B.KD.data_ptr(),
                                           B.MQ.data_ptr(), B.gc.data_ptr(), o.data_ptr(), B.ST.data_ptr(),
                                           B.UTp.data_ptr(), T, H, Hk, status, st),
        "bwd_state_walk": lambda: L_.ss_dn_bwd_state(dout.data_ptr(), B.MQ.data_ptr(), B.KD.data_ptr(),
                                                     B.QG.data_ptr(), B.WTp.data_ptr(), B.gc.data_ptr(),
                                                     B.dSpT.data_ptr(), B.dUTp.data_ptr(), T, H, Hk, status, st),
        "bwd_chunk": lambda: L_.ss_dn_bwd_chunk(B.dSpT.data_ptr(), B.ST.data_ptr(), B.UTp.data_ptr(),
                                                B.dUTp.data_ptr(), dout.data_ptr(), B.dKdTp.data_ptr(),
                                                B.dQgTp.data_ptr(), B.dWTp.data_ptr(), B.dMQ.data_ptr(),
                                                B.dgc.data_ptr(), T, H, Hk, status, st),
    }
    for name, fn in cases.items():
        out.append(report(f"deltanet_{name}_T{T}", timed(fn, a.iters, a.warmup)))
    if a.compare:
        qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))

        def torch_form():
            with seq.tf32_matmul():
                y = seq._gated_delta_rule_torch(qf, kf, vf, beta, g, None, 64, cu)
                y.backward(dout.float())
        out.append(report(f"deltanet_torch_form_fwd+bwd_T{T}_L{L}", timed(torch_form, max(1, a.iters // 3), 1)))
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("what", choices=["gemm", "attention", "elementwise", "deltanet", "all"])
    ap.add_argument("--compare", action="store_true", help="also time the PyTorch tensor-operation form")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="all", choices=["nt", "nn", "tn", "all"])
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seqlen", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--d-ff", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default="")
    a = ap.parse_args(argv)
    _lib.lib()
    rows = []
    if a.what in ("gemm", "all"):
        rows += bench_gemm(a)
    if a.what in ("attention", "all"):
        rows += bench_attention(a)
    if a.what in ("elementwise", "all"):
        rows += bench_elementwise(a)
    if a.what in ("deltanet", "all"):
        rows += bench_deltanet(a)
    _lib.check_status()
    if a.json:
        Path(a.json).parent.mkdir(parents=True, exist_ok=True)
        Path(a.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
