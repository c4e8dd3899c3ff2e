/* Attention backward for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference system.
 *
 * Who needs it. ss_attn_bwd wants a scratch buffer (fp32 [Hq, T]) from its
 * caller, and callers normally get it from an allocator. Some cannot: code that
 * runs inside a fixed-layout memory plan where every device byte is already
 * spoken for and an unplanned cudaMalloc would break the budget (or simply fail);
 * code running between other kernels where the implicit device synchronisation
 * of cudaMalloc/cudaFree would stall the whole pipeline; and embedders that call
 * this library through its C ABI from a runtime that owns all device memory and
 * gives foreign code no allocator at all. For them the scratch lives in a
 * fixed array inside the library.
 *
 * What it costs. Every GPU on which this library is loaded holds the array
 * (SS_ATTN_NOALLOC_MAX_ELEMENTS floats = 8 MiB) from load until the process
 * exits, whether or not the entry point is ever called.
 *
 * Limits and rules.
 *  - Hq * T must not exceed SS_ATTN_NOALLOC_MAX_ELEMENTS; larger problems are
 *    refused with SS_ATTN_NOALLOC_TOO_LARGE and nothing is launched. Use
 *    ss_attn_bwd with your own scratch for those.
 *  - Every call must be made with the operands' device current: the scratch
 *    used is the current device's copy of the array, and a call whose `dq` lives
 *    on another GPU (or is not device memory) is refused with
 *    SS_ATTN_NOALLOC_BAD_DEVICE before anything is launched.
 *  - The first call on each device looks up the array's device address (a
 *    one-time host-side query, no allocation). Make that first call outside any
 *    stream capture.
 *  - All calls on a device share the one array, and it keeps whatever the last
 *    call left in it. Each call rewrites every element it later reads, so
 *    nothing needs clearing, but two calls whose kernels may overlap on the GPU
 *    (different streams without ordering between them) race on it: keep calls
 *    on one stream, or order them with events.
 *  - Inputs, outputs, strides, status word and return codes are exactly those
 *    of ss_attn_bwd (bad head counts give -2 here too); the function calls no cudaMalloc, cudaFree or any
 *    allocating library routine.
 */
#ifndef SS_ATTENTION_NOALLOC_H
#define SS_ATTENTION_NOALLOC_H

#define SS_ATTN_NOALLOC_MAX_ELEMENTS (2 * 1024 * 1024)   /* Hq * T, fp32: 8 MiB per GPU */
#define SS_ATTN_NOALLOC_TOO_LARGE (-3)
#define SS_ATTN_NOALLOC_BAD_DEVICE (-4)

#ifdef __cplusplus
extern "C" {
#endif

/* The same arguments as ss_attn_bwd without the scratch pointer. */
int ss_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out,
                        const float* lse, const void* dout, void* dq, void* dk, void* dv,
                        const int* cu_seqlens, int nseq, int T, int Hq, int Hkv, int dh,
                        long long ldq, long long ldk, long long ldv, long long ldo, float scale,
                        int* status, void* stream);

/* SS_ATTN_NOALLOC_MAX_ELEMENTS as compiled into the library. */
long long ss_attn_bwd_noalloc_max_elements(void);

int ss_attn_bwd(const void* q, const void* k, const void* v, const void* out, const float* lse,
                const void* dout, void* dq, void* dk, void* dv, const int* cu_seqlens,
                float* delta_scratch, int nseq, int T, int Hq, int Hkv, int dh, long long ldq,
                long long ldk, long long ldv, long long ldo, float scale, int* status,
                void* stream);

#ifdef __cplusplus
}
#endif
#endif
