// Gated DeltaNet, chunked form, forward and backward, on tcgen05 (sm_100a).
//
// The packed token stream is cut into chunks of 64 tokens. With g the log decay, gam its running
// sum inside the chunk, R[t,i] = exp(gam_t - gam_i) for i <= t inside one sequence (0 otherwise):
//
//     A  = diag(beta) (R o K K^T), strictly lower           Tm = (I + A)^-1
//     W  = Tm diag(beta Gt) K        U0 = Tm diag(beta) V    Gt_t = exp(gam_t) [t continues the
//     U  = U0 - W S                                                 sequence of the previous chunk]
//     O  = diag(s Gt) Q S + (s R o Q K^T) U                  s = dk^-1/2
//     S' = Gc S + (diag(d) K)^T U                            d_t = exp(gam_63 - gam_t) [same
//                                                                   sequence as the chunk's end]
//
// which equals the token recurrence S <- a S; u = beta (v - k S); S <- S + k u^T; o = s q S
// (reference definition: packages/workloads/src/shadowspill_workloads/models/qwen35/
// implementations/pytorch/delta_rule/reference.py:8-41, backward :43-132; call site
// models/shared/delta_net.py:76). Sequence boundaries act only through the masks, so a packed
// batch needs no loop over sequences and no padding to chunk multiples.
//
// Kernels (dk = dv = 128; QK heads are shared by `rep` V heads, handled two V heads at a time):
//   dn_prep_kernel   per (chunk, pair of V heads): K K^T and Q K^T on the tensor cores, the
//                    64x64 triangular inverse by forward substitution in registers (one column
//                    per thread), then W^T and U0^T as MMAs; writes every per-chunk operand.
//   dn_fwd_kernel    per V head, sequential over chunks: the state S^T lives in TMEM (fp32);
//                    U^T = U0^T - S^T W^T, O^T = S^T Qg^T + U^T Mq^T, S'^T = Gc S^T + U^T Kd.
//   dn_bwd_state_kernel   the same walk in reverse for dS and dU.
//   dn_bwd_chunk_kernel   per (chunk, V head): the products that need S or dS' of one chunk.
//   dn_bwd_prep_kernel    per (chunk, pair): gradients of the chunk-local algebra -> dq dk dv
//                         dbeta dg.
// All matrices are kept transposed where that makes the M dimension 128 (features), so every MMA
// is 128 x {64,128} x 16 with operands either loaded by TMA or written one row per thread.
// No operand ever comes from another GPU; every wait is bounded.
#include "sm100_ptx.cuh"

#include <cudaTypedefs.h>
#include <math.h>

namespace ss {
int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                   long long ld, int box_rows);  // gemm_tcgen05.cu
}

namespace ss_dnc {
using namespace ss;

constexpr int CH = 64;         // tokens per chunk
constexpr int D = 128;         // dk = dv
constexpr int THREADS = 160;   // 4 row warps + 1 control warp
constexpr int CTRL = 128;      // the thread that issues TMA loads and MMAs

struct Geo {
  int T, n, H, Hk, rep, P, NP;   // P pairs of V heads per QK head, NP = Hk * P pairs per chunk
};

__device__ __forceinline__ void head_slot(const Geo& g, int h, int& pr, int& hh) {
  const int kh = h / g.rep, r = h % g.rep;
  pr = kh * g.P + (r >> 1);
  hh = r & 1;
}

// Byte offset of the 16-byte chunk holding columns [8*col8, 8*col8+8) of `row` in a tile made of
// 64-column blocks of `rows_per_blk` rows each (128-byte rows, 128B swizzle).
__device__ __forceinline__ uint32_t sw_off(int rows_per_blk, int row, int col8) {
  return static_cast<uint32_t>((col8 >> 3) * rows_per_blk * 128 + row * 128 +
                               (((col8 & 7) ^ (row & 7)) << 4));
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                    pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ float bf16_at(const uint8_t* p) {
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
}
// 32 fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_row32(uint32_t addr, float* out) {
  uint32_t r[32];
  tmem_ld_32x32(addr, r);
  tmem_ld_wait();
#pragma unroll
  for (int e = 0; e < 32; ++e) out[e] = __uint_as_float(r[e]);
}
__device__ __forceinline__ void tmem_row64(uint32_t addr, float* out) {
  tmem_row32(addr, out);
  tmem_row32(addr + 32, out + 32);
}
// Operands written by threads (shared memory, TMEM) become visible to the MMA issuer.
__device__ __forceinline__ void publish() {
  tc_fence_before();
  fence_async_proxy();
  __syncthreads();
  tc_fence_after();
}
// 64 bf16 values -> one 128-byte row of a global array.
__device__ __forceinline__ void store_row64(__nv_bfloat16* dst, const float* f) {
#pragma unroll
  for (int q = 0; q < 8; ++q) reinterpret_cast<uint4*>(dst)[q] = pack8(f + q * 8);
}
__device__ __forceinline__ void load_row64(const __nv_bfloat16* src, float* f) {
#pragma unroll
  for (int q = 0; q < 8; ++q) unpack8(reinterpret_cast<const uint4*>(src)[q], f + q * 8);
}
// Column sums over the row threads. Each row thread first writes its 64 values into its row of
// `red` ([128][65] fp32); red_sums then adds them up: per group of 64 threads into out[g*64+i]
// (per_group), or over all 128 into out[i]. red_sums must be called by every thread of the block.
__device__ __forceinline__ void red_sums(float* red, float* out, bool per_group) {
  const int tid = threadIdx.x;
  __syncthreads();
  if (tid < 128) {
    const int g = tid >> 6, i = tid & 63;
    if (per_group) {
      float s = 0.f;
      for (int t = 0; t < 64; ++t) s += red[(g * 64 + t) * 65 + i];
      out[g * 64 + i] = s;
    } else if (g == 0) {
      float s = 0.f;
      for (int t = 0; t < 128; ++t) s += red[t * 65 + i];
      out[i] = s;
    }
  }
  __syncthreads();
}

// ============================================================================ sequence ids
__global__ void dn_seq_ids_kernel(const int* __restrict__ cu, int nseq, int T, int Tp,
                                  int* __restrict__ sid) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= Tp) return;
  if (t >= T) { sid[t] = 0x7fffffff; return; }       // padding is a sequence of its own
  int lo = 0, hi = nseq;                              // boundaries cu[1..nseq] that are <= t
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid + 1] <= t) lo = mid + 1; else hi = mid;
  }
  sid[t] = lo;
}

// ============================================================================ prep (forward)
struct PrepParams {
  const float* beta; const float* g; const int* sid;
  __nv_bfloat16 *WTp, *U0Tp, *QG, *KD, *MQ, *TMT, *XW, *XU;   // TMT/XW/XU: null unless a backward follows
  float *gam, *gc;
  Geo geo; float scale; int* status;
};
namespace prep {
constexpr int OFF_KQ = 0, OFF_V = 32768, OFF_XW = 65536, OFF_XU = 81920, OFF_AF = 98304;
constexpr int OFF_MISC = OFF_AF + 2 * 64 * 65 * 4;      // 131584
constexpr int OFF_BAR = OFF_MISC + 2048;
constexpr int SMEM = OFF_BAR + 64 + 1024;
}

__global__ void __launch_bounds__(THREADS, 1)
dn_prep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const PrepParams p) {
  using namespace prep;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* Af = reinterpret_cast<float*>(smem + OFF_AF);
  float* gam_s = reinterpret_cast<float*>(smem + OFF_MISC);        // [2][64]
  float* beta_s = gam_s + 128;
  float* g_s = beta_s + 128;
  int* sid_s = reinterpret_cast<int*>(g_s + 128);                  // [65]; [64] = previous chunk's last
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* tma_bar = bars; uint64_t* mma_bar = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5;
  const Geo G = p.geo;
  const int c = blockIdx.x, pr = blockIdx.y;
  const int kh = pr / G.P, z = pr % G.P, h0 = kh * G.rep + 2 * z;
  const int nh = (2 * z + 1 < G.rep) ? 2 : 1;
  const int t0 = c * CH;

  if (tid == 0) { mbar_init(tma_bar, 1); mbar_init(mma_bar, 1); mbar_fence_init(); }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  if (tid == CTRL) {
    mbar_expect_tx(tma_bar, 32768 + nh * 16384);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + OFF_KQ + b * 16384, &tmK, tma_bar, kh * D + b * 64, t0);
      tma_load_2d(smem + OFF_KQ + b * 16384 + 64 * 128, &tmQ, tma_bar, kh * D + b * 64, t0);
    }
    for (int hh = 0; hh < nh; ++hh)
#pragma unroll
      for (int b = 0; b < 2; ++b)
        tma_load_2d(smem + OFF_V + hh * 16384 + b * 8192, &tmV, tma_bar, (h0 + hh) * D + b * 64, t0);
  }
  if (tid < 128) {
    const int hh = tid >> 6, j = tid & 63, tok = t0 + j;
    const bool live = hh < nh && tok < G.T;
    g_s[tid] = live ? p.g[static_cast<long long>(tok) * G.H + h0 + hh] : 0.f;
    beta_s[tid] = live ? p.beta[static_cast<long long>(tok) * G.H + h0 + hh] : 0.f;
  }
  if (tid < 65) sid_s[tid] = tid < 64 ? p.sid[t0 + tid] : (c > 0 ? p.sid[t0 - 1] : -1);
  __syncthreads();
  if (tid < 128) {
    const int hh = tid >> 6, j = tid & 63;
    float s = 0.f;
    for (int i = 0; i <= j; ++i) s += g_s[hh * 64 + i];
    gam_s[tid] = s;
    if (hh < nh) p.gam[(static_cast<long long>(c) * G.H + h0 + hh) * 64 + j] = s;
  }
  __syncthreads();

  // ---- [K; Q] K^T
  if (tid == CTRL) {
    mbar_wait(tma_bar, 0, p.status, KS_TIMEOUT_FULL);
    tc_fence_after();
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, false, false);
    const uint32_t s = smem_u32(smem + OFF_KQ);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t d = umma_smem_desc(s + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
      umma_bf16(tmem_base, d, d, idesc, kk != 0);
    }
    umma_commit(mma_bar);
  }
  mbar_wait(tma_bar, 0, p.status, KS_TIMEOUT_FULL);
  mbar_wait(mma_bar, 0, p.status, KS_TIMEOUT_TMEM_FULL);
  tc_fence_after();

  // ---- A (fp32, shared memory) and Mq (global)
  if (tid < 128) {
    const int t = tid & 63;
    float row[64];
    tmem_row64(lane_addr, row);
    const int my = sid_s[t];
    if (tid < 64) {
      for (int hh = 0; hh < nh; ++hh) {
        const float gt = gam_s[hh * 64 + t], bt = beta_s[hh * 64 + t];
        float* a = Af + hh * 64 * 65 + t * 65;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          a[i] = (i < t && sid_s[i] == my) ? bt * __expf(gt - gam_s[hh * 64 + i]) * row[i] : 0.f;
      }
    } else {
      for (int hh = 0; hh < nh; ++hh) {
        const float gt = gam_s[hh * 64 + t];
        float m[64];
#pragma unroll
        for (int i = 0; i < 64; ++i)
          m[i] = (i <= t && sid_s[i] == my) ? p.scale * __expf(gt - gam_s[hh * 64 + i]) * row[i] : 0.f;
        store_row64(p.MQ + ((static_cast<long long>(c) * G.NP + pr) * 128 + hh * 64 + t) * 64, m);
      }
    }
  }
  __syncthreads();

  // ---- Tm = (I + A)^-1: thread (hh, j) owns column j
  if (tid < 128) {
    const int hh = tid >> 6, j = tid & 63;
    if (hh < nh) {
      float col[64];
      const float* A = Af + hh * 64 * 65;
#pragma unroll
      for (int t = 0; t < 64; ++t) {
        float a0 = (t == j) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        const float* ar = A + t * 65;
#pragma unroll
        for (int i = 0; i < t; ++i) {
          const float v = ar[i] * col[i];
          if ((i & 3) == 0) a0 -= v; else if ((i & 3) == 1) a1 -= v;
          else if ((i & 3) == 2) a2 -= v; else a3 -= v;
        }
        col[t] = (a0 + a1) + (a2 + a3);
      }
      const float bj = beta_s[tid];
      const float gtj = (sid_s[j] == sid_s[64]) ? __expf(gam_s[tid]) : 0.f;
      const int row = hh * 64 + j;
      const long long grow = ((static_cast<long long>(c) * G.NP + pr) * 128 + row) * 64;
      float w[64];
#pragma unroll
      for (int t = 0; t < 64; ++t) w[t] = col[t] * bj * gtj;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(smem + OFF_XW + sw_off(128, row, q)) = pack8(w + q * 8);
      if (p.XW) store_row64(p.XW + grow, w);
#pragma unroll
      for (int t = 0; t < 64; ++t) w[t] = col[t] * bj;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(smem + OFF_XU + sw_off(128, row, q)) = pack8(w + q * 8);
      if (p.XU) store_row64(p.XU + grow, w);
      if (p.TMT) store_row64(p.TMT + grow, col);
    }
  }
  publish();

  // ---- W^T = K^T (Tm diag(beta Gt))^T, U0^T = V^T (Tm diag(beta))^T
  if (tid == CTRL) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, true, true);
    const uint32_t sk = smem_u32(smem + OFF_KQ), sv = smem_u32(smem + OFF_V);
    const uint32_t sxw = smem_u32(smem + OFF_XW), sxu = smem_u32(smem + OFF_XU);
    for (int hh = 0; hh < nh; ++hh) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + 64 + hh * 64, umma_smem_desc(sk + kk * 2048, 16384, 1024),
                  umma_smem_desc(sxw + hh * 8192 + kk * 2048, 8192, 1024), idesc, kk != 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + 192 + hh * 64, umma_smem_desc(sv + hh * 16384 + kk * 2048, 8192, 1024),
                  umma_smem_desc(sxu + hh * 8192 + kk * 2048, 8192, 1024), idesc, kk != 0);
    }
    umma_commit(mma_bar);
  }
  mbar_wait(mma_bar, 1, p.status, KS_TIMEOUT_TMEM_FULL);
  tc_fence_after();

  if (tid < 128) {
    const long long prow = ((static_cast<long long>(c) * G.NP + pr) * 128 + tid) * 128;
    for (int hh = 0; hh < nh; ++hh) {
      float r[64];
      tmem_row64(lane_addr + 64 + hh * 64, r);
      store_row64(p.WTp + prow + hh * 64, r);
      tmem_row64(lane_addr + 192 + hh * 64, r);
      store_row64(p.U0Tp + prow + hh * 64, r);
    }
    // Kd (threads 0..63, K rows) and Qg (threads 64..127, Q rows)
    const int t = tid & 63;
    const bool is_q = tid >= 64;
    for (int hh = 0; hh < nh; ++hh) {
      const float gt = gam_s[hh * 64 + t];
      float f;
      if (is_q) f = (sid_s[t] == sid_s[64]) ? p.scale * __expf(gt) : 0.f;
      else f = (sid_s[t] == sid_s[63]) ? __expf(gam_s[hh * 64 + 63] - gt) : 0.f;
      __nv_bfloat16* dst = (is_q ? p.QG : p.KD) +
                           ((static_cast<long long>(c) * G.H + h0 + hh) * 64 + t) * 128;
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        float v[8];
        unpack8(*reinterpret_cast<const uint4*>(smem + OFF_KQ + sw_off(128, tid, q)), v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] *= f;
        reinterpret_cast<uint4*>(dst)[q] = pack8(v);
      }
      if (tid == 63)
        p.gc[static_cast<long long>(c) * G.H + h0 + hh] =
            (sid_s[63] == sid_s[64]) ? __expf(gam_s[hh * 64 + 63]) : 0.f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ============================================================================ forward state walk
struct WalkParams {
  __nv_bfloat16* out; long long ldo;        // forward: O [T, H*D]
  const float* gc;
  __nv_bfloat16 *ST, *UTp;                  // forward saves (null = not kept)
  __nv_bfloat16 *dSpT, *dUTp;               // backward outputs
  Geo geo; int* status;
};
namespace walk {
constexpr int STAGE = 73728;
constexpr int OFF_SOP = 2 * STAGE;          // [128 x 128] K-major operand
constexpr int OFF_UOP = OFF_SOP + 32768;    // [128 x 64] K-major operand
constexpr int OFF_BAR = OFF_UOP + 16384;
constexpr int SMEM = OFF_BAR + 64 + 1024;
}

// Stage layout (forward): WT @0, U0T @16384, QG @32768, KD @49152, MQ @65536.
__global__ void __launch_bounds__(THREADS, 1)
dn_fwd_kernel(const __grid_constant__ CUtensorMap tmWT, const __grid_constant__ CUtensorMap tmU0T,
              const __grid_constant__ CUtensorMap tmQG, const __grid_constant__ CUtensorMap tmKD,
              const __grid_constant__ CUtensorMap tmMQ, const WalkParams p) {
  using namespace walk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* full = bars; uint64_t* mma_bar = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5;
  const Geo G = p.geo;
  const int h = blockIdx.x;
  int pr, hh;
  head_slot(G, h, pr, hh);

  if (tid == 0) { mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_init(mma_bar, 1); mbar_fence_init(); }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  auto load_stage = [&](int c, int st) {
    uint8_t* s = smem + st * STAGE;
    const int prow = (c * G.NP + pr) * 128, hrow = (c * G.H + h) * 64;
    mbar_expect_tx(&full[st], STAGE);
    tma_load_2d(s, &tmWT, &full[st], hh * 64, prow);
    tma_load_2d(s + 16384, &tmU0T, &full[st], hh * 64, prow);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(s + 32768 + b * 8192, &tmQG, &full[st], b * 64, hrow);
      tma_load_2d(s + 49152 + b * 8192, &tmKD, &full[st], b * 64, hrow);
    }
    tma_load_2d(s + 65536, &tmMQ, &full[st], 0, prow + hh * 64);
  };
  if (tid == CTRL) { load_stage(0, 0); if (G.n > 1) load_stage(1, 1); }
  if (tid < 128) {           // S = 0
    uint32_t zr[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) zr[e] = 0u;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) tmem_st_32x32(lane_addr + c4 * 32, zr);
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  uint32_t mma_phase = 0;
  const uint32_t sop = smem_u32(smem + OFF_SOP), uop = smem_u32(smem + OFF_UOP);
  for (int c = 0; c < G.n; ++c) {
    const int st = c & 1;
    uint8_t* stage = smem + st * STAGE;
    const uint32_t sst = smem_u32(stage);
    mbar_wait(&full[st], (c >> 1) & 1, p.status, KS_TIMEOUT_FULL);
    // 1: S^T -> bf16 operand (and the saved copy); TMEM <- Gc S^T
    if (tid < 128) {
      const float gcv = p.gc[static_cast<long long>(c) * G.H + h];
      __nv_bfloat16* save = p.ST ? p.ST + ((static_cast<long long>(c) * G.H + h) * 128 + tid) * 128 : nullptr;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        float r[32];
        tmem_row32(lane_addr + c4 * 32, r);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 v = pack8(r + q * 8);
          *reinterpret_cast<uint4*>(smem + OFF_SOP + sw_off(128, tid, c4 * 4 + q)) = v;
          if (save) reinterpret_cast<uint4*>(save)[c4 * 4 + q] = v;
        }
        uint32_t w[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) w[e] = __float_as_uint(r[e] * gcv);
        tmem_st_32x32(lane_addr + c4 * 32, w);
      }
      tmem_st_wait();
    }
    publish();
    // 2: (W S)^T = S^T W^T
    if (tid == CTRL) {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, false, true);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem_base + 128, umma_smem_desc(sop + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                  umma_smem_desc(sst + kk * 2048, 16384, 1024), idesc, kk != 0);
      umma_commit(mma_bar);
    }
    mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
    mma_phase ^= 1;
    tc_fence_after();
    // 3: U^T = U0^T - (W S)^T
    if (tid < 128) {
      float du[64];
      tmem_row64(lane_addr + 128, du);
      __nv_bfloat16* save = p.UTp ? p.UTp + ((static_cast<long long>(c) * G.NP + pr) * 128 + tid) * 128 + hh * 64
                                  : nullptr;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float u0[8];
        unpack8(*reinterpret_cast<const uint4*>(stage + 16384 + sw_off(128, tid, q)), u0);
#pragma unroll
        for (int e = 0; e < 8; ++e) u0[e] -= du[q * 8 + e];
        const uint4 v = pack8(u0);
        *reinterpret_cast<uint4*>(smem + OFF_UOP + sw_off(128, tid, q)) = v;
        if (save) reinterpret_cast<uint4*>(save)[q] = v;
      }
    }
    publish();
    // 4: O^T = S^T Qg^T + U^T Mq^T;  S'^T += U^T Kd
    if (tid == CTRL) {
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, true);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem_base + 192, umma_smem_desc(sop + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                  umma_smem_desc(sst + 32768 + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_o,
                  kk != 0);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + 192, umma_smem_desc(uop + kk * 32, 16, 1024),
                  umma_smem_desc(sst + 65536 + kk * 32, 16, 1024), idesc_o, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base, umma_smem_desc(uop + kk * 32, 16, 1024),
                  umma_smem_desc(sst + 49152 + kk * 2048, 8192, 1024), idesc_s, 1);
      umma_commit(mma_bar);
    }
    mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
    mma_phase ^= 1;
    tc_fence_after();
    if (tid == CTRL && c + 2 < G.n) load_stage(c + 2, st);
    // 5: O (transposed store: 32 consecutive features per warp and token)
    if (tid < 128) {
      float o[64];
      tmem_row64(lane_addr + 192, o);
      __nv_bfloat16* dst = p.out + static_cast<long long>(c) * CH * p.ldo + h * D + tid;
      const int lim = min(CH, G.T - c * CH);
#pragma unroll
      for (int t = 0; t < 64; ++t)
        if (t < lim) dst[static_cast<long long>(t) * p.ldo] = __float2bfloat16_rn(o[t]);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ============================================================================ backward state walk
// Stage layout: dO @0 (64 x 128), MQ @16384, KD @24576, QG @40960, WT @57344.
__global__ void __launch_bounds__(THREADS, 1)
dn_bwd_state_kernel(const __grid_constant__ CUtensorMap tmDO, const __grid_constant__ CUtensorMap tmMQ,
                    const __grid_constant__ CUtensorMap tmKD, const __grid_constant__ CUtensorMap tmQG,
                    const __grid_constant__ CUtensorMap tmWT, const WalkParams p) {
  using namespace walk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* full = bars; uint64_t* mma_bar = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5;
  const Geo G = p.geo;
  const int h = blockIdx.x;
  int pr, hh;
  head_slot(G, h, pr, hh);

  if (tid == 0) { mbar_init(&full[0], 1); mbar_init(&full[1], 1); mbar_init(mma_bar, 1); mbar_fence_init(); }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  auto load_stage = [&](int c, int st) {
    uint8_t* s = smem + st * STAGE;
    const int prow = (c * G.NP + pr) * 128, hrow = (c * G.H + h) * 64;
    mbar_expect_tx(&full[st], STAGE);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(s + b * 8192, &tmDO, &full[st], h * D + b * 64, c * CH);
      tma_load_2d(s + 24576 + b * 8192, &tmKD, &full[st], b * 64, hrow);
      tma_load_2d(s + 40960 + b * 8192, &tmQG, &full[st], b * 64, hrow);
    }
    tma_load_2d(s + 16384, &tmMQ, &full[st], 0, prow + hh * 64);
    tma_load_2d(s + 57344, &tmWT, &full[st], hh * 64, prow);
  };
  if (tid == CTRL) { load_stage(G.n - 1, 0); if (G.n > 1) load_stage(G.n - 2, 1); }
  if (tid < 128) {
    uint32_t zr[32];
#pragma unroll
    for (int e = 0; e < 32; ++e) zr[e] = 0u;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) tmem_st_32x32(lane_addr + c4 * 32, zr);
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  uint32_t mma_phase = 0;
  const uint32_t sop = smem_u32(smem + OFF_SOP), uop = smem_u32(smem + OFF_UOP);
  for (int it = 0; it < G.n; ++it) {
    const int c = G.n - 1 - it, st = it & 1;
    const uint32_t sst = smem_u32(smem + st * STAGE);
    mbar_wait(&full[st], (it >> 1) & 1, p.status, KS_TIMEOUT_FULL);
    // 1: dS'^T (gradient of the state leaving chunk c) -> operand + saved copy; TMEM <- Gc dS'^T
    if (tid < 128) {
      const float gcv = p.gc[static_cast<long long>(c) * G.H + h];
      __nv_bfloat16* save = p.dSpT + ((static_cast<long long>(c) * G.H + h) * 128 + tid) * 128;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        float r[32];
        tmem_row32(lane_addr + c4 * 32, r);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 v = pack8(r + q * 8);
          *reinterpret_cast<uint4*>(smem + OFF_SOP + sw_off(128, tid, c4 * 4 + q)) = v;
          reinterpret_cast<uint4*>(save)[c4 * 4 + q] = v;
        }
        uint32_t w[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) w[e] = __float_as_uint(r[e] * gcv);
        tmem_st_32x32(lane_addr + c4 * 32, w);
      }
      tmem_st_wait();
    }
    publish();
    // 2: dU^T = dO^T Mq + dS'^T Kd^T
    if (tid == CTRL) {
      constexpr uint32_t idesc_mn = umma_idesc_bf16(128, 64, true, true);
      constexpr uint32_t idesc_k = umma_idesc_bf16(128, 64, false, false);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + 128, umma_smem_desc(sst + kk * 2048, 8192, 1024),
                  umma_smem_desc(sst + 16384 + kk * 2048, 8192, 1024), idesc_mn, kk != 0);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma_bf16(tmem_base + 128, umma_smem_desc(sop + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                  umma_smem_desc(sst + 24576 + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_k, 1);
      umma_commit(mma_bar);
    }
    mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
    mma_phase ^= 1;
    tc_fence_after();
    // 3: save dU^T; operand <- -dU^T
    if (tid < 128) {
      float du[64];
      tmem_row64(lane_addr + 128, du);
      store_row64(p.dUTp + ((static_cast<long long>(c) * G.NP + pr) * 128 + tid) * 128 + hh * 64, du);
#pragma unroll
      for (int e = 0; e < 64; ++e) du[e] = -du[e];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(smem + OFF_UOP + sw_off(128, tid, q)) = pack8(du + q * 8);
    }
    publish();
    // 4: dS^T += dO^T Qg - dU^T W
    if (tid == CTRL) {
      constexpr uint32_t idesc_mn = umma_idesc_bf16(128, 128, true, true);
      constexpr uint32_t idesc_k = umma_idesc_bf16(128, 128, false, false);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base, umma_smem_desc(sst + kk * 2048, 8192, 1024),
                  umma_smem_desc(sst + 40960 + kk * 2048, 8192, 1024), idesc_mn, 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base, umma_smem_desc(uop + kk * 32, 16, 1024),
                  umma_smem_desc(sst + 57344 + kk * 32, 16, 1024), idesc_k, 1);
      umma_commit(mma_bar);
    }
    mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
    mma_phase ^= 1;
    tc_fence_after();
    if (tid == CTRL && it + 2 < G.n) load_stage(G.n - 1 - (it + 2), st);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ============================================================================ backward, per chunk and head
struct ChunkParams {
  __nv_bfloat16 *dKdTp, *dQgTp, *dWTp, *dMQ;
  float* dgc;
  Geo geo; int* status;
};
namespace chunkk {
constexpr int OFF_DSP = 0, OFF_ST = 32768, OFF_UT = 65536, OFF_DUT = 81920, OFF_DO = 98304;
constexpr int OFF_RED = 131072, OFF_BAR = OFF_RED + 64;
constexpr int SMEM = OFF_BAR + 64 + 1024;
}

__global__ void __launch_bounds__(THREADS, 1)
dn_bwd_chunk_kernel(const __grid_constant__ CUtensorMap tmDSP, const __grid_constant__ CUtensorMap tmST,
                    const __grid_constant__ CUtensorMap tmUT, const __grid_constant__ CUtensorMap tmDUT,
                    const __grid_constant__ CUtensorMap tmDO, const ChunkParams p) {
  using namespace chunkk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* red = reinterpret_cast<float*>(smem + OFF_RED);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* tma_bar = bars; uint64_t* mma_bar = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Geo G = p.geo;
  const int c = blockIdx.x, h = blockIdx.y;
  int pr, hh;
  head_slot(G, h, pr, hh);

  if (tid == 0) { mbar_init(tma_bar, 1); mbar_init(mma_bar, 1); mbar_fence_init(); }
  if (warp == 4) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);

  if (tid == CTRL) {
    const int prow = (c * G.NP + pr) * 128, hrow = (c * G.H + h) * 128;
    mbar_expect_tx(tma_bar, 131072);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + OFF_DSP + b * 16384, &tmDSP, tma_bar, b * 64, hrow);
      tma_load_2d(smem + OFF_ST + b * 16384, &tmST, tma_bar, b * 64, hrow);
      tma_load_2d(smem + OFF_DO + b * 16384, &tmDO, tma_bar, h * D + b * 64, c * CH);
    }
    tma_load_2d(smem + OFF_UT, &tmUT, tma_bar, hh * 64, prow);
    tma_load_2d(smem + OFF_DUT, &tmDUT, tma_bar, hh * 64, prow);
    mbar_wait(tma_bar, 0, p.status, KS_TIMEOUT_FULL);
    tc_fence_after();
    const uint32_t sdsp = smem_u32(smem + OFF_DSP), sst = smem_u32(smem + OFF_ST);
    const uint32_t sut = smem_u32(smem + OFF_UT), sdut = smem_u32(smem + OFF_DUT);
    const uint32_t sdo = smem_u32(smem + OFF_DO);
    constexpr uint32_t i_mm = umma_idesc_bf16(128, 64, true, true);
    constexpr uint32_t i_mk = umma_idesc_bf16(128, 64, true, false);
    constexpr uint32_t i_km = umma_idesc_bf16(128, 64, false, true);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t a_dsp = umma_smem_desc(sdsp + kk * 2048, 16384, 1024);
      const uint64_t a_st = umma_smem_desc(sst + kk * 2048, 16384, 1024);
      const uint64_t b_ut = umma_smem_desc(sut + kk * 2048, 16384, 1024);
      const uint64_t b_dut = umma_smem_desc(sdut + kk * 2048, 16384, 1024);
      const uint64_t k_do = umma_smem_desc(sdo + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
      umma_bf16(tmem_base, a_dsp, b_ut, i_mm, kk != 0);          // dKd^T = dS' U^T
      umma_bf16(tmem_base + 64, a_st, k_do, i_mk, kk != 0);      // dQg^T = S dO^T
      umma_bf16(tmem_base + 128, a_st, b_dut, i_mm, kk != 0);    // (S dU^T), negated below
      umma_bf16(tmem_base + 192, k_do, b_ut, i_km, kk != 0);     // dMq = dO U^T (rows 0..63)
    }
    umma_commit(mma_bar);
  }
  mbar_wait(tma_bar, 0, p.status, KS_TIMEOUT_FULL);
  // dGc = <S, dS'> while the MMAs run (both tiles share one layout, so no unswizzling)
  if (tid < 128) {
    float acc = 0.f;
    for (int idx = tid; idx < 2048; idx += 128) {
      float a[8], b[8];
      unpack8(reinterpret_cast<const uint4*>(smem + OFF_ST)[idx], a);
      unpack8(reinterpret_cast<const uint4*>(smem + OFF_DSP)[idx], b);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += a[e] * b[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) red[warp] = acc;
  }
  __syncthreads();
  if (tid == 0) p.dgc[static_cast<long long>(c) * G.H + h] = (red[0] + red[1]) + (red[2] + red[3]);
  mbar_wait(mma_bar, 0, p.status, KS_TIMEOUT_TMEM_FULL);
  tc_fence_after();
  if (tid < 128) {
    const long long prow = ((static_cast<long long>(c) * G.NP + pr) * 128 + tid) * 128 + hh * 64;
    float r[64];
    tmem_row64(lane_addr, r);
    store_row64(p.dKdTp + prow, r);
    tmem_row64(lane_addr + 64, r);
    store_row64(p.dQgTp + prow, r);
    tmem_row64(lane_addr + 128, r);
#pragma unroll
    for (int e = 0; e < 64; ++e) r[e] = -r[e];
    store_row64(p.dWTp + prow, r);
    tmem_row64(lane_addr + 192, r);
    if (tid < 64)
      store_row64(p.dMQ + ((static_cast<long long>(c) * G.NP + pr) * 128 + hh * 64 + tid) * 64, r);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ============================================================================ backward of the chunk-local algebra
struct BwdPrepParams {
  const float* beta; const int* sid; const float* gam; const float* gc; const float* dgc;
  const __nv_bfloat16 *dKdTp, *dQgTp, *dMQ;
  __nv_bfloat16 *dq, *dk, *dv;     // dq, dk: [T, NP, D] (summed over pairs by the caller); dv [T, H, D]
  float *dbeta, *dg;               // [T, H]
  Geo geo; float scale; int* status;
};
namespace bprep {
constexpr int OFF_KQ = 0, OFF_TMT = 32768, OFF_V = 49152, OFF_DWT = 81920, OFF_DUT = 114688;
constexpr int OFF_XW = 147456, OFF_XU = 163840;
// after the first group of MMAs the range [OFF_V, OFF_XU + 16384) is reused:
constexpr int OFF_KKF = 49152, OFF_QKF = OFF_KKF + 16640;          // fp32 [64][65] each
constexpr int OFF_DTM = 82944, OFF_XOP = OFF_DTM + 16384;          // operands
constexpr int OFF_SYM = OFF_XOP + 16384, OFF_DQK = OFF_SYM + 8192;
constexpr int OFF_KKA = OFF_DQK + 8192, OFF_QKA = OFF_KKA + 16640;  // fp32 accumulators over heads
constexpr int OFF_RED = OFF_QKA + 16640;                           // 165376, [128][65] fp32
constexpr int OFF_MISC = OFF_RED + 33280;                          // 198656
constexpr int OFF_BAR = OFF_MISC + 8192;
constexpr int SMEM = OFF_BAR + 64 + 1024;
static_assert(OFF_KKF >= OFF_TMT + 16384, "scratch overlaps a tile that stays live");
static_assert(SMEM <= 232448, "exceeds the shared memory of one CTA");
}

__global__ void __launch_bounds__(THREADS, 1)
dn_bwd_prep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDWT,
                   const __grid_constant__ CUtensorMap tmDUT, const __grid_constant__ CUtensorMap tmTMT,
                   const __grid_constant__ CUtensorMap tmXW, const __grid_constant__ CUtensorMap tmXU,
                   const BwdPrepParams p) {
  using namespace bprep;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* KKf = reinterpret_cast<float*>(smem + OFF_KKF);
  float* QKf = reinterpret_cast<float*>(smem + OFF_QKF);
  float* KKa = reinterpret_cast<float*>(smem + OFF_KKA);
  float* QKa = reinterpret_cast<float*>(smem + OFF_QKA);
  float* red = reinterpret_cast<float*>(smem + OFF_RED);
  float* misc = reinterpret_cast<float*>(smem + OFF_MISC);
  float* gam_s = misc;            // [2][64] each from here on
  float* beta_s = misc + 128;
  float* gt_s = misc + 256;       // exp(gam) [continues the previous chunk's sequence]
  float* d_s = misc + 384;        // exp(gam_63 - gam) [same sequence as the chunk's end]
  float* cs1 = misc + 512;
  float* cs2 = misc + 640;
  float* colG = misc + 768;
  float* dotq = misc + 896;
  float* dotk = misc + 1024;
  float* dgam_s = misc + 1152;
  int* sid_s = reinterpret_cast<int*>(misc + 1280);     // [65]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* tma_bar = bars; uint64_t* mma_bar = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5;
  const Geo G = p.geo;
  const int c = blockIdx.x, pr = blockIdx.y;
  const int kh = pr / G.P, z = pr % G.P, h0 = kh * G.rep + 2 * z;
  const int nh = (2 * z + 1 < G.rep) ? 2 : 1;
  const int t0 = c * CH;
  const long long prow0 = (static_cast<long long>(c) * G.NP + pr) * 128;

  if (tid == 0) { mbar_init(tma_bar, 1); mbar_init(mma_bar, 1); mbar_fence_init(); }
  if (warp == 4) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  uint32_t mma_phase = 0;

  if (tid == CTRL) {
    mbar_expect_tx(tma_bar, 32768 + nh * 16384 + 32768 + 32768 + 3 * 16384);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + OFF_KQ + b * 16384, &tmK, tma_bar, kh * D + b * 64, t0);
      tma_load_2d(smem + OFF_KQ + b * 16384 + 64 * 128, &tmQ, tma_bar, kh * D + b * 64, t0);
      tma_load_2d(smem + OFF_DWT + b * 16384, &tmDWT, tma_bar, b * 64, static_cast<int>(prow0));
      tma_load_2d(smem + OFF_DUT + b * 16384, &tmDUT, tma_bar, b * 64, static_cast<int>(prow0));
    }
    for (int hh = 0; hh < nh; ++hh)
#pragma unroll
      for (int b = 0; b < 2; ++b)
        tma_load_2d(smem + OFF_V + hh * 16384 + b * 8192, &tmV, tma_bar, (h0 + hh) * D + b * 64, t0);
    tma_load_2d(smem + OFF_TMT, &tmTMT, tma_bar, 0, static_cast<int>(prow0));
    tma_load_2d(smem + OFF_XW, &tmXW, tma_bar, 0, static_cast<int>(prow0));
    tma_load_2d(smem + OFF_XU, &tmXU, tma_bar, 0, static_cast<int>(prow0));
  }
  if (tid < 65) sid_s[tid] = tid < 64 ? p.sid[t0 + tid] : (c > 0 ? p.sid[t0 - 1] : -1);
  if (tid < 128) {
    const int hh = tid >> 6, j = tid & 63, tok = t0 + j;
    const bool live = hh < nh && tok < G.T;
    gam_s[tid] = hh < nh ? p.gam[(static_cast<long long>(c) * G.H + h0 + hh) * 64 + j] : 0.f;
    beta_s[tid] = live ? p.beta[static_cast<long long>(tok) * G.H + h0 + hh] : 0.f;
  }
  __syncthreads();
  if (tid < 128) {
    const int hh = tid >> 6, j = tid & 63;
    gt_s[tid] = (sid_s[j] == sid_s[64]) ? __expf(gam_s[tid]) : 0.f;
    d_s[tid] = (sid_s[j] == sid_s[63]) ? __expf(gam_s[hh * 64 + 63] - gam_s[tid]) : 0.f;
  }

  // ---- first group of products
  if (tid == CTRL) {
    mbar_wait(tma_bar, 0, p.status, KS_TIMEOUT_FULL);
    tc_fence_after();
    const uint32_t skq = smem_u32(smem + OFF_KQ), sv = smem_u32(smem + OFF_V);
    const uint32_t sdw = smem_u32(smem + OFF_DWT), sdu = smem_u32(smem + OFF_DUT);
    const uint32_t sxw = smem_u32(smem + OFF_XW), sxu = smem_u32(smem + OFF_XU);
    constexpr uint32_t i_kk = umma_idesc_bf16(128, 64, false, false);
    constexpr uint32_t i_mk = umma_idesc_bf16(128, 64, true, false);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint64_t kq = umma_smem_desc(skq + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
      umma_bf16(tmem_base, kq, kq, i_kk, kk != 0);                                   // [K;Q] K^T
      umma_bf16(tmem_base + 64, umma_smem_desc(sdw + kk * 2048, 16384, 1024), kq, i_mk, kk != 0);   // P1 = dW K^T
      for (int h2 = 0; h2 < nh; ++h2)                                                // P2 = dU V^T
        umma_bf16(tmem_base + 128 + h2 * 64, umma_smem_desc(sdu + kk * 2048, 16384, 1024),
                  umma_smem_desc(sv + h2 * 16384 + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), i_mk,
                  kk != 0);
    }
    for (int hh = 0; hh < nh; ++hh) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        umma_bf16(tmem_base + 256, umma_smem_desc(sdw + hh * 16384 + kk * 32, 16, 1024),       // dK^T
                  umma_smem_desc(sxw + hh * 8192 + kk * 32, 16, 1024), i_kk, (hh | kk) != 0);
        umma_bf16(tmem_base + 320 + hh * 64, umma_smem_desc(sdu + hh * 16384 + kk * 32, 16, 1024),  // dV^T
                  umma_smem_desc(sxu + hh * 8192 + kk * 32, 16, 1024), i_kk, kk != 0);
      }
    }
    umma_commit(mma_bar);
  }
  mbar_wait(tma_bar, 0, p.status, KS_TIMEOUT_FULL);
  mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
  mma_phase ^= 1;
  tc_fence_after();

  // ---- K K^T and Q K^T to shared memory (both heads need both)
  if (tid < 128) {
    float row[64];
    tmem_row64(lane_addr, row);
    float* dst = (tid < 64 ? KKf : QKf) + (tid & 63) * 65;
#pragma unroll
    for (int i = 0; i < 64; ++i) dst[i] = row[i];
  }
  __syncthreads();

  const int hh_me = tid >> 6, t_me = tid & 63;
  const bool live = tid < 128 && hh_me < nh;
  // ---- dTm = (P1, P2) scaled per column; column sums of Tm o P1 and Tm o P2
  {
    float z2[64];
    if (tid < 128) {
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        float p1[32], p2[32], dtm[32];
        tmem_row32(lane_addr + 64 + half * 32, p1);
        tmem_row32(lane_addr + 128 + (hh_me < nh ? hh_me : 0) * 64 + half * 32, p2);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const int i = half * 32 + e;
          const float tm = bf16_at(smem + OFF_TMT + (hh_me * 64 + i) * 128 +
                                   (((t_me >> 3) ^ (i & 7)) << 4) + (t_me & 7) * 2);
          dtm[e] = live ? beta_s[hh_me * 64 + i] * (gt_s[hh_me * 64 + i] * p1[e] + p2[e]) : 0.f;
          red[tid * 65 + i] = live ? tm * p1[e] : 0.f;
          z2[i] = live ? tm * p2[e] : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(smem + OFF_DTM + sw_off(128, tid, half * 4 + q)) = pack8(dtm + q * 8);
      }
    }
    red_sums(red, cs1, true);
    if (tid < 128) {
#pragma unroll
      for (int i = 0; i < 64; ++i) red[tid * 65 + i] = z2[i];
    }
    red_sums(red, cs2, true);
  }
  publish();

  // ---- X = dTm Tm^T
  if (tid == CTRL) {
    constexpr uint32_t i_km = umma_idesc_bf16(128, 64, false, true);
    const uint32_t sd = smem_u32(smem + OFF_DTM), st = smem_u32(smem + OFF_TMT);
    for (int h2 = 0; h2 < nh; ++h2)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + 64 + h2 * 64, umma_smem_desc(sd + kk * 32, 16, 1024),
                  umma_smem_desc(st + h2 * 8192 + kk * 2048, 8192, 1024), i_km, kk != 0);
    umma_commit(mma_bar);
  }
  mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
  mma_phase ^= 1;
  tc_fence_after();
  if (live) {
    float x[64];
    tmem_row64(lane_addr + 64 + hh_me * 64, x);
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<uint4*>(smem + OFF_XOP + hh_me * 8192 + sw_off(64, t_me, q)) = pack8(x + q * 8);
  }
  publish();

  // ---- dA = -Tm^T X
  if (tid == CTRL) {
    constexpr uint32_t i_km = umma_idesc_bf16(128, 64, false, true);
    const uint32_t st = smem_u32(smem + OFF_TMT), sx = smem_u32(smem + OFF_XOP);
    for (int h2 = 0; h2 < nh; ++h2)
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma_bf16(tmem_base + (h2 == 0 ? 192 : 0), umma_smem_desc(st + kk * 32, 16, 1024),
                  umma_smem_desc(sx + h2 * 8192 + kk * 2048, 8192, 1024), i_km, kk != 0);
    umma_commit(mma_bar);
  }
  mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
  mma_phase ^= 1;
  tc_fence_after();

  // ---- gradients through A and Mq. The two heads of the pair take turns so that dKK and dQK
  // accumulate in one pair of shared-memory matrices.
  float rowG = 0.f, rowdb = 0.f;
  for (int pass = 0; pass < 2; ++pass) {
    if (tid < 128 && hh_me == pass) {
      float acc[64], dmq[64];
      tmem_row64(lane_addr + (hh_me == 0 ? 192 : 0), acc);
      if (live) load_row64(p.dMQ + (prow0 + tid) * 64, dmq);
      const int my = sid_s[t_me];
      const float gt = gam_s[tid], bt = beta_s[tid];
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        float dkk = 0.f, dqk = 0.f, w = 0.f;
        if (live) {
          const bool same = sid_s[i] == my;
          const float R = (i <= t_me && same) ? __expf(gt - gam_s[hh_me * 64 + i]) : 0.f;
          const float da = (i < t_me && same) ? -acc[i] : 0.f;
          const float kkv = KKf[t_me * 65 + i], qkv = QKf[t_me * 65 + i];
          rowdb += da * R * kkv;
          dkk = da * bt * R;
          dqk = dmq[i] * p.scale * R;
          w = dkk * kkv + dqk * qkv;               // dR o R
          rowG += w;
        }
        red[tid * 65 + i] = w;
        if (pass == 0) { KKa[t_me * 65 + i] = dkk; QKa[t_me * 65 + i] = dqk; }
        else if (live) { KKa[t_me * 65 + i] += dkk; QKa[t_me * 65 + i] += dqk; }
      }
    }
    __syncthreads();
  }
  red_sums(red, colG, true);
  if (tid < 128) {
    float o[64];
    if (tid < 64) {
#pragma unroll
      for (int i = 0; i < 64; ++i) o[i] = KKa[t_me * 65 + i] + KKa[i * 65 + t_me];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(smem + OFF_SYM + sw_off(64, t_me, q)) = pack8(o + q * 8);
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) o[i] = QKa[t_me * 65 + i];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(smem + OFF_DQK + sw_off(64, t_me, q)) = pack8(o + q * 8);
    }
  }
  publish();

  // ---- dK^T += K^T (dKK + dKK^T) + Q^T dQK;  dQ^T = K^T dQK^T
  if (tid == CTRL) {
    constexpr uint32_t i_mm = umma_idesc_bf16(128, 64, true, true);
    constexpr uint32_t i_mk = umma_idesc_bf16(128, 64, true, false);
    const uint32_t skq = smem_u32(smem + OFF_KQ), ssym = smem_u32(smem + OFF_SYM);
    const uint32_t sdqk = smem_u32(smem + OFF_DQK);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint64_t ak = umma_smem_desc(skq + kk * 2048, 16384, 1024);
      const uint64_t aq = umma_smem_desc(skq + 8192 + kk * 2048, 16384, 1024);
      umma_bf16(tmem_base + 256, ak, umma_smem_desc(ssym + kk * 2048, 8192, 1024), i_mm, 1);
      umma_bf16(tmem_base + 256, aq, umma_smem_desc(sdqk + kk * 2048, 8192, 1024), i_mm, 1);
      umma_bf16(tmem_base + 448, ak, umma_smem_desc(sdqk + kk * 32, 16, 1024), i_mk, kk != 0);
    }
    umma_commit(mma_bar);
  }
  mbar_wait(mma_bar, mma_phase, p.status, KS_TIMEOUT_TMEM_FULL);
  mma_phase ^= 1;
  tc_fence_after();

  // ---- feature-row epilogue: dk, dq, dv and the two per-token dot products
  const int lim = min(CH, G.T - t0);
  // element [i][tid] of K (which = 0) or Q (which = 1) in the stacked tile
  auto kq_at = [&](int which, int i) {
    return bf16_at(smem + OFF_KQ + (tid >> 6) * 16384 + (which * 64 + i) * 128 +
                   (((((tid & 63) >> 3)) ^ (i & 7)) << 4) + (tid & 7) * 2);
  };
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {          // 0: dk (with Kd), 1: dq (with Qg)
    float acc[64];
    if (tid < 128) tmem_row64(lane_addr + (which == 0 ? 256 : 448), acc);
    for (int hh = 0; hh < nh; ++hh) {
      if (tid < 128) {
        float a[64];
        load_row64((which == 0 ? p.dKdTp : p.dQgTp) + (prow0 + tid) * 128 + hh * 64, a);
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float f = which == 0 ? d_s[hh * 64 + i] : p.scale * gt_s[hh * 64 + i];
          acc[i] += f * a[i];
          red[tid * 65 + i] = a[i] * kq_at(which, i);     // dKd o K  /  dQg o Q
        }
      }
      red_sums(red, (which == 0 ? dotk : dotq) + hh * 64, false);
    }
    if (tid < 128) {
      __nv_bfloat16* dst = (which == 0 ? p.dk : p.dq) + (static_cast<long long>(t0) * G.NP + pr) * D + tid;
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (i < lim) dst[static_cast<long long>(i) * G.NP * D] = __float2bfloat16_rn(acc[i]);
    }
  }
  if (tid < 128) {
    for (int hh = 0; hh < nh; ++hh) {
      float r[64];
      tmem_row64(lane_addr + 320 + hh * 64, r);
      __nv_bfloat16* dvp = p.dv + (static_cast<long long>(t0) * G.H + h0 + hh) * D + tid;
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (i < lim) dvp[static_cast<long long>(i) * G.H * D] = __float2bfloat16_rn(r[i]);
    }
  }
  __syncthreads();

  // ---- per-token scalars: dgam -> dg (suffix sum), dbeta
  if (tid < 128) {
    float dgam = 0.f;
    if (live) {
      const int o = hh_me * 64;
      dgam = rowG - colG[tid] + beta_s[tid] * gt_s[tid] * cs1[tid] + p.scale * gt_s[tid] * dotq[tid] -
             d_s[tid] * dotk[tid];
      if (t_me == 63) {
        float tail = 0.f;
        for (int i = 0; i < 64; ++i) tail += d_s[o + i] * dotk[o + i];
        const long long hi = static_cast<long long>(c) * G.H + h0 + hh_me;
        dgam += tail + p.dgc[hi] * p.gc[hi];
      }
    }
    dgam_s[tid] = dgam;
  }
  __syncthreads();
  if (live && t_me < lim) {
    float s = 0.f;
    for (int i = t_me; i < 64; ++i) s += dgam_s[hh_me * 64 + i];
    const long long o = static_cast<long long>(t0 + t_me) * G.H + h0 + hh_me;
    p.dg[o] = s;
    p.dbeta[o] = rowdb + gt_s[tid] * cs1[tid] + cs2[tid];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

static Geo make_geo(int T, int H, int Hk) {
  Geo g;
  g.T = T; g.n = (T + CH - 1) / CH; g.H = H; g.Hk = Hk; g.rep = H / Hk;
  g.P = (g.rep + 1) / 2; g.NP = Hk * g.P;
  return g;
}

}  // namespace ss_dnc

// ---------------------------------------------------------------------------- launchers
// Shapes: q, k [T, Hk, 128] bf16; v, out, dout, dv [T, H, 128] bf16; beta, g, dbeta, dg [T, H] fp32;
// sid int32 [n*64]; n = ceil(T/64); P = ceil((H/Hk)/2); NP = Hk*P.
// Pair arrays [n, NP, 128, 128] bf16: WTp U0Tp UTp dUTp dWTp dKdTp dQgTp (columns = (head of pair, token)).
// Row-stacked arrays [n, NP, 128, 64] bf16: MQ TMT XW XU dMQ (rows = (head of pair, token)).
// Per-head arrays: QG KD [n, H, 64, 128]; ST dSpT [n, H, 128, 128] bf16; gam [n, H, 64], gc dgc [n, H] fp32.
extern "C" {
using namespace ss_dnc;

int ss_dn_seq_ids(const int* cu_seqlens, int nseq, int T, int* sid, void* stream) {
  if (T <= 0) return 0;
  const int Tp = (T + CH - 1) / CH * CH;
  dn_seq_ids_kernel<<<(Tp + 255) / 256, 256, 0, (cudaStream_t)stream>>>(cu_seqlens, nseq, T, Tp, sid);
  return (int)cudaGetLastError();
}

int ss_dn_prep(const void* q, const void* k, const void* v, const float* beta, const float* g,
               const int* sid, void* WTp, void* U0Tp, void* QG, void* KD, void* MQ, void* TMT, void* XW,
               void* XU, float* gam, float* gc, int T, int H, int Hk, float scale, int* status,
               void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk) return -2;
  const Geo geo = make_geo(T, H, Hk);
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = ss::make_tmap_bf16(&tq, q, T, (long long)Hk * D, (long long)Hk * D, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tk, k, T, (long long)Hk * D, (long long)Hk * D, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tv, v, T, (long long)H * D, (long long)H * D, 64))) return r;
  PrepParams p;
  p.beta = beta; p.g = g; p.sid = sid;
  p.WTp = (__nv_bfloat16*)WTp; p.U0Tp = (__nv_bfloat16*)U0Tp; p.QG = (__nv_bfloat16*)QG;
  p.KD = (__nv_bfloat16*)KD; p.MQ = (__nv_bfloat16*)MQ; p.TMT = (__nv_bfloat16*)TMT;
  p.XW = (__nv_bfloat16*)XW; p.XU = (__nv_bfloat16*)XU; p.gam = gam; p.gc = gc;
  p.geo = geo; p.scale = scale; p.status = status;
  static ss::SmemOptIn opt_in;
  if (int e = opt_in.ensure(dn_prep_kernel, prep::SMEM)) return e;
  dn_prep_kernel<<<dim3(geo.n, geo.NP), THREADS, prep::SMEM, (cudaStream_t)stream>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

int ss_dn_fwd(const void* WTp, const void* U0Tp, const void* QG, const void* KD, const void* MQ,
              const float* gc, void* out, void* ST, void* UTp, int T, int H, int Hk, int* status,
              void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk) return -2;
  const Geo geo = make_geo(T, H, Hk);
  const long long prow = (long long)geo.n * geo.NP * 128, hrow = (long long)geo.n * H * 64;
  CUtensorMap twt, tu0, tqg, tkd, tmq;
  int r;
  if ((r = ss::make_tmap_bf16(&twt, WTp, prow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tu0, U0Tp, prow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tqg, QG, hrow, 128, 128, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tkd, KD, hrow, 128, 128, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tmq, MQ, prow, 64, 64, 64))) return r;
  WalkParams p;
  p.out = (__nv_bfloat16*)out; p.ldo = (long long)H * D; p.gc = gc;
  p.ST = (__nv_bfloat16*)ST; p.UTp = (__nv_bfloat16*)UTp; p.dSpT = nullptr; p.dUTp = nullptr;
  p.geo = geo; p.status = status;
  static ss::SmemOptIn opt_in;
  if (int e = opt_in.ensure(dn_fwd_kernel, walk::SMEM)) return e;
  dn_fwd_kernel<<<H, THREADS, walk::SMEM, (cudaStream_t)stream>>>(twt, tu0, tqg, tkd, tmq, p);
  return (int)cudaGetLastError();
}

int ss_dn_bwd_state(const void* dout, const void* MQ, const void* KD, const void* QG, const void* WTp,
                    const float* gc, void* dSpT, void* dUTp, int T, int H, int Hk, int* status,
                    void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk) return -2;
  const Geo geo = make_geo(T, H, Hk);
  const long long prow = (long long)geo.n * geo.NP * 128, hrow = (long long)geo.n * H * 64;
  CUtensorMap tdo, tmq, tkd, tqg, twt;
  int r;
  if ((r = ss::make_tmap_bf16(&tdo, dout, T, (long long)H * D, (long long)H * D, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tmq, MQ, prow, 64, 64, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tkd, KD, hrow, 128, 128, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tqg, QG, hrow, 128, 128, 64))) return r;
  if ((r = ss::make_tmap_bf16(&twt, WTp, prow, 128, 128, 128))) return r;
  WalkParams p;
  p.out = nullptr; p.ldo = 0; p.gc = gc; p.ST = nullptr; p.UTp = nullptr;
  p.dSpT = (__nv_bfloat16*)dSpT; p.dUTp = (__nv_bfloat16*)dUTp; p.geo = geo; p.status = status;
  static ss::SmemOptIn opt_in;
  if (int e = opt_in.ensure(dn_bwd_state_kernel, walk::SMEM)) return e;
  dn_bwd_state_kernel<<<H, THREADS, walk::SMEM, (cudaStream_t)stream>>>(tdo, tmq, tkd, tqg, twt, p);
  return (int)cudaGetLastError();
}

int ss_dn_bwd_chunk(const void* dSpT, const void* ST, const void* UTp, const void* dUTp, const void* dout,
                    void* dKdTp, void* dQgTp, void* dWTp, void* dMQ, float* dgc, int T, int H, int Hk,
                    int* status, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk) return -2;
  const Geo geo = make_geo(T, H, Hk);
  const long long prow = (long long)geo.n * geo.NP * 128, srow = (long long)geo.n * H * 128;
  CUtensorMap tdsp, tst, tut, tdut, tdo;
  int r;
  if ((r = ss::make_tmap_bf16(&tdsp, dSpT, srow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tst, ST, srow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tut, UTp, prow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tdut, dUTp, prow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tdo, dout, T, (long long)H * D, (long long)H * D, 128))) return r;
  ChunkParams p;
  p.dKdTp = (__nv_bfloat16*)dKdTp; p.dQgTp = (__nv_bfloat16*)dQgTp; p.dWTp = (__nv_bfloat16*)dWTp;
  p.dMQ = (__nv_bfloat16*)dMQ; p.dgc = dgc; p.geo = geo; p.status = status;
  static ss::SmemOptIn opt_in;
  if (int e = opt_in.ensure(dn_bwd_chunk_kernel, chunkk::SMEM)) return e;
  dn_bwd_chunk_kernel<<<dim3(geo.n, H), THREADS, chunkk::SMEM, (cudaStream_t)stream>>>(tdsp, tst, tut, tdut,
                                                                                      tdo, p);
  return (int)cudaGetLastError();
}

int ss_dn_bwd_prep(const void* q, const void* k, const void* v, const float* beta, const int* sid,
                   const float* gam, const float* gc, const float* dgc, const void* dWTp,
                   const void* dUTp, const void* TMT, const void* XW, const void* XU, const void* dKdTp,
                   const void* dQgTp, const void* dMQ, void* dq, void* dk, void* dv, float* dbeta,
                   float* dg, int T, int H, int Hk, float scale, int* status, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk) return -2;
  const Geo geo = make_geo(T, H, Hk);
  const long long prow = (long long)geo.n * geo.NP * 128;
  CUtensorMap tq, tk, tv, tdw, tdu, ttm, txw, txu;
  int r;
  if ((r = ss::make_tmap_bf16(&tq, q, T, (long long)Hk * D, (long long)Hk * D, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tk, k, T, (long long)Hk * D, (long long)Hk * D, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tv, v, T, (long long)H * D, (long long)H * D, 64))) return r;
  if ((r = ss::make_tmap_bf16(&tdw, dWTp, prow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&tdu, dUTp, prow, 128, 128, 128))) return r;
  if ((r = ss::make_tmap_bf16(&ttm, TMT, prow, 64, 64, 128))) return r;
  if ((r = ss::make_tmap_bf16(&txw, XW, prow, 64, 64, 128))) return r;
  if ((r = ss::make_tmap_bf16(&txu, XU, prow, 64, 64, 128))) return r;
  BwdPrepParams p;
  p.beta = beta; p.sid = sid; p.gam = gam; p.gc = gc; p.dgc = dgc;
  p.dKdTp = (const __nv_bfloat16*)dKdTp; p.dQgTp = (const __nv_bfloat16*)dQgTp;
  p.dMQ = (const __nv_bfloat16*)dMQ; p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk;
  p.dv = (__nv_bfloat16*)dv; p.dbeta = dbeta; p.dg = dg; p.geo = geo; p.scale = scale; p.status = status;
  static ss::SmemOptIn opt_in;
  if (int e = opt_in.ensure(dn_bwd_prep_kernel, bprep::SMEM)) return e;
  dn_bwd_prep_kernel<<<dim3(geo.n, geo.NP), THREADS, bprep::SMEM, (cudaStream_t)stream>>>(
      tq, tk, tv, tdw, tdu, ttm, txw, txu, p);
  return (int)cudaGetLastError();
}
}  // extern "C"
