// Packed variable-length causal GQA attention, backward, for sm_100a.
//
// Two tcgen05 kernels, neither of which needs atomics:
//
//   dQ kernel   one CTA per (128-query tile, query head); streams K/V tiles.
//               S = Q K^T and dP = dO V^T land in TMEM, the softmax warps form
//               dS = P o (dP - delta) * scale as a swizzled smem operand, and
//               dQ += dS K accumulates in TMEM.
//   dKV kernel  one CTA per (128-key tile, KV head); streams the 64-query tiles
//               of every query head of the group. S^T = K Q^T and dP^T = V dO^T
//               (keys on TMEM lanes), P^T and dS^T go to shared memory, and
//               dV += P^T dO, dK += dS^T Q accumulate in TMEM across tiles and
//               across the heads of the GQA group.
//
// For head width 256 the dK and dV accumulators do not fit TMEM together with
// the score buffers, so the dKV kernel runs twice (dV only, then dK only).
// delta[h,t] = sum_d dO*O comes from a small preprocess kernel into caller
// scratch (fp32 [Hq, T]).
//
// warps 0..7 softmax: warp w owns TMEM lanes 32*(w%4)..+31 and the 32-column half w/4 of
// every score tile, so two warps per scheduler hide each other's TMEM-load and exp latency;
// warp 8 TMA producer, warp 9 MMA.
#include "sm100_ptx.cuh"

#include <cudaTypedefs.h>
#include <math.h>

namespace ss {

int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                   long long ld, int box_rows);

constexpr int BW_THREADS = 320;
constexpr int BW_TMA_WARP = 8, BW_MMA_WARP = 9;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnBwdParams {
  void* dq; void* dk; void* dv;
  const float* lse;      // [Hq, T] natural log
  const float* delta;    // [Hq, T]
  const int* cu_seqlens;
  int nseq, T, Hq, Hkv;
  long long ldq, ldk, ldv;   // row pitches of dq / dk / dv (elements)
  float scale;
  int* status;
};

__device__ __forceinline__ bool find_tile128(const int* cu, int nseq, int tile, int& seq_start,
                                             int& seq_end, int& r0) {
  int acc = 0;
  for (int s = 0; s < nseq; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int nt = (e - b + 127) / 128;
    if (tile < acc + nt) {
      seq_start = b; seq_end = e; r0 = b + (tile - acc) * 128;
      return true;
    }
    acc += nt;
  }
  return false;
}

// Writes 32 consecutive bf16 columns [kcol, kcol+32) of row `row` into a
// K-major 128B-swizzled tile whose 64-column boxes are `box_bytes` apart.
__device__ __forceinline__ void store_swizzled_32(uint8_t* tile, int box_bytes, int row, int kcol,
                                                  const uint32_t (&pk)[16]) {
  uint8_t* box = tile + (kcol >> 6) * box_bytes + row * 128;
#pragma unroll
  for (int q8 = 0; q8 < 4; ++q8) {
    const int chunk = ((kcol & 63) >> 3) + q8;
    uint4 v = make_uint4(pk[q8 * 4], pk[q8 * 4 + 1], pk[q8 * 4 + 2], pk[q8 * 4 + 3]);
    *reinterpret_cast<uint4*>(box + ((chunk ^ (row & 7)) << 4)) = v;
  }
}

__device__ __forceinline__ void named_barrier_softmax() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// ============================================================================ preprocess
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ out,
                                  const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                  int T, int Hq, int dh, long long ld_out, long long ld_dout) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T * Hq) return;
  const int t = warp / Hq, h = warp % Hq;
  const __nv_bfloat16* o = out + static_cast<long long>(t) * ld_out + h * dh;
  const __nv_bfloat16* d = dout + static_cast<long long>(t) * ld_dout + h * dh;
  float acc = 0.f;
  for (int c = lane * 2; c < dh; c += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + c));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d + c));
    acc += a.x * b.x + a.y * b.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[static_cast<long long>(h) * T + t] = acc;
}

// ============================================================================ dQ kernel
template <int DH, int BKV, int KVS>
struct DqCfg {
  static constexpr int Q_BYTES = 128 * DH * 2;
  static constexpr int KV_BYTES = BKV * DH * 2;
  static constexpr int DS_BYTES = 128 * BKV * 2;
  static constexpr int OFF_DO = Q_BYTES;
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + KVS * KV_BYTES;
  static constexpr int OFF_DS = OFF_V + KVS * KV_BYTES;
  static constexpr int OFF_BAR = OFF_DS + 2 * DS_BYTES;   // dS is double-buffered
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int TM_S = 0, TM_DP = 2 * BKV, TM_DQ = 4 * BKV;
  static_assert(TM_DQ + DH <= 512, "TMEM budget");
};

template <int DH, int BKV, int KVS>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const AttnBwdParams p) {
  using Cfg = DqCfg<DH, BKV, KVS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* qdo_full = bars;            // 1
  uint64_t* kv_full = bars + 1;         // 2
  uint64_t* kv_empty = bars + 3;        // 2
  uint64_t* sdp_full = bars + 5;        // 2
  uint64_t* sdp_free = bars + 7;        // 2
  uint64_t* ds_full = bars + 9;         // 2
  uint64_t* dq_done = bars + 11;        // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  int seq_start, seq_end, q0;
  if (!find_tile128(p.cu_seqlens, p.nseq, blockIdx.x, seq_start, seq_end, q0)) return;
  const int q_hi = min(q0 + 128, seq_end);
  const int n_kv = (q_hi - seq_start + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1);
      mbar_init(&sdp_full[i], 1); mbar_init(&sdp_free[i], 8);
      mbar_init(&ds_full[i], 8); mbar_init(&dq_done[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == BW_MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == BW_TMA_WARP) {
    if (elect_one()) {
      mbar_expect_tx(qdo_full, 2 * Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DH / 64; ++c) {
        tma_load_2d(smem + c * (128 * 128), &tmQ, qdo_full, head * DH + c * 64, q0);
        tma_load_2d(smem + Cfg::OFF_DO + c * (128 * 128), &tmDO, qdo_full, head * DH + c * 64, q0);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % KVS;
        if (j >= KVS && !mbar_wait(&kv_empty[st], ((j / KVS) - 1) & 1, p.status, KS_TIMEOUT_EMPTY))
          break;
        uint8_t* sk = smem + Cfg::OFF_K + st * Cfg::KV_BYTES;
        uint8_t* sv = smem + Cfg::OFF_V + st * Cfg::KV_BYTES;
        mbar_expect_tx(&kv_full[st], 2 * Cfg::KV_BYTES);
        const int k0 = seq_start + j * BKV;
#pragma unroll
        for (int c = 0; c < DH / 64; ++c) {
          tma_load_2d(sk + c * (BKV * 128), &tmK, &kv_full[st], kv_head * DH + c * 64, k0);
          tma_load_2d(sv + c * (BKV * 128), &tmV, &kv_full[st], kv_head * DH + c * 64, k0);
        }
      }
    }
  } else if (warp == BW_MMA_WARP) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BKV, false, false);
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, DH, false, true);
      const uint32_t sq = smem_u32(smem), sdo = smem_u32(smem + Cfg::OFF_DO);
      const uint32_t sds = smem_u32(smem + Cfg::OFF_DS);
      bool ok = mbar_wait(qdo_full, 0, p.status, KS_TIMEOUT_FULL);
      auto issue_sdp = [&](int j) {
        const int b = j & 1, st = j % KVS;
        const uint32_t sk = smem_u32(smem + Cfg::OFF_K + st * Cfg::KV_BYTES);
        const uint32_t sv = smem_u32(smem + Cfg::OFF_V + st * Cfg::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t ao = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          const uint32_t bo = (kk >> 2) * (BKV * 128) + (kk & 3) * 32;
          umma_bf16(tmem_base + Cfg::TM_S + b * BKV, umma_smem_desc(sq + ao, 16, 1024),
                    umma_smem_desc(sk + bo, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t ao = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          const uint32_t bo = (kk >> 2) * (BKV * 128) + (kk & 3) * 32;
          umma_bf16(tmem_base + Cfg::TM_DP + b * BKV, umma_smem_desc(sdo + ao, 16, 1024),
                    umma_smem_desc(sv + bo, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&sdp_full[b]);
      };
      auto prefetch_next = [&](int j) -> bool {   // issue S/dP of tile j+1
        const int jn = j + 1, b = jn & 1;
        if (!mbar_wait(&kv_full[jn % KVS], (jn / KVS) & 1, p.status, KS_TIMEOUT_FULL)) return false;
        if (jn >= 2 && !mbar_wait(&sdp_free[b], ((jn >> 1) - 1) & 1, p.status, KS_TIMEOUT_TMEM_EMPTY))
          return false;
        tc_fence_after();
        issue_sdp(jn);
        return true;
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, p.status, KS_TIMEOUT_FULL);
      if (ok) { tc_fence_after(); issue_sdp(0); }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (KVS >= 2 && j + 1 < n_kv) { ok = prefetch_next(j); if (!ok) break; }
        ok = mbar_wait(&ds_full[j & 1], (j >> 1) & 1, p.status, KS_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + Cfg::OFF_K + (j % KVS) * Cfg::KV_BYTES);
        const uint32_t sdsj = sds + (j & 1) * Cfg::DS_BYTES;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t ad = umma_smem_desc(sdsj + (kk >> 2) * (128 * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_smem_desc(sk + kk * (16 * 128), BKV * 128, 1024);
          umma_bf16(tmem_base + Cfg::TM_DQ, ad, bd, idesc_dq, (j | kk) != 0);
        }
        umma_commit(&kv_empty[j % KVS]);
        umma_commit(&dq_done[j & 1]);
        if (KVS < 2 && j + 1 < n_kv) { ok = prefetch_next(j); }
      }
    }
  } else {
    const int quarter = warp & 3, hsel = warp >> 2;
    const int row = quarter * 32 + lane;
    const int gq = q0 + row;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const long long li = static_cast<long long>(head) * p.T + min(gq, p.T - 1);
    const float lse2 = p.lse[li] * LOG2E;
    const float dl = p.delta[li];
    const float c2 = p.scale * LOG2E;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int b = j & 1;
      uint8_t* sds = smem + Cfg::OFF_DS + b * Cfg::DS_BYTES;
      if (!mbar_wait(&sdp_full[b], (j >> 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      // this dS buffer was last read by the dQ MMAs of tile j-2
      if (j > 1 && !mbar_wait(&dq_done[b], ((j >> 1) - 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = seq_start + j * BKV;
      const bool below_diagonal = k0 + BKV - 1 <= q0;   // every key of the tile is visible to every row
#pragma unroll 1
      for (int c = hsel; c < BKV / 32; c += 2) {
        uint32_t s[32], d[32];
        tmem_ld_32x32(lane_addr + Cfg::TM_S + b * BKV + c * 32, s);
        tmem_ld_32x32(lane_addr + Cfg::TM_DP + b * BKV + c * 32, d);
        tmem_ld_wait();
        uint32_t pk[16];
        if (below_diagonal) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(s[e]), c2, -lse2));
            const float p1 = fast_exp2(fmaf(__uint_as_float(s[e + 1]), c2, -lse2));
            pk[e >> 1] = pack_bf16(p0 * (__uint_as_float(d[e]) - dl),
                                   p1 * (__uint_as_float(d[e + 1]) - dl));
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float v[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int gk = k0 + c * 32 + e + u;
              const float pr = (gk > gq) ? 0.f : fast_exp2(fmaf(__uint_as_float(s[e + u]), c2, -lse2));
              v[u] = pr * (__uint_as_float(d[e + u]) - dl);   // the softmax scale is applied to dQ once
            }
            pk[e >> 1] = pack_bf16(v[0], v[1]);
          }
        }
        store_swizzled_32(sds, 128 * 128, row, c * 32, pk);
      }
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&sdp_free[b]); mbar_arrive(&ds_full[b]); }
    }
    if (ok && n_kv > 0 && mbar_wait(&dq_done[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, p.status,
                                    KS_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.dq) +
                            static_cast<long long>(gq) * p.ldq + head * DH;
#pragma unroll 1
      for (int c = hsel; c < DH / 32; c += 2) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + Cfg::TM_DQ + c * 32, r);
        tmem_ld_wait();
        if (gq < q_hi) {
          const float sc = p.scale;
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[e]) * sc, __uint_as_float(r[e + 1]) * sc);
            v.y = pack_bf16(__uint_as_float(r[e + 2]) * sc, __uint_as_float(r[e + 3]) * sc);
            v.z = pack_bf16(__uint_as_float(r[e + 4]) * sc, __uint_as_float(r[e + 5]) * sc);
            v.w = pack_bf16(__uint_as_float(r[e + 6]) * sc, __uint_as_float(r[e + 7]) * sc);
            *reinterpret_cast<uint4*>(orow + c * 32 + e) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BW_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ============================================================================ dKV kernel
enum { MODE_BOTH = 0, MODE_DV = 1, MODE_DK = 2 };

template <int DH, int QS, int MODE>
struct DkvCfg {
  static constexpr int BQ = 64;
  static constexpr bool NEED_DP = MODE != MODE_DV;
  static constexpr bool DO_DV = MODE != MODE_DK;
  static constexpr bool DO_DK = MODE != MODE_DV;
  static constexpr int K_BYTES = 128 * DH * 2;
  static constexpr int QT_BYTES = BQ * DH * 2;
  static constexpr int PT_BYTES = 128 * BQ * 2;
  static constexpr int OFF_V = K_BYTES;
  static constexpr int OFF_Q = OFF_V + (NEED_DP ? K_BYTES : 0);
  static constexpr int OFF_DO = OFF_Q + QS * QT_BYTES;
  static constexpr int OFF_PT = OFF_DO + QS * QT_BYTES;
  static constexpr int OFF_DST = OFF_PT + (DO_DV ? 2 * PT_BYTES : 0);   // P^T, dS^T double-buffered
  static constexpr int OFF_LSE = OFF_DST + (DO_DK ? 2 * PT_BYTES : 0);
  static constexpr int OFF_BAR = OFF_LSE + 2 * 2 * BQ * 4;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int TM_ST = 0, TM_DPT = 2 * BQ;
  static constexpr int TM_ACC0 = NEED_DP ? 4 * BQ : 2 * BQ;   // dK (or dV in MODE_DV)
  static constexpr int TM_ACC1 = TM_ACC0 + DH;                // dV in MODE_BOTH
  static_assert((MODE == MODE_BOTH ? TM_ACC1 + DH : TM_ACC0 + DH) <= 512, "TMEM budget");
};

template <int DH, int QS, int MODE>
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const AttnBwdParams p) {
  using Cfg = DkvCfg<DH, QS, MODE>;
  constexpr int BQ = Cfg::BQ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;             // 1
  uint64_t* q_full = bars + 1;          // 2
  uint64_t* q_empty = bars + 3;         // 2
  uint64_t* sp_full = bars + 5;         // 2
  uint64_t* sp_free = bars + 7;         // 2
  uint64_t* pds_full = bars + 9;        // 2
  uint64_t* acc_done = bars + 11;       // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  float* s_lse = reinterpret_cast<float*>(smem + Cfg::OFF_LSE);   // [2][2][BQ]: lse2, delta

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_head = blockIdx.y;
  const int rep = p.Hq / p.Hkv;
  int seq_start, seq_end, k0;
  if (!find_tile128(p.cu_seqlens, p.nseq, blockIdx.x, seq_start, seq_end, k0)) return;
  const int n_q = (seq_end - k0 + BQ - 1) / BQ;     // query tiles at or after the key tile
  const int n_it = rep * n_q;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1);
      mbar_init(&sp_full[i], 1); mbar_init(&sp_free[i], 8);
      mbar_init(&pds_full[i], 8); mbar_init(&acc_done[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == BW_MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == BW_TMA_WARP) {
    if (elect_one()) {
      mbar_expect_tx(kv_full, Cfg::NEED_DP ? 2 * Cfg::K_BYTES : Cfg::K_BYTES);
#pragma unroll
      for (int c = 0; c < DH / 64; ++c) {
        tma_load_2d(smem + c * (128 * 128), &tmK, kv_full, kv_head * DH + c * 64, k0);
        if (Cfg::NEED_DP)
          tma_load_2d(smem + Cfg::OFF_V + c * (128 * 128), &tmV, kv_full, kv_head * DH + c * 64, k0);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % QS;
        if (it >= QS && !mbar_wait(&q_empty[st], ((it / QS) - 1) & 1, p.status, KS_TIMEOUT_EMPTY))
          break;
        const int head = kv_head * rep + it / n_q;
        const int qt0 = k0 + (it % n_q) * BQ;
        uint8_t* sq = smem + Cfg::OFF_Q + st * Cfg::QT_BYTES;
        uint8_t* sdo = smem + Cfg::OFF_DO + st * Cfg::QT_BYTES;
        mbar_expect_tx(&q_full[st], 2 * Cfg::QT_BYTES);
#pragma unroll
        for (int c = 0; c < DH / 64; ++c) {
          tma_load_2d(sq + c * (BQ * 128), &tmQ, &q_full[st], head * DH + c * 64, qt0);
          tma_load_2d(sdo + c * (BQ * 128), &tmDO, &q_full[st], head * DH + c * 64, qt0);
        }
      }
    }
  } else if (warp == BW_MMA_WARP) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BQ, false, false);
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, DH, false, true);
      const uint32_t sk = smem_u32(smem), sv = smem_u32(smem + Cfg::OFF_V);
      const uint32_t spt = smem_u32(smem + Cfg::OFF_PT), sdst = smem_u32(smem + Cfg::OFF_DST);
      bool ok = mbar_wait(kv_full, 0, p.status, KS_TIMEOUT_FULL);
      auto issue_sp = [&](int it) {
        const int b = it & 1, st = it % QS;
        const uint32_t sq = smem_u32(smem + Cfg::OFF_Q + st * Cfg::QT_BYTES);
        const uint32_t sdo = smem_u32(smem + Cfg::OFF_DO + st * Cfg::QT_BYTES);
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t ao = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          const uint32_t bo = (kk >> 2) * (BQ * 128) + (kk & 3) * 32;
          umma_bf16(tmem_base + Cfg::TM_ST + b * BQ, umma_smem_desc(sk + ao, 16, 1024),
                    umma_smem_desc(sq + bo, 16, 1024), idesc_s, kk != 0);
        }
        if (Cfg::NEED_DP) {
#pragma unroll
          for (int kk = 0; kk < DH / 16; ++kk) {
            const uint32_t ao = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
            const uint32_t bo = (kk >> 2) * (BQ * 128) + (kk & 3) * 32;
            umma_bf16(tmem_base + Cfg::TM_DPT + b * BQ, umma_smem_desc(sv + ao, 16, 1024),
                      umma_smem_desc(sdo + bo, 16, 1024), idesc_s, kk != 0);
          }
        }
        umma_commit(&sp_full[b]);
      };
      auto prefetch_next = [&](int it) -> bool {
        const int n = it + 1, b = n & 1;
        if (!mbar_wait(&q_full[n % QS], (n / QS) & 1, p.status, KS_TIMEOUT_FULL)) return false;
        if (n >= 2 && !mbar_wait(&sp_free[b], ((n >> 1) - 1) & 1, p.status, KS_TIMEOUT_TMEM_EMPTY))
          return false;
        tc_fence_after();
        issue_sp(n);
        return true;
      };
      if (ok) ok = mbar_wait(&q_full[0], 0, p.status, KS_TIMEOUT_FULL);
      if (ok) { tc_fence_after(); issue_sp(0); }
      for (int it = 0; it < n_it && ok; ++it) {
        if (QS >= 2 && it + 1 < n_it) { ok = prefetch_next(it); if (!ok) break; }
        ok = mbar_wait(&pds_full[it & 1], (it >> 1) & 1, p.status, KS_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        const int st = it % QS;
        const uint32_t spt_i = spt + (it & 1) * Cfg::PT_BYTES, sdst_i = sdst + (it & 1) * Cfg::PT_BYTES;
        const uint32_t sq = smem_u32(smem + Cfg::OFF_Q + st * Cfg::QT_BYTES);
        const uint32_t sdo = smem_u32(smem + Cfg::OFF_DO + st * Cfg::QT_BYTES);
#pragma unroll
        for (int kk = 0; kk < BQ / 16; ++kk) {
          if (Cfg::DO_DV) {
            const uint32_t acc = tmem_base + (MODE == MODE_BOTH ? Cfg::TM_ACC1 : Cfg::TM_ACC0);
            umma_bf16(acc, umma_smem_desc(spt_i + kk * 32, 16, 1024),
                      umma_smem_desc(sdo + kk * (16 * 128), BQ * 128, 1024), idesc_acc,
                      (it | kk) != 0);
          }
          if (Cfg::DO_DK) {
            umma_bf16(tmem_base + Cfg::TM_ACC0, umma_smem_desc(sdst_i + kk * 32, 16, 1024),
                      umma_smem_desc(sq + kk * (16 * 128), BQ * 128, 1024), idesc_acc,
                      (it | kk) != 0);
          }
        }
        umma_commit(&q_empty[st]);
        umma_commit(&acc_done[it & 1]);
        if (QS < 2 && it + 1 < n_it) { ok = prefetch_next(it); }
      }
    }
  } else {
    const int quarter = warp & 3, hsel = warp >> 2;
    const int row = quarter * 32 + lane;     // key row within the tile
    const int gk = k0 + row;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float c2 = p.scale * LOG2E;
    bool ok = true;
    // log-sum-exp and delta of the tile's queries: threads 0..2*BQ-1 fetch one value each, one
    // iteration ahead, so that the global-memory latency is not on the path of every tile
    auto fetch_row_stat = [&](int it) -> float {
      if (threadIdx.x >= 2 * BQ || it >= n_it) return 0.f;
      const int head_i = kv_head * rep + it / n_q;
      const int col = threadIdx.x & (BQ - 1);
      const long long li = static_cast<long long>(head_i) * p.T + min(k0 + (it % n_q) * BQ + col, p.T - 1);
      return threadIdx.x < BQ ? p.lse[li] * LOG2E : p.delta[li];
    };
    float row_stat = fetch_row_stat(0);
    for (int it = 0; it < n_it; ++it) {
      const int b = it & 1;
      const int head = kv_head * rep + it / n_q;
      const int qt0 = k0 + (it % n_q) * BQ;
      float* sl = s_lse + b * (2 * BQ);
      if (threadIdx.x < 2 * BQ) sl[threadIdx.x] = row_stat;     // [0,BQ): lse, [BQ,2BQ): delta
      row_stat = fetch_row_stat(it + 1);
      named_barrier_softmax();
      if (!mbar_wait(&sp_full[b], (it >> 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      // the P^T / dS^T buffers of this parity were last read by the MMAs of iteration it-2
      if (it > 1 && !mbar_wait(&acc_done[b], ((it >> 1) - 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = hsel; c < BQ / 32; c += 2) {
        uint32_t s[32], d[32];
        tmem_ld_32x32(lane_addr + Cfg::TM_ST + b * BQ + c * 32, s);
        if (Cfg::NEED_DP) tmem_ld_32x32(lane_addr + Cfg::TM_DPT + b * BQ + c * 32, d);
        tmem_ld_wait();
        uint32_t pkp[16], pkd[16];
        // whole tile visible: every query of the tile is at or after every key, none past the end
        const bool all_valid = (qt0 >= k0 + 127) && (qt0 + BQ <= seq_end);
        if (all_valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int col = c * 32 + e;
            const float p0 = fast_exp2(fmaf(__uint_as_float(s[e]), c2, -sl[col]));
            const float p1 = fast_exp2(fmaf(__uint_as_float(s[e + 1]), c2, -sl[col + 1]));
            pkp[e >> 1] = pack_bf16(p0, p1);
            pkd[e >> 1] = Cfg::NEED_DP
                ? pack_bf16(p0 * (__uint_as_float(d[e]) - sl[BQ + col]),
                            p1 * (__uint_as_float(d[e + 1]) - sl[BQ + col + 1]))
                : 0u;
          }
        } else
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int col = c * 32 + e + u;
            const int gqc = qt0 + col;
            const bool valid = (gqc < seq_end) && (gk <= gqc);
            const float pr = valid ? fast_exp2(fmaf(__uint_as_float(s[e + u]), c2, -sl[col])) : 0.f;
            pv[u] = pr;
            dv[u] = Cfg::NEED_DP ? pr * (__uint_as_float(d[e + u]) - sl[BQ + col]) : 0.f;   // dK scaled once at the end
          }
          pkp[e >> 1] = pack_bf16(pv[0], pv[1]);
          pkd[e >> 1] = pack_bf16(dv[0], dv[1]);
        }
        if (Cfg::DO_DV) store_swizzled_32(smem + Cfg::OFF_PT + b * Cfg::PT_BYTES, 128 * 128, row, c * 32, pkp);
        if (Cfg::DO_DK) store_swizzled_32(smem + Cfg::OFF_DST + b * Cfg::PT_BYTES, 128 * 128, row, c * 32, pkd);
      }
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&sp_free[b]); mbar_arrive(&pds_full[b]); }
    }
    if (ok && n_it > 0 && mbar_wait(&acc_done[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, p.status,
                                    KS_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const bool valid = gk < seq_end;
      auto store_acc = [&](uint32_t tm_col, void* base, long long ld, float sc) {
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(base) +
                              static_cast<long long>(gk) * ld + kv_head * DH;
#pragma unroll 1
        for (int c = hsel; c < DH / 32; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + tm_col + c * 32, r);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[e]) * sc, __uint_as_float(r[e + 1]) * sc);
              v.y = pack_bf16(__uint_as_float(r[e + 2]) * sc, __uint_as_float(r[e + 3]) * sc);
              v.z = pack_bf16(__uint_as_float(r[e + 4]) * sc, __uint_as_float(r[e + 5]) * sc);
              v.w = pack_bf16(__uint_as_float(r[e + 6]) * sc, __uint_as_float(r[e + 7]) * sc);
              *reinterpret_cast<uint4*>(orow + c * 32 + e) = v;
            }
          }
        }
      };
      if (Cfg::DO_DK) store_acc(Cfg::TM_ACC0, p.dk, p.ldk, p.scale);
      if (Cfg::DO_DV) store_acc(MODE == MODE_BOTH ? Cfg::TM_ACC1 : Cfg::TM_ACC0, p.dv, p.ldv, 1.f);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == BW_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int DH, int BKV, int KVS>
static int launch_dq(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk,
                     const CUtensorMap& tv, const AttnBwdParams& p, int tiles, cudaStream_t s) {
  using Cfg = DqCfg<DH, BKV, KVS>;
  auto kern = attn_bwd_dq_kernel<DH, BKV, KVS>;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(kern, Cfg::SMEM)) return e;
  kern<<<dim3(tiles, p.Hq), BW_THREADS, Cfg::SMEM, s>>>(tq, tdo, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

template <int DH, int QS, int MODE>
static int launch_dkv(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tk,
                      const CUtensorMap& tv, const AttnBwdParams& p, int tiles, cudaStream_t s) {
  using Cfg = DkvCfg<DH, QS, MODE>;
  auto kern = attn_bwd_dkv_kernel<DH, QS, MODE>;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(kern, Cfg::SMEM)) return e;
  kern<<<dim3(tiles, p.Hkv), BW_THREADS, Cfg::SMEM, s>>>(tq, tdo, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ss

// delta_scratch: fp32 [Hq, T] caller-provided scratch.
// lddq / lddk / lddv: row pitches of the gradient buffers, which need not be those of q, k, v
// (a fused q/k/v projection read through views, gradients written to tensors of their own).
extern "C" int ss_attn_bwd_g(const void* q, const void* k, const void* v, const void* out,
                             const float* lse, const void* dout, void* dq, void* dk, void* dv,
                             const int* cu_seqlens, float* delta_scratch, int nseq, int T, int Hq,
                             int Hkv, int dh, long long ldq, long long ldk, long long ldv,
                             long long ldo, long long lddq, long long lddk, long long lddv,
                             float scale, int* status, void* stream) {
  using namespace ss;
  if (T <= 0 || nseq <= 0) return 0;
  if (delta_scratch == nullptr) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || Hq % Hkv) return -2;
  if ((lddq % 8) || (lddk % 8) || (lddv % 8)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  {
    const long long warps = static_cast<long long>(T) * Hq;
    const int blocks = static_cast<int>((warps * 32 + 255) / 256);
    attn_delta_kernel<<<blocks, 256, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout),
        delta_scratch, T, Hq, dh, static_cast<long long>(Hq) * dh, ldo);
  }
  AttnBwdParams p;
  p.dq = dq; p.dk = dk; p.dv = dv; p.lse = lse; p.delta = delta_scratch; p.cu_seqlens = cu_seqlens;
  p.nseq = nseq; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.ldq = lddq; p.ldk = lddk; p.ldv = lddv;
  p.scale = scale; p.status = status;
  const int tiles = (T + 127) / 128 + nseq;
  const long long qc = static_cast<long long>(Hq) * dh, kc = static_cast<long long>(Hkv) * dh;
  CUtensorMap tq128, tdo128, tk64, tv64, tq64, tdo64, tk128, tv128;
  int r;
  if ((r = make_tmap_bf16(&tq128, q, T, qc, ldq, 128))) return r;
  if ((r = make_tmap_bf16(&tdo128, dout, T, qc, ldo, 128))) return r;
  if ((r = make_tmap_bf16(&tk64, k, T, kc, ldk, 64))) return r;
  if ((r = make_tmap_bf16(&tv64, v, T, kc, ldv, 64))) return r;
  if ((r = make_tmap_bf16(&tq64, q, T, qc, ldq, 64))) return r;
  if ((r = make_tmap_bf16(&tdo64, dout, T, qc, ldo, 64))) return r;
  if ((r = make_tmap_bf16(&tk128, k, T, kc, ldk, 128))) return r;
  if ((r = make_tmap_bf16(&tv128, v, T, kc, ldv, 128))) return r;
  if (dh == 128) {
    if ((r = launch_dq<128, 64, 2>(tq128, tdo128, tk64, tv64, p, tiles, s))) return r;
    return launch_dkv<128, 2, MODE_BOTH>(tq64, tdo64, tk128, tv128, p, tiles, s);
  }
  if (dh == 64) {
    if ((r = launch_dq<64, 64, 2>(tq128, tdo128, tk64, tv64, p, tiles, s))) return r;
    return launch_dkv<64, 2, MODE_BOTH>(tq64, tdo64, tk128, tv128, p, tiles, s);
  }
  if (dh == 256) {
    if ((r = launch_dq<256, 64, 1>(tq128, tdo128, tk64, tv64, p, tiles, s))) return r;
    if ((r = launch_dkv<256, 2, MODE_DV>(tq64, tdo64, tk128, tv128, p, tiles, s))) return r;
    return launch_dkv<256, 1, MODE_DK>(tq64, tdo64, tk128, tv128, p, tiles, s);
  }
  return -2;
}

// delta_scratch: fp32 [Hq, T] caller-provided scratch. Gradients have the pitches of their operands.
extern "C" int ss_attn_bwd(const void* q, const void* k, const void* v, const void* out,
                           const float* lse, const void* dout, void* dq, void* dk, void* dv,
                           const int* cu_seqlens, float* delta_scratch, int nseq, int T, int Hq,
                           int Hkv, int dh, long long ldq, long long ldk, long long ldv,
                           long long ldo, float scale, int* status, void* stream) {
  return ss_attn_bwd_g(q, k, v, out, lse, dout, dq, dk, dv, cu_seqlens, delta_scratch, nseq, T, Hq, Hkv,
                       dh, ldq, ldk, ldv, ldo, ldq, ldk, ldv, scale, status, stream);
}

// ============================================================================ no-allocation entry
// See attention_noalloc.h. The scratch that ss_attn_bwd takes from its caller
// (delta, fp32 [Hq, T]) lives here in a fixed device array instead, so the call
// performs no allocation of any kind.
#include "attention_noalloc.h"

#include <mutex>

namespace ss {

// Every GPU that loads this library holds this array until the process exits.
static __device__ __align__(256) float g_attn_delta_scratch[SS_ATTN_NOALLOC_MAX_ELEMENTS];

constexpr int kMaxDevices = 64;
static float* g_scratch_address[kMaxDevices];   // device address of the array, per device
static std::mutex g_scratch_mutex;

// In host code `g_attn_delta_scratch` is only a stand-in symbol, not an address a
// kernel can use; the device address has to be asked for, once per device, with
// that device current.
static int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return SS_ATTN_NOALLOC_BAD_DEVICE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_attn_delta_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_address[dev] = ptr;
  }
  *out = g_scratch_address[dev];
  return 0;
}

}  // namespace ss

extern "C" long long ss_attn_bwd_noalloc_max_elements(void) { return SS_ATTN_NOALLOC_MAX_ELEMENTS; }

extern "C" int ss_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out,
                                   const float* lse, const void* dout, void* dq, void* dk, void* dv,
                                   const int* cu_seqlens, int nseq, int T, int Hq, int Hkv, int dh,
                                   long long ldq, long long ldk, long long ldv, long long ldo,
                                   float scale, int* status, void* stream) {
  if (T <= 0 || nseq <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0) return -2;          // the same answer ss_attn_bwd gives
  if (static_cast<long long>(Hq) * T > SS_ATTN_NOALLOC_MAX_ELEMENTS)
    return SS_ATTN_NOALLOC_TOO_LARGE;
  // The scratch array handed to the kernels is the CURRENT device's copy. If the operands
  // live on another GPU the kernels would run there (the tensor-map set-up binds the
  // operands' device) with this GPU's array: refuse instead.
  {
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess) return SS_ATTN_NOALLOC_BAD_DEVICE;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, dq) != cudaSuccess) {
      cudaGetLastError();
      return SS_ATTN_NOALLOC_BAD_DEVICE;
    }
    if (attr.type != cudaMemoryTypeDevice || attr.device != current)
      return SS_ATTN_NOALLOC_BAD_DEVICE;
  }
  float* scratch = nullptr;
  if (int rc = ss::scratch_for_current_device(&scratch)) return rc;
  return ss_attn_bwd(q, k, v, out, lse, dout, dq, dk, dv, cu_seqlens, scratch, nseq, T, Hq, Hkv,
                     dh, ldq, ldk, ldv, ldo, scale, status, stream);
}
