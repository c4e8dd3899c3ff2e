// Packed variable-length causal GQA attention, forward, for sm_100a.
//
// One CTA per (128-query tile of one sequence, query head). K/V tiles stream
// through a two-stage TMA ring; S = Q K^T and O += P V run on tcgen05 with S
// double-buffered and O resident in TMEM; four softmax warps own one query row
// per thread (online softmax in the exp2 domain, lazy rescaling of O), write P
// as a 128B-swizzled K-major operand into shared memory, and at the end
// normalise O and store it with the log-sum-exp.
//
//   warps 0..3  softmax / correction / epilogue  (TMEM lanes 32w..32w+31)
//   warp  4     TMA producer
//   warp  5     MMA issuer + TMEM allocator
//
// Semantics: the reference's packed attention contract
// (packages/workloads/src/shadowspill_workloads/models/shared/decoder.py:251):
// each [cu_seqlens[i], cu_seqlens[i+1]) is an independent causal sequence.
#include "sm100_ptx.cuh"

#include <cudaTypedefs.h>
#include <math.h>

namespace ss {

int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                   long long ld, int box_rows);  // gemm_tcgen05.cu

constexpr int ATT_BM = 128;
constexpr int ATT_THREADS = 192;

template <int DH, int BKV>
struct AttnCfg {
  static constexpr int Q_BYTES = ATT_BM * DH * 2;
  static constexpr int KV_BYTES = BKV * DH * 2;        // one of K or V
  static constexpr int P_BYTES = ATT_BM * BKV * 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  // Two CTAs share an SM when they fit (dh <= 128 with 64-key tiles): while one CTA's softmax
  // warps work, the other CTA's MMAs keep the tensor pipe busy. Shared memory has no room for a
  // blanket alignment slack then; the kernel checks the aligned layout against what it was given.
  static constexpr int USED = OFF_BAR + 128;
  // an SM has 228 KiB of shared memory and keeps 1 KiB per resident CTA for itself
  static constexpr bool PAIR = 2 * (USED + 1024) <= 233472;
  static constexpr int SMEM = PAIR ? USED : USED + 1024;
  static constexpr int TMEM_S0 = 0;
  static constexpr int TMEM_O = 2 * BKV;
  static constexpr int TMEM_COLS = (2 * BKV + DH) <= 256 ? 256 : 512;
};

struct AttnParams {
  void* out;
  float* lse;
  const int* cu_seqlens;
  int nseq, T, Hq, Hkv;
  long long ldo;
  float scale_log2;   // softmax scale * log2(e)
  int* status;
};

// Maps a linear tile index to (sequence, tile within sequence); false if out of range.
__device__ __forceinline__ bool find_tile(const int* cu, int nseq, int tile, int& seq_start,
                                          int& seq_end, int& q0) {
  int acc = 0;
  for (int s = 0; s < nseq; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int nt = (e - b + ATT_BM - 1) / ATT_BM;
    if (tile < acc + nt) {
      seq_start = b;
      seq_end = e;
      q0 = b + (tile - acc) * ATT_BM;
      return true;
    }
    acc += nt;
  }
  return false;
}

template <int DH, int BKV>
__global__ void __launch_bounds__(ATT_THREADS, (AttnCfg<DH, BKV>::TMEM_COLS <= 256 &&
                                                AttnCfg<DH, BKV>::PAIR) ? 2 : 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using Cfg = AttnCfg<DH, BKV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  if (smem + Cfg::USED > smem_raw + Cfg::SMEM) {      // the launch gave an unaligned window
    if (threadIdx.x == 0) report(p.status, KS_BAD_ARGUMENT);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;          // 1
  uint64_t* kv_full = bars + 1;     // 2
  uint64_t* kv_empty = bars + 3;    // 2
  uint64_t* s_full = bars + 5;      // 2
  uint64_t* s_free = bars + 7;      // 2
  uint64_t* p_full = bars + 9;      // 1
  uint64_t* o_done = bars + 10;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);

  int seq_start, seq_end, q0;
  if (!find_tile(p.cu_seqlens, p.nseq, blockIdx.x, seq_start, seq_end, q0)) return;
  const int q_hi = min(q0 + ATT_BM, seq_end);           // exclusive
  const int n_kv = (q_hi - seq_start + BKV - 1) / BKV;  // tiles up to the diagonal

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DH / 64; ++c)
        tma_load_2d(smem + c * (ATT_BM * 128), &tmQ, q_full, head * DH + c * 64, q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (j >= 2 &&
            !mbar_wait(&kv_empty[st], ((j >> 1) - 1) & 1, p.status, KS_TIMEOUT_EMPTY))
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
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(ATT_BM, BKV, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(ATT_BM, DH, false, true);
      const uint32_t sq = smem_u32(smem);
      const uint32_t sp = smem_u32(smem + Cfg::OFF_P);
      bool ok = mbar_wait(q_full, 0, p.status, KS_TIMEOUT_FULL);
      auto issue_s = [&](int j) {
        const int b = j & 1;
        const uint32_t sk = smem_u32(smem + Cfg::OFF_K + b * Cfg::KV_BYTES);
        const uint32_t d = tmem_base + Cfg::TMEM_S0 + b * BKV;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint64_t ad = umma_smem_desc(sq + (kk >> 2) * (ATT_BM * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_smem_desc(sk + (kk >> 2) * (BKV * 128) + (kk & 3) * 32, 16, 1024);
          umma_bf16(d, ad, bd, idesc_s, kk != 0);
        }
        umma_commit(&s_full[b]);
      };
      if (ok) ok = mbar_wait(&kv_full[0], 0, p.status, KS_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int b = (j + 1) & 1;
          ok = mbar_wait(&kv_full[b], ((j + 1) >> 1) & 1, p.status, KS_TIMEOUT_FULL);
          if (ok && j + 1 >= 2)
            ok = mbar_wait(&s_free[b], (((j + 1) >> 1) - 1) & 1, p.status, KS_TIMEOUT_TMEM_EMPTY);
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = mbar_wait(p_full, j & 1, p.status, KS_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + Cfg::OFF_V + (j & 1) * Cfg::KV_BYTES);
        const uint32_t d = tmem_base + Cfg::TMEM_O;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t ad = umma_smem_desc(sp + (kk >> 2) * (ATT_BM * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = umma_smem_desc(sv + kk * (16 * 128), BKV * 128, 1024);
          umma_bf16(d, ad, bd, idesc_o, (j | kk) != 0);
        }
        umma_commit(&kv_empty[j & 1]);
        umma_commit(o_done);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int row = warp * 32 + lane;            // row within the tile == TMEM lane
    const int gq = q0 + row;                     // global query index
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    float m_used = -INFINITY;                    // reference max (log2 domain, scaled)
    float l = 0.f;
    bool ok = true;
    uint8_t* sp = smem + Cfg::OFF_P;
    for (int j = 0; j < n_kv; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int k0 = seq_start + j * BKV;
      const bool diag = (k0 + BKV - 1) > q0;     // some key of this tile may exceed some query
      const uint32_t s_addr = lane_addr + Cfg::TMEM_S0 + b * BKV;
      // one read of S: the row stays in registers for the maximum and for the exponentials
      float sv[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float s = __uint_as_float(r[e]) * p.scale_log2;
          if (diag && (k0 + c * 32 + e) > gq) s = -INFINITY;
          sv[c * 32 + e] = s;
        }
      }
      // S is in registers: the MMA warp may overwrite this buffer with the tile after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[b]);
      float m_t = -INFINITY;
#pragma unroll
      for (int e = 0; e < BKV; ++e) m_t = fmaxf(m_t, sv[e]);
      // lazy rescale: move the reference max only when it would grow by > 8 (2^8 headroom)
      const bool want = m_t > m_used + 8.f;
      const bool first = (j == 0);
      const bool warp_rescale = first || (__ballot_sync(0xffffffffu, want) != 0u);
      float alpha = 1.f;
      if (warp_rescale) {
        const float m_new = fmaxf(m_used, m_t);
        alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
      }
      // probabilities -> swizzled K-major P tile in shared memory. The previous P·V has to be
      // done with the tile first (o_done also covers the rescale of O below).
      if (j > 0) {
        if (!mbar_wait(o_done, (j - 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        if (warp_rescale) {
#pragma unroll 1
          for (int c = 0; c < DH / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(lane_addr + Cfg::TMEM_O + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_32x32(lane_addr + Cfg::TMEM_O + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = fast_exp2(sv[c * 32 + e] - m_used);
          const float p1 = fast_exp2(sv[c * 32 + e + 1] - m_used);
          lsum += p0 + p1;
          pk[e >> 1] = pack_bf16(p0, p1);
        }
        // columns [c*32, c*32+32) of row `row`: 64 bytes = four 16-byte chunks
        const int kcol = c * 32;
        uint8_t* box = sp + (kcol >> 6) * (ATT_BM * 128) + row * 128;
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          const int chunk = ((kcol & 63) >> 3) + q8;
          uint4 v = make_uint4(pk[q8 * 4], pk[q8 * 4 + 1], pk[q8 * 4 + 2], pk[q8 * 4 + 3]);
          *reinterpret_cast<uint4*>(box + ((chunk ^ (row & 7)) << 4)) = v;
        }
      }
      l += lsum;
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && n_kv > 0 && mbar_wait(o_done, (n_kv - 1) & 1, p.status, KS_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool valid = gq < q_hi;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) +
                            static_cast<long long>(gq) * p.ldo + head * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + Cfg::TMEM_O + c * 32, r);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + e) = v;
          }
        }
      }
      if (valid)
        p.lse[static_cast<long long>(head) * p.T + gq] =
            (m_used + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int DH, int BKV>
static int launch_fwd(const void* q, const void* k, const void* v, AttnParams p, long long ldq,
                      long long ldk, long long ldv, int max_tiles, cudaStream_t stream) {
  using Cfg = AttnCfg<DH, BKV>;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_bf16(&tq, q, p.T, static_cast<long long>(p.Hq) * DH, ldq, ATT_BM))) return r;
  if ((r = make_tmap_bf16(&tk, k, p.T, static_cast<long long>(p.Hkv) * DH, ldk, BKV))) return r;
  if ((r = make_tmap_bf16(&tv, v, p.T, static_cast<long long>(p.Hkv) * DH, ldv, BKV))) return r;
  auto kern = attn_fwd_kernel<DH, BKV>;
  static SmemOptIn opt_in;
  if (int e = opt_in.ensure(kern, Cfg::SMEM)) return e;
  dim3 grid(max_tiles, p.Hq);
  kern<<<grid, ATT_THREADS, Cfg::SMEM, stream>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ss

extern "C" int ss_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                           const int* cu_seqlens, int nseq, int T, int Hq, int Hkv, int dh,
                           long long ldq, long long ldk, long long ldv, long long ldo, float scale,
                           int* status, void* stream) {
  using namespace ss;
  if (T <= 0 || nseq <= 0) return 0;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || Hq % Hkv) return -2;
  AttnParams p;
  p.out = out; p.lse = lse; p.cu_seqlens = cu_seqlens; p.nseq = nseq; p.T = T; p.Hq = Hq;
  p.Hkv = Hkv; p.ldo = ldo; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  // every sequence adds at most one partial tile
  const int max_tiles = (T + ATT_BM - 1) / ATT_BM + nseq;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dh == 128) return launch_fwd<128, 64>(q, k, v, p, ldq, ldk, ldv, max_tiles, s);
  if (dh == 64) return launch_fwd<64, 64>(q, k, v, p, ldq, ldk, ldv, max_tiles, s);
  if (dh == 256) return launch_fwd<256, 64>(q, k, v, p, ldq, ldk, ldv, max_tiles, s);
  return -2;
}
