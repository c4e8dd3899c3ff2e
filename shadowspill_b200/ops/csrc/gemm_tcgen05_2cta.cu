// Persistent bf16 GEMM for sm_100a on CTA PAIRS: tcgen05.mma.cta_group::2.
//
// Why pairs: a 128x256x16 UMMA issued by one CTA reads 12 KB of operands from shared
// memory per 128 tensor cycles while TMA writes the same 12 KB in: 192 B/clk against a
// 128 B/clk shared-memory port, which caps a single-CTA kernel near two thirds of the
// tensor peak. In a pair each CTA holds its own 128 rows of A and only HALF of the 256
// B rows; the pair's MMA (M = 256) reads both halves, so each SM moves 8 KB in and 8 KB
// out per 128 cycles and the port stops being the limit.
//
// Cluster of 2 CTAs = one 256x256 output tile at a time, persistent over tiles.
//   CTA rank r owns output rows [256*mb + 128*r, +128) (accumulator in its own TMEM)
//   and stages A rows of that range plus B rows [256*nb + 128*r, +128).
//   warp 0      TMA producer of this CTA's operands; the byte counts of BOTH CTAs
//               complete on the LEADER's (rank 0) full barrier
//   warp 1      TMEM allocator; in the leader also the MMA issuer for the pair
//   warps 2..5  epilogue of this CTA's 128 rows
// The leader's tcgen05.commit multicasts "stage free" and "accumulator ready" to the
// same barrier in both CTAs; the peer's epilogue warps arrive remotely on the leader's
// "accumulator drained" barrier. Every wait is bounded (status word); both CTAs always
// reach the closing cluster barrier.
//
// GATHER form (ss_gemm2_gather_bf16): the weight all-gather of sharded data parallelism fused
// into the GEMM that first consumes the weight. B = W[N, K] lives as 1/world flat shards on the
// ranks of the job; four extra warps per CTA pull the shards (plain 16-byte loads from peer
// memory over NVLink, never TMA) into the LOCAL full-weight buffer in the order the tiles consume
// it, 32 KiB at a time, and count the finished pieces of every 256-row tile in a per-tile counter.
// The TMA producer waits (bounded) for a tile's counter before it loads that tile from local
// HBM, so each weight byte crosses NVLink once, the gather overlaps the MMAs tile by tile, and
// later GEMMs of the same weight read the buffer as usual. Tiles run n-major in this form, so the
// weight is needed progressively over the whole GEMM. This is what the reference does with an
// NCCL all-gather ahead of the GEMM (packages/engine/csrc/adapter/pytorch/storage/sharded.cpp:87).
//
// Same contract as ss_gemm_bf16 (operand layouts a_mn / b_mn, alpha, accumulate, bf16 or
// fp32 output); reference: shadowspill::accumulate_matmul_
// (packages/engine/src/shadowspill/pytorch/operations.py:15).
#include "sm100_ptx.cuh"

#include <cudaTypedefs.h>

namespace ss {

int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                   long long ld, int box_rows);
int make_tmap3_bf16(CUtensorMap* map, const void* base, long long experts, long long rows,
                    long long cols, long long ld, long long expert_pitch_elems, int box_rows);

namespace pair {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BN = 256;          // columns per pair tile; each CTA stages BN/2 rows of B
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = (BN / 2) * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;       // 32 KB per CTA per stage
constexpr int STAGES = 7;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 2 * BN;

struct Params {
  void* C;
  int M, N, K;
  long long ldc;
  int c_f32, accumulate;
  float alpha;
  int* status;
};

constexpr int GATHER_THREADS = 128;                  // warps 6..9 of the GATHER form
constexpr int PIECE_BYTES = 32768;
constexpr int MAX_RANKS = 16;

struct GatherArgs {
  const uint8_t* shard[MAX_RANKS];   // rank k's shard: flat elements [k*per, (k+1)*per) of W
  uint8_t* full;                     // the local full-weight buffer (= the GEMM's B)
  long long shard_bytes;             // per * 2
  long long total_bytes;             // N * K * 2
  int world, rank;
  unsigned int* counters;            // [tiles along N], zero at launch
  unsigned long long wait_ns;
};

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// ---- cluster / pair primitives
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// TMA loads of a CTA pair: data lands in THIS CTA's shared memory, the transaction bytes
// complete on `bar_cluster_addr`, which may be the barrier of the other CTA of the pair.
__device__ __forceinline__ void tma2_load_2d(void* smem_dst, const CUtensorMap* m,
                                             uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x),
      "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* smem_dst, const CUtensorMap* m,
                                             uint32_t bar_cluster_addr, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x),
      "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once every
// MMA issued so far by this thread has retired.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

template <bool GATHER>
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& mb, int& nb) {
  if (GATHER) {            // every row block of one column tile, then the next column tile
    mb = t % num_m;
    nb = t / num_m;
    return;
  }
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * num_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, num_m - first_m);
  const int r = t - g * per_group;
  mb = first_m + (r % gm);
  nb = r / gm;
}

template <bool A_MN, bool B_MN, bool GATHER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATHER ? THREADS + GATHER_THREADS : THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const Params p, const GatherArgs ga) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                    // used in the leader only
  uint64_t* empty = bars + STAGES;          // per CTA, signalled by the leader's commit
  uint64_t* tfull = bars + 2 * STAGES;      // per CTA, signalled by the leader's commit
  uint64_t* tempty = tfull + 2;             // leader only: 8 arrivals (4 warps x 2 CTAs)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers exist before anything is signalled remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        int mb, nb;
        tile_coords<GATHER>(t, num_m, num_n, mb, nb);
        const int m0 = mb * (2 * BM) + static_cast<int>(rank) * BM;
        const int n0 = nb * BN + static_cast<int>(rank) * (BN / 2);
        if (GATHER) {
          // rows [nb*BN, nb*BN + BN) of W are local once every piece of the tile is counted
          const long long tile_bytes = static_cast<long long>(BN) * p.K * 2;
          const long long lo = static_cast<long long>(nb) * tile_bytes;
          const long long hi = min(ga.total_bytes, lo + tile_bytes);
          const unsigned int need = static_cast<unsigned int>((hi - lo + PIECE_BYTES - 1) / PIECE_BYTES);
          const uint64_t t0 = globaltimer_ns();
          for (uint32_t it = 0; ld_acquire_gpu(&ga.counters[nb]) < need; ++it) {
            if ((it & 0x3f) == 0x3f) {
              if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) { ok = false; break; }
              if (globaltimer_ns() - t0 > ga.wait_ns) { report(p.status, KS_TIMEOUT_PEER); ok = false; break; }
            }
          }
          if (!ok) break;
          fence_proxy_async_global();      // the pieces were written by ordinary stores; TMA reads them
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, p.status, KS_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t fbar = map_to_rank(smem_u32(&full[stage]), 0);
          if (leader) mbar_expect_tx(&full[stage], 2 * STAGE_BYTES);
          if (!A_MN) {
            tma2_load_2d(sa, &tmA, fbar, kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma2_load_2d(sa + j * (BK * 128), &tmA, fbar, m0 + j * 64, kb * BK);
          }
          if (!B_MN) {
            tma2_load_3d(sb, &tmB, fbar, kb * BK, n0, 0);
          } else {
#pragma unroll
            for (int j = 0; j < (BN / 2) / 64; ++j)
              tma2_load_3d(sb + j * (BK * 128), &tmB, fbar, n0 + j * 64, kb * BK, 0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair_id; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, p.status, KS_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, KS_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? umma_smem_desc(sa + kk * (UMMA_K * 128), BK * 128, 1024)
                                        : umma_smem_desc(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(sb + kk * (UMMA_K * 128), BK * 128, 1024)
                                        : umma_smem_desc(sb + kk * (UMMA_K * 2), 16, 1024);
            umma2_bf16(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma2_commit_both(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit_both(&tfull[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair_id; t < num_tiles; t += num_pairs) {
      int mb, nb;
      tile_coords<GATHER>(t, num_m, num_n, mb, nb);
      if (!mbar_wait(&tfull[acc], acc_phase, p.status, KS_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = mb * (2 * BM) + static_cast<int>(rank) * BM + q * 32 + lane;
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c * 32;
        if (row < p.M && col0 < p.N) {
          const int ncols = min(32, p.N - col0);
          if (p.c_f32) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            for (int j = 0; j < ncols; j += 4) {
              float4 v = make_float4(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha,
                                     __uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha);
              if (p.accumulate) {
                const float4 o = *reinterpret_cast<const float4*>(dst + j);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              *reinterpret_cast<float4*>(dst + j) = v;
            }
          } else {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
            for (int j = 0; j < ncols; j += 8) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]) * p.alpha;
              if (p.accumulate) {
                const uint4 o = *reinterpret_cast<const uint4*>(dst + j);
                const float2 o0 = unpack_bf16(o.x), o1 = unpack_bf16(o.y), o2 = unpack_bf16(o.z),
                             o3 = unpack_bf16(o.w);
                f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
              }
              uint4 v;
              v.x = pack_bf16(f[0], f[1]);
              v.y = pack_bf16(f[2], f[3]);
              v.z = pack_bf16(f[4], f[5]);
              v.w = pack_bf16(f[6], f[7]);
              *reinterpret_cast<uint4*>(dst + j) = v;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&tempty[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  else if (GATHER) {
    // ------------------------------------------------------------ gather warps (both CTAs)
    // Piece i of the flat weight goes to CTA i mod gridDim.x; a CTA's pieces come in increasing
    // order, so the tiles fill in the order the GEMM consumes them.
    const int gt = threadIdx.x - THREADS;
    const long long n_pieces = (ga.total_bytes + PIECE_BYTES - 1) / PIECE_BYTES;
    const long long tile_bytes = static_cast<long long>(BN) * p.K * 2;
    for (long long piece = blockIdx.x; piece < n_pieces; piece += gridDim.x) {
      const long long base = piece * PIECE_BYTES;
      const long long end = min(ga.total_bytes, base + PIECE_BYTES);
#pragma unroll 4
      for (long long off = base + gt * 16; off < end; off += GATHER_THREADS * 16) {
        const int k = static_cast<int>(off / ga.shard_bytes);
        const uint4 v = *reinterpret_cast<const uint4*>(ga.shard[k] + (off - k * ga.shard_bytes));
        *reinterpret_cast<uint4*>(ga.full + off) = v;
      }
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (gt == 0) {
        fence_proxy_async_global();
        red_release_gpu_add(&ga.counters[base / tile_bytes], 1u);
      }
    }
  }

  // Neither CTA may leave while the other can still read its shared memory (the pair's
  // MMA reads both) or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int num_sms,
                  cudaStream_t stream) {
  static SmemOptIn opt_in;
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, false>;
  if (int e = opt_in.ensure(kern, SMEM)) return e;
  const long long tiles = static_cast<long long>((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  long long pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<static_cast<int>(2 * pairs), THREADS, SMEM, stream>>>(ta, tb, p, GatherArgs{});
  return static_cast<int>(cudaGetLastError());
}

static int launch_gather(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, const GatherArgs& ga,
                         int num_sms, cudaStream_t stream) {
  static SmemOptIn opt_in;
  auto kern = gemm2_bf16_kernel<false, false, true>;
  if (int e = opt_in.ensure(kern, SMEM)) return e;
  const long long tiles = static_cast<long long>((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + BN - 1) / BN);
  long long pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<static_cast<int>(2 * pairs), THREADS + GATHER_THREADS, SMEM, stream>>>(ta, tb, p, ga);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace pair
}  // namespace ss

extern "C" {

// Same arguments and return codes as ss_gemm_bf16 (without the tile-width hint).
int ss_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, int a_mn, int b_mn, int c_f32, int accumulate,
                  float alpha, int num_sms, int* status, void* stream) {
  using namespace ss;
  using namespace ss::pair;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return -2;
  if (num_sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_bf16(&ta, A, M, K, lda, BM);
  else       r = make_tmap_bf16(&ta, A, K, M, lda, BK);
  if (r) return r;
  if (!b_mn) r = make_tmap3_bf16(&tb, B, 1, N, K, ldb, static_cast<long long>(N) * ldb, BN / 2);
  else       r = make_tmap3_bf16(&tb, B, 1, K, N, ldb, static_cast<long long>(K) * ldb, BK);
  if (r) return r;
  Params p{C, M, N, K, ldc, c_f32, accumulate, alpha, status};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!a_mn && !b_mn) return launch<false, false>(ta, tb, p, num_sms, s);
  if (!a_mn && b_mn) return launch<false, true>(ta, tb, p, num_sms, s);
  if (a_mn && b_mn) return launch<true, true>(ta, tb, p, num_sms, s);
  return launch<true, false>(ta, tb, p, num_sms, s);
}

// C[M, N] (+)= alpha * A[M, K] @ W[N, K]^T where W is gathered into `full` by the same kernel.
// shard_ptrs[k]: rank k's shard (`per` elements, a multiple of 8; flat elements [k*per, (k+1)*per)
// of W, this rank's own included); counters: `ceil(N / 256)` zeroed words; wait_ns: budget of the
// wait for a tile (0 = 2 s). K must be a multiple of 64, M >= 256, ldb == K (W is contiguous).
int ss_gemm2_gather_bf16(const void* A, void* full, void* C, int M, int N, int K, long long lda,
                         long long ldc, int c_f32, int accumulate, float alpha,
                         void* const* shard_ptrs, long long per, int world, int rank,
                         unsigned int* counters, unsigned long long wait_ns, int num_sms, int* status,
                         void* stream) {
  using namespace ss;
  using namespace ss::pair;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || (per % 8) || per <= 0) return -2;
  if ((K % 64) || M < 2 * BM || (lda % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(full) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || counters == nullptr ||
      per * world < static_cast<long long>(N) * K)
    return -2;
  if (num_sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int r;
  if ((r = make_tmap_bf16(&ta, A, M, K, lda, BM))) return r;
  if ((r = make_tmap3_bf16(&tb, full, 1, N, K, K, static_cast<long long>(N) * K, BN / 2))) return r;
  Params p{C, M, N, K, ldc, c_f32, accumulate, alpha, status};
  GatherArgs ga{};
  for (int k = 0; k < world; ++k) {
    if (reinterpret_cast<uintptr_t>(shard_ptrs[k]) & 15) return -2;
    ga.shard[k] = static_cast<const uint8_t*>(shard_ptrs[k]);
  }
  ga.full = static_cast<uint8_t*>(full);
  ga.shard_bytes = per * 2;
  ga.total_bytes = static_cast<long long>(N) * K * 2;
  ga.world = world; ga.rank = rank; ga.counters = counters;
  ga.wait_ns = wait_ns ? wait_ns : 2000000000ull;
  return launch_gather(ta, tb, p, ga, num_sms, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
