// Persistent bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory ->
// tcgen05.mma (accumulators in TMEM) -> tcgen05.ld epilogue.
//
//   C[M,N] (=|+=) op(A) * op(B)      fp32 accumulation, C in bf16 or fp32
//
// Operand storage (row-major, element pitch lda/ldb):
//   a_mn = 0 : A stored [M,K]  (contraction contiguous, "K-major")
//   a_mn = 1 : A stored [K,M]  (M contiguous, "MN-major")      -> C = A^T * ...
//   b_mn = 0 : B stored [N,K]  (K-major)                       -> C = A * B^T
//   b_mn = 1 : B stored [K,N]  (MN-major)                      -> C = A * B
// which covers forward (0,0), data-gradient (0,1) and weight-gradient (1,1)
// without materialising a transpose. `accumulate` folds the existing C into the
// result in the epilogue; this is the in-place weight-gradient accumulation the
// reference expresses as shadowspill::accumulate_matmul_
// (packages/engine/src/shadowspill/pytorch/operations.py:15).
//
// One CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + MMA issuer (one elected lane)
//   warps 2..5  epilogue; warp w owns TMEM lanes 32*(w%4)..+31
// Two 128x256 fp32 accumulators (2 x 256 TMEM columns) let the epilogue of tile
// i overlap the main loop of tile i+1.
#include "sm100_ptx.cuh"

#include <cudaTypedefs.h>
#include <stdio.h>

namespace ss {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  // scatter epilogue only: per epilogue warp a 32-row x 128-column bf16 staging tile, so that
  // rows leave the SM as whole 256-byte runs (peer stores want full lines, not 16-byte pieces)
  static constexpr int SCATTER_STAGE = 4 * 32 * 256;
  static constexpr int TMEM_COLS = 2 * BN;  // 512 or 256
};

// Grouped (mixture-of-experts) forms share the kernel:
//   mode 1  rows of A/C are grouped by expert in 128-row-aligned segments; the B
//           operand of a tile is expert tile_expert[m-block] of a [E, ., .] bank
//           (forward and data-gradient of an expert bank).
//   mode 2  one output matrix per expert, contracted over that expert's padded row
//           segment [expert_offset[e], expert_offset[e+1]) (weight gradient of a bank).
// With row_dst (mode 1, bf16 output) the epilogue writes output row r to the address
// row_dst[r] instead of C + r*ldc; 0 drops the row. Addresses may point into another
// GPU's memory (plain peer stores), which is how an expert bank's output rows go
// straight back to the ranks that own their tokens: the combine transfer of expert
// parallelism rides in this kernel's epilogue, overlapped with the next tile's MMAs.
struct GroupInfo {
  int mode;
  const int* tile_expert;     // mode 1: [ceil(M/128)], -1 = tile past the used rows
  const int* expert_offset;   // mode 2: [E+1], multiples of 128
  int n_experts;
  long long c_expert_stride;  // mode 2: elements between experts' outputs
  const long long* row_dst;   // mode 1, optional: per-row destination addresses (bytes)
};

struct GemmParams {
  void* C;
  int M, N, K;
  long long ldc;
  int c_f32;
  int accumulate;
  int a_mn, b_mn;
  int* status;
  float alpha;
  GroupInfo g;
};

struct TileWork {
  int mb, nb, expert, kb0, nkb;
  long long c_off;
  bool skip;
};

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& mb, int& nb) {
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * num_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, num_m - first_m);
  const int r = t - g * per_group;
  mb = first_m + (r % gm);
  nb = r / gm;
}

__device__ __forceinline__ TileWork decode_tile(const GemmParams& p, int t, int num_m, int num_n,
                                                int num_kb) {
  TileWork w;
  w.expert = 0; w.kb0 = 0; w.nkb = num_kb; w.c_off = 0; w.skip = false;
  if (p.g.mode == 2) {
    const int per = num_m * num_n;
    w.expert = t / per;
    tile_coords(t - w.expert * per, num_m, num_n, w.mb, w.nb);
    const int lo = p.g.expert_offset[w.expert], hi = p.g.expert_offset[w.expert + 1];
    w.kb0 = lo / BK;
    w.nkb = (hi - lo) / BK;
    w.c_off = static_cast<long long>(w.expert) * p.g.c_expert_stride;
  } else {
    tile_coords(t, num_m, num_n, w.mb, w.nb);
    if (p.g.mode == 1) {
      w.expert = p.g.tile_expert[w.mb];
      w.skip = w.expert < 0;
    }
  }
  return w;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle pattern repeats every 8 rows = 1024 B.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::STAGES;
  uint64_t* tfull = bars + 2 * Cfg::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n * (p.g.mode == 2 ? p.g.n_experts : 1);
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileWork w = decode_tile(p, t, num_m, num_n, num_kb);
        if (w.skip) continue;
        const int mb = w.mb, nb = w.nb;
        for (int kr = 0; kr < w.nkb; ++kr) {
          const int kb = w.kb0 + kr;
          if (!mbar_wait(&empty[stage], phase ^ 1, p.status, KS_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sa, &tmA, &full[stage], kb * BK, mb * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmA, &full[stage], mb * BM + j * 64, kb * BK);
          }
          // B is always described by a 3-D map [expert, rows, cols]; plain GEMMs have one expert
          const int bz = p.g.mode == 1 ? w.expert : 0;
          if (!B_MN) {
            tma_load_3d(sb, &tmB, &full[stage], kb * BK, nb * BN, bz);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (BK * 128), &tmB, &full[stage], nb * BN + j * 64, kb * BK, bz);
          }
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileWork w = decode_tile(p, t, num_m, num_n, num_kb);
        if (w.skip || w.nkb == 0) continue;
        if (!mbar_wait(&tempty[acc], acc_phase ^ 1, p.status, KS_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < w.nkb; ++kb) {
          if (!mbar_wait(&full[stage], phase, p.status, KS_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? umma_smem_desc(sa + kk * (UMMA_K * 128), BK * 128, 1024)
                                        : umma_smem_desc(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc(sb + kk * (UMMA_K * 128), BK * 128, 1024)
                                        : umma_smem_desc(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // stage reusable once these MMAs retire
          if (++stage == Cfg::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const TileWork w = decode_tile(p, t, num_m, num_n, num_kb);
      if (w.skip) continue;
      const int mb = w.mb, nb = w.nb;
      if (w.nkb == 0) {
        // an expert without rows: its gradient tile is zero (nothing to add when accumulating)
        if (!p.accumulate) {
          const int zr = mb * BM + q * 32 + lane;
          for (int c = nb * BN; zr < p.M && c < min(p.N, (nb + 1) * BN); c += 8) {
            if (p.c_f32) {
              float* d = reinterpret_cast<float*>(p.C) + w.c_off + static_cast<long long>(zr) * p.ldc + c;
              *reinterpret_cast<float4*>(d) = make_float4(0, 0, 0, 0);
              *reinterpret_cast<float4*>(d + 4) = make_float4(0, 0, 0, 0);
            } else {
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + w.c_off +
                                        static_cast<long long>(zr) * p.ldc + c) = make_uint4(0, 0, 0, 0);
            }
          }
        }
        continue;
      }
      if (!mbar_wait(&tfull[acc], acc_phase, p.status, KS_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = mb * BM + q * 32 + lane;
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      if (p.g.row_dst != nullptr) {
        // Scatter epilogue. Each thread owns one accumulator row; the rows are transposed
        // through an XOR-swizzled staging tile so that 16 lanes store one row's 256
        // contiguous bytes at its destination address.
        uint8_t* stg = smem + Cfg::STAGES * Cfg::STAGE_BYTES + 256 + q * (32 * 256);
        const long long my_dst = (row < p.M) ? p.g.row_dst[row] : 0;
#pragma unroll 1
        for (int half = 0; half < BN / 128; ++half) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + half * 128 + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[8 * i + 0]) * p.alpha, __uint_as_float(r[8 * i + 1]) * p.alpha);
              v.y = pack_bf16(__uint_as_float(r[8 * i + 2]) * p.alpha, __uint_as_float(r[8 * i + 3]) * p.alpha);
              v.z = pack_bf16(__uint_as_float(r[8 * i + 4]) * p.alpha, __uint_as_float(r[8 * i + 5]) * p.alpha);
              v.w = pack_bf16(__uint_as_float(r[8 * i + 6]) * p.alpha, __uint_as_float(r[8 * i + 7]) * p.alpha);
              const int chunk = c * 4 + i;
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = v;
            }
          }
          __syncwarp();
#pragma unroll 1
          for (int rr = 0; rr < 16; ++rr) {
            const int srow = rr * 2 + (lane >> 4);
            const int chunk = lane & 15;
            const long long where = __shfl_sync(0xffffffffu, my_dst, srow);
            const int col = nb * BN + half * 128 + chunk * 8;
            if (where != 0 && col < p.N) {
              const uint4 v = *reinterpret_cast<const uint4*>(stg + srow * 256 + ((chunk ^ (srow & 15)) << 4));
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(where) + col) = v;
            }
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c * 32;
        if (row < p.M && col0 < p.N) {
          const int ncols = min(32, p.N - col0);
          if (p.c_f32) {
            float* dst = reinterpret_cast<float*>(p.C) + w.c_off + static_cast<long long>(row) * p.ldc + col0;
            for (int j = 0; j < ncols; j += 4) {
              float4 v = make_float4(__uint_as_float(r[j]) * p.alpha,
                                     __uint_as_float(r[j + 1]) * p.alpha,
                                     __uint_as_float(r[j + 2]) * p.alpha,
                                     __uint_as_float(r[j + 3]) * p.alpha);
              if (p.accumulate) {
                const float4 o = *reinterpret_cast<const float4*>(dst + j);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
              }
              *reinterpret_cast<float4*>(dst + j) = v;
            }
          } else {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(p.C) + w.c_off + static_cast<long long>(row) * p.ldc + col0;
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
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// 2-D bf16 row-major [rows, cols] with element pitch ld; box = [box_rows, 64 cols], 128B swizzle.
// The tensor-map encoder is a driver entry point and needs this thread to have a
// current context. Framework worker threads (for example an autograd engine thread)
// may not have touched the runtime yet, so bind the device that owns the operand.
static void bind_device_of(const void* ptr) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeDevice)
    cudaSetDevice(attr.device);
  else
    cudaGetLastError();   // clear the sticky "invalid value" of a non-CUDA pointer
}

int make_tmap_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                   long long ld, int box_rows) {
  bind_device_of(base);
  auto fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

// 3-D bf16 [experts, rows, cols] with row pitch ld and expert pitch `expert_rows * ld`.
int make_tmap3_bf16(CUtensorMap* map, const void* base, long long experts, long long rows,
                    long long cols, long long ld, long long expert_pitch_elems, int box_rows) {
  bind_device_of(base);
  auto fn = encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(experts)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2,
                           static_cast<cuuint64_t>(expert_pitch_elems) * 2};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int num_sms,
                  cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static SmemOptIn opt_in;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (int e = opt_in.ensure(kern, Cfg::SMEM + Cfg::SCATTER_STAGE)) return e;
  const int smem_bytes = Cfg::SMEM + (p.g.row_dst != nullptr ? Cfg::SCATTER_STAGE : 0);
  const long long tiles = static_cast<long long>((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) *
                          (p.g.mode == 2 ? p.g.n_experts : 1);
  const int grid = tiles < num_sms ? static_cast<int>(tiles) : num_sms;
  kern<<<grid, GEMM_THREADS, smem_bytes, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

static int dispatch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int bn,
                    int num_sms, cudaStream_t s) {
  const bool a_mn = p.a_mn, b_mn = p.b_mn;
#define SS_DISPATCH(BN_)                                                              \
  do {                                                                                \
    if (!a_mn && !b_mn) return launch<BN_, false, false>(ta, tb, p, num_sms, s);      \
    if (!a_mn && b_mn) return launch<BN_, false, true>(ta, tb, p, num_sms, s);        \
    if (a_mn && b_mn) return launch<BN_, true, true>(ta, tb, p, num_sms, s);          \
    return launch<BN_, true, false>(ta, tb, p, num_sms, s);                           \
  } while (0)
  if (bn == 256) SS_DISPATCH(256);
  SS_DISPATCH(128);
#undef SS_DISPATCH
}

static int sm_count() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

}  // namespace ss

extern "C" {

// Returns 0 on success, a CUDA/driver error code otherwise, -2 for bad arguments.
// `status` is an int32 in device (or mapped pinned) memory that receives a
// ss::KernelStatus if a bounded wait inside the kernel gave up; it may be null.
int ss_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int a_mn, int b_mn, int c_f32, int accumulate,
                 float alpha, int bn, int num_sms, int* status, void* stream) {
  using namespace ss;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return -2;
  if (bn != 128 && bn != 256) bn = (N <= 128) ? 128 : 256;
  if (num_sms <= 0) num_sms = sm_count();
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_bf16(&ta, A, M, K, lda, BM);
  else       r = make_tmap_bf16(&ta, A, K, M, lda, BK);
  if (r) return r;
  if (!b_mn) r = make_tmap3_bf16(&tb, B, 1, N, K, ldb, static_cast<long long>(N) * ldb, bn);
  else       r = make_tmap3_bf16(&tb, B, 1, K, N, ldb, static_cast<long long>(K) * ldb, BK);
  if (r) return r;
  GemmParams p{};
  p.C = C; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.c_f32 = c_f32; p.accumulate = accumulate;
  p.a_mn = a_mn; p.b_mn = b_mn; p.status = status; p.alpha = alpha;
  p.g.mode = 0;
  return dispatch(ta, tb, p, bn, num_sms, reinterpret_cast<cudaStream_t>(stream));
}

// Expert-bank GEMMs over token rows sorted by expert into 128-row-aligned segments.
//   mode 1, b_mn = 0: C[R,N]  = A[R,K] @ bank[e][N,K]^T     (forward through the bank)
//   mode 1, b_mn = 1: C[R,N]  = A[R,K] @ bank[e][K,N]        (data gradient)
//   mode 2          : C[e][M,N] (+)= A[rows_e, M]^T @ B[rows_e, N]   (weight gradient)
// R = padded row count; `tile_expert` (mode 1) and `expert_offset` (mode 2) are device arrays.
int ss_gemm_grouped_bf16(const void* A, const void* B, void* C, int mode, int rows, int M, int N,
                         int K, int n_experts, long long lda, long long ldb, long long ldc,
                         int b_mn, int c_f32, int accumulate, const int* tile_expert,
                         const int* expert_offset, int bn, int* status, void* stream) {
  using namespace ss;
  if (rows <= 0 || n_experts <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % (c_f32 ? 4 : 8)) || (N % 8) || (rows % BM)) return -2;
  if (bn != 128 && bn != 256) bn = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  GemmParams p{};
  int r;
  if (mode == 1) {
    if (tile_expert == nullptr) return -2;
    if ((r = make_tmap_bf16(&ta, A, rows, K, lda, BM))) return r;
    if (!b_mn) r = make_tmap3_bf16(&tb, B, n_experts, N, K, ldb, static_cast<long long>(N) * ldb, bn);
    else       r = make_tmap3_bf16(&tb, B, n_experts, K, N, ldb, static_cast<long long>(K) * ldb, BK);
    if (r) return r;
    p.M = rows; p.N = N; p.K = K; p.a_mn = 0; p.b_mn = b_mn;
  } else if (mode == 2) {
    if (expert_offset == nullptr) return -2;
    // A stored [rows, M] and B stored [rows, N]: both contraction-major over the sorted rows
    if ((r = make_tmap_bf16(&ta, A, rows, M, lda, BK))) return r;
    if ((r = make_tmap3_bf16(&tb, B, 1, rows, N, ldb, static_cast<long long>(rows) * ldb, BK))) return r;
    p.M = M; p.N = N; p.K = rows; p.a_mn = 1; p.b_mn = 1;
    p.g.c_expert_stride = static_cast<long long>(M) * ldc;
  } else {
    return -2;
  }
  p.C = C; p.ldc = ldc; p.c_f32 = c_f32; p.accumulate = accumulate; p.status = status; p.alpha = 1.f;
  p.g.mode = mode; p.g.tile_expert = tile_expert; p.g.expert_offset = expert_offset;
  p.g.n_experts = n_experts;
  return dispatch(ta, tb, p, bn, sm_count(), reinterpret_cast<cudaStream_t>(stream));
}

// Row-grouped expert GEMM whose output rows are scattered: row r of A x B[expert]^T
// (bf16) is written to the byte address row_dst[r] (16-byte aligned; 0 = dropped),
// which may lie in a peer GPU's mapped memory.
int ss_gemm_grouped_scatter_bf16(const void* A, const void* B, const long long* row_dst, int rows,
                                 int N, int K, int n_experts, long long lda, long long ldb, int b_mn,
                                 const int* tile_expert, int bn, int* status, void* stream) {
  using namespace ss;
  if (rows <= 0 || n_experts <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (rows % BM) || !tile_expert || !row_dst) return -2;
  if (bn != 128 && bn != 256) bn = (N <= 128) ? 128 : 256;
  CUtensorMap ta, tb;
  GemmParams p{};
  int r;
  if ((r = make_tmap_bf16(&ta, A, rows, K, lda, BM))) return r;
  if (!b_mn) r = make_tmap3_bf16(&tb, B, n_experts, N, K, ldb, static_cast<long long>(N) * ldb, bn);
  else       r = make_tmap3_bf16(&tb, B, n_experts, K, N, ldb, static_cast<long long>(K) * ldb, BK);
  if (r) return r;
  p.M = rows; p.N = N; p.K = K; p.a_mn = 0; p.b_mn = b_mn;
  p.C = nullptr; p.ldc = 0; p.c_f32 = 0; p.accumulate = 0; p.status = status; p.alpha = 1.f;
  p.g.mode = 1; p.g.tile_expert = tile_expert; p.g.n_experts = n_experts; p.g.row_dst = row_dst;
  return dispatch(ta, tb, p, bn, sm_count(), reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
