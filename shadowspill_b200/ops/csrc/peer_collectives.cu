// Data-parallel collectives over peer-mapped (symmetric) memory, issued from
// inside the kernels with plain P2P loads and stores across NVLink / NVSwitch.
//
//   ss_peer_barrier      every rank signals every peer's flag word and waits for
//                        all of theirs (bounded spin -> status word, never a hang)
//   ss_peer_allgather    pull all-gather: each rank copies every peer's owned
//                        slice of a tensor straight into its own full buffer
//   ss_rs_adamw          gradient reduce-scatter FUSED with the sharded AdamW
//                        update: for its owned slice, a rank loads the slice of
//                        every rank's gradient buffer over NVLink, sums in fp32,
//                        and applies AdamW with bf16 stochastic rounding to its
//                        parameter / moment shards in the same pass -- the summed
//                        gradient never exists in memory
//   ss_rs_accumulate     gradient reduce-scatter into a shard-sized fp32 sum that stays on
//                        this rank: a step that runs its microbatches in groups folds each
//                        group's gradient into it, and ss_rs_adamw_acc starts its own sum there
//   ss_peer_allreduce    one-shot all-reduce for small fp32 tensors (norm weights)
//
// These replace the NCCL calls the reference makes for sharded storage
// (packages/engine/csrc/adapter/pytorch/storage/sharded.cpp:87,94,118) and for its
// optimizer-step collective tasks (packages/engine/src/shadowspill/communication/task.py:22-71).
// No TMA is involved; peers are reached with ordinary ld/st.global.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace ss {

constexpr int MAX_RANKS = 16;
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;   // default budget of a peer wait: 2 s

struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Flag layout per rank: uint32 flags[MAX_RANKS]; flags[j] on rank r is written by rank j.
// `epoch` increases by one per barrier; a rank waits until every peer's word >= epoch.
// A wait that outlasts `wait_ns` writes KS_TIMEOUT_PEER (5) into the status word and returns.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, uint32_t epoch,
                                    unsigned long long wait_ns, int* status) {
  const int j = threadIdx.x;
  if (j >= world) return;
  __threadfence_system();
  uint32_t* theirs = reinterpret_cast<uint32_t*>(flags.p[j]) + rank;
  st_release_sys(theirs, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + j;
  const unsigned long long t0 = gtime();
  for (uint32_t it = 0;; ++it) {
    const uint32_t v = ld_acquire_sys(mine);
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if ((it & 0x3f) == 0x3f && gtime() - t0 > wait_ns) {
      if (status) atomicCAS(status, 0, 5);   // KS_TIMEOUT_PEER
      break;
    }
  }
}

// full[r] layout: the whole tensor of `numel` elements; slice k = [k*shard, min(numel,(k+1)*shard)).
// shards.p[k] points at rank k's owned slice (shard elements). 16-byte vectors.
__global__ void peer_allgather_kernel(PeerPtrs shards, uint8_t* __restrict__ full,
                                      long long shard_bytes, long long total_bytes, int rank,
                                      int world) {
  const long long vec_per_shard = shard_bytes >> 4;
  const long long nvec = vec_per_shard * world;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // four loads in flight per thread: the grid is kept small (it shares the SMs with the compute
  // stream's kernels), so the bytes in flight have to come from each thread
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec;
       i0 += 4 * stride) {
    uint4 val[4];
    long long off[4];
    bool whole[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const long long i = i0 + q * stride;
      whole[q] = false;
      off[q] = -1;
      if (i >= nvec) continue;
      // rotate the starting peer by rank so that the ranks do not all hit one peer at once
      const int k0 = static_cast<int>(i / vec_per_shard);
      const int k = (k0 + rank) % world;
      const long long v = i - static_cast<long long>(k0) * vec_per_shard;
      off[q] = static_cast<long long>(k) * shard_bytes + (v << 4);
      if (off[q] + 16 <= total_bytes) {
        whole[q] = true;
        val[q] = reinterpret_cast<const uint4*>(shards.p[k])[v];
      } else if (off[q] < total_bytes) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(shards.p[k]) + (v << 4);
        for (long long b = 0; off[q] + b < total_bytes; ++b) full[off[q] + b] = src[b];
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (whole[q]) *reinterpret_cast<uint4*>(full + off[q]) = val[q];
  }
}

// ---- AdamW pieces (same arithmetic and RNG as adamw_sr_kernel in elementwise.cu)
__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0; key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ uint16_t sr16(float f, uint32_t rnd) {
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7f800000u) == 0x7f800000u) return static_cast<uint16_t>(u >> 16);
  u += (rnd & 0xffffu);
  return static_cast<uint16_t>(u >> 16);
}
__device__ __forceinline__ uint16_t rn16(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ void up8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// g[0..8) += the eight bf16 at element `elem` of every rank's tensor. Four peers' loads are in
// flight at once, and the first peer is `rot` (a value that differs between ranks, so that the
// ranks do not all read one peer at the same moment).
__device__ __forceinline__ void add_peers_bf16x8(const PeerPtrs& grads, long long elem, int world,
                                                 int rot, float (&g)[8]) {
  for (int j0 = 0; j0 < world; j0 += 4) {
    uint4 u[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (j0 + q < world) {
        int j = j0 + q + rot;
        if (j >= world) j -= world;
        u[q] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[j]) + elem);
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (j0 + q < world) {
        float f[8];
        up8(u[q], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] += f[e];
      }
    }
  }
}

struct RsAdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
  unsigned long long seed, offset;   // offset: global element index of the tensor's element 0
  int sr_param, sr_state, g_f32;
};

// grads.p[j]: rank j's FULL gradient tensor (numel elements). This rank owns elements
// [lo, hi). p/m/v point at the owned shard (element 0 of the shard = element lo).
// full_param, when non-null, is the local full parameter buffer that also receives
// the updated owned slice (so the next all-gather source is already in place).
//
// mc_grad, when non-null, is the NVSwitch multicast address of the same bf16 gradient tensor:
// one multimem.ld_reduce returns the sum over every rank's copy, reduced inside the switch
// (fp32 accumulation, bf16 result), instead of `world` separate peer loads.
//
// acc, when non-null, is this rank's fp32 sum of earlier groups' gradients over [lo, hi)
// (element 0 = element lo): the sum starts there instead of at zero.
__global__ void rs_adamw_kernel(PeerPtrs grads, const __nv_bfloat16* __restrict__ mc_grad,
                                const float* __restrict__ acc, __nv_bfloat16* __restrict__ p,
                                __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v,
                                long long lo, long long hi, int world, RsAdamArgs a) {
  const long long n = hi - lo;
  const long long nvec = (n + 7) >> 3;
  const int rot = n > 0 ? static_cast<int>((lo / n) % world) : 0;   // the owning rank; 0 for whole tensors
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i << 3;
    const int cnt = static_cast<int>(min(8LL, n - e0));
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (acc != nullptr) {
      if (cnt == 8) {
        const float4 x = *reinterpret_cast<const float4*>(acc + e0);
        const float4 y = *reinterpret_cast<const float4*>(acc + e0 + 4);
        g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
      } else {
        for (int e = 0; e < cnt; ++e) g[e] = acc[e0 + e];
      }
    }
    if (mc_grad != nullptr && cnt == 8) {
      float f[8];
      uint4 u;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                   : "l"(mc_grad + lo + e0)
                   : "memory");
      up8(u, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] += f[e];
    } else if (!a.g_f32 && cnt == 8) {
      add_peers_bf16x8(grads, lo + e0, world, rot, g);
    } else
    for (int j = 0; j < world; ++j) {
      if (a.g_f32) {
        const float* src = reinterpret_cast<const float*>(grads.p[j]) + lo + e0;
        if (cnt == 8) {
          const float4 x = *reinterpret_cast<const float4*>(src);
          const float4 y = *reinterpret_cast<const float4*>(src + 4);
          g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
          g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
        } else {
          for (int e = 0; e < cnt; ++e) g[e] += src[e];
        }
      } else {
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(grads.p[j]) + lo + e0;
        if (cnt == 8) {
          float f[8];
          up8(*reinterpret_cast<const uint4*>(src), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] += f[e];
        } else {
          for (int e = 0; e < cnt; ++e) g[e] += __bfloat162float(src[e]);
        }
      }
    }
    float pf[8], mf[8], vf[8];
    if (cnt == 8) {
      up8(*reinterpret_cast<const uint4*>(p + e0), pf);
      up8(*reinterpret_cast<const uint4*>(m + e0), mf);
      up8(*reinterpret_cast<const uint4*>(v + e0), vf);
    } else {
      for (int e = 0; e < 8; ++e) {
        const bool in = e < cnt;
        pf[e] = in ? __bfloat162float(p[e0 + e]) : 0.f;
        mf[e] = in ? __bfloat162float(m[e0 + e]) : 0.f;
        vf[e] = in ? __bfloat162float(v[e0 + e]) : 0.f;
      }
    }
    const unsigned long long gidx = a.offset + static_cast<unsigned long long>(lo + e0);
    const uint2 key = make_uint2(static_cast<uint32_t>(a.seed), static_cast<uint32_t>(a.seed >> 32));
    uint4 r[3];
#pragma unroll
    for (int k = 0; k < 3; ++k)
      r[k] = philox(make_uint4(static_cast<uint32_t>(gidx >> 3), static_cast<uint32_t>(gidx >> 35),
                               static_cast<uint32_t>(k), 0x5353u), key);
    const uint32_t rw[12] = {r[0].x, r[0].y, r[0].z, r[0].w, r[1].x, r[1].y,
                             r[1].z, r[1].w, r[2].x, r[2].y, r[2].z, r[2].w};
    uint16_t po[8], mo[8], vo[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gg = g[e] * a.grad_scale;
      const float mn = a.beta1 * mf[e] + (1.f - a.beta1) * gg;
      const float vn = a.beta2 * vf[e] + (1.f - a.beta2) * gg * gg;
      float pn = pf[e] * (1.f - a.lr * a.weight_decay);
      // bias1 / bias2 hold reciprocals; same arithmetic as the single-GPU kernel (elementwise.cu)
      pn -= a.lr * __fdividef(mn * a.bias1, __fsqrt_rn(vn * a.bias2) + a.eps);
      const uint32_t w0 = rw[e >> 1], w1 = rw[4 + (e >> 1)], w2 = rw[8 + (e >> 1)];
      const int sh = (e & 1) * 16;
      po[e] = a.sr_param ? sr16(pn, w0 >> sh) : rn16(pn);
      mo[e] = a.sr_state ? sr16(mn, w1 >> sh) : rn16(mn);
      vo[e] = a.sr_state ? sr16(vn, w2 >> sh) : rn16(vn);
    }
    if (cnt == 8) {
      auto pack = [](const uint16_t (&x)[8]) {
        uint4 u;
        u.x = x[0] | (uint32_t(x[1]) << 16); u.y = x[2] | (uint32_t(x[3]) << 16);
        u.z = x[4] | (uint32_t(x[5]) << 16); u.w = x[6] | (uint32_t(x[7]) << 16);
        return u;
      };
      *reinterpret_cast<uint4*>(p + e0) = pack(po);
      *reinterpret_cast<uint4*>(m + e0) = pack(mo);
      *reinterpret_cast<uint4*>(v + e0) = pack(vo);
    } else {
      for (int e = 0; e < cnt; ++e) {
        p[e0 + e] = __ushort_as_bfloat16(po[e]);
        m[e0 + e] = __ushort_as_bfloat16(mo[e]);
        v[e0 + e] = __ushort_as_bfloat16(vo[e]);
      }
    }
  }
}

// acc[i] (fp32, this rank's owned slice [lo, hi)) = (first ? 0 : acc[i]) + the sum over ranks of
// grads.p[j][lo + i]: the reduce-scatter of one group's gradient, kept as a running sum.
__global__ void rs_accumulate_kernel(PeerPtrs grads, float* __restrict__ acc, long long lo,
                                     long long hi, int world, int g_f32, int first) {
  const long long n = hi - lo;
  const long long nvec = (n + 7) >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i << 3;
    const int cnt = static_cast<int>(min(8LL, n - e0));
    float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int rot = n > 0 ? static_cast<int>((lo / n) % world) : 0;
    if (!first) {
      if (cnt == 8) {
        const float4 x = *reinterpret_cast<const float4*>(acc + e0);
        const float4 y = *reinterpret_cast<const float4*>(acc + e0 + 4);
        g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
      } else {
        for (int e = 0; e < cnt; ++e) g[e] = acc[e0 + e];
      }
    }
    if (!g_f32 && cnt == 8) {
      add_peers_bf16x8(grads, lo + e0, world, rot, g);
    } else
    for (int j = 0; j < world; ++j) {
      if (g_f32) {
        const float* src = reinterpret_cast<const float*>(grads.p[j]) + lo + e0;
        if (cnt == 8) {
          const float4 x = *reinterpret_cast<const float4*>(src);
          const float4 y = *reinterpret_cast<const float4*>(src + 4);
          g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
          g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
        } else {
          for (int e = 0; e < cnt; ++e) g[e] += src[e];
        }
      } else {
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(grads.p[j]) + lo + e0;
        if (cnt == 8) {
          float f[8];
          up8(*reinterpret_cast<const uint4*>(src), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) g[e] += f[e];
        } else {
          for (int e = 0; e < cnt; ++e) g[e] += __bfloat162float(src[e]);
        }
      }
    }
    if (cnt == 8) {
      *reinterpret_cast<float4*>(acc + e0) = make_float4(g[0], g[1], g[2], g[3]);
      *reinterpret_cast<float4*>(acc + e0 + 4) = make_float4(g[4], g[5], g[6], g[7]);
    } else {
      for (int e = 0; e < cnt; ++e) acc[e0 + e] = g[e];
    }
  }
}

// One-shot all-reduce (sum) of a small fp32 tensor: every rank reads every rank.
__global__ void peer_allreduce_f32_kernel(PeerPtrs src, float* __restrict__ dst, long long n,
                                          int world) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < world; ++j) acc += reinterpret_cast<const float*>(src.p[j])[i];
    dst[i] = acc;
  }
}

// CTAs per SM that a collective kernel may take. These kernels run on the communication stream
// beside the compute stream's GEMMs and wait on NVLink latency most of the time: a grid that
// fills every thread slot of every SM (eight CTAs of 256 threads) keeps the compute kernels' CTAs
// from being scheduled for as long as it runs. Two per SM leave three quarters of the slots free;
// the bytes in flight come from four loads per thread instead. SS_COMM_CTAS_PER_SM overrides.
static inline int comm_cap() {
  static int cap = [] {
    const char* e = getenv("SS_COMM_CTAS_PER_SM");
    int v = e ? atoi(e) : 2;
    if (v < 1) v = 1;
    if (v > 8) v = 8;
    return 148 * v;
  }();
  return cap;
}

static inline int grid_of(long long work, int threads, int cap) {
  long long g = (work + threads - 1) / threads;
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace ss

extern "C" {
using namespace ss;

// wait_ns: how long a rank waits for each peer's flag before it gives up (0 = the default, 2 s).
int ss_peer_barrier_timed(void* const* flag_ptrs, int rank, int world, unsigned int epoch,
                          unsigned long long wait_ns, int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return -2;
  PeerPtrs f;
  for (int j = 0; j < world; ++j) f.p[j] = flag_ptrs[j];
  peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, rank, world, epoch,
                                                          wait_ns ? wait_ns : PEER_WAIT_NS, status);
  return (int)cudaGetLastError();
}

int ss_peer_barrier(void* const* flag_ptrs, int rank, int world, unsigned int epoch, int* status,
                    void* stream) {
  return ss_peer_barrier_timed(flag_ptrs, rank, world, epoch, 0, status, stream);
}

int ss_peer_allgather(void* const* shard_ptrs, void* full, long long shard_bytes,
                      long long total_bytes, int rank, int world, void* stream) {
  if (world < 1 || world > MAX_RANKS || (shard_bytes & 15)) return -2;
  PeerPtrs s;
  for (int j = 0; j < world; ++j) s.p[j] = shard_ptrs[j];
  const long long nvec = (shard_bytes >> 4) * world;
  if (nvec == 0) return 0;
  peer_allgather_kernel<<<grid_of((nvec + 3) / 4, 256, comm_cap()), 256, 0, (cudaStream_t)stream>>>(
      s, (uint8_t*)full, shard_bytes, total_bytes, rank, world);
  return (int)cudaGetLastError();
}

int ss_rs_accumulate(void* const* grad_ptrs, void* acc, long long lo, long long hi, int world,
                     int g_f32, int first, void* stream) {
  if (world < 1 || world > MAX_RANKS || (lo & 7) || (reinterpret_cast<uintptr_t>(acc) & 15)) return -2;
  if (hi <= lo) return 0;
  PeerPtrs g;
  for (int j = 0; j < world; ++j) g.p[j] = grad_ptrs[j];
  const long long nvec = (hi - lo + 7) >> 3;
  rs_accumulate_kernel<<<grid_of(nvec, 256, comm_cap()), 256, 0, (cudaStream_t)stream>>>(
      g, (float*)acc, lo, hi, world, g_f32, first);
  return (int)cudaGetLastError();
}

// acc: null, or this rank's fp32 sum of earlier groups' gradients over [lo, hi).
int ss_rs_adamw_acc(void* const* grad_ptrs, const void* acc, void* p, void* m, void* v, long long lo,
                    long long hi, int world, int g_f32, float lr, float beta1, float beta2, float eps,
                    float weight_decay, int step, float grad_scale, unsigned long long seed,
                    unsigned long long offset, int sr_param, int sr_state, void* stream) {
  if (world < 1 || world > MAX_RANKS || (lo & 7) || ((offset) & 7) ||
      (reinterpret_cast<uintptr_t>(acc) & 15))
    return -2;
  if (hi <= lo) return 0;
  PeerPtrs g;
  for (int j = 0; j < world; ++j) g.p[j] = grad_ptrs[j];
  RsAdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f / (1.f - powf(beta1, (float)step)); a.bias2 = 1.f / (1.f - powf(beta2, (float)step));
  a.grad_scale = grad_scale;
  a.seed = seed ^ (0x9E3779B97F4A7C15ull * (unsigned long long)(step + 1));
  a.offset = offset; a.sr_param = sr_param; a.sr_state = sr_state; a.g_f32 = g_f32;
  const long long nvec = (hi - lo + 7) >> 3;
  rs_adamw_kernel<<<grid_of(nvec, 256, comm_cap()), 256, 0, (cudaStream_t)stream>>>(
      g, nullptr, (const float*)acc, (__nv_bfloat16*)p, (__nv_bfloat16*)m, (__nv_bfloat16*)v, lo, hi,
      world, a);
  return (int)cudaGetLastError();
}

int ss_rs_adamw(void* const* grad_ptrs, void* p, void* m, void* v, long long lo, long long hi,
                int world, int g_f32, float lr, float beta1, float beta2, float eps,
                float weight_decay, int step, float grad_scale, unsigned long long seed,
                unsigned long long offset, int sr_param, int sr_state, void* stream) {
  if (world < 1 || world > MAX_RANKS || (lo & 7) || ((offset) & 7)) return -2;
  if (hi <= lo) return 0;
  PeerPtrs g;
  for (int j = 0; j < world; ++j) g.p[j] = grad_ptrs[j];
  RsAdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f / (1.f - powf(beta1, (float)step)); a.bias2 = 1.f / (1.f - powf(beta2, (float)step));
  a.grad_scale = grad_scale;
  a.seed = seed ^ (0x9E3779B97F4A7C15ull * (unsigned long long)(step + 1));
  a.offset = offset; a.sr_param = sr_param; a.sr_state = sr_state; a.g_f32 = g_f32;
  const long long nvec = (hi - lo + 7) >> 3;
  rs_adamw_kernel<<<grid_of(nvec, 256, comm_cap()), 256, 0, (cudaStream_t)stream>>>(
      g, nullptr, nullptr, (__nv_bfloat16*)p, (__nv_bfloat16*)m, (__nv_bfloat16*)v, lo, hi, world, a);
  return (int)cudaGetLastError();
}

// Same update with the gradient sum taken inside the NVSwitch: mc_grad is the multicast
// address of the bf16 gradient tensor (every rank's copy bound to one multicast object).
// grad_ptrs still serves the ragged tail (fewer than eight elements).
int ss_rs_adamw_nvls(void* const* grad_ptrs, const void* mc_grad, void* p, void* m, void* v,
                     long long lo, long long hi, int world, float lr, float beta1, float beta2,
                     float eps, float weight_decay, int step, float grad_scale,
                     unsigned long long seed, unsigned long long offset, int sr_param, int sr_state,
                     void* stream) {
  if (world < 1 || world > MAX_RANKS || (lo & 7) || ((offset) & 7) || mc_grad == nullptr ||
      (reinterpret_cast<uintptr_t>(mc_grad) & 15))
    return -2;
  if (hi <= lo) return 0;
  PeerPtrs g;
  for (int j = 0; j < world; ++j) g.p[j] = grad_ptrs[j];
  RsAdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f / (1.f - powf(beta1, (float)step)); a.bias2 = 1.f / (1.f - powf(beta2, (float)step));
  a.grad_scale = grad_scale;
  a.seed = seed ^ (0x9E3779B97F4A7C15ull * (unsigned long long)(step + 1));
  a.offset = offset; a.sr_param = sr_param; a.sr_state = sr_state; a.g_f32 = 0;
  const long long nvec = (hi - lo + 7) >> 3;
  rs_adamw_kernel<<<grid_of(nvec, 256, comm_cap()), 256, 0, (cudaStream_t)stream>>>(
      g, (const __nv_bfloat16*)mc_grad, nullptr, (__nv_bfloat16*)p, (__nv_bfloat16*)m, (__nv_bfloat16*)v,
      lo, hi, world, a);
  return (int)cudaGetLastError();
}

int ss_peer_allreduce_f32(void* const* src_ptrs, float* dst, long long n, int world, void* stream) {
  if (world < 1 || world > MAX_RANKS) return -2;
  if (n <= 0) return 0;
  PeerPtrs s;
  for (int j = 0; j < world; ++j) s.p[j] = src_ptrs[j];
  peer_allreduce_f32_kernel<<<grid_of(n, 256, 148 * 4), 256, 0, (cudaStream_t)stream>>>(s, dst, n, world);
  return (int)cudaGetLastError();
}
}  // extern "C"
