// Mixture-of-experts routing and token movement for sm_100a.
//
//   ss_moe_route      per token: top-k over the router logits, softmax over the
//                     selected logits (renormalised) or over all experts, and a
//                     per-expert histogram -- one warp per token, no sorting pass
//   ss_moe_layout     expert segments padded to 128 rows (so a GEMM tile never
//                     straddles two experts), the expert of every 128-row tile,
//                     and a destination row for every (token, slot) assignment
//   ss_moe_gather     token rows -> expert-sorted rows (optionally scaled: the
//                     backward pass scatters weight * dout the same way)
//   ss_moe_combine    expert-sorted rows -> token rows: out[t] (+)= sum_j w[t,j] *
//                     y[dest[t,j]], deterministic (a gather, no atomics); can also
//                     emit <dout[t], y[dest[t,j]]> for the router-weight gradient
//
// The same kernels serve expert parallelism: `dest` rows may live in a peer GPU's
// staging buffer (plain P2P stores / loads through the symmetric pool), which is
// how dispatch and combine cross NVLink without a separate all-to-all.
//
// Semantics: the reference's routed-expert layer (top-k then softmax for Qwen,
// softmax then top-k for OLMoE; packages/workloads/src/shadowspill_workloads/
// models/shared/qwen_moe/experts.py:31-72, router_statistics.py:9-32).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace ss {

constexpr int MOE_MAX_E = 512;
constexpr int MOE_MAX_K = 32;

__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits fp32 [T, E] (row pitch ld). ids int32 [T,k], weights fp32 [T,k], counts int32 [E].
__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, int T, int E, int k,
                                 int renormalize, int* __restrict__ ids,
                                 float* __restrict__ weights, int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + static_cast<long long>(warp) * ld;
  constexpr int PER = MOE_MAX_E / 32;
  float v[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + i * 32;
    v[i] = e < E ? row[e] : -INFINITY;
  }
  float lmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) lmax = fmaxf(lmax, v[i]);
  const float gmax = wmax(lmax);
  float denom = 0.f;
  if (!renormalize) {
#pragma unroll
    for (int i = 0; i < PER; ++i) denom += (v[i] == -INFINITY) ? 0.f : __expf(v[i] - gmax);
    denom = wsum(denom);
  }
  float sel_v[MOE_MAX_K];
  int sel_e[MOE_MAX_K];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + i * 32;
      if (v[i] > best || (v[i] == best && e < bi && v[i] != -INFINITY)) { best = v[i]; bi = e; }
    }
    // warp arg-max; ties go to the lower expert index (matches a stable top-k)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    sel_v[j] = best; sel_e[j] = bi;
    if ((bi & 31) == lane) {                          // remove the winner
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == (bi >> 5)) v[i] = -INFINITY;
    }
  }
  if (lane == 0) {
    float s = 0.f;
    if (renormalize) {
      for (int j = 0; j < k; ++j) s += __expf(sel_v[j] - sel_v[0]);
    }
    for (int j = 0; j < k; ++j) {
      const float w = renormalize ? __expf(sel_v[j] - sel_v[0]) / s : __expf(sel_v[j] - gmax) / denom;
      ids[static_cast<long long>(warp) * k + j] = sel_e[j];
      weights[static_cast<long long>(warp) * k + j] = w;
      atomicAdd(counts + sel_e[j], 1);
    }
  }
}

// One block. offsets[E+1] (padded to 128), tile_expert[max_tiles], cursor[E] zeroed.
__global__ void moe_layout_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                  int* __restrict__ tile_expert, int max_tiles,
                                  int* __restrict__ cursor) {
  __shared__ int s_off[MOE_MAX_E + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = s_off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] = 0;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * 128;
    int found = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E;            // largest e with s_off[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      found = lo;
    }
    tile_expert[t] = found;
  }
}

__global__ void moe_assign_kernel(const int* __restrict__ ids, long long n, const int* __restrict__ offsets,
                                  int* __restrict__ cursor, int* __restrict__ dest) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = ids[i];
    dest[i] = offsets[e] + atomicAdd(cursor + e, 1);
  }
}

// sorted[dest[t*k+j], :] = scale * x[t, :]   (scale = weights[t*k+j] or 1)
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                  const int* __restrict__ dest, const float* __restrict__ weights,
                                  __nv_bfloat16* __restrict__ sorted, long long lds, int T, int k,
                                  int D) {
  const int nv = D >> 3;
  const long long n = static_cast<long long>(T) * k;
  for (long long a = blockIdx.x; a < n; a += gridDim.x) {
    const long long t = a / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + t * ldx);
    uint4* dst = reinterpret_cast<uint4*>(sorted + static_cast<long long>(dest[a]) * lds);
    if (weights == nullptr) {
      for (int c = threadIdx.x; c < nv; c += blockDim.x) dst[c] = src[c];
    } else {
      const float w = weights[a];
      for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        uint4 u = src[c];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(h[e]);
          f.x *= w; f.y *= w;
          h[e] = __float22bfloat162_rn(f);
        }
        dst[c] = u;
      }
    }
  }
}

// out[t,:] (+)= sum_j w[t,j] * y[dest[t,j], :];  optionally dots[t,j] = <g[t,:], y[dest[t,j],:]>
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, long long ldy,
                                   const int* __restrict__ dest, const float* __restrict__ weights,
                                   __nv_bfloat16* __restrict__ out, long long ldo, int T, int k, int D,
                                   int accumulate, const __nv_bfloat16* __restrict__ g, long long ldg,
                                   float* __restrict__ dots) {
  const int nv = D >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    if (out != nullptr) {
      for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (accumulate) {
          const uint4 u = reinterpret_cast<const uint4*>(out + static_cast<long long>(t) * ldo)[c];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); acc[2 * e] = f.x; acc[2 * e + 1] = f.y; }
        }
        for (int j = 0; j < k; ++j) {
          const long long a = static_cast<long long>(t) * k + j;
          const float w = weights ? weights[a] : 1.f;
          const uint4 u = reinterpret_cast<const uint4*>(y + static_cast<long long>(dest[a]) * ldy)[c];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); acc[2 * e] += w * f.x; acc[2 * e + 1] += w * f.y; }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        reinterpret_cast<uint4*>(out + static_cast<long long>(t) * ldo)[c] = o;
      }
    }
    if (dots != nullptr) {
      // one warp per slot: 16-byte loads, a shuffle reduction, no block barrier
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
      const uint4* gv = reinterpret_cast<const uint4*>(g + static_cast<long long>(t) * ldg);
      for (int j = warp; j < k; j += nwarps) {
        const long long a = static_cast<long long>(t) * k + j;
        const uint4* yv = reinterpret_cast<const uint4*>(y + static_cast<long long>(dest[a]) * ldy);
        float part = 0.f;
        for (int c = lane; c < nv; c += 32) {
          const uint4 u = yv[c], w = gv[c];
          const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
          const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 fu = __bfloat1622float2(uh[e]), fw = __bfloat1622float2(wh[e]);
            part += fu.x * fw.x + fu.y * fw.y;
          }
        }
        part = wsum(part);
        if (lane == 0) dots[a] = part;
      }
    }
  }
}

}  // namespace ss

extern "C" {
using namespace ss;

int ss_moe_route(const float* logits, long long ld, int T, int E, int k, int renormalize, int* ids,
                 float* weights, int* counts, void* stream) {
  if (E > MOE_MAX_E || k > MOE_MAX_K || k > E || T <= 0) return T <= 0 ? 0 : -2;
  cudaStream_t s = (cudaStream_t)stream;
  cudaMemsetAsync(counts, 0, sizeof(int) * E, s);
  const int blocks = (T * 32 + 255) / 256;
  moe_route_kernel<<<blocks, 256, 0, s>>>(logits, ld, T, E, k, renormalize, ids, weights, counts);
  return (int)cudaGetLastError();
}

int ss_moe_layout(const int* counts, const int* ids, int T, int E, int k, int* offsets,
                  int* tile_expert, int max_tiles, int* cursor, int* dest, void* stream) {
  if (E > MOE_MAX_E) return -2;
  cudaStream_t s = (cudaStream_t)stream;
  moe_layout_kernel<<<1, 256, 0, s>>>(counts, E, offsets, tile_expert, max_tiles, cursor);
  const long long n = (long long)T * k;
  if (n > 0) {
    const int blocks = (int)((n + 255) / 256 > 1184 ? 1184 : (n + 255) / 256);
    moe_assign_kernel<<<blocks, 256, 0, s>>>(ids, n, offsets, cursor, dest);
  }
  return (int)cudaGetLastError();
}

int ss_moe_gather(const void* x, long long ldx, const int* dest, const float* weights, void* sorted,
                  long long lds, int T, int k, int D, void* stream) {
  if (D % 8 || ldx % 8 || lds % 8) return -2;
  if (T <= 0) return 0;
  const long long n = (long long)T * k;
  moe_gather_kernel<<<(int)(n > 148 * 16 ? 148 * 16 : n), 128, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, ldx, dest, weights, (__nv_bfloat16*)sorted, lds, T, k, D);
  return (int)cudaGetLastError();
}

int ss_moe_combine(const void* y, long long ldy, const int* dest, const float* weights, void* out,
                   long long ldo, int T, int k, int D, int accumulate, const void* g, long long ldg,
                   float* dots, void* stream) {
  if (D % 8 || ldy % 8 || (out && ldo % 8) || (dots && ldg % 8)) return -2;
  if (T <= 0) return 0;
  moe_combine_kernel<<<T > 148 * 8 ? 148 * 8 : T, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)y, ldy, dest, weights, (__nv_bfloat16*)out, ldo, T, k, D, accumulate,
      (const __nv_bfloat16*)g, ldg, dots);
  return (int)cudaGetLastError();
}
}  // extern "C"
