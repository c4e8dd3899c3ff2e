// Elementwise pieces of the Gated DeltaNet mixer for sm_100a (all memory-bound):
//
//   ss_conv_silu_fwd / _bwd    depthwise causal conv1d (kernel width <= 8) + SiLU over packed
//                              sequences; the window never crosses a sequence start
//                              (position-in-sequence comes with the batch)
//   ss_l2norm_fwd / _bwd       x / sqrt(sum x^2 + eps) per head row
//   ss_gated_rmsnorm_fwd/_bwd  rmsnorm(x) * w * silu(gate) per head row
//
// bf16 in/out, fp32 math, fp32 atomics for the small parameter gradients.
// Definitions: packages/workloads/src/shadowspill_workloads/models/shared/delta_net.py:13-89
// (convolution + SiLU, L2-normalised q/k, gated output norm).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ss_dn {

using bf16 = __nv_bfloat16;
constexpr int MAX_TAPS = 8;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 v = __bfloat1622float2(h[e]);
    f[2 * e] = v.x; f[2 * e + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
  return u;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// ------------------------------------------------------------------ conv + SiLU
// x,y [T, ld*] bf16, C channels (multiple of 8); w [C, K] bf16; pos[t] = index of t in its sequence.
// y[t,c] = silu(sum_{j=0..min(K-1,pos[t])} w[c, K-1-j] * x[t-j, c])
template <bool WRITE_DPRE, int KT>
__global__ void conv_silu_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                                 const int* __restrict__ pos, int T, int C, int K,
                                 bf16* __restrict__ y, long long ldy,
                                 const bf16* __restrict__ dy, long long lddy,
                                 float* __restrict__ dpre, float* __restrict__ dw, int rows_per_block) {
  const int cv = blockIdx.y * blockDim.x + threadIdx.x;     // 8-channel vector index
  if (cv * 8 >= C) return;
  float wt[KT][8];
#pragma unroll
  for (int j = 0; j < KT; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e)
      wt[j][e] = (j < K) ? __bfloat162float(w[static_cast<long long>(cv * 8 + e) * K + (K - 1 - j)]) : 0.f;
  float dwacc[KT][8];
  if (WRITE_DPRE) {
#pragma unroll
    for (int j = 0; j < KT; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) dwacc[j][e] = 0.f;
  }
  const int t0 = blockIdx.x * rows_per_block;
  const int t1 = min(T, t0 + rows_per_block);
  for (int t = t0; t < t1; ++t) {
    const int p = pos[t];
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float xs[KT][8];
#pragma unroll
    for (int j = 0; j < KT; ++j) {
      if (j < K && j <= p) {
        unpack8(*reinterpret_cast<const uint4*>(x + static_cast<long long>(t - j) * ldx + cv * 8), xs[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += wt[j][e] * xs[j][e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xs[j][e] = 0.f;
      }
    }
    if (!WRITE_DPRE) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = silu(acc[e]);
      *reinterpret_cast<uint4*>(y + static_cast<long long>(t) * ldy + cv * 8) = pack8(o);
    } else {
      float g[8], d[8];
      unpack8(*reinterpret_cast<const uint4*>(dy + static_cast<long long>(t) * lddy + cv * 8), g);
#pragma unroll
      for (int e = 0; e < 8; ++e) d[e] = g[e] * dsilu(acc[e]);
      float4* dp = reinterpret_cast<float4*>(dpre + static_cast<long long>(t) * C + cv * 8);
      dp[0] = make_float4(d[0], d[1], d[2], d[3]);
      dp[1] = make_float4(d[4], d[5], d[6], d[7]);
#pragma unroll
      for (int j = 0; j < KT; ++j)
        if (j < K)
#pragma unroll
          for (int e = 0; e < 8; ++e) dwacc[j][e] += d[e] * xs[j][e];
    }
  }
  if (WRITE_DPRE) {
#pragma unroll
    for (int j = 0; j < KT; ++j)
      if (j < K)
#pragma unroll
        for (int e = 0; e < 8; ++e)
          atomicAdd(dw + static_cast<long long>(cv * 8 + e) * K + (K - 1 - j), dwacc[j][e]);
  }
}

// dx[t,c] = sum_{j : t+j < T, pos[t+j] >= j} w[c, K-1-j] * dpre[t+j, c]
__global__ void conv_dx_kernel(const float* __restrict__ dpre, const bf16* __restrict__ w,
                               const int* __restrict__ pos, int T, int C, int K,
                               bf16* __restrict__ dx, long long lddx) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const int nv = C >> 3;
  if (idx >= static_cast<long long>(T) * nv) return;
  const int t = static_cast<int>(idx / nv), cv = static_cast<int>(idx % nv);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < K; ++j) {
    if (t + j >= T || pos[t + j] < j) break;      // later tokens belong to another sequence too
    const float4* dp = reinterpret_cast<const float4*>(dpre + static_cast<long long>(t + j) * C + cv * 8);
    const float4 a = dp[0], b = dp[1];
    const float d[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 8; ++e)
      acc[e] += __bfloat162float(w[static_cast<long long>(cv * 8 + e) * K + (K - 1 - j)]) * d[e];
  }
  *reinterpret_cast<uint4*>(dx + static_cast<long long>(t) * lddx + cv * 8) = pack8(acc);
}

// ------------------------------------------------------------------ L2 norm, one warp per row of width W
__global__ void l2norm_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long rows, int W,
                                  float eps) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * W;
  float ss = 0.f;
  for (int c = lane * 2; c < W; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    ss += v.x * v.x + v.y * v.y;
  }
  const float r = rsqrtf(warp_sum(ss) + eps);
  for (int c = lane * 2; c < W; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    *reinterpret_cast<__nv_bfloat162*>(y + row * W + c) = __floats2bfloat162_rn(v.x * r, v.y * r);
  }
}
// dx = r * (dy - xhat * <xhat, dy>),  xhat = x * r
__global__ void l2norm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ dy,
                                  bf16* __restrict__ dx, long long rows, int W, float eps) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * W;
  const bf16* gr = dy + row * W;
  float ss = 0.f, dot = 0.f;
  for (int c = lane * 2; c < W; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gr + c));
    ss += v.x * v.x + v.y * v.y;
    dot += v.x * g.x + v.y * g.y;
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss + eps);
  const float k = dot * r * r;                       // <xhat, dy> * r
  for (int c = lane * 2; c < W; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gr + c));
    *reinterpret_cast<__nv_bfloat162*>(dx + row * W + c) =
        __floats2bfloat162_rn(r * (g.x - v.x * k), r * (g.y - v.y * k));
  }
}

// ------------------------------------------------------------------ gated RMSNorm, one warp per row
// y = x * rsqrt(mean x^2 + eps) * s(w) * silu(gate),  s(w) = w or 1 + w
__global__ void gated_rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gate,
                                         const bf16* __restrict__ w, bf16* __restrict__ y,
                                         long long rows, int W, float eps, int zero_centered) {
  const long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + row * W;
  float ss = 0.f;
  for (int c = lane * 2; c < W; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    ss += v.x * v.x + v.y * v.y;
  }
  const float r = rsqrtf(warp_sum(ss) / static_cast<float>(W) + eps);
  for (int c = lane * 2; c < W; c += 64) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + row * W + c));
    const float2 ww = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + c));
    const float s0 = zero_centered ? 1.f + ww.x : ww.x, s1 = zero_centered ? 1.f + ww.y : ww.y;
    *reinterpret_cast<__nv_bfloat162*>(y + row * W + c) =
        __floats2bfloat162_rn(v.x * r * s0 * silu(g.x), v.y * r * s1 * silu(g.y));
  }
}
// dn = dy*silu(g); dgate = dy * n * silu'(g) with n = xhat*s; dx = r (dn*s - xhat*mean(dn*s*xhat));
// dw += dn * xhat (shared-memory partial sums per block, then global atomics)
__global__ void gated_rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gate,
                                         const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                         bf16* __restrict__ dx, bf16* __restrict__ dgate,
                                         float* __restrict__ dw, long long rows, int W, float eps,
                                         int zero_centered) {
  extern __shared__ float s_dw[];
  for (int c = threadIdx.x; c < W; c += blockDim.x) s_dw[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; row < rows;
       row += warps) {
    const bf16* xr = x + row * W;
    const bf16* gr = gate + row * W;
    const bf16* yr = dy + row * W;
    float ss = 0.f;
    for (int c = lane * 2; c < W; c += 64) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
      ss += v.x * v.x + v.y * v.y;
    }
    const float r = rsqrtf(warp_sum(ss) / static_cast<float>(W) + eps);
    float dot = 0.f;
    for (int c = lane * 2; c < W; c += 64) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gr + c));
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(yr + c));
      const float2 ww = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + c));
      const float s0 = zero_centered ? 1.f + ww.x : ww.x, s1 = zero_centered ? 1.f + ww.y : ww.y;
      dot += d.x * silu(g.x) * s0 * v.x * r + d.y * silu(g.y) * s1 * v.y * r;
    }
    const float mean = warp_sum(dot) / static_cast<float>(W);
    for (int c = lane * 2; c < W; c += 64) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + c));
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gr + c));
      const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(yr + c));
      const float2 ww = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + c));
      const float s0 = zero_centered ? 1.f + ww.x : ww.x, s1 = zero_centered ? 1.f + ww.y : ww.y;
      const float xh0 = v.x * r, xh1 = v.y * r;
      const float dn0 = d.x * silu(g.x), dn1 = d.y * silu(g.y);
      *reinterpret_cast<__nv_bfloat162*>(dx + row * W + c) =
          __floats2bfloat162_rn(r * (dn0 * s0 - xh0 * mean), r * (dn1 * s1 - xh1 * mean));
      *reinterpret_cast<__nv_bfloat162*>(dgate + row * W + c) =
          __floats2bfloat162_rn(d.x * xh0 * s0 * dsilu(g.x), d.y * xh1 * s1 * dsilu(g.y));
      atomicAdd(&s_dw[c], dn0 * xh0);
      atomicAdd(&s_dw[c + 1], dn1 * xh1);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < W; c += blockDim.x)
    if (s_dw[c] != 0.f) atomicAdd(dw + c, s_dw[c]);
}

}  // namespace ss_dn

extern "C" {
using namespace ss_dn;

int ss_conv_silu_fwd(const void* x, long long ldx, const void* w, const int* pos, int T, int C, int K,
                     void* y, long long ldy, void* stream) {
  if (C % 8 || ldx % 8 || ldy % 8 || K < 1 || K > MAX_TAPS) return -2;
  if (T <= 0) return 0;
  const int rows = 32, threads = 64;
  dim3 grid((T + rows - 1) / rows, (C / 8 + threads - 1) / threads);
  if (K <= 4)
    conv_silu_kernel<false, 4><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, ldx, (const bf16*)w, pos, T, C, K, (bf16*)y, ldy, nullptr, 0, nullptr, nullptr, rows);
  else
    conv_silu_kernel<false, MAX_TAPS><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, ldx, (const bf16*)w, pos, T, C, K, (bf16*)y, ldy, nullptr, 0, nullptr, nullptr, rows);
  return (int)cudaGetLastError();
}
// dpre: fp32 [T, C] scratch; dw: fp32 [C, K], ADDED into.
int ss_conv_silu_bwd(const void* x, long long ldx, const void* w, const int* pos, int T, int C, int K,
                     const void* dy, long long lddy, float* dpre, void* dx, long long lddx, float* dw,
                     void* stream) {
  if (C % 8 || ldx % 8 || lddy % 8 || lddx % 8 || K < 1 || K > MAX_TAPS) return -2;
  if (T <= 0) return 0;
  const int rows = 64, threads = 64;
  dim3 grid((T + rows - 1) / rows, (C / 8 + threads - 1) / threads);
  if (K <= 4)
    conv_silu_kernel<true, 4><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, ldx, (const bf16*)w, pos, T, C, K, nullptr, 0, (const bf16*)dy, lddy, dpre, dw, rows);
  else
    conv_silu_kernel<true, MAX_TAPS><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const bf16*)x, ldx, (const bf16*)w, pos, T, C, K, nullptr, 0, (const bf16*)dy, lddy, dpre, dw, rows);
  const long long n = (long long)T * (C / 8);
  conv_dx_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dpre, (const bf16*)w, pos, T, C,
                                                                          K, (bf16*)dx, lddx);
  return (int)cudaGetLastError();
}
int ss_l2norm_fwd(const void* x, void* y, long long rows, int W, float eps, void* stream) {
  if (W % 2) return -2;
  if (rows <= 0) return 0;
  l2norm_fwd_kernel<<<(int)((rows * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y,
                                                                                      rows, W, eps);
  return (int)cudaGetLastError();
}
int ss_l2norm_bwd(const void* x, const void* dy, void* dx, long long rows, int W, float eps, void* stream) {
  if (W % 2) return -2;
  if (rows <= 0) return 0;
  l2norm_bwd_kernel<<<(int)((rows * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)dy, (bf16*)dx, rows, W, eps);
  return (int)cudaGetLastError();
}
int ss_gated_rmsnorm_fwd(const void* x, const void* gate, const void* w, void* y, long long rows, int W,
                         float eps, int zero_centered, void* stream) {
  if (W % 2) return -2;
  if (rows <= 0) return 0;
  gated_rmsnorm_fwd_kernel<<<(int)((rows * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)gate, (const bf16*)w, (bf16*)y, rows, W, eps, zero_centered);
  return (int)cudaGetLastError();
}
// dw: fp32 [W], ADDED into.
int ss_gated_rmsnorm_bwd(const void* x, const void* gate, const void* w, const void* dy, void* dx,
                         void* dgate, float* dw, long long rows, int W, float eps, int zero_centered,
                         void* stream) {
  if (W % 2 || W > 8192) return -2;
  if (rows <= 0) return 0;
  long long blocks = (rows * 32 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  gated_rmsnorm_bwd_kernel<<<(int)blocks, 256, sizeof(float) * W, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)gate, (const bf16*)w, (const bf16*)dy, (bf16*)dx, (bf16*)dgate, dw, rows,
      W, eps, zero_centered);
  return (int)cudaGetLastError();
}
}  // extern "C"

// ============================================================================ chunk-state scan
// The only sequential part of the chunked gated delta rule: a linear recurrence over the
// chunk index for every head,
//     X_{c+1} = M_c^T X_c + B_c,        X_0 = 0,        out[c] = X_c   (the state ENTERING c)
// with M_c [dk, dk], B_c / X [dk, dv] fp32. The caller passes M = A^T for the forward
// recurrence X_{c+1} = A_c X_c + B_c and M = A itself (walking c = n-1 .. 0) for its adjoint,
// so the tile is always copied into shared memory as stored. Columns of X evolve independently:
// a block owns one head and 32 columns; each thread keeps a 4 x 4 register tile; the next
// step's matrix streams in with cp.async while the current one is multiplied.
// Everything that is parallel over chunks (building A and B, outputs, their gradients) is batched
// matrix algebra outside this kernel.
namespace ss_dn {

constexpr int SCAN_COLS = 32;
constexpr int SCAN_THREADS = 256;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(SCAN_THREADS)
linear_scan_kernel(const float* __restrict__ M, const float* __restrict__ B, float* __restrict__ out,
                   int n, int H, int dk, int dv, int reverse) {
  extern __shared__ __align__(16) float sm[];
  const int lda = dk + 4;                       // padded rows keep 16-byte alignment, spread banks
  float* Ms[2] = {sm, sm + dk * lda};           // [dk][lda] x 2 (double buffer)
  float* X = sm + 2 * dk * lda;                 // [dk][SCAN_COLS]
  float* Xn = X + dk * SCAN_COLS;
  const int slices = dv / SCAN_COLS;
  const int h = blockIdx.x / slices, col0 = (blockIdx.x % slices) * SCAN_COLS;
  const int tid = threadIdx.x;
  const int tx = tid & 7, ty = tid >> 3;        // output tile: rows 4*ty.., columns 4*tx..
  auto matrix = [&](int s) { return static_cast<long long>(reverse ? n - 1 - s : s) * H + h; };
  auto prefetch = [&](int s, float* dst) {
    const float* src = M + matrix(s) * dk * dk;
    for (int i = tid * 4; i < dk * dk; i += SCAN_THREADS * 4) {
      const int r = i / dk, cc = i - r * dk;
      cp_async16(dst + r * lda + cc, src + i);
    }
    cp_async_commit();
  };
  for (int i = tid; i < dk * SCAN_COLS; i += SCAN_THREADS) X[i] = 0.f;
  if (n > 0) prefetch(0, Ms[0]);
  for (int s = 0; s < n; ++s) {
    const long long mat = matrix(s);
    const float* Bc = B + mat * dk * dv;
    float* oc = out + mat * dk * dv;
    if (s + 1 < n) { prefetch(s + 1, Ms[(s + 1) & 1]); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();                             // this step's matrix and the current X are visible
    const float* As = Ms[s & 1];
    // the state entering this step is an output
    for (int i = tid; i < dk * SCAN_COLS / 4; i += SCAN_THREADS) {
      const int r = (i * 4) / SCAN_COLS, cc = (i * 4) - r * SCAN_COLS;
      *reinterpret_cast<float4*>(oc + static_cast<long long>(r) * dv + col0 + cc) =
          *reinterpret_cast<const float4*>(X + r * SCAN_COLS + cc);
    }
    if (ty * 4 < dk) {
      float acc[4][4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float4 b = *reinterpret_cast<const float4*>(Bc + static_cast<long long>(ty * 4 + r) * dv + col0 + tx * 4);
        acc[r][0] = b.x; acc[r][1] = b.y; acc[r][2] = b.z; acc[r][3] = b.w;
      }
#pragma unroll 8
      for (int m = 0; m < dk; ++m) {
        const float4 a = *reinterpret_cast<const float4*>(As + m * lda + ty * 4);      // M[m][4ty..]
        const float4 x = *reinterpret_cast<const float4*>(X + m * SCAN_COLS + tx * 4);
        const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          acc[r][0] += av[r] * x.x; acc[r][1] += av[r] * x.y;
          acc[r][2] += av[r] * x.z; acc[r][3] += av[r] * x.w;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float4*>(Xn + (ty * 4 + r) * SCAN_COLS + tx * 4) =
            make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
    __syncthreads();                             // everyone is done with X and with Ms[s & 1]
    float* t = X; X = Xn; Xn = t;
  }
}

}  // namespace ss_dn

// X_{c+1} = M_c^T X_c + B_c (see above). dk a multiple of 4 up to 128, dv a multiple of 32.
extern "C" int ss_linear_scan(const float* M, const float* B, float* out, int n, int H, int dk, int dv,
                              int reverse, void* stream) {
  using namespace ss_dn;
  if (dk % 4 || dk > 128 || dv % SCAN_COLS || n < 0) return -2;
  if (n == 0 || H == 0) return 0;
  const int smem = sizeof(float) * (2 * dk * (dk + 4) + 2 * dk * SCAN_COLS);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(linear_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(float) * (2 * 128 * 132 + 2 * 128 * SCAN_COLS));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  linear_scan_kernel<<<H * (dv / SCAN_COLS), SCAN_THREADS, smem, (cudaStream_t)stream>>>(
      M, B, out, n, H, dk, dv, reverse);
  return (int)cudaGetLastError();
}
