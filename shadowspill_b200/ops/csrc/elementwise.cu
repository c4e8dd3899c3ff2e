// Bandwidth-bound model ops for sm_100a: RMSNorm (+ fused residual add), rotary
// embedding, SwiGLU, embedding gather / scatter-add, masked weighted cross-entropy
// over a logits block, AdamW with bf16 stochastic rounding, sum-of-squares.
//
// All kernels move 16-byte vectors, keep reductions in fp32 and take explicit
// extents. The math follows the reference's pure-PyTorch definitions in
// packages/workloads/src/shadowspill_workloads/models/shared/decoder.py
// (RMSNorm :18, apply_rotary :232, swiglu :292, language_model_loss :320).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ss {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float2 up2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ uint32_t pk2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = up2(u.x), b = up2(u.y), c = up2(u.z), d = up2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pk2(f[0], f[1]); u.y = pk2(f[2], f[3]); u.z = pk2(f[4], f[5]); u.w = pk2(f[6], f[7]);
  return u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is >= 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// =============================================================== RMSNorm forward
// Optionally first folds `delta` into the residual stream: x <- x + delta (x is
// rewritten), then y = x * rstd * w  (zero_centered: * (1 + w)). rstd[T] is saved.
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // vectors of 8 per thread held in registers: D <= 8192

__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(bf16* __restrict__ x, const bf16* __restrict__ delta,
                   const bf16* __restrict__ w, bf16* __restrict__ y, float* __restrict__ rstd,
                   int T, int D, float eps, int zero_centered) {
  __shared__ float red[33];
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    uint4* xr = reinterpret_cast<uint4*>(x + static_cast<size_t>(row) * D);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + static_cast<size_t>(row) * D)
                            : nullptr;
    float v[NORM_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        unpack8(xr[c], v[i]);
        if (dr) {
          float d[8];
          unpack8(dr[c], d);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += d[e];
          // The residual stream is kept in bf16: round once here so that the
          // normalised value and the stored stream agree.
          const uint4 rounded = pack8(v[i]);
          xr[c] = rounded;
          unpack8(rounded, v[i]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
      }
    }
    const float tot = block_sum(ss, red);
    const float r = rsqrtf(tot / static_cast<float>(D) + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = r;
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * D);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float ww[8], o[8];
        unpack8(wr[c], ww);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          o[e] = v[i][e] * r * (zero_centered ? 1.f + ww[e] : ww[e]);
        yr[c] = pack8(o);
      }
    }
  }
}

// =============================================================== RMSNorm backward
// dx = rstd * (g*w - xhat * mean(g*w*xhat)),  dw += sum_t g * xhat   (fp32 atomics)
// dx is ADDED into dx_acc when accumulate != 0 (residual-stream gradient).
//
// One warp per row, two passes over the row (the second hits L1/L2): no block barrier
// per row and few live registers, so many rows are in flight per SM. The weight
// gradient is accumulated with shared-memory atomics (one fp32 per column per block)
// and flushed to global memory once per block.
constexpr int NORM_BWD_WARPS = 8;
__global__ void __launch_bounds__(NORM_BWD_WARPS * 32)
rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                   const bf16* __restrict__ gy, const float* __restrict__ rstd,
                   bf16* __restrict__ dx, float* __restrict__ dw, int T, int D, int zero_centered,
                   int accumulate) {
  extern __shared__ float s_dw[];          // [8][D/8]: element e of vector c at e*nv + c (conflict-free lanes)
  const int nv = D >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (dw) {
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_dw[c] = 0.f;
    __syncthreads();
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * NORM_BWD_WARPS + warp; row < T; row += gridDim.x * NORM_BWD_WARPS) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * D);
    const uint4* gr = reinterpret_cast<const uint4*>(gy + static_cast<size_t>(row) * D);
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll 4
    for (int c = lane; c < nv; c += 32) {
      float xv[8], gv[8], ww[8];
      unpack8(xr[c], xv);
      unpack8(gr[c], gv);
      unpack8(wr[c], ww);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = xv[e] * r;
        dot += gv[e] * (zero_centered ? 1.f + ww[e] : ww[e]) * xh;
        if (dw) atomicAdd(&s_dw[e * nv + c], gv[e] * xh);
      }
    }
    const float mean = warp_sum(dot) / static_cast<float>(D);
    uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * D);
#pragma unroll 4
    for (int c = lane; c < nv; c += 32) {
      float xv[8], gv[8], ww[8], o[8];
      unpack8(xr[c], xv);
      unpack8(gr[c], gv);
      unpack8(wr[c], ww);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        o[e] = r * (gv[e] * (zero_centered ? 1.f + ww[e] : ww[e]) - xv[e] * r * mean);
      if (accumulate) {
        float prev[8];
        unpack8(dr[c], prev);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] += prev[e];
      }
      dr[c] = pack8(o);
    }
  }
  if (dw) {
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      const float v = s_dw[i];
      const int e = i / nv, c = i - e * nv;
      if (v != 0.f) atomicAdd(dw + c * 8 + e, v);
    }
  }
}

// Block-per-row form for D <= 8192: a thread owns up to NORM_MAXV fixed vectors of eight columns,
// so the row is read once (x and gy stay in registers across the row reduction) and the weight
// gradient accumulates in registers over every row the block handles; one global atomic per
// column per block at the end. Same arithmetic as the warp-per-row kernel above.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS, VPT <= 2 ? 3 : 1)
rmsnorm_bwd_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                        const bf16* __restrict__ gy, const float* __restrict__ rstd,
                        bf16* __restrict__ dx, float* __restrict__ dw, int T, int D, int zero_centered,
                        int accumulate) {
  __shared__ float red[33];
  const int nv = D >> 3;
  const float wofs = zero_centered ? 1.f : 0.f;
  uint4 wq[VPT];
  float acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
    wq[i] = c < nv ? reinterpret_cast<const uint4*>(w)[c] : make_uint4(0, 0, 0, 0);
  }
  // rows are software-pipelined: the next row's x and gy are in flight while this one reduces
  uint4 xq[VPT], gq[VPT], xn[VPT], gn[VPT];
  auto fetch = [&](int row, uint4 (&xo)[VPT], uint4 (&go)[VPT]) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * D);
    const uint4* gr = reinterpret_cast<const uint4*>(gy + static_cast<size_t>(row) * D);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) { xo[i] = xr[c]; go[i] = gr[c]; }
    }
  };
  int row = blockIdx.x;
  if (row < T) fetch(row, xq, gq);
  for (; row < T; row += gridDim.x) {
    const int next = row + gridDim.x;
    if (next < T) fetch(next, xn, gn);
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float xv[8], gv[8], ww[8];
        unpack8(xq[i], xv);
        unpack8(gq[i], gv);
        unpack8(wq[i], ww);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = xv[e] * r;
          acc[i][e] += gv[e] * xh;
          dot += gv[e] * (ww[e] + wofs) * xh;
        }
      }
    }
    const float mean = block_sum(dot, red) / static_cast<float>(D);
    uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * D);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
        float xv[8], gv[8], ww[8], o[8];
        unpack8(xq[i], xv);
        unpack8(gq[i], gv);
        unpack8(wq[i], ww);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = r * (gv[e] * (ww[e] + wofs) - xv[e] * r * mean);
        if (accumulate) {
          float prev[8];
          unpack8(dr[c], prev);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += prev[e];
        }
        dr[c] = pack8(o);
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) { xq[i] = xn[i]; gq[i] = gn[i]; }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nv) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (acc[i][e] != 0.f) atomicAdd(dw + c * 8 + e, acc[i][e]);
      }
    }
  }
}

// =============================================================== rotary embedding
// In place on a [T, row_stride] buffer holding `heads` heads of width dh starting
// at column col0; rotates the first `rot` channels of each head with the
// half-split convention: (a, b) = (x[i], x[i + rot/2]) ->
// (a cos - b sin, b cos + a sin). inverse != 0 applies the transposed rotation,
// which is the backward pass.
__global__ void rope_kernel(bf16* __restrict__ buf, const int* __restrict__ positions, int T,
                            long long row_stride, int col0, int heads, int dh, int rot,
                            float log2_theta, int inverse) {
  const int half = rot >> 1;
  const int pairs_per_head = half >> 1;  // two pairs per thread (bf16x2)
  const long long total = static_cast<long long>(T) * heads * pairs_per_head;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pp = static_cast<int>(idx % pairs_per_head);
    const long long rest = idx / pairs_per_head;
    const int h = static_cast<int>(rest % heads);
    const int t = static_cast<int>(rest / heads);
    const float pos = static_cast<float>(positions[t]);
    bf16* base = buf + static_cast<long long>(t) * row_stride + col0 + h * dh;
    const int i = pp * 2;
    __nv_bfloat162 a2 = *reinterpret_cast<__nv_bfloat162*>(base + i);
    __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(base + i + half);
    float2 a = __bfloat1622float2(a2), b = __bfloat1622float2(b2);
    float s0, c0, s1, c1;
    // inv_freq_i = theta^(-2i/rot)
    const float f0 = exp2f(-log2_theta * (2.f * i) / rot);
    const float f1 = exp2f(-log2_theta * (2.f * (i + 1)) / rot);
    sincosf(pos * f0, &s0, &c0);
    sincosf(pos * f1, &s1, &c1);
    if (inverse) { s0 = -s0; s1 = -s1; }
    float2 oa, ob;
    oa.x = a.x * c0 - b.x * s0; ob.x = b.x * c0 + a.x * s0;
    oa.y = a.y * c1 - b.y * s1; ob.y = b.y * c1 + a.y * s1;
    *reinterpret_cast<__nv_bfloat162*>(base + i) = __float22bfloat162_rn(oa);
    *reinterpret_cast<__nv_bfloat162*>(base + i + half) = __float22bfloat162_rn(ob);
  }
}

// Vector form: a thread owns eight adjacent frequencies of one token (its sines and
// cosines are computed once) and walks `heads_per_thread` heads with 16-byte loads, so
// the transcendental work is amortised over the heads and the kernel runs at memory
// speed. Needs rot % 16 == 0 and 16-byte aligned heads.
__global__ void rope_vec_kernel(bf16* __restrict__ buf, const int* __restrict__ positions, int T,
                                long long row_stride, int col0, int heads, int dh, int rot,
                                float log2_theta, int inverse, int slots) {
  const int half = rot >> 1;
  const int vph = half >> 3;
  const int per_token = vph * slots;
  const long long total = static_cast<long long>(T) * per_token;
  for (long long gid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; gid < total;
       gid += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(gid / per_token);
    const int r = static_cast<int>(gid % per_token);
    const int slot = r / vph;
    const int i0 = (r % vph) * 8;
    const float pos = static_cast<float>(positions[t]);
    float sn[8], cs[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float f = exp2f(-log2_theta * (2.f * (i0 + e)) / rot);
      // sin/cos of pi*(angle/pi): the argument reduction of sincospif is exact and short
      sincospif(pos * f * 0.31830988618379067f, &sn[e], &cs[e]);
      if (inverse) sn[e] = -sn[e];
    }
    bf16* row = buf + static_cast<long long>(t) * row_stride + col0 + i0;
    // up to four heads per pass with every load issued before the first use
    for (int h0 = slot; h0 < heads; h0 += 4 * slots) {
      uint4 av[4], bv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int h = h0 + k * slots;
        if (h < heads) {
          av[k] = *reinterpret_cast<const uint4*>(row + h * dh);
          bv[k] = *reinterpret_cast<const uint4*>(row + h * dh + half);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int h = h0 + k * slots;
        if (h >= heads) continue;
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&av[k]);
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&bv[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = __bfloat1622float2(a2[e]), b = __bfloat1622float2(b2[e]);
          float2 oa, ob;
          oa.x = a.x * cs[2 * e] - b.x * sn[2 * e];
          ob.x = b.x * cs[2 * e] + a.x * sn[2 * e];
          oa.y = a.y * cs[2 * e + 1] - b.y * sn[2 * e + 1];
          ob.y = b.y * cs[2 * e + 1] + a.y * sn[2 * e + 1];
          a2[e] = __float22bfloat162_rn(oa);
          b2[e] = __float22bfloat162_rn(ob);
        }
        *reinterpret_cast<uint4*>(row + h * dh) = av[k];
        *reinterpret_cast<uint4*>(row + h * dh + half) = bv[k];
      }
    }
  }
}

// idx = t * nv + c with 32-bit arithmetic whenever idx fits (a 64-bit division costs ~100 instructions)
__device__ __forceinline__ void split_index(long long idx, int nv, long long& t, int& c) {
  if (idx < (1LL << 31)) {
    const unsigned i = static_cast<unsigned>(idx), q = i / static_cast<unsigned>(nv);
    t = q; c = static_cast<int>(i - q * static_cast<unsigned>(nv));
  } else {
    t = idx / nv; c = static_cast<int>(idx - t * nv);
  }
}

// =============================================================== SwiGLU
// gu is [T, 2F] with gate in columns [0,F) and up in [F,2F) (one fused GEMM
// output). h = bf16(silu(float(gate))) * up.
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, int T, int F) {
  const int nv = F >> 3;
  const long long total = static_cast<long long>(T) * nv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long t; int c;
    split_index(idx, nv, t, c);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    float g[8], u[8], o[8];
    unpack8(row[c], g);
    unpack8(row[nv + c], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float s = __fdividef(g[e], 1.f + __expf(-g[e]));
      o[e] = __bfloat162float(__float2bfloat16_rn(s)) * u[e];
    }
    reinterpret_cast<uint4*>(h + t * F)[c] = pack8(o);
  }
}
// dgu[T,2F] from dh[T,F] and the saved gu.
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ dh,
                                  bf16* __restrict__ dgu, int T, int F) {
  const int nv = F >> 3;
  const long long total = static_cast<long long>(T) * nv;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long t; int c;
    split_index(idx, nv, t, c);
    const uint4* row = reinterpret_cast<const uint4*>(gu + t * 2 * F);
    float g[8], u[8], d[8], og[8], ou[8];
    unpack8(row[c], g);
    unpack8(row[nv + c], u);
    unpack8(reinterpret_cast<const uint4*>(dh + t * F)[c], d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sig = __fdividef(1.f, 1.f + __expf(-g[e]));
      const float s = g[e] * sig;
      ou[e] = d[e] * s;
      og[e] = d[e] * u[e] * (sig * (1.f + g[e] * (1.f - sig)));
    }
    uint4* orow = reinterpret_cast<uint4*>(dgu + t * 2 * F);
    orow[c] = pack8(og);
    orow[nv + c] = pack8(ou);
  }
}

// =============================================================== embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ W,
                                     bf16* __restrict__ out, int T, int D, int V) {
  const int nv = D >> 3;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    long long id = ids[row];
    if (id < 0 || id >= V) id = 0;
    const uint4* src = reinterpret_cast<const uint4*>(W + id * D);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * D);
    for (int c = threadIdx.x; c < nv; c += blockDim.x) dst[c] = src[c];
  }
}
// dW[id] += g[row] (fp32 accumulator table, one atomic per element).
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const bf16* __restrict__ g,
                                     float* __restrict__ dW, int T, int D, int V) {
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    long long id = ids[row];
    if (id < 0 || id >= V) continue;
    const bf16* src = g + static_cast<size_t>(row) * D;
    float* dst = dW + id * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) atomicAdd(dst + c, __bfloat162float(src[c]));
  }
}
// bf16 gradient table variant (packed bf16x2 atomics).
__global__ void embedding_bwd_bf16_kernel(const long long* __restrict__ ids,
                                          const bf16* __restrict__ g, bf16* __restrict__ dW, int T,
                                          int D, int V) {
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    long long id = ids[row];
    if (id < 0 || id >= V) continue;
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(g + static_cast<size_t>(row) * D);
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(dW + id * D);
    for (int c = threadIdx.x; c < (D >> 1); c += blockDim.x) atomicAdd(dst + c, src[c]);
  }
}

// =============================================================== cross-entropy on a logits block
// logits [R, V] bf16 (row pitch ld). For each row: lse, loss contribution
// weight * (lse - logit[target]); then the row is REWRITTEN IN PLACE with its
// gradient weight * grad_scale * (softmax - onehot). Rows with weight 0 (masked)
// produce a zero gradient row. loss_sum / weight_sum accumulate with atomics.
//
// mode 1 is the clipped policy objective on the same block: with
// logp = logit[target] - lse, r = exp(logp - old_logp), A = advantage,
//   L = -min(r A, clamp(r, 1-clip, 1+clip) A)  [+ beta * (exp(ref-logp) - (ref-logp) - 1)]
// and the row becomes weight * grad_scale * dL/dlogp * (onehot - softmax).
struct PolicyArgs {
  int mode;                 // 0 cross-entropy, 1 clipped policy
  const float* old_logp;
  const float* advantage;
  const float* ref_logp;    // optional
  float clip, ref_beta;
  float* logp_out;          // optional: per-row log-probability of the target
};
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
cross_entropy_kernel(bf16* __restrict__ logits, const long long* __restrict__ targets,
                     const float* __restrict__ weights, float* __restrict__ loss_sum,
                     float* __restrict__ lse_out, int R, int V, long long ld, float grad_scale,
                     int write_grad, PolicyArgs pa) {
  __shared__ float red[33];
  const int row = blockIdx.x;
  if (row >= R) return;
  bf16* lr = logits + static_cast<long long>(row) * ld;
  const float wgt = weights ? weights[row] : 1.f;
  const int nv = V >> 3;
  const uint4* lv = reinterpret_cast<const uint4*>(lr);
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < nv; c += CE_THREADS) {
    float f[8];
    unpack8(lv[c], f);
    float lm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) lm = fmaxf(lm, f[e]);
    if (lm > m) {
      s *= __expf(m - lm);
      m = lm;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s += __expf(f[e] - m);
  }
  for (int c = nv * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    const float f = __bfloat162float(lr[c]);
    if (f > m) { s *= __expf(m - f); m = f; }
    s += __expf(f - m);
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + __logf(gs);
  long long tgt = targets[row];
  const bool in_vocab = tgt >= 0 && tgt < V;
  const bool valid = in_vocab && wgt != 0.f;
  const float logp = in_vocab ? __bfloat162float(lr[tgt]) - lse : 0.f;
  float row_loss = -logp, dl_dlogp = -1.f;
  if (pa.mode == 1 && valid) {
    const float r = __expf(logp - pa.old_logp[row]);
    const float A = pa.advantage[row];
    const float unclipped = r * A;
    const float clipped = fminf(fmaxf(r, 1.f - pa.clip), 1.f + pa.clip) * A;
    row_loss = -fminf(unclipped, clipped);
    dl_dlogp = (unclipped <= clipped) ? -unclipped : 0.f;
    if (pa.ref_logp != nullptr) {
      const float d = pa.ref_logp[row] - logp;
      row_loss += pa.ref_beta * (__expf(d) - d - 1.f);
      dl_dlogp += pa.ref_beta * (1.f - __expf(d));
    }
  }
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[row] = lse;
    if (pa.logp_out) pa.logp_out[row] = logp;
    if (valid) atomicAdd(loss_sum, wgt * row_loss);
  }
  if (!write_grad) return;
  __syncthreads();
  const float scale = valid ? -wgt * grad_scale * dl_dlogp : 0.f;
  uint4* gv = reinterpret_cast<uint4*>(lr);
  for (int c = threadIdx.x; c < nv; c += CE_THREADS) {
    float f[8];
    unpack8(lv[c], f);
    const int base = c * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float p = __expf(f[e] - lse);
      if (base + e == tgt) p -= 1.f;
      f[e] = p * scale;
    }
    gv[c] = pack8(f);
  }
  for (int c = nv * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    float p = __expf(__bfloat162float(lr[c]) - lse);
    if (c == tgt) p -= 1.f;
    lr[c] = __float2bfloat16_rn(p * scale);
  }
}

// =============================================================== AdamW with stochastic rounding
// Philox4x32-10 counter RNG: (seed, step) key, element index counter.
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
// fp32 -> bf16: add 16 random bits below the kept mantissa, then truncate.
__device__ __forceinline__ uint16_t sr_bf16(float f, uint32_t rnd16) {
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7f800000u) == 0x7f800000u) return static_cast<uint16_t>(u >> 16);  // inf / nan
  u += (rnd16 & 0xffffu);
  return static_cast<uint16_t>(u >> 16);
}
__device__ __forceinline__ uint16_t rn_bf16(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay, bias1, bias2, grad_scale;
  unsigned long long seed;
  unsigned long long offset;  // global element offset of this flat range (sharding-invariant RNG)
  int sr_param, sr_state;
};

// p, m, v bf16; g bf16 or fp32 (g_f32). Eight elements per thread.
__global__ void adamw_sr_kernel(bf16* __restrict__ p, const void* __restrict__ g,
                                bf16* __restrict__ m, bf16* __restrict__ v, long long n, int g_f32,
                                AdamWArgs a) {
  const long long nvec = (n + 7) >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e0 = i << 3;
    const int cnt = static_cast<int>(min(8LL, n - e0));
    float pf[8], gf[8], mf[8], vf[8];
    if (cnt == 8) {
      unpack8(*reinterpret_cast<const uint4*>(p + e0), pf);
      unpack8(*reinterpret_cast<const uint4*>(m + e0), mf);
      unpack8(*reinterpret_cast<const uint4*>(v + e0), vf);
      if (g_f32) {
        const float4 g0 = *reinterpret_cast<const float4*>(static_cast<const float*>(g) + e0);
        const float4 g1 = *reinterpret_cast<const float4*>(static_cast<const float*>(g) + e0 + 4);
        gf[0] = g0.x; gf[1] = g0.y; gf[2] = g0.z; gf[3] = g0.w;
        gf[4] = g1.x; gf[5] = g1.y; gf[6] = g1.z; gf[7] = g1.w;
      } else {
        unpack8(*reinterpret_cast<const uint4*>(static_cast<const bf16*>(g) + e0), gf);
      }
    } else {
      for (int e = 0; e < 8; ++e) {
        const bool in = e < cnt;
        pf[e] = in ? __bfloat162float(p[e0 + e]) : 0.f;
        mf[e] = in ? __bfloat162float(m[e0 + e]) : 0.f;
        vf[e] = in ? __bfloat162float(v[e0 + e]) : 0.f;
        gf[e] = in ? (g_f32 ? static_cast<const float*>(g)[e0 + e]
                            : __bfloat162float(static_cast<const bf16*>(g)[e0 + e]))
                   : 0.f;
      }
    }
    const unsigned long long gidx = a.offset + static_cast<unsigned long long>(e0);
    const uint2 key = make_uint2(static_cast<uint32_t>(a.seed), static_cast<uint32_t>(a.seed >> 32));
    uint4 r[3];
#pragma unroll
    for (int k = 0; k < 3; ++k)
      r[k] = philox4x32(make_uint4(static_cast<uint32_t>(gidx >> 3), static_cast<uint32_t>(gidx >> 35),
                                   static_cast<uint32_t>(k), 0x5353u),
                        key);
    const uint32_t rw[12] = {r[0].x, r[0].y, r[0].z, r[0].w, r[1].x, r[1].y,
                             r[1].z, r[1].w, r[2].x, r[2].y, r[2].z, r[2].w};
    uint16_t po[8], mo[8], vo[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float gg = gf[e] * a.grad_scale;
      const float mn = a.beta1 * mf[e] + (1.f - a.beta1) * gg;
      const float vn = a.beta2 * vf[e] + (1.f - a.beta2) * gg * gg;
      // bias1/bias2 hold the reciprocals of the bias corrections (set by the launcher)
      const float mhat = mn * a.bias1;
      const float vhat = vn * a.bias2;
      float pn = pf[e] * (1.f - a.lr * a.weight_decay);
      pn -= a.lr * __fdividef(mhat, __fsqrt_rn(vhat) + a.eps);
      const uint32_t w0 = rw[e >> 1], w1 = rw[4 + (e >> 1)], w2 = rw[8 + (e >> 1)];
      const int sh = (e & 1) * 16;
      po[e] = a.sr_param ? sr_bf16(pn, w0 >> sh) : rn_bf16(pn);
      mo[e] = a.sr_state ? sr_bf16(mn, w1 >> sh) : rn_bf16(mn);
      vo[e] = a.sr_state ? sr_bf16(vn, w2 >> sh) : rn_bf16(vn);
    }
    if (cnt == 8) {
      uint4 u;
      u.x = po[0] | (uint32_t(po[1]) << 16); u.y = po[2] | (uint32_t(po[3]) << 16);
      u.z = po[4] | (uint32_t(po[5]) << 16); u.w = po[6] | (uint32_t(po[7]) << 16);
      *reinterpret_cast<uint4*>(p + e0) = u;
      u.x = mo[0] | (uint32_t(mo[1]) << 16); u.y = mo[2] | (uint32_t(mo[3]) << 16);
      u.z = mo[4] | (uint32_t(mo[5]) << 16); u.w = mo[6] | (uint32_t(mo[7]) << 16);
      *reinterpret_cast<uint4*>(m + e0) = u;
      u.x = vo[0] | (uint32_t(vo[1]) << 16); u.y = vo[2] | (uint32_t(vo[3]) << 16);
      u.z = vo[4] | (uint32_t(vo[5]) << 16); u.w = vo[6] | (uint32_t(vo[7]) << 16);
      *reinterpret_cast<uint4*>(v + e0) = u;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {            // static indices keep po/mo/vo in registers
        if (e < cnt) {
          p[e0 + e] = __ushort_as_bfloat16(po[e]);
          m[e0 + e] = __ushort_as_bfloat16(mo[e]);
          v[e0 + e] = __ushort_as_bfloat16(vo[e]);
        }
      }
    }
  }
}

// fp32 state variant (master-free fp32 parameters, e.g. A_log / dt_bias exceptions).
__global__ void adamw_f32_kernel(float* __restrict__ p, const float* __restrict__ g,
                                 float* __restrict__ m, float* __restrict__ v, long long n,
                                 AdamWArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float gg = g[i] * a.grad_scale;
    const float mn = a.beta1 * m[i] + (1.f - a.beta1) * gg;
    const float vn = a.beta2 * v[i] + (1.f - a.beta2) * gg * gg;
    float pn = p[i] * (1.f - a.lr * a.weight_decay);
    pn -= a.lr * (mn / a.bias1) / (sqrtf(vn / a.bias2) + a.eps);
    p[i] = pn; m[i] = mn; v[i] = vn;
  }
}

// =============================================================== sum of squares (parameter norms)
// <=256 partials then one scalar; allocation-free, mirrors the reference's two
// diagnostic kernels (packages/engine/src/shadowspill/execution/observations/kernels.py:18,40).
__global__ void sumsq_partials_kernel(const bf16* __restrict__ x, long long n,
                                      float* __restrict__ partials) {
  __shared__ float red[33];
  float acc = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float f = __bfloat162float(x[i]);
    acc += f * f;
  }
  const float t = block_sum(acc, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = t;
}
__global__ void sumsq_final_kernel(const float* __restrict__ partials, int n, float* __restrict__ out,
                                   int accumulate) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partials[i];
  const float t = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
}

// fp32 -> bf16 cast with optional scale (used to publish fp32 accumulators).
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst,
                                     long long n, float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i] * scale);
}

static inline int grid_for(long long work, int threads, int cap = 148 * 8) {
  long long g = (work + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<int>(g);
}

}  // namespace ss

extern "C" {
using namespace ss;

int ss_rmsnorm_fwd(void* x, const void* delta, const void* w, void* y, float* rstd, int T, int D,
                   float eps, int zero_centered, void* stream) {
  if (D % 8 || D > NORM_THREADS * NORM_MAXV * 8) return -2;
  if (T <= 0) return 0;
  rmsnorm_fwd_kernel<<<T < 148 * 8 ? T : 148 * 8, NORM_THREADS, 0, (cudaStream_t)stream>>>(
      (bf16*)x, (const bf16*)delta, (const bf16*)w, (bf16*)y, rstd, T, D, eps, zero_centered);
  return (int)cudaGetLastError();
}
int ss_rmsnorm_bwd(const void* x, const void* w, const void* gy, const float* rstd, void* dx,
                   float* dw, int T, int D, int zero_centered, int accumulate, void* stream) {
  if (D % 8 || D > 12288) return -2;       // the block's fp32 column sums live in 48 KB of shared memory
  if (T <= 0) return 0;
  if (D <= NORM_THREADS * NORM_MAXV * 8 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int vpt = (D / 8 + NORM_THREADS - 1) / NORM_THREADS;
    const int grid = T < 148 * 3 ? T : 148 * 3;
    auto launch = [&](auto kern) {
      kern<<<grid, NORM_THREADS, 0, (cudaStream_t)stream>>>(
          (const bf16*)x, (const bf16*)w, (const bf16*)gy, rstd, (bf16*)dx, dw, T, D, zero_centered, accumulate);
    };
    if (vpt <= 1) launch(rmsnorm_bwd_rows_kernel<1>);
    else if (vpt == 2) launch(rmsnorm_bwd_rows_kernel<2>);
    else launch(rmsnorm_bwd_rows_kernel<4>);
    return (int)cudaGetLastError();
  }
  const int row_blocks = (T + NORM_BWD_WARPS - 1) / NORM_BWD_WARPS;
  rmsnorm_bwd_kernel<<<row_blocks < 148 * 4 ? row_blocks : 148 * 4, NORM_BWD_WARPS * 32,
                       sizeof(float) * D, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)w, (const bf16*)gy, rstd, (bf16*)dx, dw, T, D, zero_centered,
      accumulate);
  return (int)cudaGetLastError();
}
int ss_rope(void* buf, const int* positions, int T, long long row_stride, int col0, int heads,
            int dh, int rot, float theta, int inverse, void* stream) {
  if (rot % 4 || rot > dh || row_stride % 2 || col0 % 2) return -2;
  if (T <= 0) return 0;
  if (rot % 16 == 0 && dh % 8 == 0 && col0 % 8 == 0 && row_stride % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(buf) & 15) == 0) {
    const int hpt = heads >= 8 ? 4 : 1;              // heads walked by one thread
    const int slots = (heads + hpt - 1) / hpt;
    const long long threads = (long long)T * (rot >> 4) * slots;
    rope_vec_kernel<<<grid_for(threads, 256), 256, 0, (cudaStream_t)stream>>>(
        (bf16*)buf, positions, T, row_stride, col0, heads, dh, rot, log2f(theta), inverse, slots);
    return (int)cudaGetLastError();
  }
  const long long total = (long long)T * heads * (rot >> 2);
  rope_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)buf, positions, T, row_stride, col0, heads, dh, rot, log2f(theta), inverse);
  return (int)cudaGetLastError();
}
int ss_swiglu_fwd(const void* gu, void* h, int T, int F, void* stream) {
  if (F % 8) return -2;
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for((long long)T * (F >> 3), 256, 148 * 16), 256, 0,
                      (cudaStream_t)stream>>>((const bf16*)gu, (bf16*)h, T, F);
  return (int)cudaGetLastError();
}
int ss_swiglu_bwd(const void* gu, const void* dh, void* dgu, int T, int F, void* stream) {
  if (F % 8) return -2;
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for((long long)T * (F >> 3), 256, 148 * 16), 256, 0,
                      (cudaStream_t)stream>>>((const bf16*)gu, (const bf16*)dh, (bf16*)dgu, T, F);
  return (int)cudaGetLastError();
}
int ss_embedding_fwd(const long long* ids, const void* W, void* out, int T, int D, int V,
                     void* stream) {
  if (D % 8) return -2;
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<T < 148 * 8 ? T : 148 * 8, 256, 0, (cudaStream_t)stream>>>(
      ids, (const bf16*)W, (bf16*)out, T, D, V);
  return (int)cudaGetLastError();
}
int ss_embedding_bwd(const long long* ids, const void* g, void* dW, int T, int D, int V,
                     int dw_f32, void* stream) {
  if (D % 2) return -2;
  if (T <= 0) return 0;
  if (dw_f32)
    embedding_bwd_kernel<<<T < 148 * 8 ? T : 148 * 8, 256, 0, (cudaStream_t)stream>>>(
        ids, (const bf16*)g, (float*)dW, T, D, V);
  else
    embedding_bwd_bf16_kernel<<<T < 148 * 8 ? T : 148 * 8, 256, 0, (cudaStream_t)stream>>>(
        ids, (const bf16*)g, (bf16*)dW, T, D, V);
  return (int)cudaGetLastError();
}
int ss_cross_entropy(void* logits, const long long* targets, const float* weights, float* loss_sum,
                     float* lse, int R, int V, long long ld, float grad_scale, int write_grad,
                     void* stream) {
  if (ld % 8) return -2;
  if (R <= 0) return 0;
  cross_entropy_kernel<<<R, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (bf16*)logits, targets, weights, loss_sum, lse, R, V, ld, grad_scale, write_grad, PolicyArgs{});
  return (int)cudaGetLastError();
}
// Token objectives on a logits block: mode 0 cross-entropy, mode 1 clipped policy
// (old_logp and advantage required; ref_logp optional). logp_out, when given,
// receives log p(target) per row.
int ss_token_objective(void* logits, const long long* targets, const float* weights, float* loss_sum,
                       float* logp_out, int R, int V, long long ld, float grad_scale, int write_grad,
                       int mode, const float* old_logp, const float* advantage, float clip,
                       const float* ref_logp, float ref_beta, void* stream) {
  if (ld % 8 || mode < 0 || mode > 1) return -2;
  if (mode == 1 && (!old_logp || !advantage)) return -2;
  if (R <= 0) return 0;
  PolicyArgs pa{mode, old_logp, advantage, ref_logp, clip, ref_beta, logp_out};
  cross_entropy_kernel<<<R, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (bf16*)logits, targets, weights, loss_sum, nullptr, R, V, ld, grad_scale, write_grad, pa);
  return (int)cudaGetLastError();
}
int ss_adamw_sr(void* p, const void* g, void* m, void* v, long long n, int g_f32, float lr,
                float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                unsigned long long seed, unsigned long long offset, int sr_param, int sr_state,
                void* stream) {
  if (n <= 0) return 0;
  if (offset % 8) return -2;
  AdamWArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f / (1.f - powf(beta1, (float)step));     // reciprocals: the kernel multiplies
  a.bias2 = 1.f / (1.f - powf(beta2, (float)step));
  a.grad_scale = grad_scale;
  a.seed = seed ^ (0x9E3779B97F4A7C15ull * (unsigned long long)(step + 1));
  a.offset = offset; a.sr_param = sr_param; a.sr_state = sr_state;
  adamw_sr_kernel<<<grid_for((n + 7) >> 3, 256, 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)p, g, (bf16*)m, (bf16*)v, n, g_f32, a);
  return (int)cudaGetLastError();
}
int ss_adamw_f32(float* p, const float* g, float* m, float* v, long long n, float lr, float beta1,
                 float beta2, float eps, float weight_decay, int step, float grad_scale,
                 void* stream) {
  if (n <= 0) return 0;
  AdamWArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bias1 = 1.f - powf(beta1, (float)step);
  a.bias2 = 1.f - powf(beta2, (float)step);
  a.grad_scale = grad_scale; a.seed = 0; a.offset = 0; a.sr_param = 0; a.sr_state = 0;
  adamw_f32_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(p, g, m, v, n, a);
  return (int)cudaGetLastError();
}
// partials: caller-provided float[256]; out: float[1].
int ss_sumsq(const void* x, long long n, float* partials, float* out, int accumulate,
             void* stream) {
  const int blocks = grid_for(n, 256 * 16, 256);
  sumsq_partials_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, n, partials);
  sumsq_final_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(partials, blocks, out, accumulate);
  return (int)cudaGetLastError();
}
int ss_cast_f32_bf16(const float* src, void* dst, long long n, float scale, void* stream) {
  if (n <= 0) return 0;
  cast_f32_bf16_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      src, (bf16*)dst, n, scale);
  return (int)cudaGetLastError();
}
}  // extern "C"
