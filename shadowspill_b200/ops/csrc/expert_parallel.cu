// Expert parallelism over peer memory for sm_100a: the token movement of a routed
// expert layer whose banks are split across GPUs, done by kernels that read and
// write other GPUs' memory directly (NVLink / NVSwitch, plain loads and stores).
//
//   ss_ep_layout    from the routing tables of ALL ranks (ids [R*T, k]) pick the
//                   assignments whose expert lives here, lay them out in 128-row
//                   padded expert segments, and record for every local row which
//                   assignment (rank, token, slot) it serves
//   ss_ep_pull      dispatch: every local row reads its token's hidden vector from
//                   the owning rank's buffer (one NVLink crossing, the permutation
//                   into expert order happens in the same pass; optional per-row
//                   scale read from the peer's routing weights, for the backward)
//   ss_ep_row_dst   byte address, in the owning rank's staging buffer, where each
//                   local row's result must land; the grouped GEMM's scatter
//                   epilogue stores there, so combine needs no separate transfer
//
// The reference routes through an external expert-parallel provider
// (packages/workloads/src/shadowspill_workloads/models/shared/expert_parallel/
// routing.py:6-28 `parallel_forward`; ownership rules in
// packages/workloads/src/shadowspill_workloads/components/expert_parallel.py:74-140).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ss_ep {

constexpr int MAX_RANKS = 128;

struct PeerTable {
  const void* ptr[MAX_RANKS];
};

// counts[e - e_lo]++ for every assignment routed to a local expert
__global__ void ep_count_kernel(const int* __restrict__ gids, long long n, int e_lo, int e_local,
                                int* __restrict__ counts) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = gids[i] - e_lo;
    if (e >= 0 && e < e_local) atomicAdd(counts + e, 1);
  }
}

// One block: padded offsets, the expert of each 128-row tile, zeroed cursors.
__global__ void ep_offsets_kernel(const int* __restrict__ counts, int e_local, int* __restrict__ offsets,
                                  int* __restrict__ tile_expert, int max_tiles,
                                  int* __restrict__ cursor) {
  extern __shared__ int s_off[];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_off[e_local] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) offsets[e] = s_off[e];
  for (int e = threadIdx.x; e < e_local; e += blockDim.x) cursor[e] = 0;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * 128;
    int found = -1;
    if (row < s_off[e_local]) {
      int lo = 0, hi = e_local;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      // a tile inside the padding of an expert without rows still belongs to it
      found = lo;
    }
    tile_expert[t] = found;
  }
}

__global__ void ep_fill_kernel(int* __restrict__ row_src, int rows) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x)
    row_src[i] = -1;
}

// row_src[offsets[e] + slot] = assignment index (rank * T*k + t*k + j)
__global__ void ep_assign_kernel(const int* __restrict__ gids, long long n, int e_lo, int e_local,
                                 const int* __restrict__ offsets, int* __restrict__ cursor,
                                 int* __restrict__ row_src, int capacity) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int e = gids[i] - e_lo;
    if (e < 0 || e >= e_local) continue;
    const int r = offsets[e] + atomicAdd(cursor + e, 1);
    if (r < capacity) row_src[r] = static_cast<int>(i);
  }
}

// out[r, :] = scale * x_peer[rank(r)][token(r), :]; padding rows become zero.
__global__ void ep_pull_kernel(PeerTable x, long long ldx, PeerTable w, const int* __restrict__ row_src,
                               int rows, int per_rank, int k, int D,
                               __nv_bfloat16* __restrict__ out, long long ldo) {
  const int nv = D >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const int a = row_src[r];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(r) * ldo);
    if (a < 0) {
      for (int c = threadIdx.x; c < nv; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int rank = a / per_rank;
    const int idx = a - rank * per_rank;
    const int t = idx / k;
    const uint4* src = reinterpret_cast<const uint4*>(
        static_cast<const __nv_bfloat16*>(x.ptr[rank]) + static_cast<long long>(t) * ldx);
    if (w.ptr[0] == nullptr) {
      for (int c = threadIdx.x; c < nv; c += blockDim.x) dst[c] = src[c];
    } else {
      const float s = static_cast<const float*>(w.ptr[rank])[idx];
      for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        uint4 u = src[c];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(h[e]);
          f.x *= s; f.y *= s;
          h[e] = __float22bfloat162_rn(f);
        }
        dst[c] = u;
      }
    }
  }
}

__global__ void ep_row_dst_kernel(PeerTable stage, const int* __restrict__ row_src, int rows,
                                  int per_rank, long long row_bytes, long long* __restrict__ row_dst) {
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
    const int a = row_src[r];
    if (a < 0) { row_dst[r] = 0; continue; }
    const int rank = a / per_rank;
    const int idx = a - rank * per_rank;
    row_dst[r] = reinterpret_cast<long long>(stage.ptr[rank]) + static_cast<long long>(idx) * row_bytes;
  }
}

}  // namespace ss_ep

extern "C" {
using namespace ss_ep;

// gids int32 [ranks*T*k] (rank-major); experts [e_lo, e_lo+e_local) live here.
// Outputs: counts[e_local], offsets[e_local+1], tile_expert[max_tiles], cursor[e_local]
// (scratch), row_src[capacity] with capacity = max_tiles*128.
int ss_ep_layout(const int* gids, long long n, int e_lo, int e_local, int* counts, int* offsets,
                 int* tile_expert, int max_tiles, int* cursor, int* row_src, void* stream) {
  if (e_local <= 0 || e_local > 4096 || max_tiles <= 0) return -2;
  cudaStream_t s = (cudaStream_t)stream;
  const int capacity = max_tiles * 128;
  cudaMemsetAsync(counts, 0, sizeof(int) * e_local, s);
  ep_fill_kernel<<<(capacity + 255) / 256, 256, 0, s>>>(row_src, capacity);
  if (n > 0) {
    const int blocks = (int)((n + 255) / 256 > 1184 ? 1184 : (n + 255) / 256);
    ep_count_kernel<<<blocks, 256, 0, s>>>(gids, n, e_lo, e_local, counts);
    ep_offsets_kernel<<<1, 256, sizeof(int) * (e_local + 1), s>>>(counts, e_local, offsets, tile_expert,
                                                                 max_tiles, cursor);
    ep_assign_kernel<<<blocks, 256, 0, s>>>(gids, n, e_lo, e_local, offsets, cursor, row_src, capacity);
  } else {
    ep_offsets_kernel<<<1, 256, sizeof(int) * (e_local + 1), s>>>(counts, e_local, offsets, tile_expert,
                                                                 max_tiles, cursor);
  }
  return (int)cudaGetLastError();
}

int ss_ep_pull(const void* const* x_peers, long long ldx, const void* const* w_peers, int ranks,
               const int* row_src, int rows, int per_rank, int k, int D, void* out, long long ldo,
               void* stream) {
  if (ranks <= 0 || ranks > MAX_RANKS || D % 8 || ldx % 8 || ldo % 8 || k <= 0) return -2;
  if (rows <= 0) return 0;
  PeerTable x{}, w{};
  for (int r = 0; r < ranks; ++r) {
    x.ptr[r] = x_peers[r];
    w.ptr[r] = w_peers ? w_peers[r] : nullptr;
  }
  ep_pull_kernel<<<rows > 148 * 16 ? 148 * 16 : rows, 128, 0, (cudaStream_t)stream>>>(
      x, ldx, w, row_src, rows, per_rank, k, D, (__nv_bfloat16*)out, ldo);
  return (int)cudaGetLastError();
}

int ss_ep_row_dst(const void* const* stage_peers, int ranks, const int* row_src, int rows, int per_rank,
                  long long row_bytes, long long* row_dst, void* stream) {
  if (ranks <= 0 || ranks > MAX_RANKS || row_bytes % 16) return -2;
  if (rows <= 0) return 0;
  PeerTable st{};
  for (int r = 0; r < ranks; ++r) st.ptr[r] = stage_peers[r];
  ep_row_dst_kernel<<<(rows + 255) / 256, 256, 0, (cudaStream_t)stream>>>(st, row_src, rows, per_rank,
                                                                         row_bytes, row_dst);
  return (int)cudaGetLastError();
}
}  // extern "C"
