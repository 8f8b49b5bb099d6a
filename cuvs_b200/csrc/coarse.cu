// Coarse stage: choose, for every query, the n_probes nearest inverted lists.
//
// Reference: select_clusters, cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:61-168 -- one fp32 GEMM
// (queries x centers over dim_ext, the squared norm of each center riding in column `dim` against a
// query entry of -0.5) followed by select_k.  Here the exact score of a (query, list) pair is
// defined as the fp32 FMA chain over ascending k, scaled by alpha, and probes are ordered by
// (score, list id), which makes the selection deterministic.
//
// This file holds the exact SIMT path: a register-tiled fp32 product (each output accumulated by
// one thread in ascending k, so it equals the defining chain bit for bit) and a per-query radix
// select.  It is the general path (any n_probes up to 4096, any shape).
#include "search_internal.hpp"
#include "topk.cuh"

#include <algorithm>

namespace cuvs::neighbors::ivf_pq {

using namespace cuvs_b200;

namespace {

constexpr int kTile   = 64;  // queries x lists per block
constexpr int kTileK  = 16;
constexpr uint32_t kMaxProbes = 4096;

// scores[q, l] for a chunk of queries; block = 16x16 threads, 4x4 outputs per thread.
__global__ void __launch_bounds__(256)
coarse_scores_kernel(const float* __restrict__ centers, const float* __restrict__ fq, uint32_t n_lists,
                     uint32_t n_queries, uint32_t dim_ext, float alpha, int half_scores,
                     float* __restrict__ scores)
{
  __shared__ float s_c[kTileK][kTile + 1];
  __shared__ float s_q[kTileK][kTile + 1];
  const uint32_t l0 = blockIdx.x * kTile, q0 = blockIdx.y * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
#pragma unroll
    for (int j = 0; j < 4; j++) { acc[i][j] = 0.0f; }
  }
  for (uint32_t k0 = 0; k0 < dim_ext; k0 += kTileK) {
    for (int i = threadIdx.x; i < kTile * kTileK; i += 256) {
      const int row = i / kTileK, kk = i % kTileK;
      const uint32_t k = k0 + kk;
      const uint32_t l = l0 + row, q = q0 + row;
      s_c[kk][row] = (l < n_lists && k < dim_ext) ? centers[size_t(l) * dim_ext + k] : 0.0f;
      s_q[kk][row] = (q < n_queries && k < dim_ext) ? fq[size_t(q) * dim_ext + k] : 0.0f;
    }
    __syncthreads();
    const int kmax = min(kTileK, int(dim_ext - k0));
    for (int kk = 0; kk < kmax; kk++) {
      float c[4], f[4];
#pragma unroll
      for (int j = 0; j < 4; j++) { c[j] = s_c[kk][tx + 16 * j]; }
#pragma unroll
      for (int i = 0; i < 4; i++) { f[i] = s_q[kk][ty + 16 * i]; }
#pragma unroll
      for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int j = 0; j < 4; j++) { acc[i][j] = __fmaf_rn(c[j], f[i], acc[i][j]); }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t q = q0 + ty + 16 * i;
    if (q >= n_queries) { continue; }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t l = l0 + tx + 16 * j;
      if (l < n_lists) {
        float v = __fmul_rn(alpha, acc[i][j]);
        // fp16 coarse search: the score is a half-precision number
        if (half_scores) { v = __half2float(__float2half_rn(v)); }
        scores[size_t(q) * n_lists + l] = v;
      }
    }
  }
}

// One block per query: exact n_probes smallest (score, id) of a row, written in ascending order.
// Radix select on the order-preserving image of the score (4 passes of 8 bits), one gather pass,
// then a bitonic sort of the selected keys in shared memory.
__global__ void __launch_bounds__(256)
select_probes_kernel(const float* __restrict__ scores, uint32_t n_lists, uint32_t n_probes,
                     uint32_t cap /* power of two >= n_probes */, uint32_t* __restrict__ probes,
                     float* __restrict__ scores_out)
{
  extern __shared__ uint64_t s_keys[];  // [cap]
  __shared__ uint32_t s_hist[256];
  __shared__ uint32_t s_prefix, s_remaining, s_count, s_eq_taken;
  const uint32_t q   = blockIdx.x;
  const float* row   = scores + size_t(q) * n_lists;
  const uint32_t tid = threadIdx.x;

  if (tid == 0) {
    s_prefix    = 0;
    s_remaining = n_probes;
  }
  // radix select: after the passes s_prefix is the ordered image T of the n_probes-th smallest score
  for (int pass = 0; pass < 4; pass++) {
    const int shift = 24 - 8 * pass;
    s_hist[tid]     = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask   = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (uint32_t l = tid; l < n_lists; l += 256) {
      const uint32_t o = float_to_ordered(row[l]);
      if ((o & mask) == prefix) { atomicAdd(&s_hist[(o >> shift) & 0xFFu], 1u); }
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = s_remaining, d = 0;
      for (; d < 256; d++) {
        const uint32_t c = s_hist[d];
        if (c >= rem) { break; }
        rem -= c;
      }
      s_prefix    = prefix | (d << shift);
      s_remaining = rem;  // how many elements are wanted among those sharing the new prefix
    }
    __syncthreads();
  }
  const uint32_t T       = s_prefix;
  const uint32_t want_eq = s_remaining;  // elements equal to T that belong to the selection
  if (tid == 0) {
    s_count    = 0;
    s_eq_taken = 0;
  }
  for (uint32_t i = tid; i < cap; i += 256) { s_keys[i] = kEmptyKey; }
  __syncthreads();
  // gather: everything below T, plus the want_eq lowest-numbered lists equal to T
  for (uint32_t base = 0; base < n_lists; base += 256) {
    const uint32_t l = base + tid;
    uint32_t o       = 0xFFFFFFFFu;
    if (l < n_lists) { o = float_to_ordered(row[l]); }
    if (l < n_lists && o < T) { s_keys[atomicAdd(&s_count, 1u)] = (uint64_t(o) << 32) | l; }
    // ties at T are taken in list order: ballot keeps order inside a warp, warps take turns
    const bool eq = l < n_lists && o == T;
    if (__syncthreads_or(eq)) {
      for (int w = 0; w < 8; w++) {
        if (int(tid >> 5) == w) {
          const unsigned m = __ballot_sync(kFullMask, eq);
          if (m) {
            const uint32_t start = s_eq_taken;
            const uint32_t rank  = start + __popc(m & ((1u << (tid & 31)) - 1u));
            if (eq && rank < want_eq) { s_keys[atomicAdd(&s_count, 1u)] = (uint64_t(o) << 32) | l; }
            __syncwarp();
            if ((tid & 31) == 0) { s_eq_taken = start + __popc(m); }
          }
        }
        __syncthreads();
      }
    }
  }
  __syncthreads();
  // bitonic sort of cap keys
  for (uint32_t size = 2; size <= cap; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      for (uint32_t i = tid; i < cap / 2; i += 256) {
        const uint32_t lo = 2 * i - (i & (stride - 1));
        const uint32_t hi = lo + stride;
        const bool up     = (lo & size) == 0;
        const uint64_t a = s_keys[lo], b = s_keys[hi];
        if ((a > b) == up) {
          s_keys[lo] = b;
          s_keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (uint32_t p = tid; p < n_probes; p += 256) {
    const uint64_t key                  = s_keys[p];
    probes[size_t(q) * n_probes + p]    = uint32_t(key);
    if (scores_out) { scores_out[size_t(q) * n_probes + p] = ordered_to_float(uint32_t(key >> 32)); }
  }
}

// Same product as coarse_scores_kernel, but the epilogue keeps only the per-row minimum:
// atomicMin on (ordered score << 32 | list id) implements "lowest score, then lowest id".
__global__ void __launch_bounds__(256)
assign_nearest_kernel(const float* __restrict__ centers, const float* __restrict__ x, uint32_t n_lists,
                      uint32_t n_rows, uint32_t dim_ext, float alpha, unsigned long long* __restrict__ best)
{
  __shared__ float s_c[kTileK][kTile + 1];
  __shared__ float s_q[kTileK][kTile + 1];
  const uint32_t l0 = blockIdx.x * kTile, q0 = blockIdx.y * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
#pragma unroll
    for (int j = 0; j < 4; j++) { acc[i][j] = 0.0f; }
  }
  for (uint32_t k0 = 0; k0 < dim_ext; k0 += kTileK) {
    for (int i = threadIdx.x; i < kTile * kTileK; i += 256) {
      const int row = i / kTileK, kk = i % kTileK;
      const uint32_t k = k0 + kk;
      const uint32_t l = l0 + row, q = q0 + row;
      s_c[kk][row] = (l < n_lists && k < dim_ext) ? centers[size_t(l) * dim_ext + k] : 0.0f;
      s_q[kk][row] = (q < n_rows && k < dim_ext) ? x[size_t(q) * dim_ext + k] : 0.0f;
    }
    __syncthreads();
    const int kmax = min(kTileK, int(dim_ext - k0));
    for (int kk = 0; kk < kmax; kk++) {
      float c[4], f[4];
#pragma unroll
      for (int j = 0; j < 4; j++) { c[j] = s_c[kk][tx + 16 * j]; }
#pragma unroll
      for (int i = 0; i < 4; i++) { f[i] = s_q[kk][ty + 16 * i]; }
#pragma unroll
      for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int j = 0; j < 4; j++) { acc[i][j] = __fmaf_rn(c[j], f[i], acc[i][j]); }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t q = q0 + ty + 16 * i;
    unsigned long long m = ~0ull;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const uint32_t l = l0 + tx + 16 * j;
      if (l < n_lists) {
        const unsigned long long key =
          ((unsigned long long)float_to_ordered(__fmul_rn(alpha, acc[i][j])) << 32) | l;
        m = key < m ? key : m;
      }
    }
    // the 16 threads sharing a row sit in one half-warp: reduce before touching memory
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) {
      const unsigned long long o = __shfl_xor_sync(kFullMask, m, d);
      m = o < m ? o : m;
    }
    if (tx == 0 && q < n_rows) { atomicMin(best + q, m); }
  }
}

__global__ void unpack_labels_kernel(const unsigned long long* __restrict__ best, uint32_t n,
                                     uint32_t* __restrict__ labels)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { labels[i] = uint32_t(best[i]); }
}

uint32_t chunk_queries(uint32_t n_queries, uint32_t n_lists)
{
  // keep one chunk of scores around 64 MB so that the select passes read it from L2
  const uint64_t target = 64ull << 20;
  uint64_t c            = std::max<uint64_t>(kTile, target / (uint64_t(n_lists) * 4));
  c                     = (c / kTile) * kTile;
  return uint32_t(std::min<uint64_t>(c, round_up<uint32_t>(n_queries, kTile)));
}

}  // namespace

size_t coarse_workspace_bytes(uint32_t n_queries, uint32_t n_lists, uint32_t n_probes)
{
  (void)n_probes;
  return size_t(chunk_queries(n_queries, n_lists)) * n_lists * 4;
}

void select_clusters(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                     float alpha, const float* fq, uint32_t n_queries, uint32_t n_probes,
                     uint32_t* probes, float* scores_out, void* workspace, size_t workspace_bytes,
                     bool half_scores)
{
  CUVS_EXPECTS(n_probes <= kMaxProbes, "n_probes = %u: this engine supports n_probes <= %u", n_probes,
               kMaxProbes);
  CUVS_EXPECTS(n_probes <= n_lists, "n_probes must not exceed n_lists");
  const uint32_t chunk = chunk_queries(n_queries, n_lists);
  CUVS_EXPECTS(workspace_bytes >= size_t(chunk) * n_lists * 4, "coarse workspace too small");
  float* scores = static_cast<float*>(workspace);
  uint32_t cap  = 1;
  while (cap < n_probes) { cap <<= 1; }
  cap = std::max<uint32_t>(cap, 2);
  for (uint32_t q0 = 0; q0 < n_queries; q0 += chunk) {
    const uint32_t nq = std::min(chunk, n_queries - q0);
    dim3 grid(ceildiv<uint32_t>(n_lists, kTile), ceildiv<uint32_t>(nq, kTile));
    coarse_scores_kernel<<<grid, 256, 0, res.stream>>>(centers, fq + size_t(q0) * dim_ext, n_lists,
                                                       nq, dim_ext, alpha, half_scores ? 1 : 0, scores);
    select_probes_kernel<<<nq, 256, size_t(cap) * 8, res.stream>>>(
      scores, n_lists, n_probes, cap, probes + size_t(q0) * n_probes,
      scores_out ? scores_out + size_t(q0) * n_probes : nullptr);
    CUDA_TRY(cudaGetLastError());
    res.launches += 2;
  }
}

void select_rows(raft::resources& res, const float* rows, uint32_t n_rows, uint32_t row_len, uint32_t k,
                 uint32_t* out_idx, float* out_scores)
{
  CUVS_EXPECTS(k <= kMaxProbes && k <= row_len, "select_rows: k = %u out of range", k);
  if (n_rows == 0) { return; }
  uint32_t cap = 2;
  while (cap < k) { cap <<= 1; }
  select_probes_kernel<<<n_rows, 256, size_t(cap) * 8, res.stream>>>(rows, row_len, k, cap, out_idx,
                                                                     out_scores);
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

void assign_nearest(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                    float alpha, const float* x_ext, uint32_t n_rows, uint32_t* labels,
                    unsigned long long* best)
{
  if (n_rows == 0) { return; }
  CUDA_TRY(cudaMemsetAsync(best, 0xFF, size_t(n_rows) * 8, res.stream));
  // grid.y is limited to 65535 blocks of 64 rows
  const uint32_t max_rows = 65535u * kTile;
  for (uint32_t r0 = 0; r0 < n_rows; r0 += max_rows) {
    const uint32_t nr = std::min(max_rows, n_rows - r0);
    dim3 grid(ceildiv<uint32_t>(n_lists, kTile), ceildiv<uint32_t>(nr, kTile));
    assign_nearest_kernel<<<grid, 256, 0, res.stream>>>(centers, x_ext + size_t(r0) * dim_ext, n_lists,
                                                        nr, dim_ext, alpha, best + r0);
  }
  unpack_labels_kernel<<<ceildiv<uint32_t>(n_rows, 256), 256, 0, res.stream>>>(best, n_rows, labels);
  CUDA_TRY(cudaGetLastError());
  res.launches += 2;
}

}  // namespace cuvs::neighbors::ivf_pq
