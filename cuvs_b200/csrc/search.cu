// Host orchestration of IVF-PQ search and the small kernels around the two heavy ones
// (coarse selection in coarse.cu, code scan in scan.cuh).
//
// Stage map to the reference (cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh):
//   prep_queries_kernel ....... query cast + pad (:103-125) and rotation (:996-1025), one kernel
//   select_clusters ........... coarse.cu (:127-167)
//   chunk_and_count_kernel .... calc_chunk_indices (cpp/src/neighbors/ivf_common.cu:21-50) fused with
//                               the histogram of a counting sort by list (replaces the radix sort
//                               of :483-523)
//   scan_kernel ............... compute_similarity (scan.cuh)
//   final_merge_kernel ........ cross-probe select_k (:646-655) + postprocess_distances
//                               (ivf_common.cuh:175-252) + postprocess_neighbors (:112-169), fused
#include "ivf_pq.hpp"
#include "scan.cuh"
#include "search_internal.hpp"
#include "topk.cuh"

#include <algorithm>
#include <cmath>

namespace cuvs_b200 {
void launch_scan_bits_4(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_bits_5(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_bits_6(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_bits_7(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_bits_8(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);

void launch_scan_glut_bits_4(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_glut_bits_5(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_glut_bits_6(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_glut_bits_7(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);
void launch_scan_glut_bits_8(const scan_params&, int, bool, bool, int, int, size_t, cudaStream_t);

void launch_scan_glut(const scan_params& p, int pq_bits, int lut_kind, bool out_half, bool is_ip, int kpl,
                      int grid, size_t smem, cudaStream_t stream)
{
  switch (pq_bits) {
    case 4: launch_scan_glut_bits_4(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 5: launch_scan_glut_bits_5(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 6: launch_scan_glut_bits_6(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 7: launch_scan_glut_bits_7(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 8: launch_scan_glut_bits_8(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    default: fail("pq_bits must be within [4, 8]");
  }
}

void launch_scan(const scan_params& p, int pq_bits, int lut_kind, bool out_half, bool is_ip, int kpl,
                 int grid, size_t smem, cudaStream_t stream)
{
  switch (pq_bits) {
    case 4: launch_scan_bits_4(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 5: launch_scan_bits_5(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 6: launch_scan_bits_6(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 7: launch_scan_bits_7(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    case 8: launch_scan_bits_8(p, lut_kind, out_half, is_ip, kpl, grid, smem, stream); break;
    default: fail("pq_bits must be within [4, 8]");
  }
}
}  // namespace cuvs_b200

namespace cuvs::neighbors::ivf_pq {

using namespace cuvs_b200;

namespace {

// ------------------------------------------------------------------------------------------------
// query preparation
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float map_to_float(T x);
template <> __device__ __forceinline__ float map_to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float map_to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float map_to_float<int8_t>(int8_t x)
{
  return __fmul_rn(float(x), 1.0f / 128.0f);
}
template <> __device__ __forceinline__ float map_to_float<uint8_t>(uint8_t x)
{
  return __fmul_rn(float(x), 1.0f / 256.0f);
}

// mapping<int8_t> (cpp/src/neighbors/detail/ann_utils.cuh:178-209): floating types scale by 128 in
// their own precision and convert, int8 passes, uint8 halves.
template <typename T>
__device__ __forceinline__ int8_t map_to_int8(T x);
template <> __device__ __forceinline__ int8_t map_to_int8<float>(float x)
{
  // the float specialisation clamps before it converts (ann_utils.cuh:211-217)
  return static_cast<int8_t>(fminf(fmaxf(__fmul_rn(x, 128.0f), -128.0f), 127.0f));
}
template <> __device__ __forceinline__ int8_t map_to_int8<__half>(__half x)
{
  return static_cast<int8_t>(__hmul(x, __float2half(128.0f)));
}
template <> __device__ __forceinline__ int8_t map_to_int8<int8_t>(int8_t x) { return x; }
template <> __device__ __forceinline__ int8_t map_to_int8<uint8_t>(uint8_t x) { return static_cast<int8_t>(x >> 1); }

// One block per query.  fq = mapping<float>(query) padded to dim_ext with -0.5 (L2) or 0 in column
// `dim`; rot_q = R * fq[:dim], each output accumulated by one thread in ascending k with FMA.
// kInt8 (coarse_search_dtype = CUDA_R_8I, ivf_pq_search.cuh:171-256 and :996-1025): fq holds the
// int8 image of the query as numbers, dim_ext = round_up(dim + 2, 16) with 1 - m in column `dim` and
// -128 (L2) or 0 in the m - 1 columns after it; `rotation` is the int8 image of the rotation matrix
// and rot_q = (R8 * q8) / 128^2 (sums of integers below 2^24: exact in fp32 in any order).
// kMode 2 (coarse_search_dtype = CUDA_R_16F, ivf_pq_search.cuh:259-340): fq holds mapping<half> of the
// query as numbers, `rotation` is the half-rounded rotation matrix, rot_q the fp32 chain over them.
template <typename T, int kMode>
__global__ void prep_queries_kernel(const T* __restrict__ queries, uint32_t dim, uint32_t dim_ext,
                                    uint32_t rot_dim, int is_l2, int cosine, int identity,
                                    const float* __restrict__ rotation, float* __restrict__ fq,
                                    float* __restrict__ rot_q)
{
  constexpr bool kInt8 = kMode == 1;
  extern __shared__ float s_buf[];  // [dim] query, [rot_dim] rotated (cosine only)
  float* s_q         = s_buf;
  float* s_r         = s_buf + dim;
  const uint32_t q   = blockIdx.x;
  const T* src       = queries + size_t(q) * dim;
  float* dst         = fq + size_t(q) * dim_ext;
  for (uint32_t i = threadIdx.x; i < dim_ext; i += blockDim.x) {
    float v = 0.0f;
    if (i < dim) {
      v      = kInt8 ? static_cast<float>(map_to_int8<T>(src[i])) : map_to_float<T>(src[i]);
      // mapping<half>: integer types and half are exact; fp32 is rounded to nearest
      if constexpr (kMode == 2) { v = __half2float(__float2half_rn(v)); }
      s_q[i] = v;
    } else if constexpr (kInt8) {
      const uint32_t m = dim_ext - dim;
      v = (m == 1 || i > dim) ? (is_l2 ? -128.0f : 0.0f) : static_cast<float>(1 - int(m));
    } else if (i == dim && is_l2) {
      v = -0.5f;
    }
    dst[i] = v;
  }
  __syncthreads();
  float* out = rot_q + size_t(q) * rot_dim;
  for (uint32_t r = threadIdx.x; r < rot_dim; r += blockDim.x) {
    float acc;
    if (identity) {
      acc = s_q[r];
    } else {
      const float* row = rotation + size_t(r) * dim;
      acc              = 0.0f;
      for (uint32_t k = 0; k < dim; k++) { acc = __fmaf_rn(__ldg(row + k), s_q[k], acc); }
      if constexpr (kInt8) { acc = __fmul_rn(acc, 1.0f / 16384.0f); }
    }
    if (cosine) {
      s_r[r] = acc;
    } else {
      out[r] = acc;
    }
  }
  if (cosine) {
    __shared__ float s_norm;
    __syncthreads();
    if (threadIdx.x == 0) {
      float ss = 0.0f;
      for (uint32_t i = 0; i < rot_dim; i++) { ss = __fmaf_rn(s_r[i], s_r[i], ss); }
      s_norm = __fsqrt_rn(ss);
    }
    __syncthreads();
    const float nrm = s_norm;
    for (uint32_t r = threadIdx.x; r < rot_dim; r += blockDim.x) {
      out[r] = nrm > 0.0f ? __fdiv_rn(s_r[r], nrm) : s_r[r];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// per-probe sample offsets + counting sort of the (query, probe) pairs by list
// ------------------------------------------------------------------------------------------------
// One warp per query: chunk_index[q, p] = sum_{p' <= p} list_sizes[probes[q, p']]; list_count[l]++
// for every probe of a non-empty list.
__global__ void chunk_and_count_kernel(const uint32_t* __restrict__ probes,
                                       const uint32_t* __restrict__ list_sizes, uint32_t n_lists,
                                       uint32_t n_queries, uint32_t n_probes,
                                       uint32_t* __restrict__ chunk_index, uint32_t* __restrict__ list_count)
{
  const uint32_t q    = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (q >= n_queries) { return; }
  uint32_t carry = 0;
  for (uint32_t p0 = 0; p0 < n_probes; p0 += 32) {
    const uint32_t p = p0 + lane;
    uint32_t v       = 0;
    if (p < n_probes) {
      const uint32_t label = probes[size_t(q) * n_probes + p];
      v                    = label < n_lists ? list_sizes[label] : 0u;  // a list id out of range (caller-given probes) scans nothing
      // empty lists never reach the work list; the pairs of every query's nearest probe form a first
      // segment of the work list (buckets [0, n_lists)), all other pairs a second one
      if (v > 0) { atomicAdd(list_count + label + (p == 0 ? 0u : n_lists), 1u); }
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(kFullMask, v, d);
      if (lane >= uint32_t(d)) { v += t; }
    }
    if (p < n_probes) { chunk_index[size_t(q) * n_probes + p] = carry + v; }
    carry += __shfl_sync(kFullMask, v, 31);
  }
}

// Exclusive prefix sum over n values, in place, by one block of 1024 threads.  data[n] must exist:
// it receives the total; data must be 16-byte aligned.  Every thread owns one contiguous chunk: it
// sums the chunk (independent 16-byte loads), the 1024 sums are scanned once across the block, and
// the chunk is read again (from cache) to write the running prefix -- two barriers in all, where a
// loop over 4096-value slices needed three per slice (26 us for 50,000 lists; 6 us this way).
// `work_words` (optional): [0] = 0 (the scan kernel's work counter), [1] = the total.
__global__ void __launch_bounds__(1024) exclusive_scan_kernel(uint32_t* __restrict__ data, uint32_t n,
                                                              uint32_t* __restrict__ work_words)
{
  __shared__ uint32_t s_warp[32];
  const uint32_t tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const uint32_t per = round_up<uint32_t>(ceildiv<uint32_t>(n, 1024u), 4u);
  const uint32_t lo  = min(n, tid * per);
  const uint32_t hi  = min(n, lo + per);
  uint32_t mine      = 0;
  {
    uint32_t i = lo;
#pragma unroll 4
    for (; i + 4 <= hi; i += 4) {
      const uint4 v = *reinterpret_cast<const uint4*>(data + i);
      mine += v.x + v.y + v.z + v.w;
    }
    for (; i < hi; i++) { mine += data[i]; }
  }
  uint32_t x = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(kFullMask, x, d);
    if (lane >= uint32_t(d)) { x += t; }
  }
  if (lane == 31) { s_warp[wid] = x; }
  __syncthreads();
  if (wid == 0) {
    uint32_t w = s_warp[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t t = __shfl_up_sync(kFullMask, w, d);
      if (lane >= uint32_t(d)) { w += t; }
    }
    s_warp[lane] = w;
  }
  __syncthreads();
  uint32_t run = (wid > 0 ? s_warp[wid - 1] : 0u) + (x - mine);
  {
    uint32_t i = lo;
    for (; i + 4 <= hi; i += 4) {
      const uint4 v = *reinterpret_cast<const uint4*>(data + i);
      uint4 o;
      o.x = run;
      o.y = o.x + v.x;
      o.z = o.y + v.y;
      o.w = o.z + v.z;
      run = o.w + v.w;
      *reinterpret_cast<uint4*>(data + i) = o;
    }
    for (; i < hi; i++) {
      const uint32_t v = data[i];
      data[i]          = run;
      run += v;
    }
  }
  if (tid == 0) {
    data[n] = s_warp[31];
    if (work_words) {
      work_words[0] = 0u;
      work_words[1] = s_warp[31];
    }
  }
}

__global__ void copy_u32_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src) { *dst = *src; }

// Counters for the benchmark: sum over pairs, and over distinct probed lists, of ceil(size / 32).
__global__ void scan_stats_kernel(const uint32_t* __restrict__ list_count,
                                  const uint32_t* __restrict__ list_sizes, uint32_t n_lists,
                                  unsigned long long* __restrict__ stats)
{
  const uint32_t l = blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long a = 0, b = 0;
  const uint32_t cnt = l < n_lists ? list_count[l] + list_count[n_lists + l] : 0u;  // both segments
  if (cnt > 0) {
    const unsigned long long g = (list_sizes[l] + 31u) >> 5;
    a = g * cnt;
    b = g;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    a += __shfl_xor_sync(kFullMask, a, d);
    b += __shfl_xor_sync(kFullMask, b, d);
  }
  if ((threadIdx.x & 31) == 0 && a) {
    atomicAdd(stats, a);
    atomicAdd(stats + 1, b);
  }
}

// Work list of the scan kernel: first the pairs of every query's nearest probe, ordered by list, then all
// other pairs, ordered by list.  The first segment gives every query a bound on its k-th best score
// early, so that the rest of the scan discards most candidates (and, for L2, stops their look-ups)
// sooner; within a segment the order by list keeps concurrent groups on the same bytes in L2.
// One 32-byte descriptor per (query, probe) pair
// {pair id, query, list, list size, sample offset, first row of the list (lo, hi), 0}.
__global__ void scatter_pairs_kernel(const uint32_t* __restrict__ probes,
                                     const uint32_t* __restrict__ chunk_index,
                                     const uint32_t* __restrict__ list_sizes, uint32_t n_lists,
                                     const uint64_t* __restrict__ row_off, uint32_t n_pairs,
                                     uint32_t n_probes, uint32_t* __restrict__ cursor,
                                     uint4* __restrict__ work, uint64_t* __restrict__ out_keys, uint32_t k,
                                     uint32_t* __restrict__ query_kth, uint32_t n_queries)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) { return; }
  if (i < n_queries) { query_kth[i] = kEmptyScore; }  // no bound on any query's k-th best yet
  const uint32_t label = probes[i];
  if (label >= n_lists || list_sizes[label] == 0) {
    // nothing to scan (e.g. a list owned by another GPU): the pair's result slots are empty
    if (out_keys) {
      for (uint32_t t = 0; t < k; t++) { out_keys[size_t(i) * k + t] = kEmptyKey; }
    }
    return;
  }
  const uint32_t q     = i / n_probes;
  const uint32_t pi    = i - q * n_probes;
  const uint32_t pos   = atomicAdd(cursor + label + (pi == 0 ? 0u : n_lists), 1u);
  const uint64_t ro    = row_off[label];
  work[2 * size_t(pos)]     = make_uint4(i, q, label, list_sizes[label]);
  work[2 * size_t(pos) + 1] = make_uint4(pi > 0 ? chunk_index[i - 1] : 0u, uint32_t(ro), uint32_t(ro >> 32), 0u);
}

// Small batches: sample offsets, work descriptors (in arrival order: no sort by list), empty result
// slots and the per-query bounds in one launch.  One warp per query; `n_work` counts the non-empty
// pairs and must be zero on entry.
__global__ void small_batch_pairs_kernel(const uint32_t* __restrict__ probes,
                                         const uint32_t* __restrict__ list_sizes, uint32_t n_lists,
                                         const uint64_t* __restrict__ row_off, uint32_t n_queries,
                                         uint32_t n_probes, uint32_t* __restrict__ chunk_index,
                                         uint4* __restrict__ work, uint32_t* __restrict__ n_work,
                                         uint32_t* __restrict__ query_kth, uint64_t* __restrict__ out_keys,
                                         uint32_t k)
{
  const uint32_t q    = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (q >= n_queries) { return; }
  uint32_t carry = 0;
  for (uint32_t p0 = 0; p0 < n_probes; p0 += 32) {
    const uint32_t p = p0 + lane;
    uint32_t label = 0, size = 0;
    if (p < n_probes) {
      label = probes[size_t(q) * n_probes + p];
      size  = label < n_lists ? list_sizes[label] : 0u;
    }
    uint32_t v = size;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t t = __shfl_up_sync(kFullMask, v, d);
      if (lane >= uint32_t(d)) { v += t; }
    }
    if (p < n_probes) {
      const uint32_t pair = q * n_probes + p;
      chunk_index[pair]   = carry + v;
      if (size > 0) {
        const uint32_t pos = atomicAdd(n_work, 1u);
        const uint64_t ro  = row_off[label];
        work[2 * size_t(pos)]     = make_uint4(pair, q, label, size);
        work[2 * size_t(pos) + 1] = make_uint4(carry + v - size, uint32_t(ro), uint32_t(ro >> 32), 0u);
      } else if (out_keys) {
        for (uint32_t t = 0; t < k; t++) { out_keys[size_t(pair) * k + t] = kEmptyKey; }
      }
    }
    carry += __shfl_sync(kFullMask, v, 31);
  }
  if (lane == 0) { query_kth[q] = kEmptyScore; }
}

__global__ void fill_u32_kernel(uint32_t* p, size_t n, uint32_t v)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i < n) { p[i] = v; }
}

// ------------------------------------------------------------------------------------------------
// final selection across probes + post-processing
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float postprocess_distance(float score, int metric, float scale)
{
  switch (metric) {
    case 0: return scale != 1.0f ? __fmul_rn(score, __fmul_rn(scale, scale)) : score;
    case 1: return scale != 1.0f ? __fmul_rn(__fsqrt_rn(score), scale) : __fsqrt_rn(score);
    case 6: return __fmul_rn(score, __fmul_rn(__fmul_rn(-1.0f, scale), scale));
    default: {
      const float f = __fmul_rn(scale, scale);
      return f != 1.0f ? __fmul_rn(score, f) : score;
    }
  }
}

// One warp per query: k smallest of the n_probes * k keys, then id translation
// (binary search of the sample index in chunk_index, as find_chunk_ix does) and distance scaling.
template <int KPL>
__global__ void final_merge_kernel(const uint64_t* __restrict__ keys,
                                   const uint32_t* __restrict__ probes,
                                   const uint32_t* __restrict__ chunk_index,
                                   const uint64_t* __restrict__ row_off,
                                   const int64_t* __restrict__ ids, uint32_t n_queries,
                                   uint32_t n_probes, uint32_t k, int metric, float scale,
                                   int64_t* __restrict__ neighbors, float* __restrict__ distances)
{
  const uint32_t q    = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (q >= n_queries) { return; }
  warp_topk<KPL> queue;
  queue.init(int(k));
  const uint64_t* src = keys + size_t(q) * n_probes * k;
  const uint32_t n    = n_probes * k;
  for (uint32_t t0 = 0; t0 < n; t0 += 32) {
    const uint32_t t = t0 + lane;
    uint64_t key     = t < n ? src[t] : kEmptyKey;
    queue.offer(key, t < n);
  }
  const uint32_t* ci = chunk_index + size_t(q) * n_probes;
  const uint32_t* pr = probes + size_t(q) * n_probes;
#pragma unroll
  for (int r = 0; r < KPL; r++) {
    const uint32_t pos = uint32_t(r) * 32u + lane;
    if (pos >= k) { continue; }
    const uint64_t key = queue.a[r];
    int64_t id         = kOutOfBoundsRecord;
    float score        = INFINITY;
    if (uint32_t(key >> 32) != kEmptyScore) {
      score              = ordered_to_float(uint32_t(key >> 32));
      uint32_t sample    = uint32_t(key);
      uint32_t lo = 0, hi = n_probes;
      while (lo < hi) {
        uint32_t mid = (lo + hi) >> 1;
        if (ci[mid] <= sample) {
          lo = mid + 1;
        } else {
          hi = mid;
        }
      }
      if (lo < n_probes) {
        if (lo > 0) { sample -= ci[lo - 1]; }
        id = ids[row_off[pr[lo]] + sample];
      }
    }
    neighbors[size_t(q) * k + pos] = id;
    distances[size_t(q) * k + pos] = postprocess_distance(score, metric, scale);
  }
}

// Store-all path (k > 128): selected (score, sample index) pairs -> ids and final distances.
__global__ void translate_selected_kernel(const float* __restrict__ sel_scores,
                                          const uint32_t* __restrict__ sel_idx,
                                          const uint32_t* __restrict__ probes,
                                          const uint32_t* __restrict__ chunk_index,
                                          const uint64_t* __restrict__ row_off,
                                          const int64_t* __restrict__ ids, uint32_t n_queries,
                                          uint32_t n_probes, uint32_t k, int metric, float scale,
                                          int64_t* __restrict__ neighbors, float* __restrict__ distances)
{
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (i >= uint64_t(n_queries) * k) { return; }
  const uint32_t q   = uint32_t(i / k);
  const uint32_t* ci = chunk_index + size_t(q) * n_probes;
  const uint32_t* pr = probes + size_t(q) * n_probes;
  uint32_t sample    = sel_idx[i];
  float score        = sel_scores[i];
  int64_t id         = kOutOfBoundsRecord;
  uint32_t lo = 0, hi = n_probes;
  while (lo < hi) {
    uint32_t mid = (lo + hi) >> 1;
    if (ci[mid] <= sample) {
      lo = mid + 1;
    } else {
      hi = mid;
    }
  }
  if (lo < n_probes && score < INFINITY) {
    if (lo > 0) { sample -= ci[lo - 1]; }
    id = ids[row_off[pr[lo]] + sample];
  } else {
    score = INFINITY;
  }
  neighbors[i] = id;
  distances[i] = postprocess_distance(score, metric, scale);
}

__global__ void fill_f32_kernel(float* p, size_t n, float v)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i < n) { p[i] = v; }
}

// knn_merge_parts (cpp/src/neighbors/detail/knn_merge_parts.cuh:24-97): one warp per query.
template <int KPL>
__global__ void merge_parts_kernel(const float* __restrict__ in_dist,
                                   const int64_t* __restrict__ in_ids, size_t stride_d, size_t stride_i,
                                   uint32_t n_parts, uint32_t n_queries, uint32_t k, int select_min,
                                   float* __restrict__ out_dist, int64_t* __restrict__ out_ids)
{
  const uint32_t q    = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (q >= n_queries) { return; }
  warp_topk<KPL> queue;
  queue.init(int(k));
  const uint32_t n = n_parts * k;
  for (uint32_t t0 = 0; t0 < n; t0 += 32) {
    const uint32_t t = t0 + lane;
    uint64_t key     = kEmptyKey;
    bool valid       = false;
    if (t < n) {
      const uint32_t part = t / k, pos = t - part * k;
      const size_t src    = size_t(q) * k + pos;
      const int64_t id    = in_ids[part * stride_i + src];
      if (id != kOutOfBoundsRecord) {
        float d = in_dist[part * stride_d + src];
        key     = make_key(select_min ? d : -d, t);
        valid   = true;
      }
    }
    queue.offer(key, valid);
  }
#pragma unroll
  for (int r = 0; r < KPL; r++) {
    const uint32_t pos = uint32_t(r) * 32u + lane;
    if (pos >= k) { continue; }
    const uint64_t key = queue.a[r];
    int64_t id         = kOutOfBoundsRecord;
    float d            = select_min ? INFINITY : -INFINITY;
    if (uint32_t(key >> 32) != kEmptyScore) {
      const uint32_t t    = uint32_t(key);
      const uint32_t part = t / k, p = t - part * k;
      const size_t src    = size_t(q) * k + p;
      id                  = in_ids[part * stride_i + src];
      d                   = in_dist[part * stride_d + src];
    }
    out_ids[size_t(q) * k + pos]  = id;
    out_dist[size_t(q) * k + pos] = d;
  }
}

int kpl_for_k(uint32_t k) { return k <= 32 ? 1 : (k <= 64 ? 2 : 4); }

// Process-wide override of the coarse path (diagnostics): 0 automatic, 1 exact SIMT, 2 tensor core.
int& coarse_mode_ref()
{
  static int mode = 0;
  return mode;
}
int coarse_mode() { return coarse_mode_ref(); }

// `rotation_alt`: the int8 (mode 1) or half-rounded (mode 2) image of the rotation matrix.
void launch_prep(raft::resources& res, const index<int64_t>& idx, const void* qptr, elem_t qtype,
                 uint32_t nq, float* d_fq, float* d_rq, const float* rotation_alt = nullptr, int mode = 0)
{
  const DistanceType metric = idx.metric();
  const int is_l2  = metric == DistanceType::L2Expanded || metric == DistanceType::L2SqrtExpanded;
  const int cosine = metric == DistanceType::CosineExpanded;
  if (rotation_alt != nullptr && mode == 0) { mode = 1; }
  // the int8 image of an identity rotation is 127 on the diagonal: no shortcut there (the half image
  // of an identity matrix is the identity)
  const int ident  = mode != 1 && idx.rotation_is_identity();
  const float* rot = mode != 0 ? rotation_alt : idx.rotation_matrix();
  const uint32_t dim_ext = mode == 1 ? idx.dim_ext_int8() : idx.dim_ext();
  const size_t smem = (size_t(idx.dim()) + idx.rot_dim()) * 4;
  const int threads = 128;
  cudaStream_t stream = res.stream;
  auto launch = [&](auto* q) {
    using T = std::remove_const_t<std::remove_pointer_t<decltype(q)>>;
    if (mode == 1) {
      prep_queries_kernel<T, 1><<<nq, threads, smem, stream>>>(q, idx.dim(), dim_ext, idx.rot_dim(), is_l2,
                                                               cosine, ident, rot, d_fq, d_rq);
    } else if (mode == 2) {
      prep_queries_kernel<T, 2><<<nq, threads, smem, stream>>>(q, idx.dim(), dim_ext, idx.rot_dim(), is_l2,
                                                               cosine, ident, rot, d_fq, d_rq);
    } else {
      prep_queries_kernel<T, 0><<<nq, threads, smem, stream>>>(q, idx.dim(), dim_ext, idx.rot_dim(), is_l2,
                                                               cosine, ident, rot, d_fq, d_rq);
    }
  };
  switch (qtype) {
    case elem_t::f32: launch(reinterpret_cast<const float*>(qptr)); break;
    case elem_t::f16: launch(reinterpret_cast<const __half*>(qptr)); break;
    case elem_t::i8: launch(reinterpret_cast<const int8_t*>(qptr)); break;
    default: launch(reinterpret_cast<const uint8_t*>(qptr));
  }
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// shared-memory plan of the scan kernel
// ------------------------------------------------------------------------------------------------
int& scan_codebook_home()
{
  // 0 = choose, 1 = never tensor memory (shared or global memory instead), 2 = choose, but never an
  // instantiation made for one exact shape (tests compare it with the general kernel), 3 = behave as
  // if no look-up table fitted shared memory (the variant with the table in global memory)
  static int home = 0;
  return home;
}

scan_plan plan_scan(const raft::resources& res, const index<int64_t>& idx, int lut_kind, bool is_ip,
                    uint32_t k)
{
  scan_plan plan{};
  const size_t lut_elem  = lut_kind == LUT_F32 ? 4 : (lut_kind == LUT_F16 ? 2 : 1);
  const size_t lut_bytes = round_up<size_t>(size_t(idx.pq_dim()) * idx.pq_book_size() * lut_elem, 16);
  // base differences are stored pre-duplicated: (d, d) or (-q, -q, q*c, q*c) per rotated dimension
  const size_t base_bytes = round_up<size_t>(size_t(idx.rot_dim()) * (is_ip ? 16 : 8), 16);
  const size_t pqc_bytes =
    idx.codebook_kind() == codebook_gen::PER_SUBSPACE
      ? round_up<size_t>(size_t(idx.pq_dim()) * idx.pq_len() * idx.pq_book_size() * 4, 16)
      : 0;
  const size_t limit = size_t(res.smem_optin) - 1024;
  // Where the per-subspace codebook lives while the kernel runs: 2 = tensor memory (pq_len 1, 2 or
  // 4 and at most 128 lanes x 512 columns of fp32), 1 = shared memory, 0 = global memory.
  const uint32_t upj      = idx.pq_book_size() / 4;
  const uint32_t n_m      = ceildiv<uint32_t>(idx.pq_dim(), 128 / upj);
  const uint32_t need_col = n_m * idx.pq_len() * 4;
  const bool tmem_ok      = pqc_bytes > 0 && scan_codebook_home() != 1 && need_col <= 512 &&
                       (idx.pq_len() == 1 || idx.pq_len() == 2 || idx.pq_len() == 4);
  // (test override 3: behave as if no table fitted shared memory)
  for (int home = tmem_ok ? 2 : (pqc_bytes > 0 ? 1 : 0); home >= 0 && scan_codebook_home() != 3; home--) {
    if (home == 1 && pqc_bytes == 0) { continue; }
    for (int g = (home == 2 ? 8 : 4); g >= 1; g >>= 1) {
      const size_t merge_bytes = round_up<size_t>(size_t(1024 / g / 32) * k * 8, 16);
      const size_t fixed_part  = (home == 1 ? pqc_bytes : 0) + 16;
      // a second base-difference buffer per group where it fits (the next pair's vector is prepared
      // while the current pair's queues are merged)
      const bool base_double   = fixed_part + size_t(g) * (lut_bytes + 2 * base_bytes + merge_bytes + 16) <= limit;
      const size_t group_bytes = lut_bytes + (base_double ? 2 : 1) * base_bytes + merge_bytes + 16;
      const size_t total       = fixed_part + size_t(g) * group_bytes;
      if (total <= limit) {
        plan.n_groups      = g;
        plan.group_threads = 1024 / g;
        plan.pqc_in_smem   = home == 1;
        plan.pqc_bytes     = home == 1 ? uint32_t(pqc_bytes) : 0;
        plan.group_bytes   = uint32_t(group_bytes);
        plan.lut_bytes     = uint32_t(lut_bytes);
        plan.base_bytes    = uint32_t((base_double ? 2 : 1) * base_bytes);
        plan.base_double   = base_double ? 1 : 0;
        plan.merge_bytes   = uint32_t(merge_bytes);
        plan.total_bytes   = total;
        plan.tmem_slot_off = uint32_t(total - 16);
        plan.tmem_cols     = 0;
        if (home == 2) {
          // blocks of one thread's successive subspaces side by side, plus slack for the last
          // 16-column load of a thread, rounded to a power of two
          const uint32_t m_stride = plan.group_threads / 128;
          const uint32_t ipt      = ceildiv<uint32_t>(n_m, m_stride);
          const uint32_t need     = m_stride * ipt * idx.pq_len() * 4 + 16;
          if (need > 512) { continue; }
          uint32_t cols = 32;
          while (cols < need) { cols <<= 1; }
          plan.tmem_cols = cols;
        }
        return plan;
      }
    }
  }
  // no table fits shared memory (ivf_pq_compute_similarity_impl.cuh:441-460, conf_no_smem_lut): the
  // table of a CTA lives in global memory; shared memory holds base differences and the merge buffer
  plan.lut_global  = 1;
  plan.n_groups    = 1;
  plan.group_threads = 256;
  plan.lut_bytes   = uint32_t(lut_bytes);
  plan.base_bytes  = uint32_t(round_up<size_t>(size_t(idx.rot_dim()) * (is_ip ? 8 : 4), 16));
  plan.merge_bytes = uint32_t(round_up<size_t>(size_t(8) * k * 8, 16));
  plan.total_bytes = size_t(plan.base_bytes) + plan.merge_bytes;
  CUVS_EXPECTS(plan.total_bytes <= limit, "IVF-PQ search: rot_dim = %u is too large for this engine", idx.rot_dim());
  return plan;
}

// ------------------------------------------------------------------------------------------------
// search
// ------------------------------------------------------------------------------------------------
void check_search_params(const raft::resources& res, const search_params& params, const index<int64_t>& idx,
                         uint32_t k, bool shard)
{
  // ivf_pq_search.cuh:901-917
  CUVS_EXPECTS(params.internal_distance_dtype == CUDA_R_16F ||
                 params.internal_distance_dtype == CUDA_R_32F,
               "internal_distance_dtype must be either CUDA_R_16F or CUDA_R_32F");
  CUVS_EXPECTS(params.lut_dtype == CUDA_R_16F || params.lut_dtype == CUDA_R_32F ||
                 params.lut_dtype == CUDA_R_8U,
               "lut_dtype must be CUDA_R_16F, CUDA_R_32F or CUDA_R_8U");
  CUVS_EXPECTS(k > 0, "parameter `k` in top-k must be positive.");
  // (a shard of a list-sharded index may hold fewer than k rows: its result is padded, and an error on
  // one rank alone would leave the other ranks waiting in a collective)
  CUVS_EXPECTS(shard || int64_t(k) <= idx.size(),
               "parameter `k` (%u) in top-k must not be larger that the total size of the index (%zu)",
               k, size_t(idx.size()));
  CUVS_EXPECTS(params.n_probes > 0,
               "n_probes (number of clusters to probe in the search) must be positive.");
  CUVS_EXPECTS(idx.codes_layout() == list_layout::INTERLEAVED,
               "IVF-PQ search requires INTERLEAVED codes layout. FLAT layout is not supported for GPU search.");
  // ivf_pq_search.cuh:958-966
  CUVS_EXPECTS(params.coarse_search_dtype == CUDA_R_32F || params.coarse_search_dtype == CUDA_R_16F ||
                 params.coarse_search_dtype == CUDA_R_8I,
               "Unsupported coarse_search_dtype (only CUDA_R_32F, CUDA_R_16F, and CUDA_R_8I are supported)");
  // integer scores and rotated queries stay exact in fp32 while dim_ext * 128 * 128 <= 2^24
  CUVS_EXPECTS(params.coarse_search_dtype != CUDA_R_8I || idx.dim_ext_int8() <= 1024,
               "coarse_search_dtype CUDA_R_8I: dim = %u is too large for this engine (at most 1022)", idx.dim());
  const bool out_half = params.internal_distance_dtype == CUDA_R_16F;
  const int lut_kind =
    params.lut_dtype == CUDA_R_32F ? LUT_F32 : (params.lut_dtype == CUDA_R_16F ? LUT_F16 : LUT_FP8);
  // ivf_pq_search.cuh:697-708
  CUVS_EXPECTS(!(out_half && lut_kind == LUT_F32),
               "Unexpected lut_dtype / internal_distance_dtype combination (%d, %d). Size of the "
               "internal_distance_dtype should be not smaller than the size of the lut_dtype.",
               int(params.lut_dtype), int(params.internal_distance_dtype));
  CUVS_EXPECTS(k <= 4096, "k = %u: this engine supports k <= 4096", k);
  const uint32_t n_probes = std::min<uint32_t>(params.n_probes, idx.n_lists());
  CUVS_EXPECTS(uint64_t(idx.accum_sorted_sizes()[n_probes]) <= 0xFFFFFFFFull,
               "The maximum sample size is too big.");
  const DistanceType metric = idx.metric();
  const bool is_l2 = metric == DistanceType::L2Expanded || metric == DistanceType::L2SqrtExpanded;
  (void)plan_scan(res, idx, lut_kind, !is_l2, k > 128 ? 1 : k);  // throws when no plan exists
}

void search_any(raft::resources& res, const search_params& params, const index<int64_t>& idx,
                const void* queries, elem_t qtype, uint32_t n_queries, uint32_t k,
                int64_t* neighbors, float* distances, const uint32_t* given_probes, bitset_view filter)
{
  nvtx_range fun_scope("ivf_pq::search(n_queries = %u, n_probes = %u, k = %u, dim = %zu)", n_queries,
                       params.n_probes, k, size_t(idx.dim()));
  check_search_params(res, params, idx, k, /*shard=*/given_probes != nullptr);
  const bool coarse_i8 = params.coarse_search_dtype == CUDA_R_8I;
  const bool coarse_h  = params.coarse_search_dtype == CUDA_R_16F;
  const bool out_half = params.internal_distance_dtype == CUDA_R_16F;
  const int lut_kind =
    params.lut_dtype == CUDA_R_32F ? LUT_F32 : (params.lut_dtype == CUDA_R_16F ? LUT_F16 : LUT_FP8);
  // k <= 128: top-k fused into the scan (registers).  Larger k: the scan stores every score and a
  // separate selection follows (the reference's non-fused mode, ivf_pq_compute_similarity_impl.cuh:34-45).
  const bool store_all = k > 128;
  if (n_queries == 0) { return; }
  {
    cudaPointerAttributes a{};
    for (const void* ptr : {queries, (const void*)neighbors, (const void*)distances}) {
      cudaError_t e = cudaPointerGetAttributes(&a, ptr);
      if (e != cudaSuccess || a.type == cudaMemoryTypeUnregistered) {
        cudaGetLastError();
        fail("all pointers must be accessible from the device.");
      }
    }
  }

  const cudaStream_t stream = res.stream;
  const uint32_t n_lists    = idx.n_lists();
  const uint32_t n_probes   = std::min<uint32_t>(params.n_probes, n_lists);
  const DistanceType metric = idx.metric();
  const bool is_l2  = metric == DistanceType::L2Expanded || metric == DistanceType::L2SqrtExpanded;
  const bool is_ip  = !is_l2;
  const bool cosine = metric == DistanceType::CosineExpanded;
  const int kpl     = store_all ? 0 : kpl_for_k(k);
  const float scale = qtype == elem_t::u8 ? 256.0f : (qtype == elem_t::i8 ? 128.0f : 1.0f);

  const scan_plan plan = plan_scan(res, idx, lut_kind, is_ip, store_all ? 1 : k);
  uint32_t batch = std::min<uint32_t>(n_queries, std::max<uint32_t>(1, params.max_internal_batch_size));
  // worst-case samples per query: the n_probes largest lists (ivf_pq_search.cuh:934-940)
  const uint32_t max_samples =
    round_up<uint32_t>(std::max<uint32_t>(uint32_t(idx.accum_sorted_sizes()[n_probes]), k), 128);
  if (store_all) {
    // keep the score matrix of one internal batch within 1 GiB
    const uint64_t cap_q = std::max<uint64_t>(1, (1ull << 30) / (uint64_t(max_samples) * 4));
    batch                = uint32_t(std::min<uint64_t>(batch, cap_q));
  }
  const size_t n_pairs_max = size_t(batch) * n_probes;
  CUVS_EXPECTS(n_pairs_max < (1ull << 31), "max_internal_batch_size * n_probes is too large");

  // ---- workspace ----
  ws_layout lay;
  // the coarse stage works on the padded fp32 rows, or on the int8 images of queries and centers
  const uint32_t cdim_ext = coarse_i8 ? idx.dim_ext_int8() : idx.dim_ext();
  index<int64_t>::int8_operands op8{};
  if (coarse_i8) { op8 = idx.int8_coarse_operands(stream); }
  index<int64_t>::half_operands oph{};
  if (coarse_h) { oph = idx.half_coarse_operands(stream); }
  const size_t o_fq      = lay.add(size_t(batch) * cdim_ext * 4);
  const size_t o_rq      = lay.add(size_t(batch) * idx.rot_dim() * 4);
  const size_t o_probes  = lay.add(n_pairs_max * 4);
  const size_t o_chunk   = lay.add(n_pairs_max * 4);
  const size_t o_order   = lay.add(n_pairs_max * 32);
  const size_t o_count   = lay.add((size_t(n_lists) * 2 + 1) * 4);  // two segments of buckets, one per list each
  const size_t o_kth     = lay.add(size_t(batch) * 4);
  const size_t o_counter = lay.add(256);
  const size_t o_keys    = lay.add(store_all ? size_t(batch) * k * 8 : n_pairs_max * k * 8);
  const size_t o_all     = lay.add(store_all ? size_t(batch) * max_samples * 4 : 0);
  // half-precision scores tie in large groups, which the tensor-core path's guard (made for fp32
  // scores) does not settle: the fp16 coarse search runs on the exact SIMT path
  const bool use_tc = !coarse_h && coarse_mode() != 1 && coarse_tc_usable(n_lists, n_probes, cdim_ext);
  const size_t coarse_ws =
    given_probes ? 0
                 : (use_tc ? coarse_tc_workspace_bytes(batch, n_lists, cdim_ext)
                           : coarse_workspace_bytes(batch, n_lists, n_probes));
  const size_t o_coarse  = lay.add(coarse_ws);
  // tables in global memory: one per CTA of the (smaller) grid of that variant
  const uint32_t glut_grid = uint32_t(std::min<size_t>(n_pairs_max, size_t(res.sm_count) * 4));
  const size_t o_glut      = lay.add(plan.lut_global ? size_t(glut_grid) * plan.lut_bytes : 0);
  res.ws.reserve(lay.total());
  char* ws = res.ws.base();
  auto* d_fq      = reinterpret_cast<float*>(ws + o_fq);
  auto* d_rq      = reinterpret_cast<float*>(ws + o_rq);
  auto* d_probes  = reinterpret_cast<uint32_t*>(ws + o_probes);
  auto* d_chunk   = reinterpret_cast<uint32_t*>(ws + o_chunk);
  auto* d_order   = reinterpret_cast<uint4*>(ws + o_order);
  auto* d_count   = reinterpret_cast<uint32_t*>(ws + o_count);
  auto* d_kth     = reinterpret_cast<uint32_t*>(ws + o_kth);
  auto* d_counter = reinterpret_cast<uint32_t*>(ws + o_counter);
  auto* d_keys    = reinterpret_cast<uint64_t*>(ws + o_keys);
  auto* d_all     = reinterpret_cast<float*>(ws + o_all);
  void* d_coarse  = ws + o_coarse;

  for (uint32_t q0 = 0; q0 < n_queries; q0 += batch) {
    const uint32_t nq      = std::min(batch, n_queries - q0);
    const uint32_t n_pairs = nq * n_probes;
    const char* qptr       = static_cast<const char*>(queries) + size_t(q0) * idx.dim() * elem_size(qtype);

    nvtx_range batch_scope("ivf_pq::search-batch(queries: %u - %u)", q0, q0 + nq);
    raft::resources::stage_events ev{};
    const bool stats = res.stats_enabled;
    if (stats) { res.stats_mark(ev, 0); }

    // 1. cast / pad / rotate
    launch_prep(res, idx, qptr, qtype, nq, d_fq, d_rq, coarse_i8 ? op8.rotation : (coarse_h ? oph.rotation : nullptr),
                coarse_i8 ? 1 : (coarse_h ? 2 : 0));

    if (stats) { res.stats_mark(ev, 1); }
    // 2. coarse selection: probes sorted by (score, list id)
    {
    nvtx_range select_scope("ivf_pq::search::select_clusters(n_probes = %u, n_queries = %u, n_lists = %u, dim = %u)",
                            n_probes, nq, n_lists, idx.dim());
    if (given_probes) {
      CUDA_TRY(cudaMemcpyAsync(d_probes, given_probes + size_t(q0) * n_probes, size_t(nq) * n_probes * 4,
                               cudaMemcpyDeviceToDevice, stream));
    } else if (coarse_h) {
      select_clusters(res, oph.centers, n_lists, cdim_ext, is_l2 ? -2.0f : -1.0f, d_fq, nq, n_probes, d_probes,
                      nullptr, d_coarse, coarse_ws, /*half_scores=*/true);
    } else if (coarse_i8) {
      // integer operands are exact in TF32 and their sums in fp32: one product, no split error
      if (use_tc) {
        select_clusters_tc(res, op8.centers, op8.centers, op8.centers, op8.centers_max_norm, n_lists, cdim_ext,
                           is_l2 ? -2.0f : -1.0f, d_fq, nq, n_probes, d_probes, nullptr, d_coarse, coarse_ws,
                           /*exact_operands=*/true);
      } else {
        select_clusters(res, op8.centers, n_lists, cdim_ext, is_l2 ? -2.0f : -1.0f, d_fq, nq, n_probes,
                        d_probes, nullptr, d_coarse, coarse_ws);
      }
    } else if (use_tc) {
      select_clusters_tc(res, idx.centers(), idx.centers_hi(), idx.centers_lo(), idx.centers_max_norm(),
                         n_lists, idx.dim_ext(), is_l2 ? -2.0f : -1.0f, d_fq, nq, n_probes, d_probes,
                         nullptr, d_coarse, coarse_ws, false, idx.dim(), idx.centers_ext_scale());
    } else {
      select_clusters(res, idx.centers(), n_lists, idx.dim_ext(), is_l2 ? -2.0f : -1.0f, d_fq, nq,
                      n_probes, d_probes, nullptr, d_coarse, coarse_ws);
    }
    }

    nvtx_range worker_scope("ivf_pq::search-worker(n_queries = %u, n_probes = %u, k = %u, dim = %zu)", nq, n_probes,
                            k, size_t(idx.dim()));
    if (stats) { res.stats_mark(ev, 2); }
    // 3. sample offsets + work list of the scan
    const bool sorted_pairs = stats || n_pairs > 4096;
    if (!sorted_pairs) {
      // small batch: one launch, pairs in arrival order (a sort by list has nothing to gain here)
      CUDA_TRY(cudaMemsetAsync(d_counter, 0, 8, stream));
      small_batch_pairs_kernel<<<ceildiv<uint32_t>(nq * 32, 128), 128, 0, stream>>>(
        d_probes, idx.list_sizes(), n_lists, idx.row_offsets(), nq, n_probes, d_chunk, d_order, d_counter + 1, d_kth,
        store_all ? nullptr : d_keys, k);
      CUDA_TRY(cudaGetLastError());
      res.launches += 1;
    } else {
      // counting sort of the pairs by list
      CUDA_TRY(cudaMemsetAsync(d_count, 0, (size_t(n_lists) * 2 + 1) * 4, stream));
      chunk_and_count_kernel<<<ceildiv<uint32_t>(nq * 32, 256), 256, 0, stream>>>(
        d_probes, idx.list_sizes(), n_lists, nq, n_probes, d_chunk, d_count);
      if (stats) {
        scan_stats_kernel<<<ceildiv<uint32_t>(n_lists, 256), 256, 0, stream>>>(d_count, idx.list_sizes(),
                                                                                n_lists, res.d_stats);
        res.stat_pairs += n_pairs;
      }
      // d_counter[0] = 0 (work counter), d_counter[1] = d_count[2 * n_lists] = number of work items
      exclusive_scan_kernel<<<1, 1024, 0, stream>>>(d_count, n_lists * 2, d_counter);
      scatter_pairs_kernel<<<ceildiv<uint32_t>(n_pairs, 256), 256, 0, stream>>>(
        d_probes, d_chunk, idx.list_sizes(), n_lists, idx.row_offsets(), n_pairs, n_probes, d_count, d_order,
        store_all ? nullptr : d_keys, k, d_kth, nq);
      CUDA_TRY(cudaGetLastError());
      res.launches += 3;
    }

    if (stats) { res.stats_mark(ev, 3); }
    // 4. LUT + scan + per-pair top-k
    if (store_all) {
      const size_t n_all = size_t(nq) * max_samples;
      fill_f32_kernel<<<unsigned(ceildiv<size_t>(n_all, 256)), 256, 0, stream>>>(d_all, n_all, INFINITY);
      res.launches++;
    }
    {
      scan_params sp{};
      sp.pq_centers     = idx.pq_centers();
      sp.centers_rot    = idx.centers_rot();
      sp.codes          = idx.codes();
      sp.pq_dim         = idx.pq_dim();
      sp.pq_len         = idx.pq_len();
      sp.rot_dim        = idx.rot_dim();
      sp.n_pieces       = idx.n_pieces();
      sp.per_cluster    = idx.codebook_kind() == codebook_gen::PER_CLUSTER;
      sp.cosine         = cosine;
      sp.rot_q          = d_rq;
      sp.work           = d_order;
      sp.n_pairs        = n_pairs;
      sp.n_probes       = n_probes;
      sp.k              = k;
      sp.query_kth      = d_kth;
      sp.out_keys       = d_keys;
      sp.all_scores     = d_all;
      sp.max_samples    = max_samples;
      sp.work_counter   = d_counter;
      sp.n_work         = d_counter + 1;
      sp.ids            = idx.ids();
      sp.filter_bits    = filter.bits;
      sp.filter_nbits   = filter.n_bits;
      sp.n_groups       = plan.n_groups;
      sp.group_threads  = plan.group_threads;
      sp.pqc_in_smem    = plan.pqc_in_smem;
      sp.tmem_cols      = plan.tmem_cols;
      sp.tmem_slot_off  = plan.tmem_slot_off;
      sp.smem_pqc_bytes = plan.pqc_bytes;
      sp.smem_group_bytes = plan.group_bytes;
      sp.lut_bytes      = plan.lut_bytes;
      sp.base_bytes     = plan.base_bytes;
      sp.base_double    = plan.base_double;
      sp.merge_bytes    = plan.merge_bytes;
      sp.allow_fixed_shape = scan_codebook_home() != 2;
      if (plan.lut_global) {
        sp.lut_global = ws + o_glut;
        launch_scan_glut(sp, int(idx.pq_bits()), lut_kind, out_half, is_ip, store_all ? 0 : 4,
                         int(std::min<uint32_t>(glut_grid, n_pairs)), plan.total_bytes, stream);
      } else if (res.scan_phase_hook && n_pairs > 4096 && !store_all && n_lists >= 1) {
        // (every condition here is the same on every rank: the hook is a collective)
        // List-sharded search: every rank knows a query's k-th best only over the lists it owns, which
        // prunes less than the single-GPU search does.  So: the segment of nearest-probe pairs first
        // (after the scatter the cursor of its last bucket is the segment's end), the ranks exchange
        // the bounds they have (a min-reduction: any rank's k-th best bounds the global one from
        // above), then the other pairs with the shared bound.
        sp.n_work = d_count + (n_lists - 1);
        const int grid1 = int(std::min<uint32_t>(uint32_t(res.sm_count), ceildiv<uint32_t>(nq, plan.n_groups)));
        launch_scan(sp, int(idx.pq_bits()), lut_kind, out_half, is_ip, kpl, grid1, plan.total_bytes, stream);
        res.scan_phase_hook(stream, d_kth, nq);
        copy_u32_kernel<<<1, 1, 0, stream>>>(d_counter, d_count + (n_lists - 1));  // claims restart at segment two
        sp.n_work      = d_counter + 1;
        const int grid = int(std::min<uint32_t>(uint32_t(res.sm_count), ceildiv<uint32_t>(n_pairs, plan.n_groups)));
        launch_scan(sp, int(idx.pq_bits()), lut_kind, out_half, is_ip, kpl, grid, plan.total_bytes, stream);
        res.launches += 2;
      } else {
        const int grid = int(std::min<uint32_t>(uint32_t(res.sm_count), ceildiv<uint32_t>(n_pairs, plan.n_groups)));
        launch_scan(sp, int(idx.pq_bits()), lut_kind, out_half, is_ip, kpl, grid, plan.total_bytes, stream);
      }
      res.launches++;
    }

    if (stats) { res.stats_mark(ev, 4); }
    // 5. final selection + id translation + distance post-processing
    if (store_all) {
      auto* sel_scores = reinterpret_cast<float*>(d_keys);
      auto* sel_idx    = reinterpret_cast<uint32_t*>(d_keys) + size_t(nq) * k;
      select_rows(res, d_all, nq, max_samples, k, sel_idx, sel_scores);
      translate_selected_kernel<<<unsigned(ceildiv<uint64_t>(uint64_t(nq) * k, 256)), 256, 0, stream>>>(
        sel_scores, sel_idx, d_probes, d_chunk, idx.row_offsets(), idx.ids(), nq, n_probes, k,
        int(metric), scale, neighbors + size_t(q0) * k, distances + size_t(q0) * k);
      CUDA_TRY(cudaGetLastError());
      res.launches++;
    } else {
      const int blocks = int(ceildiv<uint32_t>(nq * 32, 128));
      int64_t* nb      = neighbors + size_t(q0) * k;
      float* ds        = distances + size_t(q0) * k;
      switch (kpl) {
        case 1:
          final_merge_kernel<1><<<blocks, 128, 0, stream>>>(d_keys, d_probes, d_chunk,
                                                            idx.row_offsets(), idx.ids(), nq, n_probes,
                                                            k, int(metric), scale, nb, ds);
          break;
        case 2:
          final_merge_kernel<2><<<blocks, 128, 0, stream>>>(d_keys, d_probes, d_chunk,
                                                            idx.row_offsets(), idx.ids(), nq, n_probes,
                                                            k, int(metric), scale, nb, ds);
          break;
        default:
          final_merge_kernel<4><<<blocks, 128, 0, stream>>>(d_keys, d_probes, d_chunk,
                                                            idx.row_offsets(), idx.ids(), nq, n_probes,
                                                            k, int(metric), scale, nb, ds);
      }
      CUDA_TRY(cudaGetLastError());
      res.launches++;
    }
    if (stats) {
      res.stats_mark(ev, 5);
      res.pending.push_back(ev);
    }
  }
}

void set_coarse_mode(int mode)
{
  // 0 auto, 1 exact SIMT path, 2 tensor-core path; 11 / 12 / 13: tensor-core path with 1 / 2 / 3
  // products of the TF32 split; 21 / 22: the same with 1 / 2 products and every operand streamed
  // (no query tile kept resident in shared memory)
  set_coarse_tc_resident(!(mode == 21 || mode == 22));
  if (mode == 21 || mode == 22) { mode -= 10; }
  if (mode >= 11 && mode <= 13) {
    set_coarse_tc_products(mode - 10);
    mode = 2;
  } else {
    set_coarse_tc_products(0);  // every handle chooses (and adapts) the number of products itself
  }
  coarse_mode_ref() = mode;
}
void set_scan_codebook_home(int home) { scan_codebook_home() = home; }

void select_probes_any(raft::resources& res, const index<int64_t>& idx, const void* queries,
                       elem_t qtype, uint32_t n_queries, uint32_t n_probes, uint32_t* probes,
                       cudaDataType_t coarse_search_dtype)
{
  if (n_queries == 0) { return; }
  const uint32_t n_lists = idx.n_lists();
  CUVS_EXPECTS(n_probes > 0 && n_probes <= n_lists, "n_probes must be within [1, n_lists]");
  CUVS_EXPECTS(coarse_search_dtype == CUDA_R_32F || coarse_search_dtype == CUDA_R_16F ||
                 coarse_search_dtype == CUDA_R_8I,
               "Unsupported coarse_search_dtype (only CUDA_R_32F, CUDA_R_16F, and CUDA_R_8I are supported)");
  const bool coarse_i8 = coarse_search_dtype == CUDA_R_8I;
  const bool coarse_h  = coarse_search_dtype == CUDA_R_16F;
  CUVS_EXPECTS(!coarse_i8 || idx.dim_ext_int8() <= 1024,
               "coarse_search_dtype CUDA_R_8I: dim = %u is too large for this engine (at most 1022)", idx.dim());
  const DistanceType metric = idx.metric();
  const bool is_l2  = metric == DistanceType::L2Expanded || metric == DistanceType::L2SqrtExpanded;
  const uint32_t cdim_ext = coarse_i8 ? idx.dim_ext_int8() : idx.dim_ext();
  index<int64_t>::int8_operands op8{};
  if (coarse_i8) { op8 = idx.int8_coarse_operands(res.stream); }
  index<int64_t>::half_operands oph{};
  if (coarse_h) { oph = idx.half_coarse_operands(res.stream); }
  const bool use_tc = !coarse_h && coarse_mode() != 1 && coarse_tc_usable(n_lists, n_probes, cdim_ext);
  const uint32_t batch = std::min<uint32_t>(n_queries, 16384);
  ws_layout lay;
  const size_t o_fq = lay.add(size_t(batch) * cdim_ext * 4);
  const size_t o_rq = lay.add(size_t(batch) * idx.rot_dim() * 4);
  const size_t cws  = use_tc ? coarse_tc_workspace_bytes(batch, n_lists, cdim_ext)
                             : coarse_workspace_bytes(batch, n_lists, n_probes);
  const size_t o_c  = lay.add(cws);
  res.ws.reserve(lay.total());
  char* ws   = res.ws.base();
  auto* d_fq = reinterpret_cast<float*>(ws + o_fq);
  auto* d_rq = reinterpret_cast<float*>(ws + o_rq);
  const float alpha = is_l2 ? -2.0f : -1.0f;
  for (uint32_t q0 = 0; q0 < n_queries; q0 += batch) {
    const uint32_t nq = std::min(batch, n_queries - q0);
    const char* qptr  = static_cast<const char*>(queries) + size_t(q0) * idx.dim() * elem_size(qtype);
    uint32_t* out     = probes + size_t(q0) * n_probes;
    launch_prep(res, idx, qptr, qtype, nq, d_fq, d_rq, coarse_i8 ? op8.rotation : (coarse_h ? oph.rotation : nullptr),
                coarse_i8 ? 1 : (coarse_h ? 2 : 0));
    if (coarse_h) {
      select_clusters(res, oph.centers, n_lists, cdim_ext, alpha, d_fq, nq, n_probes, out, nullptr, ws + o_c,
                      cws, /*half_scores=*/true);
    } else if (coarse_i8) {
      if (use_tc) {
        select_clusters_tc(res, op8.centers, op8.centers, op8.centers, op8.centers_max_norm, n_lists, cdim_ext,
                           alpha, d_fq, nq, n_probes, out, nullptr, ws + o_c, cws, /*exact_operands=*/true);
      } else {
        select_clusters(res, op8.centers, n_lists, cdim_ext, alpha, d_fq, nq, n_probes, out, nullptr,
                        ws + o_c, cws);
      }
    } else if (use_tc) {
      select_clusters_tc(res, idx.centers(), idx.centers_hi(), idx.centers_lo(), idx.centers_max_norm(),
                         n_lists, idx.dim_ext(), alpha, d_fq, nq, n_probes, out, nullptr, ws + o_c, cws, false,
                         idx.dim(), idx.centers_ext_scale());
    } else {
      select_clusters(res, idx.centers(), n_lists, idx.dim_ext(), alpha, d_fq, nq, n_probes, out, nullptr,
                      ws + o_c, cws);
    }
  }
}

void coarse_only(raft::resources& res, const index<int64_t>& idx, const void* queries, elem_t qtype,
                 uint32_t n_queries, uint32_t n_probes_in, int mode, uint32_t* probes, float* scores,
                 uint32_t* status)
{
  CUVS_EXPECTS(n_queries > 0 && n_probes_in > 0, "coarse_only: empty request");
  const uint32_t n_lists  = idx.n_lists();
  const uint32_t n_probes = std::min(n_probes_in, n_lists);
  CUVS_EXPECTS(n_probes == n_probes_in, "coarse_only: n_probes exceeds n_lists");
  const DistanceType metric = idx.metric();
  const bool is_l2 = metric == DistanceType::L2Expanded || metric == DistanceType::L2SqrtExpanded;
  const bool tc_ok = coarse_tc_usable(n_lists, n_probes, idx.dim_ext());
  CUVS_EXPECTS(mode != 2 || tc_ok, "coarse_only: the tensor-core path does not cover this shape");
  const bool use_tc = mode == 2 || (mode == 0 && tc_ok);
  ws_layout lay;
  const size_t o_fq = lay.add(size_t(n_queries) * idx.dim_ext() * 4);
  const size_t o_rq = lay.add(size_t(n_queries) * idx.rot_dim() * 4);
  const size_t cws  = use_tc ? coarse_tc_workspace_bytes(n_queries, n_lists, idx.dim_ext())
                             : coarse_workspace_bytes(n_queries, n_lists, n_probes);
  const size_t o_c  = lay.add(cws);
  res.ws.reserve(lay.total());
  char* ws    = res.ws.base();
  auto* d_fq  = reinterpret_cast<float*>(ws + o_fq);
  auto* d_rq  = reinterpret_cast<float*>(ws + o_rq);
  launch_prep(res, idx, queries, qtype, n_queries, d_fq, d_rq);
  status[0] = status[1] = 0;
  if (use_tc) {
    select_clusters_tc(res, idx.centers(), idx.centers_hi(), idx.centers_lo(), idx.centers_max_norm(),
                       n_lists, idx.dim_ext(), is_l2 ? -2.0f : -1.0f, d_fq, n_queries, n_probes, probes,
                       scores, ws + o_c, cws, false, idx.dim(), idx.centers_ext_scale());
    coarse_tc_status(res, ws + o_c, n_queries, n_lists, idx.dim_ext(), &status[0], &status[1]);
  } else {
    select_clusters(res, idx.centers(), n_lists, idx.dim_ext(), is_l2 ? -2.0f : -1.0f, d_fq, n_queries,
                    n_probes, probes, scores, ws + o_c, cws);
    res.sync();
  }
}

namespace {
// Large-k merge, step 1: part-major results -> one row of n_parts * k scores per query, smallest
// wanted first (inner-product results negated), absent results (id INT64_MAX) at +inf.
__global__ void merge_rows_kernel(const float* __restrict__ in_dist, const int64_t* __restrict__ in_ids,
                                  size_t stride_d, size_t stride_i, uint32_t n_parts, uint32_t n_queries,
                                  uint32_t k, int select_min, float* __restrict__ rows)
{
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  const uint64_t n = uint64_t(n_queries) * n_parts * k;
  if (i >= n) { return; }
  const uint32_t q    = uint32_t(i / (uint64_t(n_parts) * k));
  const uint32_t t    = uint32_t(i - uint64_t(q) * n_parts * k);
  const uint32_t part = t / k, pos = t - part * k;
  const size_t src    = size_t(q) * k + pos;
  const int64_t id    = in_ids[part * stride_i + src];
  const float d       = in_dist[part * stride_d + src];
  rows[i]             = id == kOutOfBoundsRecord ? INFINITY : (select_min ? d : -d);
}
// step 3: selected positions -> ids and distances
__global__ void merge_take_kernel(const float* __restrict__ in_dist, const int64_t* __restrict__ in_ids,
                                  size_t stride_d, size_t stride_i, uint32_t n_queries, uint32_t k,
                                  int select_min, const uint32_t* __restrict__ sel_idx,
                                  const float* __restrict__ sel_scores, float* __restrict__ out_dist,
                                  int64_t* __restrict__ out_ids)
{
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (i >= uint64_t(n_queries) * k) { return; }
  const uint32_t q = uint32_t(i / k);
  int64_t id       = kOutOfBoundsRecord;
  float d          = select_min ? INFINITY : -INFINITY;
  if (sel_scores[i] < INFINITY) {
    const uint32_t t    = sel_idx[i];
    const uint32_t part = t / k, pos = t - part * k;
    const size_t src    = size_t(q) * k + pos;
    id                  = in_ids[part * stride_i + src];
    d                   = in_dist[part * stride_d + src];
  }
  out_ids[i]  = id;
  out_dist[i] = d;
}
}  // namespace

namespace detail {
void knn_merge_parts(raft::resources& res, const float* in_dist, const int64_t* in_ids,
                     float* out_dist, int64_t* out_ids, uint32_t n_parts, uint32_t n_queries,
                     uint32_t k, bool select_min, size_t part_stride_dist, size_t part_stride_ids)
{
  CUVS_EXPECTS(k > 0 && k <= 4096, "knn_merge_parts supports 0 < k <= 4096, got %u", k);
  if (n_queries == 0) { return; }
  const size_t sd = part_stride_dist ? part_stride_dist : size_t(n_queries) * k;
  const size_t si = part_stride_ids ? part_stride_ids : size_t(n_queries) * k;
  if (k > 128) {
    // beyond the register top-k: the row selection of the store-all search path over the n_parts * k
    // candidates of a query (the reference's warp-sort merge stops at 1024,
    // cpp/src/neighbors/detail/knn_merge_parts.cuh:133-170)
    const uint32_t row_len = n_parts * k;
    ws_layout lay;
    const size_t o_rows = lay.add(size_t(n_queries) * row_len * 4);
    const size_t o_idx  = lay.add(size_t(n_queries) * k * 4);
    const size_t o_sc   = lay.add(size_t(n_queries) * k * 4);
    res.ws.reserve(lay.total());
    auto* rows = reinterpret_cast<float*>(res.ws.base() + o_rows);
    auto* idx  = reinterpret_cast<uint32_t*>(res.ws.base() + o_idx);
    auto* sc   = reinterpret_cast<float*>(res.ws.base() + o_sc);
    const uint64_t n = uint64_t(n_queries) * row_len;
    merge_rows_kernel<<<unsigned(ceildiv<uint64_t>(n, 256)), 256, 0, res.stream>>>(
      in_dist, in_ids, sd, si, n_parts, n_queries, k, select_min, rows);
    select_rows(res, rows, n_queries, row_len, k, idx, sc);
    merge_take_kernel<<<unsigned(ceildiv<uint64_t>(uint64_t(n_queries) * k, 256)), 256, 0, res.stream>>>(
      in_dist, in_ids, sd, si, n_queries, k, select_min, idx, sc, out_dist, out_ids);
    CUDA_TRY(cudaGetLastError());
    res.launches += 2;
    return;
  }
  const int blocks = int(ceildiv<uint32_t>(n_queries * 32, 128));
  const int kpl    = kpl_for_k(k);
  switch (kpl) {
    case 1:
      merge_parts_kernel<1><<<blocks, 128, 0, res.stream>>>(in_dist, in_ids, sd, si, n_parts, n_queries, k,
                                                            select_min, out_dist, out_ids);
      break;
    case 2:
      merge_parts_kernel<2><<<blocks, 128, 0, res.stream>>>(in_dist, in_ids, sd, si, n_parts, n_queries, k,
                                                            select_min, out_dist, out_ids);
      break;
    default:
      merge_parts_kernel<4><<<blocks, 128, 0, res.stream>>>(in_dist, in_ids, sd, si, n_parts, n_queries, k,
                                                            select_min, out_dist, out_ids);
  }
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}
}  // namespace detail

}  // namespace cuvs::neighbors::ivf_pq
