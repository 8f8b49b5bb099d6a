// Refinement: re-rank candidate neighbours with exact distances on the original vectors.
//
// Reference: cuvs::neighbors::refine (cpp/src/neighbors/refine/refine_device.cuh:30-138, C entry
// c/src/neighbors/refine.cpp) -- there an IVF-Flat scan over a fake one-list-per-query index; here
// one warp per query: the lanes split the dimensions of each candidate vector (coalesced row reads),
// a shuffle tree sums the partial distances and the warp keeps the k best in its register top-k.
// Candidates equal to INT64_MAX (the search's "no such neighbour" marker) or outside the dataset
// are ignored.  Results are sorted best first.
//   L2Expanded / L2Unexpanded : sum (q - x)^2        L2Sqrt*: its square root
//   InnerProduct              : sum q * x (largest first)
//   CosineExpanded            : 1 - q.x / (|q| |x|)
#include "ivf_pq.hpp"
#include "topk.cuh"

namespace cuvs::neighbors {

using namespace cuvs_b200;
using ivf_pq::elem_t;

namespace {

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p, uint32_t i);
template <> __device__ __forceinline__ float ld_as_float<float>(const float* p, uint32_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_as_float<__half>(const __half* p, uint32_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float ld_as_float<int8_t>(const int8_t* p, uint32_t i) { return float(p[i]); }
template <> __device__ __forceinline__ float ld_as_float<uint8_t>(const uint8_t* p, uint32_t i) { return float(p[i]); }

enum { REF_L2 = 0, REF_L2SQRT = 1, REF_IP = 2, REF_COS = 3 };

template <typename T, int KPL>
__global__ void refine_kernel(const T* __restrict__ dataset, int64_t n_rows, uint32_t dim,
                              const T* __restrict__ queries, uint32_t n_queries,
                              const int64_t* __restrict__ candidates, uint32_t n_cand, uint32_t k,
                              int mode, int64_t* __restrict__ indices, float* __restrict__ distances)
{
  extern __shared__ float s_query[];  // [warps per block][dim]
  const uint32_t wib  = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q    = blockIdx.x * (blockDim.x >> 5) + wib;
  if (q >= n_queries) { return; }
  float* sq     = s_query + size_t(wib) * dim;
  const T* qrow = queries + size_t(q) * dim;
  float qn      = 0.0f;
  for (uint32_t d = lane; d < dim; d += 32) {
    const float v = ld_as_float<T>(qrow, d);
    sq[d]         = v;
    qn            = __fmaf_rn(v, v, qn);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { qn += __shfl_xor_sync(kFullMask, qn, o); }
  __syncwarp();
  warp_topk<KPL> queue;
  queue.init(int(k));
  const int64_t* cand = candidates + size_t(q) * n_cand;
  for (uint32_t c0 = 0; c0 < n_cand; c0 += 32) {
    // every lane ends up with the score of candidate c0 + lane
    float my_score = INFINITY;
    bool my_valid  = false;
    const uint32_t n_here = min(32u, n_cand - c0);
    // four candidates at a time, so that their rows are in flight together (each candidate's own
    // summation order is unchanged)
    for (uint32_t j = 0; j < n_here; j += 4) {
      const T* x[4];
      bool ok[4];  // uniform across the warp
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, xn[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int64_t id = j + u < n_here ? cand[c0 + j + u] : int64_t(-1);
        ok[u]            = id >= 0 && id < n_rows;
        x[u]             = dataset + size_t(ok[u] ? id : 0) * dim;
      }
      for (uint32_t d = lane; d < dim; d += 32) {
        const float qv = sq[d];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          if (!ok[u]) { continue; }
          const float xv = ld_as_float<T>(x[u], d);
          if (mode == REF_IP) {
            acc[u] = __fmaf_rn(qv, xv, acc[u]);
          } else if (mode == REF_COS) {
            acc[u] = __fmaf_rn(qv, xv, acc[u]);
            xn[u]  = __fmaf_rn(xv, xv, xn[u]);
          } else {
            const float t = qv - xv;
            acc[u]        = __fmaf_rn(t, t, acc[u]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (!ok[u]) { continue; }
        float a = acc[u], b = xn[u];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          a += __shfl_xor_sync(kFullMask, a, o);
          b += __shfl_xor_sync(kFullMask, b, o);
        }
        float score = a;                       // smaller is better
        if (mode == REF_IP) { score = -a; }
        if (mode == REF_COS) { score = 1.0f - a / (sqrtf(qn) * sqrtf(b) + 1e-30f); }
        if (lane == j + uint32_t(u)) {
          my_score = score;
          my_valid = true;
        }
      }
    }
    queue.offer(make_key(my_score, c0 + lane), my_valid);
  }
#pragma unroll
  for (int r = 0; r < KPL; r++) {
    const uint32_t pos = uint32_t(r) * 32u + lane;
    if (pos >= k) { continue; }
    const uint64_t key = queue.a[r];
    int64_t id         = ivf_pq::kOutOfBoundsRecord;
    float d            = mode == REF_IP ? -INFINITY : INFINITY;
    if (uint32_t(key >> 32) != kEmptyScore) {
      id = cand[uint32_t(key)];
      d  = ordered_to_float(uint32_t(key >> 32));
      if (mode == REF_IP) { d = -d; }
      if (mode == REF_L2SQRT) { d = sqrtf(d); }
    }
    indices[size_t(q) * k + pos]   = id;
    distances[size_t(q) * k + pos] = d;
  }
}

template <typename T>
void launch_refine(raft::resources& res, const void* dataset, int64_t n_rows, uint32_t dim,
                   const void* queries, uint32_t n_queries, const int64_t* candidates, uint32_t n_cand,
                   uint32_t k, int mode, int64_t* indices, float* distances)
{
  const int warps   = 4;
  const size_t smem = size_t(warps) * dim * 4;
  CUVS_EXPECTS(smem <= 48 * 1024, "refine: dim = %u is too large", dim);
  const int blocks = int(ceildiv<uint32_t>(n_queries, warps));
  const T* ds      = static_cast<const T*>(dataset);
  const T* qs      = static_cast<const T*>(queries);
  if (k <= 32) {
    refine_kernel<T, 1><<<blocks, warps * 32, smem, res.stream>>>(ds, n_rows, dim, qs, n_queries, candidates,
                                                                  n_cand, k, mode, indices, distances);
  } else if (k <= 64) {
    refine_kernel<T, 2><<<blocks, warps * 32, smem, res.stream>>>(ds, n_rows, dim, qs, n_queries, candidates,
                                                                  n_cand, k, mode, indices, distances);
  } else {
    refine_kernel<T, 4><<<blocks, warps * 32, smem, res.stream>>>(ds, n_rows, dim, qs, n_queries, candidates,
                                                                  n_cand, k, mode, indices, distances);
  }
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

}  // namespace

void refine_any(raft::resources& res, const void* dataset, elem_t dtype, int64_t n_rows, uint32_t dim,
                const void* queries, uint32_t n_queries, const int64_t* candidates, uint32_t n_cand,
                ivf_pq::DistanceType metric, int64_t* indices, float* distances, uint32_t k)
{
  // refine_check_input of the reference (cpp/src/neighbors/refine/refine_common.hpp)
  CUVS_EXPECTS(k > 0 && k <= n_cand,
               "Number of neighbors cannot be smaller than k (candidates %u, k %u)", n_cand, k);
  CUVS_EXPECTS(k <= 128, "k must be less than topk::kMaxCapacity (%d).", 128);
  int mode;
  switch (metric) {
    case ivf_pq::DistanceType::L2Expanded:
    case ivf_pq::DistanceType::L2Unexpanded: mode = REF_L2; break;
    case ivf_pq::DistanceType::L2SqrtExpanded:
    case ivf_pq::DistanceType::L2SqrtUnexpanded: mode = REF_L2SQRT; break;
    case ivf_pq::DistanceType::InnerProduct: mode = REF_IP; break;
    case ivf_pq::DistanceType::CosineExpanded: mode = REF_COS; break;
    default: fail("refine: unsupported metric %d", int(metric));
  }
  if (n_queries == 0) { return; }
  switch (dtype) {
    case elem_t::f32:
      launch_refine<float>(res, dataset, n_rows, dim, queries, n_queries, candidates, n_cand, k, mode, indices, distances);
      break;
    case elem_t::f16:
      launch_refine<__half>(res, dataset, n_rows, dim, queries, n_queries, candidates, n_cand, k, mode, indices, distances);
      break;
    case elem_t::i8:
      launch_refine<int8_t>(res, dataset, n_rows, dim, queries, n_queries, candidates, n_cand, k, mode, indices, distances);
      break;
    default:
      launch_refine<uint8_t>(res, dataset, n_rows, dim, queries, n_queries, candidates, n_cand, k, mode, indices, distances);
  }
}

}  // namespace cuvs::neighbors
