// Oracle pin, device build: compiles the scoring code of the reference's IVF-PQ search, unmodified
// and from where it lies in the reference checkout, with nvcc into a small library that runs on the
// GPU.  The parity tests run it next to the C restatement (ivfpq_oracle.c) and next to the product's
// scan kernel and compare bytes.  TEST INFRASTRUCTURE ONLY; built into oracle/_ref/ by the Makefile.
//
// Reference code compiled here (paths inside the reference project):
//   cpp/src/neighbors/ivf_pq/ivf_pq_fp_8bit.cuh                                   fp_8bit<5, Signed>
//   cpp/src/neighbors/ivf_pq/detail/jit_lto_kernels/precompute_base_diff_impl.cuh base differences
//   cpp/src/neighbors/ivf_pq/detail/jit_lto_kernels/create_lut_impl.cuh           look-up table
//   cpp/src/neighbors/ivf_pq/detail/jit_lto_kernels/compute_score_impl.cuh        code unpack + score
//   cpp/src/neighbors/ivf_pq/detail/jit_lto_kernels/increment_score_impl.cuh      cosine increment
//   cpp/src/neighbors/ivf_pq/detail/jit_lto_kernels/get_line_width_impl.cuh       bytes per 32 rows
//   cpp/src/neighbors/detail/ann_utils.cuh      config<> and mapping<> (an excerpt: the rest of that
//                                               header manages memory through un-vendored libraries)
//   cpp/src/neighbors/ivf_common.cuh            kOutOfBoundsRecord, find_chunk_ix,
//                                               postprocess_neighbors, postprocess_distances (excerpt)
// The two excerpts are cut out of the reference files at build time (oracle.py, build_ref_pin_dev)
// into oracle/_ref/extract/, which is not tracked.  Everything these files include from
// un-vendored libraries (RAFT, RMM) is replaced by the stand-ins in ref_shims/.
//
// The driver kernel below does what compute_similarity_impl.cuh:110-170 and
// compute_distances_impl.cuh:52-93 do for one (query, probe) pair -- base differences, table,
// barrier, one score per row addressed as the reference addresses the interleaved list -- without
// the top-k (every score is written out) and without pruning (early-stop limit = +inf).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <type_traits>
#include <vector>

#include <raft/linalg/map.cuh>
#include <raft/util/cuda_utils.cuh>
#include <raft/util/pow2_utils.cuh>
#include <raft/util/vectorized.cuh>
#include <cuvs/distance/distance.hpp>

#include "ivf_pq_fp_8bit.cuh"
#include "detail/jit_lto_kernels/precompute_base_diff_impl.cuh"
#include "detail/jit_lto_kernels/create_lut_impl.cuh"
#include "detail/jit_lto_kernels/compute_score_impl.cuh"
#include "detail/jit_lto_kernels/increment_score_impl.cuh"
#include "detail/jit_lto_kernels/get_line_width_impl.cuh"

namespace cuvs::spatial::knn::detail::utils {
#include "extract/ann_utils_mapping.inc"
}
namespace cuvs::neighbors::ivf::detail {
#include "extract/ivf_common_postprocess.inc"
}

namespace pin {
using namespace cuvs::neighbors::ivf_pq;
using namespace cuvs::neighbors::ivf_pq::detail;
using vec_t = raft::TxN_t<uint32_t, kIndexGroupVecLen / sizeof(uint32_t)>;  // device_functions.cuh:17

template <typename T>
__device__ float widen(T v)
{
  return float(v);
}

template <typename OutT, typename LutT, typename MetricTag, bool Precomp, uint32_t PqBits, bool Increment>
__global__ void pair_kernel(uint32_t rot_dim, uint32_t pq_dim, uint32_t pq_len, int per_cluster,
                            const float* pair_query, const uint32_t* pair_label, const float* centers_rot,
                            const float* pq_centers, const uint8_t* codes, const uint64_t* code_off,
                            const uint32_t* list_sizes, uint32_t max_rows, uint8_t* lut_out, float* scores_out)
{
  extern __shared__ __align__(256) uint8_t smem_buf[];
  const uint32_t pair         = blockIdx.x;
  const uint32_t label        = pair_label[pair];
  const float* query          = pair_query + size_t(pair) * rot_dim;
  const float* cluster_center = centers_rot + size_t(label) * rot_dim;
  const uint32_t lut_size     = pq_dim << PqBits;
  // prepare_lut_impl.cuh:24-26 with the table in shared memory
  LutT* lut_scores = reinterpret_cast<LutT*>(smem_buf);
  uint8_t* lut_end = reinterpret_cast<uint8_t*>(lut_scores + lut_size);
  if constexpr (Precomp) {
    if constexpr (std::is_same_v<MetricTag, tag_metric_euclidean>) {
      precompute_base_diff_euclidean_impl(rot_dim, lut_end, query, cluster_center);
    } else {
      precompute_base_diff_inner_product_impl(rot_dim, lut_end, query, cluster_center);
    }
  } else {
    precompute_base_diff_none_impl(rot_dim, lut_end, query, cluster_center);
  }
  create_lut_impl<LutT, MetricTag, Precomp, PqBits>(
    pq_dim, pq_len, label, pq_centers, per_cluster ? codebook_gen::PER_CLUSTER : codebook_gen::PER_SUBSPACE,
    lut_scores, lut_end, query, cluster_center);
  __threadfence_block();
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < lut_size * sizeof(LutT); i += blockDim.x) {
    lut_out[size_t(pair) * lut_size * sizeof(LutT) + i] = reinterpret_cast<const uint8_t*>(lut_scores)[i];
  }
  // compute_distances_impl.cuh:47-93
  using group_align            = raft::Pow2<kIndexGroupSize>;
  using vec_align              = raft::Pow2<kIndexGroupVecLen>;
  const uint32_t n_samples     = list_sizes[label];
  uint32_t n_samples_aligned   = group_align::roundUp(n_samples);
  uint32_t pq_line_width       = get_line_width_impl<PqBits>(pq_dim);
  const uint8_t* pq_thread_data = codes + code_off[label] + group_align::roundDown(threadIdx.x) * pq_line_width +
                                  group_align::mod(threadIdx.x) * vec_align::Value;
  pq_line_width *= blockDim.x;
  const OutT early_stop_limit = OutT(std::numeric_limits<float>::infinity());
  for (uint32_t i = threadIdx.x; i < n_samples_aligned; i += blockDim.x, pq_thread_data += pq_line_width) {
    if (i < n_samples) {
      OutT score = compute_score_impl<OutT, LutT, vec_t, PqBits>(
        pq_dim, reinterpret_cast<const vec_t::io_t*>(pq_thread_data), lut_scores, early_stop_limit);
      score = increment_score_impl<OutT, Increment>(score);
      scores_out[size_t(pair) * max_rows + i] = widen(score);
    }
  }
}

struct pair_args {
  uint32_t rot_dim, pq_dim, pq_len;
  int per_cluster;
  const float *pair_query, *centers_rot, *pq_centers;
  const uint32_t *pair_label, *list_sizes;
  const uint8_t* codes;
  const uint64_t* code_off;
  uint32_t max_rows, n_pairs;
  uint8_t* lut_out;
  float* scores_out;
  int threads;
};

template <typename OutT, typename LutT, typename MetricTag, bool Precomp, uint32_t PqBits, bool Increment>
int launch(const pair_args& a)
{
  auto kernel = pair_kernel<OutT, LutT, MetricTag, Precomp, PqBits, Increment>;
  const size_t smem = (size_t(a.pq_dim) << PqBits) * sizeof(LutT) + size_t(a.rot_dim) * 8 + 256;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
    cudaGetLastError();
    return -3;  // table does not fit in shared memory
  }
  kernel<<<a.n_pairs, a.threads, smem>>>(a.rot_dim, a.pq_dim, a.pq_len, a.per_cluster, a.pair_query,
                                        a.pair_label, a.centers_rot, a.pq_centers, a.codes, a.code_off,
                                        a.list_sizes, a.max_rows, a.lut_out, a.scores_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <typename OutT, typename LutT, typename MetricTag, bool Precomp, uint32_t PqBits>
int by_increment(const pair_args& a, int increment)
{
  if constexpr (std::is_same_v<MetricTag, tag_metric_inner_product>) {
    if (increment) { return launch<OutT, LutT, MetricTag, Precomp, PqBits, true>(a); }
  }
  return launch<OutT, LutT, MetricTag, Precomp, PqBits, false>(a);
}
template <typename OutT, typename LutT, typename MetricTag, bool Precomp>
int by_bits(const pair_args& a, uint32_t bits, int increment)
{
  switch (bits) {
    case 4: return by_increment<OutT, LutT, MetricTag, Precomp, 4>(a, increment);
    case 5: return by_increment<OutT, LutT, MetricTag, Precomp, 5>(a, increment);
    case 6: return by_increment<OutT, LutT, MetricTag, Precomp, 6>(a, increment);
    case 7: return by_increment<OutT, LutT, MetricTag, Precomp, 7>(a, increment);
    case 8: return by_increment<OutT, LutT, MetricTag, Precomp, 8>(a, increment);
    default: return -2;
  }
}
template <typename OutT, typename LutT, typename MetricTag>
int by_precomp(const pair_args& a, int precomp, uint32_t bits, int increment)
{
  return precomp ? by_bits<OutT, LutT, MetricTag, true>(a, bits, increment)
                 : by_bits<OutT, LutT, MetricTag, false>(a, bits, increment);
}
// the table types the reference pairs with each metric (ivf_pq_search.cuh:720-731): the unsigned
// 8-bit float for L2, the signed one for inner product and cosine
template <typename OutT, typename MetricTag>
int by_lut(const pair_args& a, int lut_kind, int precomp, uint32_t bits, int increment)
{
  constexpr bool kSigned = std::is_same_v<MetricTag, tag_metric_inner_product>;
  switch (lut_kind) {
    case 0:
      if constexpr (std::is_same_v<OutT, float>) {
        return by_precomp<OutT, float, MetricTag>(a, precomp, bits, increment);
      } else {
        return -2;
      }
    case 1: return by_precomp<OutT, half, MetricTag>(a, precomp, bits, increment);
    case 2: return by_precomp<OutT, fp_8bit<5, kSigned>, MetricTag>(a, precomp, bits, increment);
    default: return -2;
  }
}

template <typename T>
struct dev_buf {
  T* p = nullptr;
  size_t n = 0;
  explicit dev_buf(size_t count) : n(count) { cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)); }
  dev_buf(const T* host, size_t count) : dev_buf(count)
  {
    if (count) { cudaMemcpy(p, host, count * sizeof(T), cudaMemcpyHostToDevice); }
  }
  ~dev_buf() { cudaFree(p); }
  void to_host(T* host) const
  {
    if (n) { cudaMemcpy(host, p, n * sizeof(T), cudaMemcpyDeviceToHost); }
  }
};

// ---- element-wise kernels over the reference's small value types --------------------------------
template <bool Signed>
__global__ void fp8_kernel(const float* in, size_t n, uint8_t* enc, float* dec32, uint16_t* dec16)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i >= n) { return; }
  fp_8bit<5, Signed> v(in[i]);
  enc[i]   = v.bitstring;
  dec32[i] = float(v);
  half h   = half(v);
  dec16[i] = *reinterpret_cast<uint16_t*>(&h);
}
template <bool Signed>
__global__ void fp8_decode_kernel(const uint8_t* in, size_t n, float* dec32, uint16_t* dec16)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i >= n) { return; }
  fp_8bit<5, Signed> v(in[i]);
  dec32[i] = float(v);
  half h   = half(v);
  dec16[i] = *reinterpret_cast<uint16_t*>(&h);
}
template <typename D, typename S>
__global__ void mapping_kernel(const S* in, size_t n, D* out)
{
  size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i < n) { out[i] = cuvs::spatial::knn::detail::utils::mapping<D>{}(in[i]); }
}
template <typename D, typename S>
int run_mapping(const void* in, size_t n, void* out)
{
  dev_buf<S> d_in(static_cast<const S*>(in), n);
  dev_buf<D> d_out(n);
  mapping_kernel<D, S><<<unsigned((n + 255) / 256), 256>>>(d_in.p, n, d_out.p);
  if (cudaDeviceSynchronize() != cudaSuccess) { return -4; }
  d_out.to_host(static_cast<D*>(out));
  return 0;
}
}  // namespace pin

#define PIN_EXPORT extern "C" __attribute__((visibility("default")))

// Scores and tables of n_pairs (query, list) pairs.  lut_kind: 0 fp32, 1 fp16, 2 8-bit; scores come
// back widened to fp32 (exact for fp16).  Returns 0, or a negative code (-2 unsupported combination,
// -3 table larger than shared memory, -4 CUDA error).
PIN_EXPORT int refdev_pairs(int lut_kind, int out_half, int is_ip, int increment, int precomp, uint32_t pq_bits,
                            int per_cluster, uint32_t pq_dim, uint32_t pq_len, uint32_t n_pairs,
                            const float* pair_query, const uint32_t* pair_label, uint32_t n_lists,
                            const float* centers_rot, const float* pq_centers, uint64_t pq_centers_count,
                            const uint8_t* codes, uint64_t codes_bytes, const uint64_t* code_off,
                            const uint32_t* list_sizes, uint32_t max_rows, uint8_t* lut_out,
                            float* scores_out, int threads)
{
  using namespace pin;
  const uint32_t rot_dim = pq_dim * pq_len;
  const size_t lut_elem  = lut_kind == 0 ? 4 : (lut_kind == 1 ? 2 : 1);
  const size_t lut_bytes = (size_t(pq_dim) << pq_bits) * lut_elem;
  dev_buf<float> d_q(pair_query, size_t(n_pairs) * rot_dim), d_c(centers_rot, size_t(n_lists) * rot_dim),
    d_pq(pq_centers, pq_centers_count);
  dev_buf<uint32_t> d_label(pair_label, n_pairs), d_sizes(list_sizes, n_lists);
  dev_buf<uint8_t> d_codes(codes, codes_bytes), d_lut(size_t(n_pairs) * lut_bytes);
  dev_buf<uint64_t> d_off(code_off, n_lists);
  dev_buf<float> d_scores(size_t(n_pairs) * max_rows);
  cudaMemset(d_scores.p, 0xff, d_scores.n * sizeof(float));
  pair_args a{rot_dim, pq_dim, pq_len, per_cluster, d_q.p, d_c.p, d_pq.p, d_label.p, d_sizes.p, d_codes.p,
              d_off.p, max_rows, n_pairs, d_lut.p, d_scores.p, threads};
  int rc;
  if (is_ip) {
    rc = out_half ? by_lut<half, tag_metric_inner_product>(a, lut_kind, precomp, pq_bits, increment)
                  : by_lut<float, tag_metric_inner_product>(a, lut_kind, precomp, pq_bits, increment);
  } else {
    rc = out_half ? by_lut<half, tag_metric_euclidean>(a, lut_kind, precomp, pq_bits, 0)
                  : by_lut<float, tag_metric_euclidean>(a, lut_kind, precomp, pq_bits, 0);
  }
  if (rc != 0) { return rc; }
  if (cudaDeviceSynchronize() != cudaSuccess) { return -4; }
  d_lut.to_host(lut_out);
  d_scores.to_host(scores_out);
  return 0;
}

PIN_EXPORT int refdev_fp8(const float* in, uint64_t n, int is_signed, uint8_t* enc, float* dec32, uint16_t* dec16)
{
  using namespace pin;
  dev_buf<float> d_in(in, n), d_32(n);
  dev_buf<uint8_t> d_enc(n);
  dev_buf<uint16_t> d_16(n);
  const unsigned blocks = unsigned((n + 255) / 256);
  if (is_signed) {
    fp8_kernel<true><<<blocks, 256>>>(d_in.p, n, d_enc.p, d_32.p, d_16.p);
  } else {
    fp8_kernel<false><<<blocks, 256>>>(d_in.p, n, d_enc.p, d_32.p, d_16.p);
  }
  if (cudaDeviceSynchronize() != cudaSuccess) { return -4; }
  d_enc.to_host(enc);
  d_32.to_host(dec32);
  d_16.to_host(dec16);
  return 0;
}

PIN_EXPORT int refdev_fp8_decode(const uint8_t* in, uint64_t n, int is_signed, float* dec32, uint16_t* dec16)
{
  using namespace pin;
  dev_buf<uint8_t> d_in(in, n);
  dev_buf<float> d_32(n);
  dev_buf<uint16_t> d_16(n);
  const unsigned blocks = unsigned((n + 255) / 256);
  if (is_signed) {
    fp8_decode_kernel<true><<<blocks, 256>>>(d_in.p, n, d_32.p, d_16.p);
  } else {
    fp8_decode_kernel<false><<<blocks, 256>>>(d_in.p, n, d_32.p, d_16.p);
  }
  if (cudaDeviceSynchronize() != cudaSuccess) { return -4; }
  d_32.to_host(dec32);
  d_16.to_host(dec16);
  return 0;
}

// mapping<dst>(src value): element types 0 fp32, 1 fp16, 2 int8, 3 uint8; dst fp32 or int8.
PIN_EXPORT int refdev_mapping(int src, int dst, const void* in, uint64_t n, void* out)
{
  using namespace pin;
  if (dst == 0) {
    switch (src) {
      case 0: return run_mapping<float, float>(in, n, out);
      case 1: return run_mapping<float, half>(in, n, out);
      case 2: return run_mapping<float, int8_t>(in, n, out);
      case 3: return run_mapping<float, uint8_t>(in, n, out);
    }
  } else if (dst == 2) {
    switch (src) {
      case 0: return run_mapping<int8_t, float>(in, n, out);
      case 1: return run_mapping<int8_t, half>(in, n, out);
      case 2: return run_mapping<int8_t, int8_t>(in, n, out);
      case 3: return run_mapping<int8_t, uint8_t>(in, n, out);
    }
  }
  return -2;
}

// postprocess_distances (ivf_common.cuh) on fp32 scores, in place as the search calls it when the
// internal distance type is fp32, or from a separate input (in != out on the device).
PIN_EXPORT int refdev_postprocess_distances(const float* in, float* out, uint32_t n_queries, uint32_t topk,
                                            int metric, float scaling_factor, int account_for_max_close,
                                            int in_place)
{
  using namespace pin;
  const size_t n = size_t(n_queries) * topk;
  dev_buf<float> d_in(in, n), d_out(n);
  raft::resources res;
  try {
    if (in_place) {
      cuvs::neighbors::ivf::detail::postprocess_distances<float, float>(
        res, d_in.p, d_in.p, cuvs::distance::DistanceType(metric), n_queries, topk, scaling_factor,
        account_for_max_close != 0);
    } else {
      cudaMemset(d_out.p, 0xff, n * sizeof(float));
      cuvs::neighbors::ivf::detail::postprocess_distances<float, float>(
        res, d_out.p, d_in.p, cuvs::distance::DistanceType(metric), n_queries, topk, scaling_factor,
        account_for_max_close != 0);
    }
  } catch (...) {
    return -2;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) { return -4; }
  (in_place ? d_in : d_out).to_host(out);
  return 0;
}

// postprocess_neighbors (ivf_common.cuh): sample indices -> source ids through the per-list id arrays.
PIN_EXPORT int refdev_postprocess_neighbors(const uint32_t* neighbors_in, const int64_t* ids,
                                            const uint64_t* id_off, uint32_t n_lists, uint64_t n_ids,
                                            const uint32_t* clusters_to_probe, const uint32_t* chunk_indices,
                                            uint32_t n_queries, uint32_t n_probes, uint32_t topk,
                                            int64_t* neighbors_out)
{
  using namespace pin;
  dev_buf<uint32_t> d_in(neighbors_in, size_t(n_queries) * topk),
    d_probe(clusters_to_probe, size_t(n_queries) * n_probes), d_chunk(chunk_indices, size_t(n_queries) * n_probes);
  dev_buf<int64_t> d_ids(ids, n_ids), d_out(size_t(n_queries) * topk);
  std::vector<const int64_t*> ptrs(n_lists);
  for (uint32_t l = 0; l < n_lists; l++) { ptrs[l] = d_ids.p + id_off[l]; }
  dev_buf<const int64_t*> d_ptrs(ptrs.data(), n_lists);
  cuvs::neighbors::ivf::detail::postprocess_neighbors<int64_t, int64_t>(
    d_out.p, d_in.p, d_ptrs.p, d_probe.p, d_chunk.p, n_queries, n_probes, topk, rmm::cuda_stream_view{});
  if (cudaDeviceSynchronize() != cudaSuccess) { return -4; }
  d_out.to_host(neighbors_out);
  return 0;
}
