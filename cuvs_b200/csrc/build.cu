// Index construction on the GPU: coarse k-means, rotation, PQ codebooks, encoding (extend),
// transform and the code unpack helper.
//
// What is kept from the reference (cpp/src/neighbors/ivf_pq/ivf_pq_build.cuh) is the data contract
// of the result, not the training procedure:
//   - trainset size rule .................. :1283-1290
//   - IP trains and predicts with L2 ....... :70-76
//   - rotation: identity when dim == rot_dim and not forced, else a random orthogonal matrix
//     (cpp/src/neighbors/ivf_pq/ivf_pq_build_common.cu:235-261)
//   - centers[l, dim] = |c_l|^2, zero tail; centers_rot = centers * R^T ........ :262-300
//   - codebooks stored [part, pq_len, book] with the book index fastest ........ :303-325
//   - encoding: residual = R (x - c_label); per subspace the codebook entry with the smallest
//     squared distance, lowest code on ties
//     (cpp/src/neighbors/ivf_pq/ivf_pq_process_and_fill_codes.cuh:84-126); codes written in the
//     interleaved layout (cpp/src/neighbors/ivf_pq/ivf_pq_codepacking.cuh:135-168)
// The coarse clustering is Lloyd k-means over all lists at once with the reference's balancing step
// between iterations (underfull clusters restart next to overfull ones, size-sorted donors,
// cpp/src/cluster/detail/kmeans_balanced.cuh:616-720) and re-seeding of empty clusters; the reference
// first clusters hierarchically (mesoclusters) to make training cheap, which the tensor-core
// labelling makes unnecessary here.  Unlike the reference's atomic slot allocation, vectors are placed
// in a list in input order, so extend is deterministic.
#include "ivf_pq.hpp"
#include "search_internal.hpp"
#include "topk.cuh"

#include <cub/device/device_radix_sort.cuh>

#include <algorithm>
#include <cmath>
#include <random>

namespace cuvs::neighbors::ivf_pq {

using namespace cuvs_b200;

namespace {

// ------------------------------------------------------------------------------------------------
// element conversion
// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_float<int8_t>(int8_t x) { return float(x) * (1.0f / 128.0f); }
template <> __device__ __forceinline__ float to_float<uint8_t>(uint8_t x) { return float(x) * (1.0f / 256.0f); }

// One warp per row: out[r, :dim] = mapping<float>(in[r * row_stride, :]) (optionally L2-normalised),
// out[r, dim] = pad, zero tail.
template <typename T>
__global__ void to_float_ext_kernel(const T* __restrict__ in, uint64_t n, uint64_t row_stride,
                                    uint32_t dim, uint32_t dim_ext, float pad, int normalize,
                                    float* __restrict__ out)
{
  const uint64_t r    = (blockIdx.x * uint64_t(blockDim.x) + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (r >= n) { return; }
  const T* src = in + r * row_stride * dim;
  float* dst   = out + r * dim_ext;
  float inv    = 1.0f;
  if (normalize) {
    float ss = 0.0f;
    for (uint32_t i = lane; i < dim; i += 32) {
      float v = to_float<T>(src[i]);
      ss += v * v;
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) { ss += __shfl_xor_sync(kFullMask, ss, d); }
    inv = ss > 0.0f ? 1.0f / sqrtf(ss) : 1.0f;
  }
  for (uint32_t i = lane; i < dim_ext; i += 32) {
    float v = 0.0f;
    if (i < dim) {
      v = to_float<T>(src[i]) * inv;
    } else if (i == dim) {
      v = pad;
    }
    dst[i] = v;
  }
}

void to_float_ext(raft::resources& res, const void* in, elem_t t, uint64_t n, uint64_t row_stride,
                  uint32_t dim, uint32_t dim_ext, float pad, bool normalize, float* out)
{
  if (n == 0) { return; }
  const unsigned blocks = unsigned(ceildiv<uint64_t>(n * 32, 256));
  switch (t) {
    case elem_t::f32:
      to_float_ext_kernel<float><<<blocks, 256, 0, res.stream>>>(static_cast<const float*>(in), n, row_stride, dim, dim_ext, pad, normalize, out);
      break;
    case elem_t::f16:
      to_float_ext_kernel<__half><<<blocks, 256, 0, res.stream>>>(static_cast<const __half*>(in), n, row_stride, dim, dim_ext, pad, normalize, out);
      break;
    case elem_t::i8:
      to_float_ext_kernel<int8_t><<<blocks, 256, 0, res.stream>>>(static_cast<const int8_t*>(in), n, row_stride, dim, dim_ext, pad, normalize, out);
      break;
    default:
      to_float_ext_kernel<uint8_t><<<blocks, 256, 0, res.stream>>>(static_cast<const uint8_t*>(in), n, row_stride, dim, dim_ext, pad, normalize, out);
  }
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

// ------------------------------------------------------------------------------------------------
// k-means update
// ------------------------------------------------------------------------------------------------
__global__ void accumulate_kernel(const float* __restrict__ x_ext, const uint32_t* __restrict__ labels,
                                  uint64_t n, uint32_t dim, uint32_t dim_ext, float* __restrict__ sums,
                                  uint32_t* __restrict__ counts)
{
  const uint64_t r    = (blockIdx.x * uint64_t(blockDim.x) + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (r >= n) { return; }
  const uint32_t l = labels[r];
  const float* src = x_ext + r * dim_ext;
  float* dst       = sums + size_t(l) * dim;
  for (uint32_t i = lane; i < dim; i += 32) { atomicAdd(dst + i, src[i]); }
  if (lane == 0) { atomicAdd(counts + l, 1u); }
}

// One block per center: mean (or a re-seed from a pseudo-random row when the cluster is empty),
// squared norm into column `dim`, zero tail.
__global__ void finalize_centers_kernel(const float* __restrict__ sums, const uint32_t* __restrict__ counts,
                                        uint32_t dim, uint32_t dim_ext, const float* __restrict__ x_ext,
                                        uint64_t n, uint32_t seed, int normalize,
                                        float* __restrict__ centers)
{
  __shared__ float s_red[32];
  const uint32_t l   = blockIdx.x;
  const uint32_t cnt = counts[l];
  float* c           = centers + size_t(l) * dim_ext;
  const uint64_t rr  = (uint64_t(l) * 2654435761ull + uint64_t(seed) * 40503ull + 12345ull) % n;
  float ss           = 0.0f;
  for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = cnt > 0 ? sums[size_t(l) * dim + i] / float(cnt) : x_ext[rr * dim_ext + i];
    c[i]    = v;
    ss += v * v;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) { ss += __shfl_xor_sync(kFullMask, ss, d); }
  if ((threadIdx.x & 31) == 0) { s_red[threadIdx.x >> 5] = ss; }
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : 0.0f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) { v += __shfl_xor_sync(kFullMask, v, d); }
    if (threadIdx.x == 0) { s_red[0] = v; }
  }
  __syncthreads();
  float norm2 = s_red[0];
  if (normalize && norm2 > 0.0f) {
    const float inv = 1.0f / sqrtf(norm2);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) { c[i] *= inv; }
    norm2 = 1.0f;
  }
  for (uint32_t i = dim + threadIdx.x; i < dim_ext; i += blockDim.x) { c[i] = i == dim ? norm2 : 0.0f; }
}

// centers_ext rows <- strided rows of x_ext (k-means initialisation)
__global__ void init_centers_kernel(const float* __restrict__ x_ext, uint64_t n, uint32_t n_lists,
                                    uint32_t dim_ext, float* __restrict__ centers)
{
  const uint32_t l = blockIdx.x;
  const uint64_t r = (uint64_t(l) * n) / n_lists;
  for (uint32_t i = threadIdx.x; i < dim_ext; i += blockDim.x) {
    centers[size_t(l) * dim_ext + i] = x_ext[r * dim_ext + i];
  }
}

// out[l, r] = sum_k R[r, k] * centers[l, k]
__global__ void rotate_centers_kernel(const float* __restrict__ centers, const float* __restrict__ rot,
                                      uint32_t n_lists, uint32_t dim, uint32_t dim_ext, uint32_t rot_dim,
                                      float* __restrict__ out)
{
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (i >= uint64_t(n_lists) * rot_dim) { return; }
  const uint32_t l = uint32_t(i / rot_dim), r = uint32_t(i % rot_dim);
  const float* c = centers + size_t(l) * dim_ext;
  const float* R = rot + size_t(r) * dim;
  float acc      = 0.0f;
  for (uint32_t k = 0; k < dim; k++) { acc = __fmaf_rn(R[k], c[k], acc); }
  out[i] = acc;
}

// Balancing step of the coarse k-means (the reference's adjust_centers with size-sorted donors,
// cpp/src/cluster/detail/kmeans_balanced.cuh:520-720): one pseudo-random member row per cluster ...
__global__ void pick_member_kernel(const uint32_t* __restrict__ labels, uint64_t n, uint32_t seed,
                                   unsigned long long* __restrict__ member /* [n_lists], zeroed */)
{
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (i >= n) { return; }
  // the row with the largest hash wins: a different member every iteration
  uint32_t h = uint32_t(i) * 2654435761u + seed * 40503u;
  h ^= h >> 15;
  h *= 2246822519u;
  h ^= h >> 13;
  atomicMax(member + labels[i], (static_cast<unsigned long long>(h) << 32) | uint32_t(i));
}

// ... and, per (receiver, donor) pair, the receiver's centre re-initialised next to the donor's centre,
// a small step (`offset`) towards one of the donor's rows, so that the next assignment splits the large
// cluster.  One block per pair; norm column and zero tail rewritten.
__global__ void adjust_centers_kernel(float* __restrict__ centers, const uint32_t* __restrict__ pairs /* [n_pairs][2] */,
                                      const unsigned long long* __restrict__ member,
                                      const float* __restrict__ x_ext, uint32_t dim, uint32_t dim_ext,
                                      float offset, int normalize)
{
  __shared__ float s_red[4];
  const uint32_t receiver = pairs[2 * blockIdx.x], donor = pairs[2 * blockIdx.x + 1];
  const uint64_t row      = member[donor] & 0xFFFFFFFFull;
  float* c                = centers + size_t(receiver) * dim_ext;
  const float* d          = centers + size_t(donor) * dim_ext;
  const float* x          = x_ext + row * dim_ext;
  float ss                = 0.0f;
  for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = d[i] + offset * (x[i] - d[i]);
    c[i]          = v;
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(kFullMask, ss, o); }
  if ((threadIdx.x & 31) == 0) { s_red[threadIdx.x >> 5] = ss; }
  __syncthreads();
  float norm2 = 0.0f;
  for (uint32_t w = 0; w < (blockDim.x >> 5); w++) { norm2 += s_red[w]; }
  if (normalize && norm2 > 0.0f) {
    const float inv = 1.0f / sqrtf(norm2);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) { c[i] *= inv; }
    norm2 = 1.0f;
  }
  for (uint32_t i = dim + threadIdx.x; i < dim_ext; i += blockDim.x) { c[i] = i == dim ? norm2 : 0.0f; }
}

// Recompute column `dim` (squared norm) and the zero tail of padded centers in place.
__global__ void center_norms_kernel(float* __restrict__ centers, uint32_t n_lists, uint32_t dim,
                                    uint32_t dim_ext)
{
  const uint32_t l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= n_lists) { return; }
  float* c = centers + size_t(l) * dim_ext;
  float ss = 0.0f;
  for (uint32_t k = 0; k < dim; k++) { ss = __fmaf_rn(c[k], c[k], ss); }
  for (uint32_t k = dim; k < dim_ext; k++) { c[k] = k == dim ? ss : 0.0f; }
}

// Pad [n_lists, dim] centers to [n_lists, dim_ext] with the squared norm in column dim.
__global__ void pad_centers_kernel(const float* __restrict__ in, uint32_t n_lists, uint32_t dim,
                                   uint32_t dim_ext, float* __restrict__ out)
{
  const uint32_t l = blockIdx.x * blockDim.x + threadIdx.x;
  if (l >= n_lists) { return; }
  float ss = 0.0f;
  for (uint32_t k = 0; k < dim; k++) {
    float v                       = in[size_t(l) * dim + k];
    out[size_t(l) * dim_ext + k] = v;
    ss                            = __fmaf_rn(v, v, ss);
  }
  for (uint32_t k = dim; k < dim_ext; k++) { out[size_t(l) * dim_ext + k] = k == dim ? ss : 0.0f; }
}

// ------------------------------------------------------------------------------------------------
// residuals
// ------------------------------------------------------------------------------------------------
// One block per selected row: out[i, :] = R * (x[rows[i]] - centers[label]) with each output
// accumulated in ascending k by FMA (identity rotation copies the difference).
__global__ void residual_kernel(const float* __restrict__ x_ext, const uint32_t* __restrict__ labels,
                                uint64_t row_stride, const float* __restrict__ centers,
                                const float* __restrict__ rot, int identity, uint32_t dim,
                                uint32_t dim_ext, uint32_t rot_dim, float* __restrict__ out)
{
  extern __shared__ float s_diff[];
  const uint64_t i   = blockIdx.x;
  const uint64_t row = i * row_stride;
  const float* x     = x_ext + row * dim_ext;
  const float* c     = centers + size_t(labels[row]) * dim_ext;
  for (uint32_t k = threadIdx.x; k < dim; k += blockDim.x) { s_diff[k] = __fsub_rn(x[k], c[k]); }
  __syncthreads();
  for (uint32_t r = threadIdx.x; r < rot_dim; r += blockDim.x) {
    float acc;
    if (identity) {
      acc = s_diff[r];
    } else {
      const float* R = rot + size_t(r) * dim;
      acc            = 0.0f;
      for (uint32_t k = 0; k < dim; k++) { acc = __fmaf_rn(R[k], s_diff[k], acc); }
    }
    out[i * rot_dim + r] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// PQ codebook training: one block per codebook, Lloyd iterations entirely in shared memory
// ------------------------------------------------------------------------------------------------
// Problem b trains `book` centers of `len` dims.
//   per_cluster == 0: b = subspace; points are slice b of every residual row (n_rows of them).
//   per_cluster == 1: b = list; points are all pq_dim slices of the residual rows
//                     row_ids[row_begin[b] .. row_begin[b+1]) (capped at max_rows).
__global__ void train_codebooks_kernel(const float* __restrict__ resid, uint32_t n_rows,
                                       uint32_t rot_dim, uint32_t pq_dim, uint32_t len, uint32_t book,
                                       int per_cluster, const uint32_t* __restrict__ row_ids,
                                       const uint32_t* __restrict__ row_begin, uint32_t max_rows,
                                       int n_iters, float* __restrict__ pq_centers)
{
  extern __shared__ float s_mem[];
  float* s_c       = s_mem;               // [book, len]
  float* s_sum     = s_c + book * len;    // [book, len]
  uint32_t* s_cnt  = reinterpret_cast<uint32_t*>(s_sum + book * len);  // [book]
  const uint32_t b = blockIdx.x;
  uint32_t rows0 = 0, nr = n_rows;
  if (per_cluster) {
    rows0 = row_begin[b];
    nr    = min(row_begin[b + 1] - rows0, max_rows);
  }
  const uint32_t n_pts = per_cluster ? nr * pq_dim : nr;
  float* out           = pq_centers + size_t(b) * len * book;
  if (n_pts == 0) {
    for (uint32_t i = threadIdx.x; i < len * book; i += blockDim.x) { out[i] = 0.0f; }
    return;
  }
  auto point = [&](uint32_t p) -> const float* {
    if (per_cluster) {
      const uint32_t row = row_ids[rows0 + p / pq_dim];
      return resid + size_t(row) * rot_dim + (p % pq_dim) * len;
    }
    return resid + size_t(p) * rot_dim + b * len;
  };
  // init: evenly strided points
  for (uint32_t i = threadIdx.x; i < book * len; i += blockDim.x) {
    const uint32_t c = i / len, k = i % len;
    s_c[i]           = point(uint32_t((uint64_t(c) * n_pts) / book))[k];
  }
  __syncthreads();
  for (int it = 0; it < n_iters; it++) {
    for (uint32_t i = threadIdx.x; i < book * len; i += blockDim.x) { s_sum[i] = 0.0f; }
    for (uint32_t i = threadIdx.x; i < book; i += blockDim.x) { s_cnt[i] = 0; }
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pts; p += blockDim.x) {
      const float* x = point(p);
      float best     = INFINITY;
      uint32_t bc    = 0;
      for (uint32_t c = 0; c < book; c++) {
        float d2 = 0.0f;
        for (uint32_t k = 0; k < len; k++) {
          float t = x[k] - s_c[c * len + k];
          d2 += t * t;
        }
        if (d2 < best) {
          best = d2;
          bc   = c;
        }
      }
      for (uint32_t k = 0; k < len; k++) { atomicAdd(&s_sum[bc * len + k], x[k]); }
      atomicAdd(&s_cnt[bc], 1u);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < book * len; i += blockDim.x) {
      const uint32_t c = i / len, k = i % len;
      if (s_cnt[c] > 0) {
        s_c[i] = s_sum[i] / float(s_cnt[c]);
      } else {
        // empty: re-seed from a pseudo-random point, nudged so that duplicates separate
        const uint32_t p = uint32_t((uint64_t(c) * 2654435761ull + uint64_t(it + 1) * 97003ull) % n_pts);
        s_c[i]           = point(p)[k] * (1.0f + 1e-3f * float((c % 7) + 1));
      }
    }
    __syncthreads();
  }
  // stored transposed: [len, book]
  for (uint32_t i = threadIdx.x; i < book * len; i += blockDim.x) {
    const uint32_t c = i / len, k = i % len;
    out[size_t(k) * book + c] = s_c[i];
  }
}

// ------------------------------------------------------------------------------------------------
// encoder
// ------------------------------------------------------------------------------------------------
// One warp per vector (taken in `order`): residual into shared memory, per-subspace argmin over the
// codebook split across lanes, then the lanes pack the codes.
//   interleaved != 0: write into the list arena at row (row_off[label] + slot[i]); ids too.
//   interleaved == 0: write a flat little-endian bit stream of ceil(pq_dim*bits/8) bytes per vector.
__global__ void encode_kernel(const float* __restrict__ x_ext, const uint32_t* __restrict__ labels,
                              const uint32_t* __restrict__ order, const uint32_t* __restrict__ slots,
                              uint32_t n, const float* __restrict__ centers,
                              const float* __restrict__ rot, int identity,
                              const float* __restrict__ pq_centers, int per_cluster, uint32_t dim,
                              uint32_t dim_ext, uint32_t rot_dim, uint32_t pq_dim, uint32_t len,
                              uint32_t bits, int interleaved, const uint64_t* __restrict__ row_off,
                              uint8_t* __restrict__ codes_out, int64_t* __restrict__ ids_out,
                              const int64_t* __restrict__ src_ids, int64_t id_base,
                              uint32_t flat_row_bytes)
{
  extern __shared__ float s_enc[];
  const uint32_t warps = blockDim.x >> 5;
  const uint32_t wid   = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t per_warp_floats = round_up<uint32_t>(dim, 4) + round_up<uint32_t>(rot_dim, 4) + round_up<uint32_t>(pq_dim, 16) / 4;
  float* s_diff   = s_enc + size_t(wid) * per_warp_floats;
  float* s_res    = s_diff + round_up<uint32_t>(dim, 4);
  uint8_t* s_code = reinterpret_cast<uint8_t*>(s_res + round_up<uint32_t>(rot_dim, 4));
  const uint32_t i = blockIdx.x * warps + wid;
  if (i >= n) { return; }
  const uint32_t row   = order ? order[i] : i;
  const uint32_t label = labels[row];
  const uint32_t book  = 1u << bits;
  const float* x       = x_ext + size_t(row) * dim_ext;
  const float* c       = centers + size_t(label) * dim_ext;
  for (uint32_t k = lane; k < dim; k += 32) { s_diff[k] = __fsub_rn(x[k], c[k]); }
  __syncwarp();
  for (uint32_t r = lane; r < rot_dim; r += 32) {
    float acc;
    if (identity) {
      acc = s_diff[r];
    } else {
      const float* R = rot + size_t(r) * dim;
      acc            = 0.0f;
      for (uint32_t k = 0; k < dim; k++) { acc = __fmaf_rn(R[k], s_diff[k], acc); }
    }
    s_res[r] = acc;
  }
  __syncwarp();
  const float* pqc0 = per_cluster ? pq_centers + size_t(label) * len * book : pq_centers;
  for (uint32_t j = 0; j < pq_dim; j++) {
    const float* pqc = pqc0 + (per_cluster ? 0 : size_t(j) * len * book);
    float best       = INFINITY;
    uint32_t best_b  = 0xFFFFFFFFu;
    for (uint32_t b = lane; b < book; b += 32) {
      float d2 = 0.0f;
      for (uint32_t k = 0; k < len; k++) {
        const float t = __fsub_rn(s_res[j * len + k], __ldg(pqc + size_t(k) * book + b));
        d2            = __fmaf_rn(t, t, d2);
      }
      if (d2 < best) {
        best   = d2;
        best_b = b;
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ob    = __shfl_xor_sync(kFullMask, best, d);
      const uint32_t oc = __shfl_xor_sync(kFullMask, best_b, d);
      if (ob < best || (ob == best && oc < best_b)) {
        best   = ob;
        best_b = oc;
      }
    }
    if (lane == 0) { s_code[j] = uint8_t(best_b == 0xFFFFFFFFu ? 0 : best_b); }
  }
  __syncwarp();
  if (interleaved == 1) {
    const uint32_t cpp      = 128u / bits;
    const uint32_t n_pieces = ceildiv(pq_dim, cpp);
    const uint64_t arow     = row_off[label] + slots[i];
    for (uint32_t p = lane; p < n_pieces; p += 32) {
      uint32_t w[4] = {0, 0, 0, 0};
      for (uint32_t t = 0; t < cpp && p * cpp + t < pq_dim; t++) {
        const uint32_t code = s_code[p * cpp + t];
        const uint32_t bit  = t * bits;
        w[bit >> 5] |= code << (bit & 31);
        if ((bit & 31) + bits > 32) { w[(bit >> 5) + 1] |= code >> (32 - (bit & 31)); }
      }
      uint4* dst = reinterpret_cast<uint4*>(codes_out + (((arow >> 5) * n_pieces + p) * 32 + (arow & 31)) * 16);
      *dst       = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (lane == 0) { ids_out[arow] = src_ids ? src_ids[row] : id_base + int64_t(row); }
  } else {
    // interleaved == 0: row `row` of a plain output matrix (transform); == 2: a slot of a FLAT list
    uint8_t* dst = codes_out + size_t(row) * flat_row_bytes;
    if (interleaved == 2) {
      const uint64_t arow = row_off[label] + slots[i];
      dst                 = codes_out + arow * flat_row_bytes;
      if (lane == 0) { ids_out[arow] = src_ids ? src_ids[row] : id_base + int64_t(row); }
    }
    for (uint32_t byte = lane; byte < flat_row_bytes; byte += 32) {
      uint32_t v = 0;
      // collect the bits [byte*8, byte*8+8) of the stream
      const uint32_t first = (byte * 8) / bits;
      for (uint32_t j = first; j < pq_dim && j * bits < byte * 8 + 8; j++) {
        const int shift = int(j * bits) - int(byte * 8);
        const uint32_t code = s_code[j];
        v |= shift >= 0 ? (code << shift) : (code >> (-shift));
      }
      dst[byte] = uint8_t(v & 0xFFu);
    }
  }
}

// Interleaved list rows [offset, offset + n) -> flat bit-packed rows.
__global__ void unpack_contiguous_kernel(const uint8_t* __restrict__ list, uint32_t n, uint32_t offset,
                                         uint32_t pq_dim, uint32_t bits, uint32_t flat_row_bytes,
                                         uint8_t* __restrict__ out)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) { return; }
  const uint32_t row      = offset + i;
  const uint32_t cpp      = 128u / bits;
  const uint32_t n_pieces = ceildiv(pq_dim, cpp);
  uint8_t* dst            = out + size_t(i) * flat_row_bytes;
  for (uint32_t b = 0; b < flat_row_bytes; b++) { dst[b] = 0; }
  for (uint32_t j = 0; j < pq_dim; j++) {
    const uint32_t p = j / cpp, t = j % cpp;
    const uint8_t* piece = list + ((size_t(row >> 5) * n_pieces + p) * 32 + (row & 31)) * 16;
    const uint32_t bit   = t * bits;
    uint32_t pair        = piece[bit >> 3];
    if ((bit & 7) + bits > 8) { pair |= uint32_t(piece[(bit >> 3) + 1]) << 8; }
    const uint32_t code = (pair >> (bit & 7)) & ((1u << bits) - 1u);
    const uint32_t ob   = j * bits;
    dst[ob >> 3] |= uint8_t((code << (ob & 7)) & 0xFFu);
    if ((ob & 7) + bits > 8) { dst[(ob >> 3) + 1] |= uint8_t(code >> (8 - (ob & 7))); }
  }
}

// Code j of one interleaved list row.
__device__ __forceinline__ uint32_t list_code(const uint8_t* __restrict__ list, uint32_t row, uint32_t j,
                                              uint32_t n_pieces, uint32_t bits)
{
  const uint32_t cpp = 128u / bits;
  const uint32_t p = j / cpp, bit = (j % cpp) * bits;
  const uint8_t* piece = list + ((size_t(row >> 5) * n_pieces + p) * 32 + (row & 31)) * 16;
  uint32_t pair        = piece[bit >> 3];
  if ((bit & 7) + bits > 8) { pair |= uint32_t(piece[(bit >> 3) + 1]) << 8; }
  return (pair >> (bit & 7)) & ((1u << bits) - 1u);
}

// One thread per (row, subspace): interleaved list rows -> one code per byte.
__global__ void unpack_codes_kernel(const uint8_t* __restrict__ list, uint32_t n, uint32_t offset,
                                    const uint32_t* __restrict__ indices, uint32_t pq_dim, uint32_t bits,
                                    uint32_t n_pieces, uint8_t* __restrict__ out)
{
  const uint64_t t = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (t >= uint64_t(n) * pq_dim) { return; }
  const uint32_t i = uint32_t(t / pq_dim), j = uint32_t(t % pq_dim);
  const uint32_t row = indices ? indices[i] : offset + i;
  out[t] = uint8_t(list_code(list, row, j, n_pieces, bits));
}

// One thread per (row, 16-byte piece): codes (one per byte, or bit-packed rows when kContiguous)
// -> interleaved list rows [offset, offset + n).  Unused bits of the last piece are zero.
template <bool kContiguous>
__global__ void pack_codes_kernel(const uint8_t* __restrict__ codes, uint32_t n, uint32_t offset,
                                  uint32_t pq_dim, uint32_t bits, uint32_t n_pieces,
                                  uint32_t flat_row_bytes, uint8_t* __restrict__ list)
{
  const uint64_t t = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (t >= uint64_t(n) * n_pieces) { return; }
  const uint32_t i = uint32_t(t / n_pieces), p = uint32_t(t % n_pieces);
  const uint32_t cpp = 128u / bits, mask = (1u << bits) - 1u;
  const uint8_t* src = codes + size_t(i) * (kContiguous ? flat_row_bytes : pq_dim);
  uint32_t w[4] = {0, 0, 0, 0};
  for (uint32_t c = 0; c < cpp && p * cpp + c < pq_dim; c++) {
    const uint32_t j = p * cpp + c;
    uint32_t code;
    if (kContiguous) {
      const uint32_t ib = j * bits;
      uint32_t pair     = src[ib >> 3];
      if ((ib & 7) + bits > 8) { pair |= uint32_t(src[(ib >> 3) + 1]) << 8; }
      code = (pair >> (ib & 7)) & mask;
    } else {
      code = src[j] & mask;
    }
    const uint32_t bit = c * bits;
    w[bit >> 5] |= code << (bit & 31);
    if ((bit & 31) + bits > 32) { w[(bit >> 5) + 1] |= code >> (32 - (bit & 31)); }
  }
  const uint32_t row = offset + i;
  *reinterpret_cast<uint4*>(list + ((size_t(row >> 5) * n_pieces + p) * 32 + (row & 31)) * 16) =
    make_uint4(w[0], w[1], w[2], w[3]);
}

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
// mapping<int8_t>(float) clamps before it converts (ann_utils.cuh:211-217); the uint8 mapping does not
template <> __device__ __forceinline__ int8_t from_float<int8_t>(float x)
{
  return static_cast<int8_t>(fminf(fmaxf(__fmul_rn(x, 128.0f), -128.0f), 127.0f));
}
template <> __device__ __forceinline__ uint8_t from_float<uint8_t>(float x) { return static_cast<uint8_t>(__fmul_rn(x, 256.0f)); }

// One block per row: decode the row in the rotated space (codeword + rotated list center, one add
// per component), then out[i, d] = sum over r, in order, of rotation[r, d] * decoded[r] (fp32 fma).
template <typename T>
__global__ void reconstruct_kernel(const uint8_t* __restrict__ list, uint32_t offset,
                                   const uint32_t* __restrict__ indices, const float* __restrict__ pq_centers,
                                   int per_cluster, const float* __restrict__ center_rot,
                                   const float* __restrict__ rot, uint32_t label, uint32_t dim,
                                   uint32_t rot_dim, uint32_t pq_dim, uint32_t len, uint32_t bits,
                                   uint32_t n_pieces, T* __restrict__ out)
{
  extern __shared__ float s_dec[];
  const uint32_t i    = blockIdx.x;
  const uint32_t row  = indices ? indices[i] : offset + i;
  const uint32_t book = 1u << bits;
  for (uint32_t r = threadIdx.x; r < rot_dim; r += blockDim.x) {
    const uint32_t j = r / len, k = r % len;
    const uint32_t code = list_code(list, row, j, n_pieces, bits);
    const float* pqc    = pq_centers + size_t(per_cluster ? label : j) * len * book;
    s_dec[r]            = __fadd_rn(pqc[size_t(k) * book + code], center_rot[r]);
  }
  __syncthreads();
  for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
    float acc = 0.0f;
    for (uint32_t r = 0; r < rot_dim; r++) { acc = __fmaf_rn(rot[size_t(r) * dim + d], s_dec[r], acc); }
    out[size_t(i) * dim + d] = from_float<T>(acc);
  }
}

__global__ void fill_u32_kernel(uint32_t* p, uint32_t n, uint32_t v)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { p[i] = v; }
}

__global__ void add_scalar_u32_kernel(uint32_t* p, uint32_t n, uint32_t v)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { p[i] += v; }
}

// ------------------------------------------------------------------------------------------------
// extend helpers
// ------------------------------------------------------------------------------------------------
__global__ void histogram_kernel(const uint32_t* __restrict__ labels, uint64_t n, uint32_t* __restrict__ counts)
{
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (i < n) { atomicAdd(counts + labels[i], 1u); }
}

__global__ void iota_kernel(uint32_t* p, uint32_t n)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { p[i] = i; }
}

// slots[i] = base[label] + (i - first index of label in the sorted order)
__global__ void slots_kernel(const uint32_t* __restrict__ sorted_labels, uint32_t n,
                             const uint32_t* __restrict__ base, uint32_t* __restrict__ slots)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) { return; }
  const uint32_t l = sorted_labels[i];
  // first position of l: binary search for the lower bound
  uint32_t lo = 0, hi = i;
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if (sorted_labels[mid] < l) {
      lo = mid + 1;
    } else {
      hi = mid;
    }
  }
  slots[i] = base[l] + (i - lo);
}

// One block per list: copy the old list payload (whole 32-row groups) and ids to the new arena.
__global__ void relocate_lists_kernel(const uint8_t* __restrict__ old_codes, const int64_t* __restrict__ old_ids,
                                      const uint64_t* __restrict__ old_off, const uint32_t* __restrict__ old_sizes,
                                      const uint64_t* __restrict__ new_off, uint32_t row_bytes,
                                      uint8_t* __restrict__ new_codes, int64_t* __restrict__ new_ids)
{
  const uint32_t l = blockIdx.x;
  const uint32_t n = old_sizes[l];
  if (n == 0) { return; }
  const uint64_t rows  = round_up<uint64_t>(n, 32);
  const uint4* src     = reinterpret_cast<const uint4*>(old_codes + old_off[l] * row_bytes);
  uint4* dst           = reinterpret_cast<uint4*>(new_codes + new_off[l] * row_bytes);
  const uint64_t n_vec = rows * row_bytes / 16;
  for (uint64_t i = threadIdx.x; i < n_vec; i += blockDim.x) { dst[i] = src[i]; }
  for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) { new_ids[new_off[l] + i] = old_ids[old_off[l] + i]; }
}

__global__ void add_u32_kernel(uint32_t* a, const uint32_t* b, uint32_t n)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { a[i] += b[i]; }
}

uint64_t chunk_rows_for(uint32_t dim_ext)
{
  const uint64_t budget = 1ull << 30;  // bytes of converted rows per chunk
  return std::max<uint64_t>(1024, std::min<uint64_t>(1u << 20, budget / (uint64_t(dim_ext) * 4)));
}

// balanced k-means defaults of the reference (cpp/include/cuvs/cluster/kmeans.hpp:181-204)
constexpr double kBalanceLower  = 0.333;
constexpr double kBalanceUpper  = 3.0;
constexpr float kCentroidOffset = 0.01f;

struct label_ctx {
  float alpha;
  float pad;
  bool normalize;
};
label_ctx labeling_of(DistanceType m)
{
  // IP trains/predicts with L2 (ivf_pq_build.cuh:70-76); cosine works on normalised rows.
  return {-2.0f, -0.5f, m == DistanceType::CosineExpanded};
}

// Labelling of many rows against one set of centres.  Where the shape allows, the tensor-core coarse
// path does it (probe selection with n_probes = 1: exact rescoring and guard make its answer the
// defining one, ties to the lowest list id) -- an order of magnitude faster than the SIMT product on
// the 10^5 .. 10^6 lists of the large configurations; otherwise the SIMT kernel.
class nearest_labeler {
 public:
  // `dim`: index of the |c|^2 column of the centre rows (rows carry -0.5 there)
  nearest_labeler(raft::resources& res, const float* centers, uint32_t n_lists, uint32_t dim, uint32_t dim_ext,
                  float alpha)
    : res_(res), centers_(centers), n_lists_(n_lists), dim_ext_(dim_ext), ext_col_(dim), alpha_(alpha)
  {
    use_tc_ = coarse_tc_usable(n_lists, 1, dim_ext);
    if (!use_tc_) { return; }
    const size_t nc = size_t(n_lists) * dim_ext;
    hi_.resize(nc);
    lo_.resize(nc);
    prepare_tc_centers(res.stream, centers, n_lists, dim_ext, ext_col_, hi_.data(), lo_.data(), &cmax_, &ext_scale_);
    res.launches += 2;
  }
  // labels[i] = nearest list of row i of x_ext [n_rows, dim_ext]; `best` is scratch of n_rows * 8 bytes
  void run(const float* x_ext, uint32_t n_rows, uint32_t* labels, unsigned long long* best)
  {
    if (!use_tc_) {
      assign_nearest(res_, centers_, n_lists_, dim_ext_, alpha_, x_ext, n_rows, labels, best);
      return;
    }
    const uint32_t batch = std::min<uint32_t>(n_rows, 16384);
    const size_t need    = coarse_tc_workspace_bytes(batch, n_lists_, dim_ext_);
    if (ws_.size() < need) { ws_.resize(need); }
    for (uint32_t r0 = 0; r0 < n_rows; r0 += batch) {
      const uint32_t nr = std::min(batch, n_rows - r0);
      select_clusters_tc(res_, centers_, hi_.data(), lo_.data(), cmax_, n_lists_, dim_ext_, alpha_,
                         x_ext + size_t(r0) * dim_ext_, nr, 1, labels + r0, nullptr, ws_.data(), ws_.size(), false,
                         ext_col_, ext_scale_);
    }
  }

 private:
  raft::resources& res_;
  const float* centers_;
  uint32_t n_lists_, dim_ext_, ext_col_;
  float alpha_;
  bool use_tc_     = false;
  float cmax_      = 0.0f;
  float ext_scale_ = 1.0f;
  dev_array<float> hi_, lo_;
  dev_array<uint8_t> ws_;
};

// Host rows -> device staging (no-op for device data).
const void* stage_rows(raft::resources& res, const void* data, elem_t t, uint64_t r0, uint64_t nr,
                       uint32_t dim, bool on_device, dev_array<uint8_t>& staging)
{
  const size_t es = elem_size(t);
  const char* src = static_cast<const char*>(data) + r0 * dim * es;
  if (on_device) { return src; }
  if (staging.size() < nr * dim * es) { staging.resize(nr * dim * es); }
  CUDA_TRY(cudaMemcpyAsync(staging.data(), src, nr * dim * es, cudaMemcpyHostToDevice, res.stream));
  return staging.data();
}

void make_rotation(uint32_t rot_dim, uint32_t dim, bool force_random, std::vector<float>& out)
{
  out.assign(size_t(rot_dim) * dim, 0.0f);
  if (rot_dim == dim && !force_random) {
    for (uint32_t i = 0; i < dim; i++) { out[size_t(i) * dim + i] = 1.0f; }
    return;
  }
  // random orthogonal: Gaussian matrix, columns orthonormalised (modified Gram-Schmidt, twice)
  const uint32_t n = rot_dim;
  std::vector<double> a(size_t(n) * n);
  std::mt19937_64 gen(7);
  std::normal_distribution<double> nd(0.0, 1.0);
  for (auto& v : a) { v = nd(gen); }
  for (uint32_t c = 0; c < n; c++) {
    for (int pass = 0; pass < 2; pass++) {
      for (uint32_t p = 0; p < c; p++) {
        double dot = 0;
        for (uint32_t r = 0; r < n; r++) { dot += a[size_t(r) * n + c] * a[size_t(r) * n + p]; }
        for (uint32_t r = 0; r < n; r++) { a[size_t(r) * n + c] -= dot * a[size_t(r) * n + p]; }
      }
    }
    double nn = 0;
    for (uint32_t r = 0; r < n; r++) { nn += a[size_t(r) * n + c] * a[size_t(r) * n + c]; }
    nn = std::sqrt(nn);
    for (uint32_t r = 0; r < n; r++) { a[size_t(r) * n + c] /= nn; }
  }
  for (uint32_t r = 0; r < rot_dim; r++) {
    for (uint32_t c = 0; c < dim; c++) { out[size_t(r) * dim + c] = float(a[size_t(r) * n + c]); }
  }
}

void launch_encode(raft::resources& res, const index<int64_t>& idx, const float* x_ext,
                   const uint32_t* labels, const uint32_t* order, const uint32_t* slots, uint32_t n,
                   bool interleaved, uint8_t* codes_out, int64_t* ids_out, const int64_t* src_ids,
                   int64_t id_base)
{
  if (n == 0) { return; }
  const uint32_t warps = 4;
  const uint32_t per_warp_floats = round_up<uint32_t>(idx.dim(), 4) + round_up<uint32_t>(idx.rot_dim(), 4) +
                                   round_up<uint32_t>(idx.pq_dim(), 16) / 4;
  const size_t smem = size_t(warps) * per_warp_floats * 4;
  CUVS_EXPECTS(smem <= 48 * 1024, "dim = %u is too large for the encoder", idx.dim());
  encode_kernel<<<ceildiv(n, warps), warps * 32, smem, res.stream>>>(
    x_ext, labels, order, slots, n, idx.centers(), idx.rotation_matrix(), idx.rotation_is_identity(),
    idx.pq_centers(), idx.codebook_kind() == codebook_gen::PER_CLUSTER, idx.dim(), idx.dim_ext(),
    idx.rot_dim(), idx.pq_dim(), idx.pq_len(), idx.pq_bits(),
    // 0: rows of a plain output matrix; 1: slots of interleaved lists; 2: slots of flat lists
    interleaved ? (idx.codes_layout() == list_layout::FLAT ? 2 : 1) : 0, idx.row_offsets(), codes_out,
    ids_out, src_ids, id_base, ceildiv(idx.pq_dim() * idx.pq_bits(), 8u));
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}


// Re-create the arenas for `new_sizes`, keeping the first min(old, new) rows (codes and ids) of every list.
void resize_lists(raft::resources& res, index<int64_t>* idx, const std::vector<uint32_t>& new_sizes)
{
  const uint32_t n_lists    = idx->n_lists();
  const cudaStream_t stream = res.stream;
  std::vector<uint32_t> keep(n_lists);
  bool any = false;
  for (uint32_t l = 0; l < n_lists; l++) {
    keep[l] = std::min(idx->host_list_sizes()[l], new_sizes[l]);
    any |= keep[l] > 0;
  }
  dev_array<uint8_t> old_codes = std::move(idx->codes_);
  dev_array<int64_t> old_ids   = std::move(idx->ids_);
  dev_array<uint64_t> old_off(size_t(n_lists) + 1);
  dev_array<uint32_t> keep_d(n_lists);
  CUDA_TRY(cudaMemcpyAsync(old_off.data(), idx->row_offsets(), (size_t(n_lists) + 1) * 8, cudaMemcpyDeviceToDevice, stream));
  CUDA_TRY(cudaMemcpyAsync(keep_d.data(), keep.data(), size_t(n_lists) * 4, cudaMemcpyHostToDevice, stream));
  idx->allocate_lists(new_sizes, stream);
  if (any) {
    relocate_lists_kernel<<<n_lists, 128, 0, stream>>>(old_codes.data(), old_ids.data(), old_off.data(),
                                                       keep_d.data(), idx->row_offsets(),
                                                       idx->list_row_bytes(), idx->codes(), idx->ids());
    CUDA_TRY(cudaGetLastError());
    res.launches++;
  }
  res.sync();  // the old arenas are released on return
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// helpers
// ------------------------------------------------------------------------------------------------
namespace helpers {

void unpack_contiguous_list_data(raft::resources& res, const index<int64_t>& idx, uint8_t* out_codes,
                                 uint32_t n_rows, uint32_t label, uint32_t offset)
{
  CUVS_EXPECTS(label < idx.n_lists(), "label %u is out of range", label);
  CUVS_EXPECTS(uint64_t(offset) + n_rows <= idx.host_list_sizes()[label],
               "rows [%u, %u) exceed the size of list %u (%u)", offset, offset + n_rows, label,
               idx.host_list_sizes()[label]);
  if (n_rows == 0) { return; }
  if (idx.codes_layout() == list_layout::FLAT) {
    // the rows already are what the caller asks for
    const size_t bpv = idx.bytes_per_vector();
    CUDA_TRY(cudaMemcpyAsync(out_codes, idx.codes() + (idx.host_row_offsets()[label] + offset) * bpv,
                             size_t(n_rows) * bpv, cudaMemcpyDeviceToDevice, res.stream));
    return;
  }
  const uint8_t* list = idx.codes() + idx.host_row_offsets()[label] * size_t(idx.n_pieces()) * 16;
  unpack_contiguous_kernel<<<ceildiv(n_rows, 128u), 128, 0, res.stream>>>(
    list, n_rows, offset, idx.pq_dim(), idx.pq_bits(), ceildiv(idx.pq_dim() * idx.pq_bits(), 8u), out_codes);
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

void set_model(raft::resources& res, index<int64_t>* idx, const float* pq_centers, const float* centers,
               uint32_t centers_cols, const float* centers_rot, const float* rotation_matrix)
{
  CUDA_TRY(cudaMemcpyAsync(idx->pq_centers(), pq_centers, idx->pq_centers_size() * 4,
                           cudaMemcpyDefault, res.stream));
  if (centers_cols == idx->dim_ext()) {
    CUDA_TRY(cudaMemcpyAsync(idx->centers(), centers, size_t(idx->n_lists()) * idx->dim_ext() * 4,
                             cudaMemcpyDefault, res.stream));
  } else {
    pad_centers_kernel<<<ceildiv(idx->n_lists(), 128u), 128, 0, res.stream>>>(
      centers, idx->n_lists(), idx->dim(), idx->dim_ext(), idx->centers());
    res.launches++;
  }
  CUDA_TRY(cudaMemcpyAsync(idx->centers_rot(), centers_rot, size_t(idx->n_lists()) * idx->rot_dim() * 4,
                           cudaMemcpyDefault, res.stream));
  CUDA_TRY(cudaMemcpyAsync(idx->rotation_matrix(), rotation_matrix,
                           size_t(idx->rot_dim()) * idx->dim() * 4, cudaMemcpyDefault, res.stream));
  res.sync();
  idx->allocate_lists(std::vector<uint32_t>(idx->n_lists(), 0), res.stream);
}

namespace {
void check_rows(const index<int64_t>& idx, uint32_t label, uint32_t offset, uint32_t n_rows)
{
  CUVS_EXPECTS(label < idx.n_lists(), "label %u is out of range", label);
  // ivf_pq_build.cuh:611-612
  CUVS_EXPECTS(uint64_t(offset) + n_rows <= idx.host_list_sizes()[label],
               "offset + output size must be not bigger than the cluster size.");
}
uint8_t* list_base(const index<int64_t>& idx, uint32_t label)
{
  // the helpers that read or write single codes address the interleaved layout (as the reference's do)
  CUVS_EXPECTS(idx.codes_layout() == list_layout::INTERLEAVED,
               "this helper supports the INTERLEAVED codes layout only");
  return idx.codes() + idx.host_row_offsets()[label] * size_t(idx.n_pieces()) * kIndexGroupVecLen;
}
// Grow list `label` by n_rows, write the new source ids; returns the first new row.
uint32_t extend_list_prepare(raft::resources& res, index<int64_t>* idx, const int64_t* new_indices,
                             uint32_t n_rows, uint32_t label)
{
  CUVS_EXPECTS(idx != nullptr && label < idx->n_lists(), "label %u is out of range", label);
  const uint32_t offset = idx->host_list_sizes()[label];
  CUVS_EXPECTS(uint64_t(offset) + n_rows < (1ull << 32), "list %u grows beyond 2^32 rows", label);
  std::vector<uint32_t> sizes = idx->host_list_sizes();
  sizes[label] += n_rows;
  resize_lists(res, idx, sizes);
  CUDA_TRY(cudaMemcpyAsync(idx->ids() + idx->host_row_offsets()[label] + offset, new_indices,
                           size_t(n_rows) * 8, cudaMemcpyDefault, res.stream));
  return offset;
}
}  // namespace

namespace codepacker {

void unpack_list_data(raft::resources& res, const index<int64_t>& idx, uint8_t* out_codes,
                      uint32_t n_rows, uint32_t label, uint32_t offset,
                      const uint32_t* in_cluster_indices)
{
  check_rows(idx, label, in_cluster_indices ? 0 : offset, in_cluster_indices ? 0 : n_rows);
  if (n_rows == 0) { return; }
  const uint64_t n_threads = uint64_t(n_rows) * idx.pq_dim();
  unpack_codes_kernel<<<unsigned(ceildiv<uint64_t>(n_threads, 256)), 256, 0, res.stream>>>(
    list_base(idx, label), n_rows, offset, in_cluster_indices, idx.pq_dim(), idx.pq_bits(),
    idx.n_pieces(), out_codes);
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

namespace {
template <bool kContiguous>
void pack_rows(raft::resources& res, index<int64_t>* idx, const uint8_t* codes, uint32_t n_rows,
               uint32_t label, uint32_t offset)
{
  CUVS_EXPECTS(idx != nullptr, "null index");
  check_rows(*idx, label, offset, n_rows);
  if (n_rows == 0) { return; }
  if (kContiguous && idx->codes_layout() == list_layout::FLAT) {
    const size_t bpv = idx->bytes_per_vector();
    CUDA_TRY(cudaMemcpyAsync(idx->codes() + (idx->host_row_offsets()[label] + offset) * bpv, codes,
                             size_t(n_rows) * bpv, cudaMemcpyDefault, res.stream));
    return;
  }
  const uint64_t n_threads = uint64_t(n_rows) * idx->n_pieces();
  pack_codes_kernel<kContiguous><<<unsigned(ceildiv<uint64_t>(n_threads, 256)), 256, 0, res.stream>>>(
    codes, n_rows, offset, idx->pq_dim(), idx->pq_bits(), idx->n_pieces(),
    ceildiv(idx->pq_dim() * idx->pq_bits(), 8u), list_base(*idx, label));
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}
}  // namespace

void pack_list_data(raft::resources& res, index<int64_t>* idx, const uint8_t* codes, uint32_t n_rows,
                    uint32_t label, uint32_t offset)
{
  pack_rows<false>(res, idx, codes, n_rows, label, offset);
}

void pack_contiguous_list_data(raft::resources& res, index<int64_t>* idx, const uint8_t* codes,
                               uint32_t n_rows, uint32_t label, uint32_t offset)
{
  pack_rows<true>(res, idx, codes, n_rows, label, offset);
}

void reconstruct_list_data(raft::resources& res, const index<int64_t>& idx, void* out_vectors,
                           elem_t out_type, uint32_t n_rows, uint32_t label, uint32_t offset,
                           const uint32_t* in_cluster_indices)
{
  if (n_rows == 0) { return; }
  check_rows(idx, label, in_cluster_indices ? 0 : offset, in_cluster_indices ? 0 : n_rows);
  const size_t smem = size_t(idx.rot_dim()) * 4;
  CUVS_EXPECTS(smem <= 48 * 1024, "rot_dim = %u is too large to reconstruct", idx.rot_dim());
  auto launch = [&](auto* out) {
    using T = std::remove_pointer_t<decltype(out)>;
    reconstruct_kernel<T><<<n_rows, 128, smem, res.stream>>>(
      list_base(idx, label), offset, in_cluster_indices, idx.pq_centers(),
      idx.codebook_kind() == codebook_gen::PER_CLUSTER, idx.centers_rot() + size_t(label) * idx.rot_dim(),
      idx.rotation_matrix(), label, idx.dim(), idx.rot_dim(), idx.pq_dim(), idx.pq_len(), idx.pq_bits(),
      idx.n_pieces(), out);
  };
  switch (out_type) {
    case elem_t::f32: launch(static_cast<float*>(out_vectors)); break;
    case elem_t::f16: launch(static_cast<__half*>(out_vectors)); break;
    case elem_t::i8: launch(static_cast<int8_t*>(out_vectors)); break;
    default: launch(static_cast<uint8_t*>(out_vectors));
  }
  CUDA_TRY(cudaGetLastError());
  res.launches++;
}

void extend_list_with_codes(raft::resources& res, index<int64_t>* idx, const uint8_t* new_codes,
                            const int64_t* new_indices, uint32_t n_rows, uint32_t label)
{
  const uint32_t offset = extend_list_prepare(res, idx, new_indices, n_rows, label);
  pack_rows<false>(res, idx, new_codes, n_rows, label, offset);
  res.sync();
}

void extend_list_with_contiguous_codes(raft::resources& res, index<int64_t>* idx,
                                       const uint8_t* new_codes, const int64_t* new_indices,
                                       uint32_t n_rows, uint32_t label)
{
  const uint32_t offset = extend_list_prepare(res, idx, new_indices, n_rows, label);
  pack_rows<true>(res, idx, new_codes, n_rows, label, offset);
  res.sync();
}

void extend_list(raft::resources& res, index<int64_t>* idx, const void* new_vectors, elem_t dtype,
                 const int64_t* new_indices, uint32_t n_rows, uint32_t label)
{
  const uint32_t offset = extend_list_prepare(res, idx, new_indices, n_rows, label);
  if (n_rows == 0) { return; }
  const label_ctx lc = labeling_of(idx->metric());
  dev_array<float> x_ext(size_t(n_rows) * idx->dim_ext());
  dev_array<uint32_t> labels(n_rows), slots(n_rows);
  to_float_ext(res, new_vectors, dtype, n_rows, 1, idx->dim(), idx->dim_ext(), lc.pad, lc.normalize,
               x_ext.data());
  fill_u32_kernel<<<ceildiv(n_rows, 256u), 256, 0, res.stream>>>(labels.data(), n_rows, label);
  iota_kernel<<<ceildiv(n_rows, 256u), 256, 0, res.stream>>>(slots.data(), n_rows);
  add_scalar_u32_kernel<<<ceildiv(n_rows, 256u), 256, 0, res.stream>>>(slots.data(), n_rows, offset);
  res.launches += 3;
  // ids were written by extend_list_prepare: the encoder gets the same array, so it rewrites them
  launch_encode(res, *idx, x_ext.data(), labels.data(), nullptr, slots.data(), n_rows, true, idx->codes(),
                idx->ids(), new_indices, 0);
  res.sync();
}

}  // namespace codepacker

void erase_list(raft::resources& res, index<int64_t>* idx, uint32_t label)
{
  CUVS_EXPECTS(idx != nullptr && label < idx->n_lists(), "label %u is out of range", label);
  std::vector<uint32_t> sizes = idx->host_list_sizes();
  sizes[label]                = 0;
  resize_lists(res, idx, sizes);
}

void reset_index(raft::resources& res, index<int64_t>* idx)
{
  CUVS_EXPECTS(idx != nullptr, "null index");
  idx->allocate_lists(std::vector<uint32_t>(idx->n_lists(), 0), res.stream);
}

}  // namespace helpers

// ------------------------------------------------------------------------------------------------
// extend
// ------------------------------------------------------------------------------------------------
void extend_any(raft::resources& res, const void* new_vectors, elem_t dtype, int64_t n_rows_i,
                const int64_t* new_indices, bool on_device, index<int64_t>* idx)
{
  CUVS_EXPECTS(idx != nullptr && idx->n_lists() > 0, "extend: the index is not trained");
  CUVS_EXPECTS(n_rows_i >= 0 && n_rows_i < (1ll << 32), "extend: unsupported number of rows");
  // ivf_pq_build.cuh:1011-1012
  CUVS_EXPECTS(new_indices != nullptr || idx->size() == 0,
               "You must pass data indices when the index is non-empty.");
  const uint64_t n = uint64_t(n_rows_i);
  if (n == 0) { return; }
  const cudaStream_t stream = res.stream;
  const uint32_t dim = idx->dim(), dim_ext = idx->dim_ext(), n_lists = idx->n_lists();
  const label_ctx lc   = labeling_of(idx->metric());
  const uint64_t chunk = std::min<uint64_t>(n, chunk_rows_for(dim_ext));

  dev_array<uint8_t> staging;
  dev_array<float> x_ext(chunk * dim_ext);
  dev_array<unsigned long long> best(chunk);
  dev_array<uint32_t> labels(n);
  dev_array<uint32_t> counts(n_lists);
  CUDA_TRY(cudaMemsetAsync(counts.data(), 0, size_t(n_lists) * 4, stream));

  // pass 1: labels + histogram
  nearest_labeler labeler(res, idx->centers(), n_lists, dim, dim_ext, lc.alpha);
  for (uint64_t r0 = 0; r0 < n; r0 += chunk) {
    const uint64_t nr = std::min(chunk, n - r0);
    const void* src   = stage_rows(res, new_vectors, dtype, r0, nr, dim, on_device, staging);
    to_float_ext(res, src, dtype, nr, 1, dim, dim_ext, lc.pad, lc.normalize, x_ext.data());
    labeler.run(x_ext.data(), uint32_t(nr), labels.data() + r0, best.data());
    if (!on_device) { res.sync(); }
  }
  histogram_kernel<<<unsigned(ceildiv<uint64_t>(n, 256)), 256, 0, stream>>>(labels.data(), n, counts.data());
  std::vector<uint32_t> h_counts(n_lists);
  CUDA_TRY(cudaMemcpyAsync(h_counts.data(), counts.data(), size_t(n_lists) * 4, cudaMemcpyDeviceToHost, stream));
  res.sync();

  // new arenas, old payload moved over
  std::vector<uint32_t> old_sizes = idx->host_list_sizes();
  std::vector<uint32_t> new_sizes(n_lists);
  for (uint32_t l = 0; l < n_lists; l++) {
    CUVS_EXPECTS(uint64_t(old_sizes[l]) + h_counts[l] < (1ull << 32), "list %u grows beyond 2^32 rows", l);
    new_sizes[l] = old_sizes[l] + h_counts[l];
  }
  resize_lists(res, idx, new_sizes);

  // pass 2: per chunk, order rows by list (stable), give each its slot, encode
  dev_array<uint32_t> fill(n_lists);  // rows already placed in each list
  CUDA_TRY(cudaMemcpyAsync(fill.data(), old_sizes.data(), size_t(n_lists) * 4, cudaMemcpyHostToDevice, stream));
  dev_array<uint32_t> iota(chunk), order(chunk), sorted_labels(chunk), slots(chunk), chunk_counts(n_lists);
  size_t cub_bytes = 0;
  int end_bit      = 1;
  while ((1ull << end_bit) < n_lists) { end_bit++; }
  cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, labels.data(), sorted_labels.data(), iota.data(),
                                  order.data(), int(chunk), 0, end_bit, stream);
  dev_array<uint8_t> cub_tmp(cub_bytes);
  for (uint64_t r0 = 0; r0 < n; r0 += chunk) {
    const uint32_t nr = uint32_t(std::min(chunk, n - r0));
    const void* src   = stage_rows(res, new_vectors, dtype, r0, nr, dim, on_device, staging);
    to_float_ext(res, src, dtype, nr, 1, dim, dim_ext, lc.pad, lc.normalize, x_ext.data());
    iota_kernel<<<ceildiv(nr, 256u), 256, 0, stream>>>(iota.data(), nr);
    cub::DeviceRadixSort::SortPairs(cub_tmp.data(), cub_bytes, labels.data() + r0, sorted_labels.data(),
                                    iota.data(), order.data(), int(nr), 0, end_bit, stream);
    slots_kernel<<<ceildiv(nr, 256u), 256, 0, stream>>>(sorted_labels.data(), nr, fill.data(), slots.data());
    const int64_t* ids_chunk = new_indices ? new_indices + r0 : nullptr;
    dev_array<int64_t> ids_staging;
    if (new_indices && !on_device) {
      ids_staging.resize(nr);
      CUDA_TRY(cudaMemcpyAsync(ids_staging.data(), new_indices + r0, size_t(nr) * 8, cudaMemcpyHostToDevice, stream));
      ids_chunk = ids_staging.data();
    }
    launch_encode(res, *idx, x_ext.data(), labels.data() + r0, order.data(), slots.data(), nr, true,
                  idx->codes(), idx->ids(), ids_chunk, int64_t(r0));
    CUDA_TRY(cudaMemsetAsync(chunk_counts.data(), 0, size_t(n_lists) * 4, stream));
    histogram_kernel<<<ceildiv(nr, 256u), 256, 0, stream>>>(labels.data() + r0, nr, chunk_counts.data());
    add_u32_kernel<<<ceildiv(n_lists, 256u), 256, 0, stream>>>(fill.data(), chunk_counts.data(), n_lists);
    CUDA_TRY(cudaGetLastError());
    res.launches += 5;
    res.sync();  // staging buffers are reused by the next chunk
  }
}

// ------------------------------------------------------------------------------------------------
// transform
// ------------------------------------------------------------------------------------------------
void transform_any(raft::resources& res, const index<int64_t>& idx, const void* dataset, elem_t dtype,
                   int64_t n_rows_i, uint32_t* out_labels, uint8_t* out_codes)
{
  CUVS_EXPECTS(n_rows_i >= 0 && n_rows_i < (1ll << 32), "transform: unsupported number of rows");
  const uint64_t n = uint64_t(n_rows_i);
  if (n == 0) { return; }
  const uint32_t dim = idx.dim(), dim_ext = idx.dim_ext();
  const label_ctx lc   = labeling_of(idx.metric());
  const uint64_t chunk = std::min<uint64_t>(n, chunk_rows_for(dim_ext));
  const uint32_t flat  = ceildiv(idx.pq_dim() * idx.pq_bits(), 8u);
  dev_array<float> x_ext(chunk * dim_ext);
  dev_array<unsigned long long> best(chunk);
  nearest_labeler labeler(res, idx.centers(), idx.n_lists(), dim, dim_ext, lc.alpha);
  for (uint64_t r0 = 0; r0 < n; r0 += chunk) {
    const uint32_t nr = uint32_t(std::min(chunk, n - r0));
    const char* src   = static_cast<const char*>(dataset) + r0 * dim * elem_size(dtype);
    to_float_ext(res, src, dtype, nr, 1, dim, dim_ext, lc.pad, lc.normalize, x_ext.data());
    labeler.run(x_ext.data(), nr, out_labels + r0, best.data());
    launch_encode(res, idx, x_ext.data(), out_labels + r0, nullptr, nullptr, nr, false,
                  out_codes + r0 * flat, nullptr, nullptr, 0);
    res.sync();
  }
}

// ------------------------------------------------------------------------------------------------
// build
// ------------------------------------------------------------------------------------------------
void build_any(raft::resources& res, const index_params& params, const void* dataset, elem_t dtype,
               int64_t n_rows_i, uint32_t dim, bool on_device, index<int64_t>* out)
{
  CUVS_EXPECTS(n_rows_i > 0 && dim > 0, "build: empty dataset");
  CUVS_EXPECTS(params.n_lists > 0, "n_lists must be positive");
  const uint64_t n_rows     = uint64_t(n_rows_i);
  const cudaStream_t stream = res.stream;
  index<int64_t> idx(params.metric, params.codebook_kind, params.n_lists, dim, params.pq_bits,
                     params.pq_dim, params.conservative_memory_allocation, params.codes_layout);
  const uint32_t n_lists = idx.n_lists(), dim_ext = idx.dim_ext(), rot_dim = idx.rot_dim();
  const uint32_t book = idx.pq_book_size(), len = idx.pq_len(), pq_dim = idx.pq_dim();
  const label_ctx lc  = labeling_of(idx.metric());

  // ---- trainset (ivf_pq_build.cuh:1283-1290): every `stride`-th row ----
  const double frac      = std::min(1.0, std::max(0.0, params.kmeans_trainset_fraction));
  const uint64_t want    = std::max<uint64_t>(uint64_t(frac * double(n_rows)), n_lists);
  const uint64_t stride  = std::max<uint64_t>(1, n_rows / std::max<uint64_t>(1, want));
  const uint64_t n_train = n_rows / stride;
  CUVS_EXPECTS(n_train < (1ull << 32), "trainset too large");
  dev_array<float> train(n_train * dim_ext);
  {
    dev_array<uint8_t> staging;
    const void* src = dataset;
    if (!on_device) {
      const size_t rb = size_t(dim) * elem_size(dtype);
      staging.resize(n_train * rb);
      CUDA_TRY(cudaMemcpy2DAsync(staging.data(), rb, dataset, rb * stride, rb, n_train,
                                 cudaMemcpyHostToDevice, stream));
      src = staging.data();
      to_float_ext(res, src, dtype, n_train, 1, dim, dim_ext, lc.pad, lc.normalize, train.data());
      res.sync();
    } else {
      to_float_ext(res, src, dtype, n_train, stride, dim, dim_ext, lc.pad, lc.normalize, train.data());
    }
  }

  // ---- coarse k-means ----
  dev_array<uint32_t> labels(n_train);
  dev_array<unsigned long long> best(n_train);
  dev_array<float> sums(size_t(n_lists) * dim);
  dev_array<uint32_t> counts(n_lists);
  init_centers_kernel<<<n_lists, 128, 0, stream>>>(train.data(), n_train, n_lists, dim_ext, idx.centers());
  center_norms_kernel<<<ceildiv(n_lists, 128u), 128, 0, stream>>>(idx.centers(), n_lists, dim, dim_ext);
  res.launches += 2;
  const uint32_t iters = std::max<uint32_t>(1, params.kmeans_n_iters);
  for (uint32_t it = 0; it < iters; it++) {
    nearest_labeler(res, idx.centers(), n_lists, dim, dim_ext, lc.alpha)
      .run(train.data(), uint32_t(n_train), labels.data(), best.data());
    CUDA_TRY(cudaMemsetAsync(sums.data(), 0, sums.size() * 4, stream));
    CUDA_TRY(cudaMemsetAsync(counts.data(), 0, size_t(n_lists) * 4, stream));
    accumulate_kernel<<<unsigned(ceildiv<uint64_t>(n_train * 32, 256)), 256, 0, stream>>>(
      train.data(), labels.data(), n_train, dim, dim_ext, sums.data(), counts.data());
    finalize_centers_kernel<<<n_lists, 128, 0, stream>>>(sums.data(), counts.data(), dim, dim_ext,
                                                         train.data(), n_train, it + 1, lc.normalize,
                                                         idx.centers());
    CUDA_TRY(cudaGetLastError());
    res.launches += 2;
    // Balancing (not after the last step, whose means are final): clusters sorted by size, the i-th
    // smallest paired with the i-th largest; where the small one is underfull (< 1/3 of the average)
    // or the large one overfull (> 3 x the average), the small one restarts next to the large one.
    if (it + 1 < iters && n_lists >= 2) {
      std::vector<uint32_t> h_counts(n_lists);
      CUDA_TRY(cudaMemcpyAsync(h_counts.data(), counts.data(), size_t(n_lists) * 4, cudaMemcpyDeviceToHost, stream));
      res.sync();
      std::vector<uint32_t> order(n_lists);
      for (uint32_t l = 0; l < n_lists; l++) { order[l] = l; }
      std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
        return h_counts[a] != h_counts[b] ? h_counts[a] < h_counts[b] : a < b;
      });
      const double avg = double(n_train) / double(n_lists);
      std::vector<uint32_t> h_pairs;
      for (uint32_t i = 0; i < n_lists / 2; i++) {
        const uint32_t small = order[i], large = order[n_lists - 1 - i];
        const bool underfull = double(h_counts[small]) < avg * kBalanceLower;
        const bool overfull  = double(h_counts[large]) > avg * kBalanceUpper;
        if (!underfull && !overfull) { break; }  // sizes are sorted: no later pair qualifies either
        if (h_counts[large] < 2) { break; }
        h_pairs.push_back(small);
        h_pairs.push_back(large);
      }
      if (!h_pairs.empty()) {
        dev_array<uint32_t> d_pairs(h_pairs.size());
        dev_array<unsigned long long> member(n_lists);
        CUDA_TRY(cudaMemcpyAsync(d_pairs.data(), h_pairs.data(), h_pairs.size() * 4, cudaMemcpyHostToDevice, stream));
        CUDA_TRY(cudaMemsetAsync(member.data(), 0, size_t(n_lists) * 8, stream));
        pick_member_kernel<<<unsigned(ceildiv<uint64_t>(n_train, 256)), 256, 0, stream>>>(labels.data(), n_train,
                                                                                         it + 1, member.data());
        adjust_centers_kernel<<<unsigned(h_pairs.size() / 2), 128, 0, stream>>>(
          idx.centers(), d_pairs.data(), member.data(), train.data(), dim, dim_ext, kCentroidOffset, lc.normalize);
        CUDA_TRY(cudaGetLastError());
        res.sync();  // the pair list and the member table are released here
        res.launches += 2;
      }
    }
  }
  nearest_labeler(res, idx.centers(), n_lists, dim, dim_ext, lc.alpha)
    .run(train.data(), uint32_t(n_train), labels.data(), best.data());

  // ---- rotation, rotated centers ----
  {
    std::vector<float> rot;
    make_rotation(rot_dim, dim, params.force_random_rotation, rot);
    CUDA_TRY(cudaMemcpyAsync(idx.rotation_matrix(), rot.data(), rot.size() * 4, cudaMemcpyHostToDevice, stream));
    res.sync();
  }
  rotate_centers_kernel<<<unsigned(ceildiv<uint64_t>(uint64_t(n_lists) * rot_dim, 256)), 256, 0, stream>>>(
    idx.centers(), idx.rotation_matrix(), n_lists, dim, dim_ext, rot_dim, idx.centers_rot());
  res.launches++;
  idx.allocate_lists(std::vector<uint32_t>(n_lists, 0), stream);  // also detects an identity rotation

  // ---- PQ codebooks ----
  {
    const uint64_t max_pts = uint64_t(std::max<uint32_t>(1, params.max_train_points_per_pq_code)) * book;
    const bool per_cluster = idx.codebook_kind() == codebook_gen::PER_CLUSTER;
    const uint64_t n_pq    = per_cluster ? n_train : std::min<uint64_t>(n_train, max_pts);
    const uint64_t pstride = std::max<uint64_t>(1, n_train / n_pq);
    dev_array<float> resid(n_pq * rot_dim);
    residual_kernel<<<unsigned(n_pq), 128, size_t(dim) * 4, stream>>>(
      train.data(), labels.data(), pstride, idx.centers(), idx.rotation_matrix(),
      idx.rotation_is_identity(), dim, dim_ext, rot_dim, resid.data());
    res.launches++;
    const size_t smem = size_t(book) * len * 8 + size_t(book) * 4;
    CUVS_EXPECTS(smem <= 200 * 1024, "pq_len = %u is too large for codebook training", len);
    ensure_dynamic_smem(reinterpret_cast<const void*>(train_codebooks_kernel), smem);
    const int pq_iters = 25;
    if (!per_cluster) {
      train_codebooks_kernel<<<pq_dim, 1024, smem, stream>>>(resid.data(), uint32_t(n_pq), rot_dim, pq_dim,
                                                             len, book, 0, nullptr, nullptr, 0, pq_iters,
                                                             idx.pq_centers());
    } else {
      // rows of each list: stable sort of the trainset labels
      dev_array<uint32_t> iota(n_train), order(n_train), sorted_labels(n_train), begin(size_t(n_lists) + 1);
      iota_kernel<<<unsigned(ceildiv<uint64_t>(n_train, 256)), 256, 0, stream>>>(iota.data(), uint32_t(n_train));
      size_t cub_bytes = 0;
      int end_bit      = 1;
      while ((1ull << end_bit) < n_lists) { end_bit++; }
      cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, labels.data(), sorted_labels.data(), iota.data(),
                                      order.data(), int(n_train), 0, end_bit, stream);
      dev_array<uint8_t> tmp(cub_bytes);
      cub::DeviceRadixSort::SortPairs(tmp.data(), cub_bytes, labels.data(), sorted_labels.data(), iota.data(),
                                      order.data(), int(n_train), 0, end_bit, stream);
      CUDA_TRY(cudaMemsetAsync(begin.data(), 0, (size_t(n_lists) + 1) * 4, stream));
      histogram_kernel<<<unsigned(ceildiv<uint64_t>(n_train, 256)), 256, 0, stream>>>(labels.data(), n_train, begin.data());
      std::vector<uint32_t> hb(size_t(n_lists) + 1);
      CUDA_TRY(cudaMemcpyAsync(hb.data(), begin.data(), (size_t(n_lists) + 1) * 4, cudaMemcpyDeviceToHost, stream));
      res.sync();
      uint32_t run = 0;
      for (uint32_t l = 0; l <= n_lists; l++) {
        uint32_t c = hb[l];
        hb[l]      = run;
        run += (l < n_lists ? c : 0);
      }
      CUDA_TRY(cudaMemcpyAsync(begin.data(), hb.data(), (size_t(n_lists) + 1) * 4, cudaMemcpyHostToDevice, stream));
      const uint32_t max_rows = uint32_t(std::max<uint64_t>(1, ceildiv<uint64_t>(max_pts, pq_dim)));
      train_codebooks_kernel<<<n_lists, 256, smem, stream>>>(resid.data(), uint32_t(n_pq), rot_dim, pq_dim,
                                                             len, book, 1, order.data(), begin.data(),
                                                             max_rows, pq_iters, idx.pq_centers());
      res.sync();
    }
    CUDA_TRY(cudaGetLastError());
    res.launches++;
    res.sync();
  }

  // ---- fill ----
  if (params.add_data_on_build) {
    train.reset();
    extend_any(res, dataset, dtype, n_rows_i, nullptr, on_device, &idx);
  }
  *out = std::move(idx);
}

}  // namespace cuvs::neighbors::ivf_pq
