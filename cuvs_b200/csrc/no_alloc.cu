// cuvsIvfPqPredictNoAlloc: nearest-list labels for a batch of vectors without allocating anything.
//
// Who this is for.  Some hosts of this library are not allowed to allocate device memory while they
// serve traffic: a process whose GPU memory was handed out in full to a framework allocator at
// start-up (a cudaMalloc from a plug-in would fail or fragment it), a latency-critical thread that
// must not take the driver-wide lock and implicit synchronisation that cudaMalloc / cudaFree imply,
// or a sandboxed extension that is only given pre-existing buffers.  The regular entry points size
// a workspace on demand; this one never does.
//
// How.  The labelling kernel needs one 64-bit scratch word per input row (the running
// "best (score, list)" that thread blocks combine with atomicMin).  Here that scratch is a
// file-scope __device__ array of fixed size, so it is part of the loaded module: every GPU that
// loads the library holds kNoAllocMaxRows * 8 bytes (512 KiB) until the process exits.
//   * Batches larger than kNoAllocMaxRows rows are rejected with an error; split them.
//   * The array is shared by every call in the process and keeps the previous call's contents; each
//     call re-initialises the part it uses.  Two calls that overlap on the GPU (different streams or
//     threads) would race on it -- issue them one after the other.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
//     caches it; that first call should happen before any stream capture begins.
// Arithmetic is the same FMA chain as the regular labelling path, so labels are identical to the
// ones cuvsIvfPqTransform returns.
#include "../../include/cuvs_ivf_pq.h"

#include "ivf_pq.hpp"
#include "topk.cuh"

#include <mutex>

namespace {

using namespace cuvs_b200;
namespace ivf_pq = cuvs::neighbors::ivf_pq;

constexpr uint32_t kNoAllocMaxRows = 65536;
constexpr int kMaxDevices          = 64;

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress, never a
// device pointer.
static __device__ __align__(256) unsigned long long g_best_scratch[kNoAllocMaxRows];

std::mutex g_setup_mutex;
unsigned long long* g_scratch_ptr[kMaxDevices] = {};

unsigned long long* scratch_for_current_device()
{
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  CUVS_EXPECTS(dev >= 0 && dev < kMaxDevices, "device ordinal %d is out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    unsigned long long* ptr = nullptr;
    CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_best_scratch));
    CUVS_EXPECTS(ptr != nullptr, "could not resolve the scratch array on device %d", dev);
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

template <typename T>
__device__ __forceinline__ float as_float(T x);
template <> __device__ __forceinline__ float as_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float as_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float as_float<int8_t>(int8_t x) { return float(x) * (1.0f / 128.0f); }
template <> __device__ __forceinline__ float as_float<uint8_t>(uint8_t x) { return float(x) * (1.0f / 256.0f); }

constexpr int kTile  = 64;
constexpr int kTileK = 16;

__global__ void reset_scratch_kernel(unsigned long long* __restrict__ best, uint32_t n)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { best[i] = ~0ull; }
}

// 64 rows x 64 lists per block, 4 x 4 outputs per thread, ascending-k FMA chain per output.
// Rows are read in their source type; column `dim` of the padded row is -0.5 and the tail is zero.
template <typename T>
__global__ void __launch_bounds__(256)
predict_kernel(const float* __restrict__ centers, const T* __restrict__ x, uint32_t n_lists,
               uint32_t n_rows, uint32_t dim, uint32_t dim_ext, unsigned long long* __restrict__ best)
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
      float v      = 0.0f;
      if (q < n_rows) {
        if (k < dim) {
          v = as_float<T>(x[size_t(q) * dim + k]);
        } else if (k == dim) {
          v = -0.5f;
        }
      }
      s_q[kk][row] = v;
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
          ((unsigned long long)float_to_ordered(__fmul_rn(-2.0f, acc[i][j])) << 32) | l;
        m = key < m ? key : m;
      }
    }
#pragma unroll
    for (int d = 8; d > 0; d >>= 1) {
      const unsigned long long o = __shfl_xor_sync(kFullMask, m, d);
      m = o < m ? o : m;
    }
    if (tx == 0 && q < n_rows) { atomicMin(best + q, m); }
  }
}

__global__ void write_labels_kernel(const unsigned long long* __restrict__ best, uint32_t n,
                                    uint32_t* __restrict__ labels)
{
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { labels[i] = uint32_t(best[i]); }
}

template <typename T>
void launch_predict(cudaStream_t stream, const ivf_pq::index<int64_t>& ix, const void* x, uint32_t n,
                    uint32_t* labels, unsigned long long* best)
{
  reset_scratch_kernel<<<ceildiv(n, 256u), 256, 0, stream>>>(best, n);
  dim3 grid(ceildiv<uint32_t>(ix.n_lists(), kTile), ceildiv<uint32_t>(n, kTile));
  predict_kernel<T><<<grid, 256, 0, stream>>>(ix.centers(), static_cast<const T*>(x), ix.n_lists(), n,
                                              ix.dim(), ix.dim_ext(), best);
  write_labels_kernel<<<ceildiv(n, 256u), 256, 0, stream>>>(best, n, labels);
  CUDA_TRY(cudaGetLastError());
}

bool device_accessible(const DLTensor& t)
{
  return t.device.device_type == kDLCUDA || t.device.device_type == kDLCUDAHost ||
         t.device.device_type == kDLCUDAManaged;
}
bool compact(const DLTensor& t)
{
  if (!t.strides) { return true; }
  int64_t expected = 1;
  for (int64_t i = t.ndim - 1; i >= 0; --i) {
    if (t.strides[i] != expected) { return false; }
    expected *= t.shape[i];
  }
  return true;
}

}  // namespace

extern "C" cuvsError_t cuvsIvfPqPredictNoAlloc(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                               DLManagedTensor* vectors, DLManagedTensor* labels)
{
  try {
    CUVS_EXPECTS(res != 0 && index != nullptr && index->addr != 0 && vectors && labels, "null argument");
    auto* r        = reinterpret_cast<cuvs_b200::resources*>(res);
    const auto& ix = *reinterpret_cast<ivf_pq::index<int64_t>*>(index->addr);
    const DLTensor& v = vectors->dl_tensor;
    const DLTensor& l = labels->dl_tensor;
    CUVS_EXPECTS(device_accessible(v) && device_accessible(l),
                 "vectors and labels should have device compatible memory");
    CUVS_EXPECTS(compact(v) && compact(l), "Expected a row-major matrix");
    CUVS_EXPECTS(v.ndim == 2 && l.ndim == 1 && v.dtype.lanes == 1 && l.dtype.lanes == 1,
                 "vectors must be a matrix and labels a vector");
    CUVS_EXPECTS(l.dtype.code == kDLUInt && l.dtype.bits == 32, "labels should be of type uint32_t");
    CUVS_EXPECTS(v.shape[1] == int64_t(ix.dim()),
                 "Number of columns of vectors should equal number of dimensions in the index.");
    CUVS_EXPECTS(l.shape[0] == v.shape[0], "labels must have one entry per vector");
    CUVS_EXPECTS(v.shape[0] >= 0 && v.shape[0] <= int64_t(kNoAllocMaxRows),
                 "cuvsIvfPqPredictNoAlloc handles at most %u rows per call (got %lld); split the batch",
                 kNoAllocMaxRows, (long long)v.shape[0]);
    CUVS_EXPECTS(ix.metric() != ivf_pq::DistanceType::CosineExpanded,
                 "cuvsIvfPqPredictNoAlloc does not support CosineExpanded indexes");
    const uint32_t n = uint32_t(v.shape[0]);
    if (n > 0) {
      unsigned long long* best = scratch_for_current_device();
      const void* x            = static_cast<const char*>(v.data) + v.byte_offset;
      auto* out = reinterpret_cast<uint32_t*>(static_cast<char*>(l.data) + l.byte_offset);
      if (v.dtype.code == kDLFloat && v.dtype.bits == 32) {
        launch_predict<float>(r->stream, ix, x, n, out, best);
      } else if (v.dtype.code == kDLFloat && v.dtype.bits == 16) {
        launch_predict<__half>(r->stream, ix, x, n, out, best);
      } else if (v.dtype.code == kDLInt && v.dtype.bits == 8) {
        launch_predict<int8_t>(r->stream, ix, x, n, out, best);
      } else if (v.dtype.code == kDLUInt && v.dtype.bits == 8) {
        launch_predict<uint8_t>(r->stream, ix, x, n, out, best);
      } else {
        fail("Unsupported vectors DLtensor dtype: %d and bits: %d", int(v.dtype.code), int(v.dtype.bits));
      }
      r->launches += 3;
    }
    cuvsSetLastErrorText(nullptr);
    return CUVS_SUCCESS;
  } catch (const std::exception& e) {
    cuvsSetLastErrorText(e.what());
  } catch (...) {
    cuvsSetLastErrorText("unknown exception");
  }
  return CUVS_ERROR;
}
