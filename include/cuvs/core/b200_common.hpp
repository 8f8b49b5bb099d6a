// Shared host-side plumbing of the IVF-PQ engine: error type and checks, resources handle, and the
// grow-only device workspace that lets a steady-state search run without any allocation.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#pragma GCC visibility push(default)

namespace cuvs_b200 {

// Same role as raft::logic_error in the reference: argument/format errors surfaced to the caller.
struct error : public std::runtime_error {
  using std::runtime_error::runtime_error;
};

[[noreturn]] inline void fail(const char* fmt, ...)
{
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  throw error(buf);
}

#define CUVS_EXPECTS(cond, ...)                       \
  do {                                                \
    if (!(cond)) { ::cuvs_b200::fail(__VA_ARGS__); }  \
  } while (0)

#define CUDA_TRY(call)                                                                       \
  do {                                                                                       \
    cudaError_t e__ = (call);                                                                \
    if (e__ != cudaSuccess) {                                                                \
      ::cuvs_b200::fail("CUDA error %s at %s:%d: %s", cudaGetErrorName(e__), __FILE__,       \
                        __LINE__, cudaGetErrorString(e__));                                  \
    }                                                                                        \
  } while (0)

#ifdef __CUDACC__
#define CUVS_HD __host__ __device__
#else
#define CUVS_HD
#endif

template <typename T>
CUVS_HD constexpr T ceildiv(T a, T b)
{
  return (a + b - 1) / b;
}
template <typename T>
CUVS_HD constexpr T round_up(T a, T b)
{
  return ceildiv(a, b) * b;
}

// Raises a kernel's limit of dynamic shared memory to `bytes` on the current device unless it has
// already been raised that far there.  The attribute belongs to the device's context -- one value for
// all threads of the process, one per device -- and setting it again LOWERS it if the new value is
// smaller, so the record of what has been set is process-wide and the limit only ever grows.
void ensure_dynamic_smem(const void* kernel, size_t bytes);

// A named range in the NVTX domain "cuvs" for the lifetime of the object (the ranges of the reference's
// search, cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:74, 436, 894, 974).  NVTX v3 is header-only and
// does nothing unless a profiler is attached; the text is only formatted when one is.
class nvtx_range {
 public:
  explicit nvtx_range(const char* fmt, ...);
  ~nvtx_range();
  nvtx_range(const nvtx_range&)            = delete;
  nvtx_range& operator=(const nvtx_range&) = delete;

 private:
  bool pushed_ = false;
};

// One grow-only device buffer carved into aligned slices per call.
class workspace {
 public:
  ~workspace() { release(); }
  void reserve(size_t bytes)
  {
    if (bytes <= cap_) { return; }
    release();
    CUDA_TRY(cudaMalloc(&base_, bytes));
    cap_ = bytes;
  }
  void release()
  {
    if (base_) { cudaFree(base_); }
    base_ = nullptr;
    cap_  = 0;
  }
  size_t capacity() const { return cap_; }
  char* base() const { return static_cast<char*>(base_); }

 private:
  void* base_ = nullptr;
  size_t cap_ = 0;
};

// Computes slice offsets first (dry run), then hands out pointers from a workspace.
class ws_layout {
 public:
  size_t add(size_t bytes)
  {
    size_t off = total_;
    total_ += round_up<size_t>(bytes ? bytes : 1, 256);
    return off;
  }
  size_t total() const { return total_; }

 private:
  size_t total_ = 0;
};

// The opaque object behind cuvsResources_t (raft::resources in the reference): device, stream,
// workspace.  One per host thread, like the reference handle.
struct resources {
  int kind              = 0;        // 0 = one device; 1 = the multi-GPU clique handle (mg.hpp)
  int device            = 0;
  cudaStream_t stream   = nullptr;  // caller-set; default stream otherwise
  int sm_count          = 0;
  int smem_optin        = 0;        // max dynamic shared memory per block (opt-in)
  int cc_major          = 0;
  workspace ws;
  // small pinned host word for an occasional device->host scalar
  uint32_t* pinned = nullptr;
  // counters read by the benchmark ("how many kernels of ours ran")
  uint64_t launches = 0;

  // Optional stage timing (off by default): five events per internal batch, resolved on demand.
  struct stage_events {
    cudaEvent_t e[6];
  };
  bool stats_enabled = false;
  std::vector<stage_events> pending;
  double stage_ms[5]      = {0, 0, 0, 0, 0};
  uint64_t stat_batches   = 0;
  uint64_t stat_pairs     = 0;
  unsigned long long* d_stats = nullptr;  // [2] device counters: scan groups, unique groups
  void stats_enable(bool on);
  void stats_mark(stage_events& ev, int i);
  void stats_resolve();

  // Tensor-core coarse stage: products of the TF32 split per K step used by this handle (start at
  // two; raised when a finished batch had to redo more than 1/256 of its queries exactly, lowered when
  // all but 1/1024 of a batch would have passed the guard with one product less); the counters of the
  // last batch arrive in pinned[8..11] once tc_redo_event has completed.
  // List-sharded multi-GPU search: when set, the fine search scans the pairs of every query's nearest
  // probe first, calls this with (stream, per-query bounds on the k-th best ordered score, n_queries)
  // -- the caller enqueues a min-reduction of the bounds over the ranks -- and then scans the rest.
  std::function<void(cudaStream_t, uint32_t*, uint32_t)> scan_phase_hook;
  // The level is kept per n_probes (the guard's margin depends on it: a handle that once served
  // n_probes = 200 must not pay for that when it serves n_probes = 20).
  struct tc_level {
    int products = 2;
    int floor    = 1;  // raised when a level produced too many exact redos
  };
  std::map<uint32_t, tc_level> tc_levels;
  uint32_t tc_redo_n_probes  = 0;  // n_probes of the batch whose counters are in flight
  cudaEvent_t tc_redo_event  = nullptr;
  bool tc_redo_pending       = false;
  uint32_t tc_redo_queries   = 0;
  bool tc_redo_adapts        = false;
  void adopt_tc_verdict();
  // batches whose coarse GEMM gave up on a bounded wait (their probes were recomputed exactly)
  uint64_t tc_timeouts       = 0;

  resources();
  ~resources();
  resources(const resources&)            = delete;
  resources& operator=(const resources&) = delete;
  void sync();
};

}  // namespace cuvs_b200

#pragma GCC visibility pop
