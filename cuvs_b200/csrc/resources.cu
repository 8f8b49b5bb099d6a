#include "common.hpp"

#include <nvtx3/nvToolsExt.h>

#include <mutex>

namespace cuvs_b200 {

namespace {
nvtxDomainHandle_t nvtx_domain()
{
  static nvtxDomainHandle_t d = nvtxDomainCreateA("cuvs");
  return d;
}
}  // namespace

nvtx_range::nvtx_range(const char* fmt, ...)
{
  nvtxDomainHandle_t d = nvtx_domain();
  if (d == nullptr) { return; }  // no tool attached: the domain handle is null and nothing is recorded
  char buf[256];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  nvtxEventAttributes_t attr{};
  attr.version       = NVTX_VERSION;
  attr.size          = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
  attr.messageType   = NVTX_MESSAGE_TYPE_ASCII;
  attr.message.ascii = buf;
  nvtxDomainRangePushEx(d, &attr);
  pushed_ = true;
}

nvtx_range::~nvtx_range()
{
  if (pushed_) { nvtxDomainRangePop(nvtx_domain()); }
}

void ensure_dynamic_smem(const void* kernel, size_t bytes)
{
  static std::mutex lock;
  static std::map<std::pair<const void*, int>, size_t> done;
  int dev = 0;
  CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> guard(lock);
  size_t& have = done[{kernel, dev}];
  if (bytes > have) {
    CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
    have = bytes;
  }
}

resources::resources()
{
  CUDA_TRY(cudaGetDevice(&device));
  cudaDeviceProp prop{};
  CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  sm_count   = prop.multiProcessorCount;
  smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
  cc_major   = prop.major;
  CUDA_TRY(cudaMallocHost(&pinned, 64));
}

resources::~resources()
{
  for (auto& ev : pending) {
    for (auto& e : ev.e) { cudaEventDestroy(e); }
  }
  if (tc_redo_event) { cudaEventDestroy(tc_redo_event); }
  if (d_stats) { cudaFree(d_stats); }
  if (pinned) { cudaFreeHost(pinned); }
}

void resources::adopt_tc_verdict()
{
  if (!tc_redo_pending || cudaEventQuery(tc_redo_event) != cudaSuccess) { return; }
  tc_redo_pending = false;
  if (pinned[8] != 0u) {
    // the coarse GEMM of that batch gave up on a bounded wait; its probes were all recomputed exactly
    tc_timeouts++;
  } else if (tc_redo_adapts) {
    tc_level& lv = tc_levels[tc_redo_n_probes];
    if (uint64_t(pinned[9]) * 256 > tc_redo_queries && lv.products < 3) {
      // more than 1/256 of the batch failed the exactness guard: one more product of the TF32 split,
      // and never fewer again on this handle for this n_probes
      lv.products++;
      lv.floor = lv.products;
    } else if (lv.products > lv.floor && uint64_t(pinned[11]) * 1024 <= tc_redo_queries) {
      // (almost) every query of the batch would have passed the guard with one product less
      lv.products--;
    }
  }
}

void resources::sync()
{
  CUDA_TRY(cudaStreamSynchronize(stream));
  adopt_tc_verdict();
}

void resources::stats_enable(bool on)
{
  if (on && !d_stats) {
    CUDA_TRY(cudaMalloc(&d_stats, 16));
    CUDA_TRY(cudaMemset(d_stats, 0, 16));
  }
  stats_enabled = on;
}

void resources::stats_mark(stage_events& ev, int i)
{
  if (i == 0) {
    for (auto& e : ev.e) { CUDA_TRY(cudaEventCreate(&e)); }
  }
  CUDA_TRY(cudaEventRecord(ev.e[i], stream));
}

void resources::stats_resolve()
{
  CUDA_TRY(cudaStreamSynchronize(stream));
  for (auto& ev : pending) {
    for (int i = 0; i < 5; i++) {
      float ms = 0.0f;
      CUDA_TRY(cudaEventElapsedTime(&ms, ev.e[i], ev.e[i + 1]));
      stage_ms[i] += ms;
    }
    for (auto& e : ev.e) { cudaEventDestroy(e); }
    stat_batches++;
  }
  pending.clear();
}

}  // namespace cuvs_b200
