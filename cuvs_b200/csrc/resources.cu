#include "common.hpp"

namespace cuvs_b200 {

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
  if (pinned) { cudaFreeHost(pinned); }
}

}  // namespace cuvs_b200
