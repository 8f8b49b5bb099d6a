// Instantiations of the fine-search kernel for one code width (compiled once per PQ_BITS = 4..8).
#include "common.hpp"
#include "scan.cuh"

#ifndef PQ_BITS
#error "compile with -DPQ_BITS=4..8"
#endif

namespace cuvs_b200 {

namespace {

template <int LutKind, bool OutHalf, bool IsIP, int KPL>
void launch_one(const scan_params& p, int grid, size_t smem, cudaStream_t stream)
{
  auto kernel = scan_kernel<PQ_BITS, LutKind, OutHalf, IsIP, KPL>;
  ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
  kernel<<<grid, 1024, smem, stream>>>(p);
  CUDA_TRY(cudaGetLastError());
}

template <int LutKind, bool OutHalf, bool IsIP>
void launch_kpl(const scan_params& p, int kpl, int grid, size_t smem, cudaStream_t stream)
{
  switch (kpl) {
    case 0: launch_one<LutKind, OutHalf, IsIP, 0>(p, grid, smem, stream); break;
    case 1: launch_one<LutKind, OutHalf, IsIP, 1>(p, grid, smem, stream); break;
    case 2: launch_one<LutKind, OutHalf, IsIP, 2>(p, grid, smem, stream); break;
    default: launch_one<LutKind, OutHalf, IsIP, 4>(p, grid, smem, stream); break;
  }
}

template <bool IsIP>
void launch_types(const scan_params& p, int lut_kind, bool out_half, int kpl, int grid, size_t smem,
                  cudaStream_t stream)
{
  if (!out_half) {
    switch (lut_kind) {
      case LUT_F32: launch_kpl<LUT_F32, false, IsIP>(p, kpl, grid, smem, stream); break;
      case LUT_F16: launch_kpl<LUT_F16, false, IsIP>(p, kpl, grid, smem, stream); break;
      default: launch_kpl<LUT_FP8, false, IsIP>(p, kpl, grid, smem, stream); break;
    }
  } else {
    switch (lut_kind) {
      case LUT_F16: launch_kpl<LUT_F16, true, IsIP>(p, kpl, grid, smem, stream); break;
      case LUT_FP8: launch_kpl<LUT_FP8, true, IsIP>(p, kpl, grid, smem, stream); break;
      default: fail("fp32 look-up table with fp16 internal distances is not a valid combination");
    }
  }
}

}  // namespace

#define SCAN_FN_NAME2(b) launch_scan_bits_##b
#define SCAN_FN_NAME(b) SCAN_FN_NAME2(b)

void SCAN_FN_NAME(PQ_BITS)(const scan_params& p, int lut_kind, bool out_half, bool is_ip, int kpl,
                           int grid, size_t smem, cudaStream_t stream)
{
  if (is_ip) {
    launch_types<true>(p, lut_kind, out_half, kpl, grid, smem, stream);
  } else {
    launch_types<false>(p, lut_kind, out_half, kpl, grid, smem, stream);
  }
}

}  // namespace cuvs_b200
