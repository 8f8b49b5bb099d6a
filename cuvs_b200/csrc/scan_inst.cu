// Instantiations of the fine-search kernel for one code width (compiled once per PQ_BITS = 4..8).
#include "common.hpp"
#include "scan.cuh"

#ifndef PQ_BITS
#error "compile with -DPQ_BITS=4..8"
#endif

namespace cuvs_b200 {

namespace {

template <typename Kernel>
void launch_kernel(Kernel kernel, const scan_params& p, int grid, size_t smem, cudaStream_t stream)
{
  ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
  kernel<<<grid, 1024, smem, stream>>>(p);
  CUDA_TRY(cudaGetLastError());
}

// Instantiations with pq_dim, threads per group and pq_len fixed at compile time, for the shapes of the
// five benchmark configurations (table loop and piece loop become straight-line code).  Taken when the
// plan of the launch is the one the instantiation was made for; every other shape runs the general one.
template <int LutKind, bool OutHalf, bool IsIP, int KPL>
bool launch_fixed(const scan_params& p, int grid, size_t smem, cudaStream_t stream)
{
  if (p.tmem_cols == 0 || p.per_cluster) { return false; }
  [[maybe_unused]] auto is = [&](uint32_t pq_dim, uint32_t gthreads, uint32_t len) {
    return p.pq_dim == pq_dim && p.group_threads == gthreads && p.pq_len == len;
  };
#if PQ_BITS == 8
  if constexpr (LutKind == LUT_F16 && !OutHalf && !IsIP && KPL == 1) {
    if (is(48, 128, 2)) {  // 96-d embeddings, pq 48 x 8, fp16 table
      launch_kernel(scan_kernel<8, LutKind, OutHalf, IsIP, KPL, 48, 128, 2>, p, grid, smem, stream);
      return true;
    }
  }
  if constexpr (LutKind == LUT_FP8 && !OutHalf && !IsIP && (KPL == 1 || KPL == 4)) {
    if (is(64, 128, 2)) {  // 128-d integer data, pq 64 x 8, 8-bit table, k = 10 or 100
      launch_kernel(scan_kernel<8, LutKind, OutHalf, IsIP, KPL, 64, 128, 2>, p, grid, smem, stream);
      return true;
    }
  }
  if constexpr (LutKind == LUT_F32 && !OutHalf && !IsIP && KPL == 1) {
    if (is(64, 512, 2)) {  // 128-d fp32 data, pq 64 x 8, fp32 table (two groups per CTA)
      launch_kernel(scan_kernel<8, LutKind, OutHalf, IsIP, KPL, 64, 512, 2>, p, grid, smem, stream);
      return true;
    }
  }
#elif PQ_BITS == 4
  if constexpr (LutKind == LUT_F16 && !OutHalf && IsIP && KPL == 1) {
    if (is(384, 128, 2)) {  // 768-d embeddings, pq 384 x 4, inner product, fp16 table
      launch_kernel(scan_kernel<4, LutKind, OutHalf, IsIP, KPL, 384, 128, 2>, p, grid, smem, stream);
      return true;
    }
  }
#endif
  return false;
}

template <int LutKind, bool OutHalf, bool IsIP, int KPL>
void launch_one(const scan_params& p, int grid, size_t smem, cudaStream_t stream)
{
  if (p.allow_fixed_shape && launch_fixed<LutKind, OutHalf, IsIP, KPL>(p, grid, smem, stream)) { return; }
  launch_kernel(scan_kernel<PQ_BITS, LutKind, OutHalf, IsIP, KPL>, p, grid, smem, stream);
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

template <int LutKind, bool OutHalf, bool IsIP>
void launch_glut_kpl(const scan_params& p, int kpl, int grid, size_t smem, cudaStream_t stream)
{
  auto go = [&](auto kernel) {
    ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    kernel<<<grid, 256, smem, stream>>>(p);
    CUDA_TRY(cudaGetLastError());
  };
  if (kpl == 0) {
    go(scan_glut_kernel<PQ_BITS, LutKind, OutHalf, IsIP, 0>);
  } else {
    go(scan_glut_kernel<PQ_BITS, LutKind, OutHalf, IsIP, 4>);
  }
}

template <bool IsIP>
void launch_glut_types(const scan_params& p, int lut_kind, bool out_half, int kpl, int grid, size_t smem,
                       cudaStream_t stream)
{
  if (!out_half) {
    switch (lut_kind) {
      case LUT_F32: launch_glut_kpl<LUT_F32, false, IsIP>(p, kpl, grid, smem, stream); break;
      case LUT_F16: launch_glut_kpl<LUT_F16, false, IsIP>(p, kpl, grid, smem, stream); break;
      default: launch_glut_kpl<LUT_FP8, false, IsIP>(p, kpl, grid, smem, stream); break;
    }
  } else {
    switch (lut_kind) {
      case LUT_F16: launch_glut_kpl<LUT_F16, true, IsIP>(p, kpl, grid, smem, stream); break;
      case LUT_FP8: launch_glut_kpl<LUT_FP8, true, IsIP>(p, kpl, grid, smem, stream); break;
      default: fail("fp32 look-up table with fp16 internal distances is not a valid combination");
    }
  }
}

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

#define GLUT_FN_NAME2(b) launch_scan_glut_bits_##b
#define GLUT_FN_NAME(b) GLUT_FN_NAME2(b)

void GLUT_FN_NAME(PQ_BITS)(const scan_params& p, int lut_kind, bool out_half, bool is_ip, int kpl,
                           int grid, size_t smem, cudaStream_t stream)
{
  if (is_ip) {
    launch_glut_types<true>(p, lut_kind, out_half, kpl, grid, smem, stream);
  } else {
    launch_glut_types<false>(p, lut_kind, out_half, kpl, grid, smem, stream);
  }
}

}  // namespace cuvs_b200
