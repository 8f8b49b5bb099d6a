// Coarse stage on the tensor cores: queries x list-centers as a TF32-split GEMM (tcgen05.mma, TMEM
// accumulators, operands staged by TMA), fused with candidate selection, followed by an exact
// rescoring so that the chosen probes are bit-identical to the exact SIMT path of coarse.cu.
//
// Reference semantics: select_clusters, cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:61-168
// (fp32 GEMM + select_k).  The full [n_queries, n_lists] score matrix of the reference is never
// materialised here.
//
// Pipeline per batch
//   1. operand split: every fp32 operand x is written as hi = tf32(x), lo = tf32(x - hi) (centres once
//      per index, prepare_tc_centers; queries per batch, split_queries_kernel).  Two exact power-of-two
//      rescalings ride on it: the |c|^2 column of the L2 operands is balanced against the queries'
//      -0.5 (tightens the norm product the guard's error bound scales with), and every query row is
//      scaled so that its dot products lie in (-0.5, 0.5) (lets the epilogue build keys with float adds).
//   2. coarse_tc_kernel: one persistent CTA per SM walks the output tiles (128 queries x 256
//      lists); K in blocks of 16 floats (one 64-byte swizzle atom), four pipeline stages.  Per K
//      step one, two or three products of the split accumulate into TMEM: hi*hi (+ lo*hi (+ hi*lo)).
//      Warp 0 issues TMA loads (no multicast), warp 1 issues the MMAs, sixteen epilogue warps read
//      the accumulator with tcgen05.ld (thread = query row, warp = 32 rows x 64 columns) and keep,
//      per row and per 64-list unit, the eight largest dot products in registers, as packed
//      32-bit keys (the value in fixed point with 16 fractional bits, low 7 bits the column tag;
//      built with four float additions): insertion is a branch-free chain of integer max/min.  Two variants: two independent
//      top-4 chains (column % 2) or one top-8 chain; the last key of a chain bounds everything the
//      chain dropped.  Two TMEM accumulators let the epilogue of one tile overlap the MMAs of the
//      next.
//      Every mbarrier wait is bounded; on a time-out the kernel raises an error word, lets its
//      in-flight copies land, frees its TMEM and returns.
//   3. finish kernel (one block per query): candidates at or above a threshold (the C-th largest
//      half-tile maximum, C = n_probes + margin; or, for large C, the C best keys by radix select)
//      are rescored with the defining fp32 FMA chain, sorted by (score, id), and the first
//      n_probes become the probes.  A guard proves the selection exact: every list that was not
//      rescored has a tensor-core score <= T, and T + eps < exact score of the last probe, eps
//      bounding |tensor-core - exact| for the number of products in use.  A query whose guard
//      fails is queued.
//   4. coarse_fallback_kernel: queued queries (rare) are redone exactly over all lists.
#include "search_internal.hpp"
#include "topk.cuh"

#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <type_traits>
#include <mutex>

namespace cuvs::neighbors::ivf_pq {

using namespace cuvs_b200;

namespace {

constexpr int kBM       = 128;  // queries per tile
constexpr int kBN       = 256;  // lists per tile
constexpr int kBK       = 16;   // floats per K block (64 bytes: four pipeline stages fit, and more bytes
                                // stay in flight than with two 128-byte stages)
constexpr int kStages   = 4;
// Epilogue: sixteen warps, one per (32-row lane quarter, 64-column unit) of the accumulator; every
// unit contributes eight keys per row.  Variants <STREAMS, KEEP> (STREAMS * KEEP = 8): the columns of
// a unit are dealt to STREAMS independent chains (column % STREAMS), each keeping its KEEP largest
// keys.  <2, 4> is the cheaper one (8 min/max per column, two independent chains of 32 lists);
// <1, 8> keeps more per chain and is chosen when many wanted lists per unit are likely (large
// n_probes relative to n_lists).  Keys are stored per 128-column half tile (two units side by side).
constexpr int kMaxKph   = 16;   // keys written per row per half tile
constexpr int kHalf     = kBN / 2;
constexpr int kUnit     = 64;   // columns per epilogue warp
constexpr int kEpiWarps = 16;
constexpr int kThreads  = (2 + kEpiWarps) * 32;  // warp 0 TMA, warp 1 MMA, warps 2..17 epilogue
constexpr uint32_t kStageBytes = (2 * kBM + 2 * kBN) * kBK * 4;  // 48 KB
constexpr uint32_t kSmemBytes  = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit  = 1u << 21;  // bounded waits (each try_wait sleeps up to ~1 us)

enum { ERR_NONE = 0, ERR_TIMEOUT = 1 };


// ------------------------------------------------------------------------------------------------
// operand split
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_tf32(float x)
{
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Column `ext_col` of every row (row length `dim_ext`) is multiplied by `col_scale`, a power of two
// (exact, and it commutes with the split); ext_col >= dim_ext leaves every column alone.
__global__ void split_tf32_kernel(const float* __restrict__ in, size_t n, uint32_t dim_ext, uint32_t ext_col,
                                  float col_scale, float* __restrict__ hi, float* __restrict__ lo)
{
  const size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
  if (i >= n) { return; }
  float x = in[i];
  if (uint32_t(i % dim_ext) == ext_col) { x *= col_scale; }
  const float h = to_tf32(x);
  hi[i]         = h;
  lo[i]         = to_tf32(x - h);
}

// The query operand of the GEMM, one warp per query row: the norm column multiplied by `col_scale`
// (see prepare_tc_centers), then the whole row by a power of two 2^e chosen per query so that every
// product of the row, |u| <= |q'| * cmax, lands in (-0.5, 0.5):  |q'| * cmax * (1 + 2^-9) * 2^e in
// [0.25, 0.5).  The GEMM's epilogue turns such a value into a sortable key with float additions alone
// (see there); the finish kernels undo the scale (row_scale[q] = 2^e, exact).  Then the TF32 split.
__global__ void split_queries_kernel(const float* __restrict__ fq, uint32_t n_queries, uint32_t dim_ext,
                                     uint32_t ext_col, float col_scale, float cmax, float* __restrict__ hi,
                                     float* __restrict__ lo, float* __restrict__ row_scale)
{
  const uint32_t q    = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  if (q >= n_queries) { return; }
  const float* src = fq + size_t(q) * dim_ext;
  float ss         = 0.0f;
  for (uint32_t k = lane; k < dim_ext; k += 32) {
    float v = src[k];
    if (k == ext_col) { v *= col_scale; }
    ss = __fmaf_rn(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(kFullMask, ss, o); }
  // bound = m * 2^(E - 126), m in [0.5, 1)  ->  scale 2^(125 - E) puts it in [0.25, 0.5)
  const float bound = sqrtf(ss) * cmax * 1.002f;
  const int E       = int((__float_as_uint(bound) >> 23) & 0xFFu);
  float scale       = 1.0f;
  if (E >= 1 && E <= 250) { scale = __uint_as_float(uint32_t(252 - E) << 23); }
  for (uint32_t k = lane; k < dim_ext; k += 32) {
    float v = src[k];
    if (k == ext_col) { v *= col_scale; }
    v *= scale;
    const float h                = to_tf32(v);
    hi[size_t(q) * dim_ext + k] = h;
    lo[size_t(q) * dim_ext + k] = to_tf32(v - h);
  }
  if (lane == 0) { row_scale[q] = scale; }
}

// One warp per row: bits of the largest sum of squares of a row, the column `ext_col` multiplied by
// `col_scale` first (col_scale = 0 leaves it out).  Non-negative floats order as integers.
__global__ void max_row_sumsq_scaled_kernel(const float* __restrict__ rows, uint32_t n_rows, uint32_t dim_ext,
                                            uint32_t ext_col, float col_scale, uint32_t* __restrict__ out_bits)
{
  const uint32_t row  = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  if (row >= n_rows) { return; }
  float ss = 0.0f;
  for (uint32_t k = lane; k < dim_ext; k += 32) {
    float v = rows[size_t(row) * dim_ext + k];
    if (k == ext_col) { v *= col_scale; }
    ss = __fmaf_rn(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { ss += __shfl_xor_sync(kFullMask, ss, o); }
  if (lane == 0) { atomicMax(out_bits, __float_as_uint(ss)); }
}

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
  return uint32_t(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false on time-out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit)
{
  for (uint32_t it = 0; it < limit; it++) {
    uint32_t done;
    asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 1000;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
    if (done) { return true; }
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x,
                                            int y)
{
  asm volatile(
    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
    ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
    : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate)
{
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "setp.ne.b32 p, %4, 0;\n\t"
    "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
    ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
    : "memory");
}
// Shared-memory matrix descriptor of a K-major tile stored as rows of 64 bytes with the 64-byte
// swizzle: 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr)
{
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= uint64_t(1) << 16;                  // leading byte offset (unused for swizzled K-major)
  d |= uint64_t((8 * kBK * 4) >> 4) << 32; // stride byte offset between 8-row groups
  d |= uint64_t(1) << 46;                  // descriptor version of this architecture
  d |= uint64_t(4) << 61;                  // 64-byte swizzle
  return d;
}
static_assert(kBK * 4 == 64, "descriptor and tensor maps are written for 64-byte rows");
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
  asm volatile(
    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
      "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
      "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
      "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
    : "r"(taddr)
    : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// the GEMM + candidate kernel
// ------------------------------------------------------------------------------------------------
struct tc_params {
  uint32_t n_queries, n_lists, k_blocks, n_tiles /* list tiles */, n_work /* query tiles x list tiles */;
  uint32_t* cand_key;    // [n_queries, n_tiles, 2, keys per half tile] packed keys (larger = closer)
  uint32_t* cand_bound;  // [n_queries, n_tiles, 2, 2] key bounding everything a 64-column unit dropped
  uint32_t* error;     // error word
  uint32_t spin_limit;  // iterations a bounded wait may take (about a microsecond each)
  uint32_t skip_kb;     // test only: 1 + index of an operand stage the producer leaves unfilled, 0 = none
};

// kARes ("query operand resident"): the whole K extent of the 128-query operand tile (hi and lo) stays
// in shared memory while the CTA walks consecutive list tiles of that query tile, and only the list
// operand streams through the stages -- half the operand bytes out of L2 per output tile.  Needs the
// query tile to leave room for at least four list stages (k_blocks <= 8 with two products).
template <int kStreams, int kKeep, int kProducts, bool kARes>
__global__ void __launch_bounds__(kThreads, 1)
coarse_tc_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                 const tc_params p)
{
  static_assert(!kARes || kProducts <= 2, "the resident-query variant stages one list operand");
  // Only the operands the chosen number of products reads are staged, and the 192 KB of stage memory
  // hold as many stages of that size as fit: 4 x 48 KB (three products), 6 x 32 KB (two), 8 x 24 KB
  // (one).  With fewer than three products the loop is bound by the latency of the operand loads,
  // so more of them in flight is what shortens it.
  constexpr uint32_t kATile  = kBM * kBK * 4;  // one K block of the query tile: 8 KB
  constexpr uint32_t kOffALo = kATile;
  constexpr uint32_t kOffBHi = kARes ? 0u : kATile * (kProducts >= 2 ? 2 : 1);
  constexpr uint32_t kOffBLo = kOffBHi + kBN * kBK * 4;
  constexpr uint32_t kStageB = kOffBHi + kBN * kBK * 4 * (kProducts >= 3 ? 2 : 1);
  constexpr int kMaxNS       = 8;
  // resident variant: [query tile: k_blocks x hi, k_blocks x lo][list stages]
  const uint32_t a_bytes = kARes ? p.k_blocks * kATile * (kProducts >= 2 ? 2u : 1u) : 0u;
  const int kNS = kARes ? int(min(uint32_t(kMaxNS), (kStages * kStageBytes - a_bytes) / kStageB))
                        : int((kStages * kStageBytes) / kStageB);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_a  = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;             // tiles need 1024-byte alignment
  uint8_t* base_p       = smem_raw + (base_a - raw_a);
  uint64_t* bars        = reinterpret_cast<uint64_t*>(base_p + kStages * kStageBytes);
  // bars: full[8], empty[8], tmem_full[2], tmem_empty[2], query tile full / empty, then the TMEM address slot
  const uint32_t bar_full   = smem_u32(bars);
  const uint32_t bar_empty  = bar_full + kMaxNS * 8;
  const uint32_t bar_tfull  = bar_empty + kMaxNS * 8;
  const uint32_t bar_tempty = bar_tfull + 2 * 8;
  const uint32_t bar_afull  = bar_tempty + 2 * 8;
  const uint32_t bar_aempty = bar_afull + 8;
  uint32_t* tmem_slot       = reinterpret_cast<uint32_t*>(bars + 2 * kMaxNS + 6);
  const uint32_t stage_base = base_a + a_bytes;
  __shared__ uint32_t s_failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kNS; s++) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, 1);
    }
    for (int a = 0; a < 2; a++) {
      mbar_init(bar_tfull + a * 8, 1);
      mbar_init(bar_tempty + a * 8, kEpiWarps);  // one arrival per epilogue warp
    }
    mbar_init(bar_afull, 1);
    mbar_init(bar_aempty, 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  // Persistent CTAs (one per SM) over the n_work = query tiles x list tiles, list tile fastest, every SM
  // the same number of tiles to within one: tiles blockIdx.x, blockIdx.x + gridDim.x, ... -- or, with
  // the query operand resident, one contiguous run of tiles (the query tile changes once or twice).
  uint32_t n_my_tiles = 0, first_tile = blockIdx.x, tile_step = gridDim.x;
  if constexpr (kARes) {
    first_tile = uint32_t(uint64_t(p.n_work) * blockIdx.x / gridDim.x);
    n_my_tiles = uint32_t(uint64_t(p.n_work) * (blockIdx.x + 1) / gridDim.x) - first_tile;
    tile_step  = 1;
  } else {
    if (blockIdx.x < p.n_work) { n_my_tiles = (p.n_work - blockIdx.x + gridDim.x - 1) / gridDim.x; }
  }

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, a_loads = 0, q_tile_now = 0xFFFFFFFFu;
      bool ok = true;
      for (uint32_t i = 0; ok && i < n_my_tiles; i++) {
        const uint32_t g  = first_tile + i * tile_step;
        const uint32_t q0 = (g / p.n_tiles) * kBM;
        const int n0      = int((g % p.n_tiles) * kBN);
        if constexpr (kARes) {
          if (g / p.n_tiles != q_tile_now) {
            // a new query tile: once the MMAs that read the old one have finished, load all its K blocks
            q_tile_now = g / p.n_tiles;
            if (!mbar_wait(bar_aempty, (a_loads & 1u) ^ 1u, p.spin_limit)) {
              ok = false;
              break;
            }
            a_loads++;
            mbar_arrive_expect_tx(bar_afull, a_bytes);
            for (uint32_t kb = 0; kb < p.k_blocks; kb++) {
              tma_load_2d(base_a + kb * kATile, &map_a_hi, bar_afull, int(kb * kBK), int(q0));
              if constexpr (kProducts >= 2) {
                tma_load_2d(base_a + (p.k_blocks + kb) * kATile, &map_a_lo, bar_afull, int(kb * kBK), int(q0));
              }
            }
          }
        }
        for (uint32_t kb = 0; kb < p.k_blocks; kb++) {
          if (!mbar_wait(bar_empty + stage * 8, phase ^ 1u, p.spin_limit)) {
            ok = false;
            break;
          }
          if (p.skip_kb != 0 && i == 0 && kb + 1 == p.skip_kb) {
            // test only: this stage is never filled, so the wait for it runs out (bounded) and the
            // kernel reports a time-out instead of finishing
            if (++stage == kNS) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          const uint32_t dst = stage_base + stage * kStageB;
          const uint32_t bar = bar_full + stage * 8;
          // operands the chosen number of products needs: 1: hi*hi; 2: + lo*hi; 3: + hi*lo
          constexpr uint32_t kBytes =
            ((kARes ? 0 : kBM + (kProducts >= 2 ? kBM : 0)) + kBN + (kProducts >= 3 ? kBN : 0)) * kBK * 4;
          mbar_arrive_expect_tx(bar, kBytes);
          if constexpr (!kARes) {
            tma_load_2d(dst, &map_a_hi, bar, int(kb * kBK), int(q0));
            if constexpr (kProducts >= 2) { tma_load_2d(dst + kOffALo, &map_a_lo, bar, int(kb * kBK), int(q0)); }
          }
          tma_load_2d(dst + kOffBHi, &map_b_hi, bar, int(kb * kBK), n0);
          if constexpr (kProducts >= 3) {
            tma_load_2d(dst + kOffBLo, &map_b_lo, bar, int(kb * kBK), n0);
          }
          if (++stage == kNS) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        atomicExch(p.error, ERR_TIMEOUT);
        s_failed = 1;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, tf32 x tf32, both K-major, N = 256, M = 128
      constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(kBN >> 3) << 17) |
                                 (uint32_t(kBM >> 4) << 24);
      uint32_t stage = 0, phase = 0, a_loads = 0, q_tile_now = 0xFFFFFFFFu;
      bool ok = true;
      for (uint32_t i = 0; ok && i < n_my_tiles; i++) {
        const uint32_t acc       = i & 1u;
        const uint32_t acc_phase = (i >> 1) & 1u;
        if (!mbar_wait(bar_tempty + acc * 8, acc_phase ^ 1u, p.spin_limit)) {
          ok = false;
          break;
        }
        if constexpr (kARes) {
          const uint32_t g = first_tile + i * tile_step;
          if (g / p.n_tiles != q_tile_now) {
            q_tile_now = g / p.n_tiles;
            if (!mbar_wait(bar_afull, a_loads & 1u, p.spin_limit)) {
              ok = false;
              break;
            }
            a_loads++;
          }
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        for (uint32_t kb = 0; kb < p.k_blocks; kb++) {
          if (!mbar_wait(bar_full + stage * 8, phase, p.spin_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa      = stage_base + stage * kStageB;
          const uint64_t d_a_hi  = make_desc(kARes ? base_a + kb * kATile : sa);
          const uint64_t d_a_lo  = make_desc(kARes ? base_a + (p.k_blocks + kb) * kATile : sa + kOffALo);
          const uint64_t d_b_hi  = make_desc(sa + kOffBHi);
          const uint64_t d_b_lo  = make_desc(sa + kOffBLo);
#pragma unroll
          for (uint32_t k8 = 0; k8 < kBK / 8; k8++) {
            const uint64_t adv = uint64_t(k8 * 2);  // 32 bytes per MMA along K, in 16-byte units
            if constexpr (kProducts >= 2) { tc_mma_tf32(tmem_d, d_a_lo + adv, d_b_hi + adv, idesc, (kb | k8) != 0); }
            if constexpr (kProducts >= 3) { tc_mma_tf32(tmem_d, d_a_hi + adv, d_b_lo + adv, idesc, 1); }
            tc_mma_tf32(tmem_d, d_a_hi + adv, d_b_hi + adv, idesc, kProducts >= 2 || (kb | k8) != 0);
          }
          tc_commit(bar_empty + stage * 8);  // the stage may be refilled once these MMAs have read it
          if (++stage == kNS) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) { tc_commit(bar_tfull + acc * 8); }
        if constexpr (kARes) {
          // last tile of this query tile: the query operand may be replaced once these MMAs are done
          const uint32_t g = first_tile + i * tile_step;
          if (ok && i + 1 < n_my_tiles && (g + tile_step) / p.n_tiles != q_tile_now) { tc_commit(bar_aempty); }
        }
      }
      if (!ok) {
        atomicExch(p.error, ERR_TIMEOUT);
        s_failed = 1;
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: thread = query row, warp = (lane quarter, 64-column unit) ----------------
    const uint32_t quarter = uint32_t(warp) & 3u;        // TMEM lanes a warp may read: 32 * (warp % 4)
    const uint32_t unit    = uint32_t(warp - 2) >> 2;    // warps 2..5 -> columns 0..63, 6..9 -> 64..127, ...
    const uint32_t half    = unit >> 1;                  // 128-column half tile the unit belongs to
    const uint32_t sub     = unit & 1u;                  // first or second unit of the half tile
    const uint32_t row     = quarter * 32 + lane;
    bool ok = true;
    for (uint32_t i = 0; i < n_my_tiles; i++) {
      const uint32_t g         = first_tile + i * tile_step;
      const uint32_t tile      = g % p.n_tiles;
      const uint32_t q         = (g / p.n_tiles) * kBM + row;
      const uint32_t acc       = i & 1u;
      const uint32_t acc_phase = (i >> 1) & 1u;
      if (ok && !mbar_wait(bar_tfull + acc * 8, acc_phase, p.spin_limit)) { ok = false; }
      // a time-out on any lane ends the loop for the whole warp
      if (__any_sync(kFullMask, !ok)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // Packed key.  The query rows were scaled so that every dot product u lies in (-0.5, 0.5)
      // (split_queries_kernel).  u + 192 rounds u to a multiple of 2^-16 (the ulp of [128, 256)),
      // - 192 is exact, + (1.5 + tag * 2^-23) is exact and lands in [1, 2): the bits of the result are a
      // sortable key whose low 7 bits are tag = 127 - column in the 128-column half tile.  Four float
      // additions on the FMA pipe instead of shift / logic operations on the integer pipe, which the
      // min / max chains below already fill.  Empty / out-of-range columns are key 0.
      uint32_t key[kStreams][kKeep];
#pragma unroll
      for (int st = 0; st < kStreams; st++) {
#pragma unroll
        for (int t = 0; t < kKeep; t++) { key[st][t] = 0u; }
      }
      const uint32_t col0 = unit * kUnit;
      const uint32_t n0   = tile * kBN + col0;
#pragma unroll 1
      for (uint32_t c = 0; c < kUnit; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((quarter * 32u) << 16) + acc * kBN + col0 + c, r);
        const uint32_t list0 = n0 + c;
        const bool full      = list0 + 32 <= p.n_lists;
        // The range check exists only in the version used by the last, partial list tile.
        const float tag_base = 1.5f + float(127u - (sub * kUnit + c)) * 0x1p-23f;
        auto take = [&](auto full_c) {
          constexpr bool kFull = decltype(full_c)::value;
#pragma unroll
          for (int e = 0; e < 32; e++) {
            float t = __fadd_rn(__uint_as_float(r[e]), 192.0f);
            t       = __fadd_rn(t, -192.0f);
            t       = __fadd_rn(t, tag_base);
            t       = __fadd_rn(t, -float(e) * 0x1p-23f);
            uint32_t k = __float_as_uint(t);
            if constexpr (!kFull) {
              if (list0 + e >= p.n_lists) { k = 0u; }
            }
            // sorted insert (key[.][0] >= key[.][1] >= ...): new key[t] = min(old key[t-1], max(old
            // key[t], k)) -- 2 * kKeep - 1 independent min/max
            uint32_t up[kKeep];
#pragma unroll
            for (int t2 = 0; t2 < kKeep; t2++) { up[t2] = max(key[e % kStreams][t2], k); }
#pragma unroll
            for (int t2 = kKeep - 1; t2 > 0; t2--) {
              key[e % kStreams][t2] = min(key[e % kStreams][t2 - 1], up[t2]);
            }
            key[e % kStreams][0] = up[0];
          }
        };
        if (full) {
          take(std::true_type{});
        } else {
          take(std::false_type{});
        }
      }
      // the accumulator may be overwritten now
      tc_fence_before();
      __syncwarp();
      if (lane == 0) { mbar_arrive(bar_tempty + acc * 8); }
      if (q < p.n_queries) {
        // whatever a chain dropped is not larger than its last key
        uint32_t bound = key[0][kKeep - 1];
#pragma unroll
        for (int st = 1; st < kStreams; st++) { bound = max(bound, key[st][kKeep - 1]); }
        const size_t slot = (size_t(q) * p.n_tiles + tile) * 2 + half;
        uint4* o          = reinterpret_cast<uint4*>(p.cand_key + slot * kMaxKph + sub * (kStreams * kKeep));
#pragma unroll
        for (int st = 0; st < kStreams; st++) {
#pragma unroll
          for (int u = 0; u < kKeep / 4; u++) {
            o[st * (kKeep / 4) + u] =
              make_uint4(key[st][4 * u], key[st][4 * u + 1], key[st][4 * u + 2], key[st][4 * u + 3]);
          }
        }
        p.cand_bound[slot * 2 + sub] = bound;
      }
    }
    if (!ok && lane == 0) {
      atomicExch(p.error, ERR_TIMEOUT);
      s_failed = 1;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (s_failed) {
    // give copies that are still in flight time to land before the shared memory is released
    for (int i = 0; i < 64; i++) { __nanosleep(1000); }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// finish: select C best candidates by tensor-core score, rescore exactly, sort, guard
// ------------------------------------------------------------------------------------------------
constexpr uint32_t kMaxC = 1024;

// Key helpers shared with the GEMM epilogue.
__device__ __forceinline__ bool key_valid(uint32_t key) { return key >= 0x00800000u; }
// the dot product a key stands for (to within 2^-17 / row scale): key bits = 1.5 + u * scale + tag * 2^-23
__device__ __forceinline__ float key_value(uint32_t key, float inv_row_scale)
{
  return __fmul_rn(__fadd_rn(__uint_as_float(key & ~127u), -1.5f), inv_row_scale);
}

__global__ void __launch_bounds__(256)
coarse_finish_kernel(const uint32_t* __restrict__ cand_key, const uint32_t* __restrict__ cand_bound,
                     uint32_t n_cand /* per query */, uint32_t kph /* keys per half tile */,
                     const float* __restrict__ centers, const float* __restrict__ fq,
                     uint32_t n_lists, uint32_t dim_ext, float alpha, uint32_t n_probes, uint32_t C,
                     uint32_t cap /* pow2 >= C */, float cmax, float eps_rel,
                     uint32_t* __restrict__ probes, float* __restrict__ scores_out,
                     uint32_t* __restrict__ redo_list, uint32_t* __restrict__ redo_count,
                     const uint32_t* __restrict__ error_word, uint32_t ext_col, float ext_scale,
                     const float* __restrict__ row_scale, float down_thr, int by_maxima)
{
  // the GEMM gave up on a wait: its candidates are incomplete, every query is redone exactly
  if (*error_word != 0u) { return; }
  extern __shared__ uint64_t s_keys[];                 // [cap] keys; the query; the values to select among
  float* s_q      = reinterpret_cast<float*>(s_keys + cap);
  // by_maxima: [n_cand / kph] largest key of every half tile; else [n_cand] every candidate key
  uint32_t* key   = reinterpret_cast<uint32_t*>(s_q + dim_ext);
  __shared__ uint32_t s_hist[256];
  __shared__ uint32_t s_prefix, s_remaining, s_count;
  __shared__ float s_red[8];
  __shared__ uint32_t s_tb[8];
  const uint32_t q    = blockIdx.x;
  const uint32_t tid  = threadIdx.x;
  // by_maxima (C small against the number of half tiles): the threshold comes from the half-tile maxima
  // alone -- at least C keys are >= the C-th largest maximum, so every key at or above it is taken (a
  // superset of the C best keys, little larger); the candidate keys stay in global memory, read once
  // here and again only for the half tiles that qualify.  Otherwise all keys are staged and the C-th
  // largest key itself is the threshold.
  const uint32_t n_half  = n_cand / kph;
  const uint32_t n_sel_from = by_maxima ? n_half : n_cand;
  const uint32_t* my_key = cand_key + size_t(q) * n_cand;
  if (by_maxima) {
    for (uint32_t h = tid; h < n_half; h += 256) {
      const uint4* src = reinterpret_cast<const uint4*>(my_key + size_t(h) * kph);
      uint32_t mx      = 0;
      for (uint32_t i = 0; i < kph / 4; i++) {
        const uint4 v = __ldg(src + i);
        mx            = max(max(mx, v.x), max(v.y, max(v.z, v.w)));
      }
      key[h] = mx;
    }
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(my_key);
    uint4* dst       = reinterpret_cast<uint4*>(key);
    for (uint32_t i = tid; i < n_cand / 4; i += 256) { dst[i] = __ldg(src + i); }
  }

  const float inv_row_scale = 1.0f / __ldg(row_scale + q);  // a power of two: exact
  float qq = 0.0f;
  for (uint32_t i = tid; i < dim_ext; i += 256) {
    const float v = fq[size_t(q) * dim_ext + i];
    s_q[i]        = v;
    const float w = i == ext_col ? v * ext_scale : v;  // the norm of the row the GEMM multiplied
    qq += w * w;
  }
  if (tid == 0) {
    s_prefix    = 0;
    s_remaining = C;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) { qq += __shfl_xor_sync(kFullMask, qq, d); }
  if ((tid & 31) == 0) { s_red[tid >> 5] = qq; }

  // radix select of the C LARGEST keys: ascending order of the complement
  for (int pass = 0; pass < 4; pass++) {
    const int shift = 24 - 8 * pass;
    s_hist[tid]     = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask   = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (uint32_t i = tid; i < n_sel_from; i += 256) {
      const uint32_t kk = key[i];
      if (!key_valid(kk)) { continue; }
      const uint32_t o = ~kk;
      if ((o & mask) == prefix) { atomicAdd(&s_hist[(o >> shift) & 0xFFu], 1u); }
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = s_remaining, d = 0;
      for (; d < 256; d++) {
        const uint32_t c = s_hist[d];
        if (c >= rem) { break; }
        rem -= c;
      }
      if (d == 256) {  // fewer valid candidates than C: take everything
        d   = 255;
        rem = 0xFFFFFFFFu;
      }
      s_prefix    = prefix | (d << shift);
      s_remaining = rem;
    }
    __syncthreads();
  }
  const uint32_t T = s_prefix;  // complement of the C-th largest key (half-tile maximum)
  if (tid == 0) { s_count = 0; }
  for (uint32_t i = tid; i < cap; i += 256) { s_keys[i] = kEmptyKey; }
  __syncthreads();
  // gather everything at least as good as the threshold; then the bound on what the half tiles dropped
  uint32_t tb = 0;
  if (by_maxima) {
    for (uint32_t h = tid; h < n_half; h += 256) {
      const uint32_t mx = key[h];
      if (!key_valid(mx) || ~mx > T) { continue; }
      for (uint32_t i = 0; i < kph; i++) {
        const uint32_t kk = __ldg(my_key + size_t(h) * kph + i);
        if (key_valid(kk) && ~kk <= T) {
          const uint32_t slot = atomicAdd(&s_count, 1u);
          // list id = tile * 256 + half * 128 + column; h enumerates (tile, half)
          if (slot < cap) { s_keys[slot] = h * kHalf + (127u - (kk & 127u)); }
        }
      }
    }
  } else {
    for (uint32_t i = tid; i < n_cand; i += 256) {
      const uint32_t kk = key[i];
      if (!key_valid(kk)) { continue; }
      if (~kk <= T) {
        const uint32_t slot = atomicAdd(&s_count, 1u);
        if (slot < cap) { s_keys[slot] = (i / kph) * kHalf + (127u - (kk & 127u)); }
      }
    }
  }
  {
    const uint32_t n_bnd = 2 * n_half;  // one bound per 64-column unit
    const uint32_t* bnd  = cand_bound + size_t(q) * n_bnd;
    for (uint32_t i = tid; i < n_bnd; i += 256) { tb = max(tb, bnd[i]); }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) { tb = max(tb, __shfl_xor_sync(kFullMask, tb, d)); }
  if ((tid & 31) == 0) { s_tb[tid >> 5] = tb; }
  __syncthreads();
  uint32_t tile_key = s_tb[0];
#pragma unroll
  for (int w = 1; w < 8; w++) { tile_key = max(tile_key, s_tb[w]); }
  const float tilebound = key_valid(tile_key) ? key_value(tile_key, inv_row_scale) : -INFINITY;
  const uint32_t n_sel  = min(s_count, cap);
  const bool overflow   = s_count > cap;
  // exact rescoring: the defining FMA chain, ascending k
  for (uint32_t i = tid; i < n_sel; i += 256) {
    const uint32_t l = uint32_t(s_keys[i]);
    const float4* c  = reinterpret_cast<const float4*>(centers + size_t(l) * dim_ext);
    float acc        = 0.0f;
    for (uint32_t k4 = 0; k4 < dim_ext / 4; k4++) {  // dim_ext is a multiple of 8
      const float4 cv = __ldg(c + k4);
      acc             = __fmaf_rn(cv.x, s_q[4 * k4], acc);
      acc             = __fmaf_rn(cv.y, s_q[4 * k4 + 1], acc);
      acc             = __fmaf_rn(cv.z, s_q[4 * k4 + 2], acc);
      acc             = __fmaf_rn(cv.w, s_q[4 * k4 + 3], acc);
    }
    s_keys[i] = (uint64_t(float_to_ordered(__fmul_rn(alpha, acc))) << 32) | l;
  }
  __syncthreads();
  for (uint32_t size = 2; size <= cap; size <<= 1) {
    for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
      for (uint32_t i = tid; i < cap / 2; i += 256) {
        const uint32_t lo = 2 * i - (i & (stride - 1));
        const uint32_t hi = lo + stride;
        const bool up     = (lo & size) == 0;
        const uint64_t a = s_keys[lo], b = s_keys[hi];
        if ((a > b) == up) {
          s_keys[lo] = b;
          s_keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
  for (uint32_t pi = tid; pi < n_probes; pi += 256) {
    const uint64_t key               = s_keys[pi];
    probes[size_t(q) * n_probes + pi] = uint32_t(key);
    if (scores_out) { scores_out[size_t(q) * n_probes + pi] = ordered_to_float(uint32_t(key >> 32)); }
  }
  if (tid == 0) {
    // guard, in dot-product units (score = alpha * dot, alpha < 0)
    float qnorm = 0.0f;
    for (int w = 0; w < 8; w++) { qnorm += s_red[w]; }
    qnorm = sqrtf(qnorm);
    // |tensor-core - exact| (accumulation order, dropped lo*lo term) plus the rounding of the packed
    // keys (2^-17 of the scaled row, i.e. at most 2^-15 * 1.002 of |q| * cmax)
    const float eps       = eps_rel * qnorm * cmax;
    const float t_c       = key_valid(~T) ? key_value(~T, inv_row_scale) : -INFINITY;  // C-th largest key, as a value
    const float unseen    = fmaxf(t_c, tilebound);
    bool ok               = !overflow && n_sel >= n_probes;
    if (ok) {
      const float last_dot = ordered_to_float(uint32_t(s_keys[n_probes - 1] >> 32)) / alpha;
      // all lists rescored (n_sel == every valid candidate == every list) needs no proof
      ok = (last_dot - unseen > eps) || (n_sel >= n_lists);
      // would the guard also hold with one product less (a wider error bound)?  Counted for the
      // handle's choice of the number of products; no effect on this batch.
      if (ok && n_sel < n_lists && !(last_dot - unseen > down_thr * eps)) { atomicAdd(redo_count + 1, 1u); }
    }
    if (!ok) {
      redo_list[atomicAdd(redo_count, 1u)] = q;
      atomicAdd(redo_count + 1, 1u);
    }
  }
}

// Faster finish for the common case (at most 512 half tiles, C <= 64 and small against the number of
// half tiles).  Instead of a radix select over every candidate key:
//   A. every thread keeps the keys of up to two half tiles in registers and finds their maxima;
//   B. the 64 largest maxima are found with register bitonic sorts (64 values per warp, two per
//      lane) and three rounds of pairwise merges through shared memory; the C-th largest maximum
//      is the threshold t0: at least C keys are >= t0;
//   C. every key >= t0 is a list to rescore (usually little more than C lists);
//   D. their rows are copied to shared memory with coalesced loads and the defining FMA chains run
//      out of shared memory, one thread per list;
//   E. one warp sorts the rescored lists by (exact score, list id) in registers.
// Same result contract as coarse_finish_kernel: the guard proves the probes exact or the query is
// queued for the exact redo.
constexpr uint32_t kFinMaxHalfTiles = 512;
constexpr uint32_t kFinMaxC         = 64;
constexpr uint32_t kFinRows         = 64;  // most rows rescored per round (all selected lists at once)

// 64 values per warp, value e = r * 32 + lane in register a<r>: full bitonic sort.
template <typename T, bool Desc>
__device__ __forceinline__ void warp_sort64(T& a0, T& a1)
{
  const uint32_t lane = threadIdx.x & 31u;
  auto shfl = [](T v, int j) {
    if constexpr (sizeof(T) == 8) {
      const uint32_t lo = __shfl_xor_sync(kFullMask, uint32_t(v), j);
      const uint32_t hi = __shfl_xor_sync(kFullMask, uint32_t(uint64_t(v) >> 32), j);
      return T((uint64_t(hi) << 32) | lo);
    } else {
      return T(__shfl_xor_sync(kFullMask, v, j));
    }
  };
#pragma unroll
  for (uint32_t k = 2; k <= 64; k <<= 1) {
#pragma unroll
    for (uint32_t j = k >> 1; j > 0; j >>= 1) {
      if (j == 32) {  // k == 64: partner is the other register of the same lane, ascending block
        const T lo = a0 < a1 ? a0 : a1, hi = a0 < a1 ? a1 : a0;
        a0 = Desc ? hi : lo;
        a1 = Desc ? lo : hi;
      } else {
        const T o0 = shfl(a0, int(j)), o1 = shfl(a1, int(j));
        // value index e = r * 32 + lane; block direction from bit k of e (k == 64: one block)
        const bool up0 = ((lane & k) == 0) || k >= 32;         // r = 0: bit 5 of e is 0
        const bool up1 = k == 64 || (k < 32 && (lane & k) == 0);  // r = 1: bit 5 of e is 1
        const bool low = (lane & j) == 0;
        const bool min0 = (low == up0) != Desc, min1 = (low == up1) != Desc;
        a0 = min0 ? (a0 < o0 ? a0 : o0) : (a0 < o0 ? o0 : a0);
        a1 = min1 ? (a1 < o1 ? a1 : o1) : (a1 < o1 ? o1 : a1);
      }
    }
  }
}
// (a0, a1) sorted descending, `other` = 64 values sorted descending in shared memory: afterwards
// (a0, a1) = the 64 largest of the union, sorted descending.
__device__ __forceinline__ void warp_merge_top64_desc(uint32_t& a0, uint32_t& a1, const uint32_t* other)
{
  const uint32_t lane = threadIdx.x & 31u;
  a0 = max(a0, other[63u - lane]);
  a1 = max(a1, other[31u - lane]);
  // bitonic sequence -> descending
  {
    const uint32_t hi = max(a0, a1), lo = min(a0, a1);
    a0 = hi;
    a1 = lo;
  }
#pragma unroll
  for (uint32_t j = 16; j > 0; j >>= 1) {
    const uint32_t o0 = __shfl_xor_sync(kFullMask, a0, int(j)), o1 = __shfl_xor_sync(kFullMask, a1, int(j));
    const bool keep_max = (lane & j) == 0;
    a0 = keep_max ? max(a0, o0) : min(a0, o0);
    a1 = keep_max ? max(a1, o1) : min(a1, o1);
  }
}

template <int KPH>
__global__ void __launch_bounds__(256)
coarse_finish_small_kernel(const uint32_t* __restrict__ cand_key, const uint32_t* __restrict__ cand_bound,
                           uint32_t n_cand /* per query */, const float* __restrict__ centers,
                           const float* __restrict__ fq, uint32_t n_lists, uint32_t dim_ext, float alpha,
                           uint32_t n_probes, uint32_t C, float cmax, float eps_rel,
                           uint32_t* __restrict__ probes, float* __restrict__ scores_out,
                           uint32_t* __restrict__ redo_list, uint32_t* __restrict__ redo_count,
                           uint32_t rows_per_round, const uint32_t* __restrict__ error_word, uint32_t ext_col,
                           float ext_scale, const float* __restrict__ row_scale, float down_thr)
{
  // the GEMM gave up on a wait: its candidates are incomplete, every query is redone exactly
  if (*error_word != 0u) { return; }
  // dynamic: query [dim_ext] | rows to rescore [rows_per_round][dim_ext + 1]
  extern __shared__ float s_dyn[];
  float* s_q    = s_dyn;
  float* s_rows = s_dyn + dim_ext;
  __shared__ uint32_t s_top[8][64];
  __shared__ uint64_t s_keys[128];  // lists to rescore, then (ordered exact score << 32 | list)
  __shared__ uint32_t s_count, s_t0;
  __shared__ float s_red[8];
  __shared__ uint32_t s_tb[8];
  const uint32_t q      = blockIdx.x;
  const uint32_t tid    = threadIdx.x;
  const uint32_t lane   = tid & 31u;
  const uint32_t warp   = tid >> 5;
  const uint32_t n_half = n_cand / KPH;

  // ---- A: the keys of half tiles tid and tid + 256, their maxima (invalid keys count as 0) ----
  uint32_t keys[2][KPH];
  uint32_t mx[2];
#pragma unroll
  for (int s = 0; s < 2; s++) {
    const uint32_t h = tid + uint32_t(s) * 256u;
    mx[s]            = 0;
    if (h < n_half) {
      const uint4* src = reinterpret_cast<const uint4*>(cand_key + size_t(q) * n_cand + size_t(h) * KPH);
#pragma unroll
      for (int i = 0; i < KPH / 4; i++) {
        const uint4 v      = __ldg(src + i);
        keys[s][4 * i]     = v.x;
        keys[s][4 * i + 1] = v.y;
        keys[s][4 * i + 2] = v.z;
        keys[s][4 * i + 3] = v.w;
        mx[s]              = max(max(mx[s], v.x), max(v.y, max(v.z, v.w)));
      }
      if (!key_valid(mx[s])) { mx[s] = 0; }
    } else {
#pragma unroll
      for (int i = 0; i < KPH; i++) { keys[s][i] = 0; }
    }
  }
  const float inv_row_scale = 1.0f / __ldg(row_scale + q);  // a power of two: exact
  float qq = 0.0f;
  for (uint32_t i = tid; i < dim_ext; i += 256) {
    const float v = fq[size_t(q) * dim_ext + i];
    s_q[i]        = v;
    const float w = i == ext_col ? v * ext_scale : v;  // the norm of the row the GEMM multiplied
    qq += w * w;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) { qq += __shfl_xor_sync(kFullMask, qq, d); }
  if (lane == 0) { s_red[warp] = qq; }
  if (tid == 0) { s_count = 0; }
  if (tid < 128) { s_keys[tid] = kEmptyKey; }
  uint32_t tb = 0;  // bound on what the half tiles dropped
  {
    const uint32_t* bnd = cand_bound + size_t(q) * 2 * n_half;  // one bound per 64-column unit
    for (uint32_t i = tid; i < 2 * n_half; i += 256) { tb = max(tb, __ldg(bnd + i)); }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) { tb = max(tb, __shfl_xor_sync(kFullMask, tb, d)); }
  if (lane == 0) { s_tb[warp] = tb; }

  // ---- B: the 64 largest maxima, descending; t0 = the C-th largest ----
  uint32_t a0 = mx[0], a1 = mx[1];
  warp_sort64<uint32_t, true>(a0, a1);
#pragma unroll
  for (uint32_t half = 4; half > 0; half >>= 1) {
    if (warp >= half && warp < 2 * half) {
      s_top[warp][lane]       = a0;
      s_top[warp][32u + lane] = a1;
    }
    __syncthreads();
    if (warp < half) { warp_merge_top64_desc(a0, a1, s_top[warp + half]); }
  }
  if (warp == 0) {
    // the C-th largest maximum (0 = fewer than C valid half tiles: every valid key is taken)
    const uint32_t pos = C - 1;
    const uint32_t v   = __shfl_sync(kFullMask, pos < 32 ? a0 : a1, int(pos & 31u));
    if (lane == 0) { s_t0 = v; }
  }
  __syncthreads();
  const uint32_t t0 = s_t0;

  // ---- C: every key >= t0 names a list to rescore ----
#pragma unroll
  for (int s = 0; s < 2; s++) {
    const uint32_t h = tid + uint32_t(s) * 256u;
    if (mx[s] >= t0 && mx[s] != 0) {
#pragma unroll
      for (int i = 0; i < KPH; i++) {
        const uint32_t kk = keys[s][i];
        if (key_valid(kk) && kk >= t0) {
          const uint32_t slot = atomicAdd(&s_count, 1u);
          // list id = tile * 256 + half * 128 + column; h enumerates (tile, half)
          if (slot < 128u) { s_keys[slot] = h * kHalf + (127u - (kk & 127u)); }
        }
      }
    }
  }
  __syncthreads();
  uint32_t tile_key = s_tb[0];
#pragma unroll
  for (int w = 1; w < 8; w++) { tile_key = max(tile_key, s_tb[w]); }
  const float tilebound = key_valid(tile_key) ? key_value(tile_key, inv_row_scale) : -INFINITY;
  const uint32_t n_sel  = min(s_count, 64u);
  const bool overflow   = s_count > 64u;

  // ---- D: exact rescoring out of shared memory (rows padded against bank conflicts) ----
  const uint32_t row_words = dim_ext + 1;
  for (uint32_t r0 = 0; r0 < n_sel; r0 += rows_per_round) {
    const uint32_t n_rows = min(rows_per_round, n_sel - r0);
    const uint32_t per4   = dim_ext / 4;  // dim_ext is a multiple of 4
    for (uint32_t e = tid; e < n_rows * per4; e += 256) {
      const uint32_t r = e / per4, c4 = e - r * per4;
      const uint32_t l = uint32_t(s_keys[r0 + r]);
      const float4 v   = __ldg(reinterpret_cast<const float4*>(centers + size_t(l) * dim_ext) + c4);
      float* dst       = s_rows + r * row_words + 4 * c4;
      dst[0] = v.x;
      dst[1] = v.y;
      dst[2] = v.z;
      dst[3] = v.w;
    }
    __syncthreads();
    if (tid < n_rows) {
      const uint32_t l = uint32_t(s_keys[r0 + tid]);
      const float* c   = s_rows + tid * row_words;
      float acc        = 0.0f;
      uint32_t k       = 0;
      for (; k + 4 <= dim_ext; k += 4) {
        acc = __fmaf_rn(c[k], s_q[k], acc);
        acc = __fmaf_rn(c[k + 1], s_q[k + 1], acc);
        acc = __fmaf_rn(c[k + 2], s_q[k + 2], acc);
        acc = __fmaf_rn(c[k + 3], s_q[k + 3], acc);
      }
      s_keys[r0 + tid] = (uint64_t(float_to_ordered(__fmul_rn(alpha, acc))) << 32) | l;
    }
    __syncthreads();
  }

  // ---- E: sort by (exact score, list id), write the probes, guard ----
  if (warp == 0) {
    uint64_t b0 = s_keys[lane], b1 = s_keys[32u + lane];
    warp_sort64<uint64_t, false>(b0, b1);
    for (uint32_t pi = lane; pi < n_probes; pi += 32) {
      const uint64_t kk                 = pi < 32 ? b0 : b1;  // n_probes <= C <= 64
      probes[size_t(q) * n_probes + pi] = uint32_t(kk);
      if (scores_out) { scores_out[size_t(q) * n_probes + pi] = ordered_to_float(uint32_t(kk >> 32)); }
    }
    const uint32_t last_pos = n_probes - 1;
    const uint64_t last_key = (uint64_t(__shfl_sync(kFullMask, uint32_t((last_pos < 32 ? b0 : b1) >> 32),
                                                    int(last_pos & 31u)))
                               << 32);
    if (lane == 0) {
      // guard, in dot-product units (score = alpha * dot, alpha < 0)
      float qnorm = 0.0f;
      for (int w = 0; w < 8; w++) { qnorm += s_red[w]; }
      qnorm = sqrtf(qnorm);
      const float eps = eps_rel * qnorm * cmax;
      // every list that was not rescored has a key below t0 or was dropped by its half tile
      const float t_c    = key_valid(t0) ? key_value(t0, inv_row_scale) : -INFINITY;
      const float unseen = fmaxf(t_c, tilebound);
      bool ok            = !overflow && n_sel >= n_probes;
      if (ok) {
        const float last_dot = ordered_to_float(uint32_t(last_key >> 32)) / alpha;
        // all lists rescored (n_sel == every valid candidate == every list) needs no proof
        ok = (last_dot - unseen > eps) || (n_sel >= n_lists);
        if (ok && n_sel < n_lists && !(last_dot - unseen > down_thr * eps)) { atomicAdd(redo_count + 1, 1u); }
      }
      if (!ok) {
        redo_list[atomicAdd(redo_count, 1u)] = q;
        atomicAdd(redo_count + 1, 1u);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// exact redo of flagged queries
// ------------------------------------------------------------------------------------------------
constexpr uint32_t kFbSlots = 64;  // queries redone per round = blocks of coarse_fallback_kernel = scratch rows
constexpr uint32_t kFbGroup = 8;   // queries whose chains one thread carries at a time

// Exact scores of the first kFbSlots queries to redo, spread over the whole grid: one block per 256
// lists; 256 lists x 32 columns at a time go through shared memory (a warp reads 128 contiguous bytes
// of one row), every thread continues the defining chain (ascending k, fused multiply-add) of its own
// list for up to kFbGroup queries.  scratch[slot][list] = alpha * dot.
__global__ void __launch_bounds__(256)
coarse_fallback_scores_kernel(const uint32_t* __restrict__ redo_list, const uint32_t* __restrict__ redo_count,
                              const float* __restrict__ centers, const float* __restrict__ fq,
                              uint32_t n_queries, uint32_t n_lists, uint32_t dim_ext, float alpha,
                              float* __restrict__ scratch, uint32_t n_slots,
                              const uint32_t* __restrict__ error_word)
{
  extern __shared__ float s_f[];
  float* s_tile = s_f;             // [256 lists][32 columns + 1]
  float* s_qs   = s_f + 256 * 33;  // [kFbGroup][dim_ext]
  const uint32_t tid    = threadIdx.x;
  const bool redo_all   = *error_word != 0u;
  const uint32_t n_redo = redo_all ? n_queries : min(*redo_count, n_queries);
  const uint32_t R      = min(n_redo, n_slots);
  const uint32_t l0     = blockIdx.x * 256u;
  for (uint32_t j0 = 0; j0 < R; j0 += kFbGroup) {
    const uint32_t nj = min(kFbGroup, R - j0);
    __syncthreads();
    for (uint32_t i = tid; i < nj * dim_ext; i += 256) {
      const uint32_t j = i / dim_ext, k = i - j * dim_ext;
      const uint32_t q = redo_all ? (j0 + j) : redo_list[j0 + j];
      s_qs[i]          = fq[size_t(q) * dim_ext + k];
    }
    float acc[kFbGroup];
#pragma unroll
    for (uint32_t j = 0; j < kFbGroup; j++) { acc[j] = 0.0f; }
    for (uint32_t k0 = 0; k0 < dim_ext; k0 += 32) {
      const uint32_t kc = min(32u, dim_ext - k0);
      __syncthreads();
      for (uint32_t r = tid >> 5; r < 256; r += 8) {
        const uint32_t l = l0 + r, lane = tid & 31u;
        if (l < n_lists && lane < kc) { s_tile[r * 33 + lane] = __ldg(centers + size_t(l) * dim_ext + k0 + lane); }
      }
      __syncthreads();
      if (l0 + tid < n_lists) {
        for (uint32_t k = 0; k < kc; k++) {
          const float c = s_tile[tid * 33 + k];
#pragma unroll
          for (uint32_t j = 0; j < kFbGroup; j++) {
            if (j < nj) { acc[j] = __fmaf_rn(c, s_qs[j * dim_ext + k0 + k], acc[j]); }
          }
        }
      }
    }
    if (l0 + tid < n_lists) {
#pragma unroll
      for (uint32_t j = 0; j < kFbGroup; j++) {
        if (j < nj) { scratch[size_t(j0 + j) * n_lists + l0 + tid] = __fmul_rn(alpha, acc[j]); }
      }
    }
  }
}

__global__ void __launch_bounds__(256)
coarse_fallback_kernel(const uint32_t* __restrict__ redo_list, const uint32_t* __restrict__ redo_count,
                       const float* __restrict__ centers,
                       const float* __restrict__ fq, uint32_t n_queries, uint32_t n_lists,
                       uint32_t dim_ext, float alpha, uint32_t n_probes, uint32_t cap,
                       float* __restrict__ scratch /* [gridDim.x, n_lists] */,
                       uint32_t* __restrict__ probes, float* __restrict__ scores_out,
                       uint32_t* __restrict__ n_fallback, const uint32_t* __restrict__ error_word)
{
  extern __shared__ uint64_t s_keys[];  // [cap], then the query
  float* s_q = reinterpret_cast<float*>(s_keys + cap);
  __shared__ uint32_t s_hist[256];
  __shared__ uint32_t s_prefix, s_remaining, s_count, s_eq_taken;
  const uint32_t tid = threadIdx.x;
  float* row         = scratch + size_t(blockIdx.x) * n_lists;
  // after a time-out of the GEMM nothing it produced is trusted: all queries are redone here
  const bool redo_all   = *error_word != 0u;
  const uint32_t n_redo = redo_all ? n_queries : min(*redo_count, n_queries);
  if (blockIdx.x == 0 && tid == 0) { *n_fallback = n_redo; }
  for (uint32_t ri = blockIdx.x; ri < n_redo; ri += gridDim.x) {
    const uint32_t q = redo_all ? ri : redo_list[ri];
    for (uint32_t i = tid; i < dim_ext; i += 256) { s_q[i] = fq[size_t(q) * dim_ext + i]; }
    __syncthreads();
    // the first gridDim.x queries were scored by coarse_fallback_scores_kernel (row = slot); later
    // rounds (many queries to redo: rare) score here, one chain per thread
    if (ri >= gridDim.x) {
      for (uint32_t l = tid; l < n_lists; l += 256) {
        const float* c = centers + size_t(l) * dim_ext;
        float acc      = 0.0f;
        for (uint32_t k = 0; k < dim_ext; k++) { acc = __fmaf_rn(__ldg(c + k), s_q[k], acc); }
        row[l] = __fmul_rn(alpha, acc);
      }
    }
    if (tid == 0) {
      s_prefix    = 0;
      s_remaining = n_probes;
    }
    __syncthreads();
    for (int pass = 0; pass < 4; pass++) {
      const int shift = 24 - 8 * pass;
      s_hist[tid]     = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask   = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (uint32_t l = tid; l < n_lists; l += 256) {
        const uint32_t o = float_to_ordered(row[l]);
        if ((o & mask) == prefix) { atomicAdd(&s_hist[(o >> shift) & 0xFFu], 1u); }
      }
      __syncthreads();
      if (tid == 0) {
        uint32_t rem = s_remaining, d = 0;
        for (; d < 256; d++) {
          const uint32_t c = s_hist[d];
          if (c >= rem) { break; }
          rem -= c;
        }
        s_prefix    = prefix | (d << shift);
        s_remaining = rem;
      }
      __syncthreads();
    }
    const uint32_t T = s_prefix, want_eq = s_remaining;
    if (tid == 0) {
      s_count    = 0;
      s_eq_taken = 0;
    }
    for (uint32_t i = tid; i < cap; i += 256) { s_keys[i] = kEmptyKey; }
    __syncthreads();
    for (uint32_t base = 0; base < n_lists; base += 256) {
      const uint32_t l = base + tid;
      uint32_t o       = 0xFFFFFFFFu;
      if (l < n_lists) { o = float_to_ordered(row[l]); }
      if (l < n_lists && o < T) { s_keys[atomicAdd(&s_count, 1u)] = (uint64_t(o) << 32) | l; }
      const bool eq = l < n_lists && o == T;
      if (__syncthreads_or(eq)) {
        for (int w = 0; w < 8; w++) {
          if (int(tid >> 5) == w) {
            const unsigned m = __ballot_sync(kFullMask, eq);
            if (m) {
              const uint32_t start = s_eq_taken;
              const uint32_t rank  = start + __popc(m & ((1u << (tid & 31)) - 1u));
              if (eq && rank < want_eq) { s_keys[atomicAdd(&s_count, 1u)] = (uint64_t(o) << 32) | l; }
              __syncwarp();
              if ((tid & 31) == 0) { s_eq_taken = start + __popc(m); }
            }
          }
          __syncthreads();
        }
      }
    }
    __syncthreads();
    for (uint32_t size = 2; size <= cap; size <<= 1) {
      for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
        for (uint32_t i = tid; i < cap / 2; i += 256) {
          const uint32_t lo = 2 * i - (i & (stride - 1));
          const uint32_t hi = lo + stride;
          const bool up     = (lo & size) == 0;
          const uint64_t a = s_keys[lo], b = s_keys[hi];
          if ((a > b) == up) {
            s_keys[lo] = b;
            s_keys[hi] = a;
          }
        }
        __syncthreads();
      }
    }
    for (uint32_t pi = tid; pi < n_probes; pi += 256) {
      const uint64_t key               = s_keys[pi];
      probes[size_t(q) * n_probes + pi] = uint32_t(key);
      if (scores_out) { scores_out[size_t(q) * n_probes + pi] = ordered_to_float(uint32_t(key >> 32)); }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
using encode_fn_t = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

encode_fn_t get_encode_fn()
{
  static encode_fn_t fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<encode_fn_t>(p);
    }
  });
  CUVS_EXPECTS(fn != nullptr, "cuTensorMapEncodeTiled is not available in this driver");
  return fn;
}

// 2-D fp32 row-major [rows, cols] tensor, box [box_rows, kBK columns], 64-byte swizzle, zero fill.
CUtensorMap make_map(const float* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
  CUtensorMap m;
  const cuuint64_t dims[2]    = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2]     = {kBK, box_rows};
  const cuuint32_t elem[2]    = {1, 1};
  CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(ptr), dims,
                               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CUVS_EXPECTS(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", int(r));
  return m;
}

uint32_t margin_for(uint32_t n_probes) { return std::max<uint32_t>(16, n_probes / 4); }

int& tc_products_ref()
{
  static int products = 0;  // 0 = every handle adapts on its own, 1..3 = forced (tests)
  return products;
}

bool& tc_resident_ref()
{
  static bool on = true;
  return on;
}

// test hook: a shorter limit for the bounded waits and one operand stage left unfilled
struct tc_fault {
  uint32_t spin_limit = 0, skip_kb = 0;
};
tc_fault& tc_fault_ref()
{
  static tc_fault f;
  return f;
}

}  // namespace

void set_coarse_tc_products(int products) { tc_products_ref() = products; }
void set_coarse_tc_resident(bool on) { tc_resident_ref() = on; }
void set_coarse_tc_wait_test(uint32_t spin_limit, uint32_t skip_kb)
{
  tc_fault_ref().spin_limit = spin_limit;
  tc_fault_ref().skip_kb    = skip_kb;
}

bool coarse_tc_usable(uint32_t n_lists, uint32_t n_probes, uint32_t dim_ext)
{
  if (n_lists < 2048 || (dim_ext % 4) != 0) { return false; }
  const uint32_t C = n_probes + margin_for(n_probes);
  if (C > kMaxC / 2) { return false; }
  // expected number of wanted lists per 128-list half tile; the 8 kept per half tile must cover
  // it, and the candidates of one query must fit the finish kernel's shared memory
  const double lambda = double(C) * kHalf / double(n_lists);
  const size_t n_cand = size_t(ceildiv<uint32_t>(n_lists, kBN)) * 2 * kMaxKph;
  return lambda <= 1.5 && n_cand * 4 <= 160 * 1024;
}

size_t coarse_tc_workspace_bytes(uint32_t n_queries, uint32_t n_lists, uint32_t dim_ext)
{
  const size_t n_tiles = ceildiv<uint32_t>(n_lists, kBN);
  ws_layout lay;
  lay.add(size_t(n_queries) * dim_ext * 4);  // fq hi
  lay.add(size_t(n_queries) * dim_ext * 4);  // fq lo
  lay.add(size_t(n_queries) * n_tiles * 2 * kMaxKph * 4);  // candidate keys
  lay.add(size_t(n_queries) * n_tiles * 4 * 4);          // bound per 64-column unit
  lay.add(size_t(n_queries) * 4);            // queries to redo exactly
  lay.add(256);                              // error word, fallback counter, redo counter
  lay.add(size_t(kFbSlots) * n_lists * 4);   // fallback scratch rows
  lay.add(size_t(n_queries) * 4);            // power-of-two scale of every query row
  return lay.total();
}

// Derived operands of the tensor-core coarse search: TF32 split of the centre rows with the norm
// column (`ext_col`, holding |c|^2 for L2 metrics) divided by a power of two s ~ max |c|, and the
// largest norm of a row so prepared.  The query side multiplies its own entry of that column by s, so
// the products are unchanged while the Cauchy-Schwarz bound |q'||c'| that the guard's error term
// scales with no longer carries |c|^2 against 0.5: on data with large norms (8-bit integer vectors)
// the bound tightens by about |c|.  ext_col >= dim_ext: nothing is rescaled.  Synchronises the stream.
void prepare_tc_centers(cudaStream_t stream, const float* centers, uint32_t n_lists, uint32_t dim_ext,
                        uint32_t ext_col, float* hi, float* lo, float* cmax, float* ext_scale)
{
  *cmax      = 0.0f;
  *ext_scale = 1.0f;
  const size_t n = size_t(n_lists) * dim_ext;
  if (n == 0) { return; }
  dev_array<uint32_t> bits_buf(2);
  uint32_t* d_bits = bits_buf.data();
  CUDA_TRY(cudaMemsetAsync(d_bits, 0, 8, stream));
  const unsigned blocks = ceildiv<uint32_t>(n_lists * 32u, 256u);
  uint32_t bits[2]      = {0, 0};
  float s               = 1.0f;
  if (ext_col < dim_ext) {
    max_row_sumsq_scaled_kernel<<<blocks, 256, 0, stream>>>(centers, n_lists, dim_ext, ext_col, 0.0f, d_bits);
    CUDA_TRY(cudaMemcpyAsync(bits, d_bits, 4, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaStreamSynchronize(stream));
    float ss;
    std::memcpy(&ss, &bits[0], 4);
    const float nrm = std::sqrt(ss);
    if (std::isfinite(nrm) && nrm > 0.0f) {
      int e = 0;
      std::frexp(nrm, &e);  // nrm = m * 2^e, m in [0.5, 1)
      s = std::ldexp(1.0f, std::max(-60, std::min(60, e)));
    }
  }
  max_row_sumsq_scaled_kernel<<<blocks, 256, 0, stream>>>(centers, n_lists, dim_ext, ext_col, 1.0f / s, d_bits + 1);
  split_tf32_kernel<<<unsigned(ceildiv<size_t>(n, 256)), 256, 0, stream>>>(centers, n, dim_ext, ext_col, 1.0f / s,
                                                                          hi, lo);
  CUDA_TRY(cudaGetLastError());
  CUDA_TRY(cudaMemcpyAsync(bits + 1, d_bits + 1, 4, cudaMemcpyDeviceToHost, stream));
  CUDA_TRY(cudaStreamSynchronize(stream));
  float ss;
  std::memcpy(&ss, &bits[1], 4);
  // the lanes sum in another order than a sequential loop: a margin on the bound
  *cmax      = std::sqrt(ss) * 1.001f;
  *ext_scale = s;
}

void select_clusters_tc(raft::resources& res, const float* centers, const float* centers_hi,
                        const float* centers_lo, float cmax, uint32_t n_lists, uint32_t dim_ext,
                        float alpha, const float* fq, uint32_t n_queries, uint32_t n_probes,
                        uint32_t* probes, float* scores_out, void* workspace, size_t workspace_bytes,
                        bool exact_operands, uint32_t ext_col, float ext_scale)
{
  CUVS_EXPECTS(alpha < 0.0f, "the tensor-core coarse search expects a negative scale");
  CUVS_EXPECTS(workspace_bytes >= coarse_tc_workspace_bytes(n_queries, n_lists, dim_ext),
               "coarse workspace too small");
  const uint32_t n_tiles = ceildiv<uint32_t>(n_lists, kBN);
  const uint32_t C = std::min<uint32_t>(n_probes + margin_for(n_probes), n_lists);
  // <2,4> drops a wanted list when more than 4 of the 32 lists of a chain are wanted: expected
  // fraction of queries hit = n_chains * C(32,4) * (C/L)^4; above 0.02% use one top-8 chain per
  // 64-column unit instead
  const double frac    = double(C) / double(n_lists);
  const bool four_by_4 = (double(n_lists) / 32.0) * 35960.0 * frac * frac * frac * frac <= 2e-4;
  const uint32_t kph   = kMaxKph;
  const uint32_t n_cand  = n_tiles * 2 * kph;
  ws_layout lay;
  char* ws        = static_cast<char*>(workspace);
  float* fq_hi    = reinterpret_cast<float*>(ws + lay.add(size_t(n_queries) * dim_ext * 4));
  float* fq_lo    = reinterpret_cast<float*>(ws + lay.add(size_t(n_queries) * dim_ext * 4));
  auto* cand_key  = reinterpret_cast<uint32_t*>(ws + lay.add(size_t(n_queries) * n_tiles * 2 * kMaxKph * 4));
  auto* cand_bnd  = reinterpret_cast<uint32_t*>(ws + lay.add(size_t(n_queries) * n_tiles * 4 * 4));
  auto* redo_list = reinterpret_cast<uint32_t*>(ws + lay.add(size_t(n_queries) * 4));
  auto* words     = reinterpret_cast<uint32_t*>(ws + lay.add(256));
  float* scratch  = reinterpret_cast<float*>(ws + lay.add(size_t(kFbSlots) * n_lists * 4));
  float* row_scale = reinterpret_cast<float*>(ws + lay.add(size_t(n_queries) * 4));
  cudaStream_t stream = res.stream;

  if (ext_scale == 1.0f) { ext_col = dim_ext; }
  split_queries_kernel<<<ceildiv<uint32_t>(n_queries * 32u, 256u), 256, 0, stream>>>(
    fq, n_queries, dim_ext, ext_col, ext_scale, cmax, fq_hi, fq_lo, row_scale);
  CUDA_TRY(cudaMemsetAsync(words, 0, 16, stream));  // error, queries redone, redo counter, would-fail counter

  const CUtensorMap m_a_hi = make_map(fq_hi, n_queries, dim_ext, kBM);
  const CUtensorMap m_a_lo = make_map(fq_lo, n_queries, dim_ext, kBM);
  const CUtensorMap m_b_hi = make_map(centers_hi, n_lists, dim_ext, kBN);
  const CUtensorMap m_b_lo = make_map(centers_lo, n_lists, dim_ext, kBN);

  tc_params p{};
  p.n_queries = n_queries;
  p.n_lists   = n_lists;
  p.k_blocks  = ceildiv<uint32_t>(dim_ext, kBK);
  p.n_tiles   = n_tiles;
  p.cand_key  = cand_key;
  p.cand_bound = cand_bnd;
  p.error     = words;
  p.spin_limit = tc_fault_ref().spin_limit ? tc_fault_ref().spin_limit : kSpinLimit;
  p.skip_kb    = tc_fault_ref().skip_kb;
  const uint32_t q_tiles = ceildiv<uint32_t>(n_queries, kBM);
  p.n_work               = q_tiles * n_tiles;
  const uint32_t grid    = std::min<uint32_t>(uint32_t(res.sm_count), p.n_work);
  // Products of the TF32 split per K step: 3 (hi*hi + lo*hi + hi*lo, error ~ fp32 rounding),
  // 2 (without hi*lo: |error| <= 2^-11 |q||c|) or 1 (hi*hi only: <= 2^-10 |q||c|).  Fewer products
  // make the GEMM cheaper and the guard's error bound wider; the probes stay exact either way.
  res.adopt_tc_verdict();  // what the last batch of this handle reported, if it has arrived
  int products = exact_operands ? 1 : tc_products_ref();
  if (products == 0) { products = res.tc_levels[n_probes].products; }
  const float eps_base = float(dim_ext + 8) * 2.4e-7f + 3.1e-5f;
  const float eps_split[4] = {0.0f, 9.8e-4f, 4.9e-4f, 0.0f};
  const float eps_rel = eps_base + (exact_operands ? 0.0f : eps_split[products]);
  // A query would pass the guard with one product less if its margin exceeds that level's bound plus
  // the largest change of the unseen maximum between the two levels (the sum of both bounds).
  const float down_thr = (exact_operands || products == 1)
                           ? 0.0f
                           : 1.5f + 2.0f * (eps_base + eps_split[products - 1]) / eps_rel;
  auto launch = [&](auto kernel) {
    // every instantiation needs its shared-memory limit raised once per device
    ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kSmemBytes);
    kernel<<<grid, kThreads, kSmemBytes, stream>>>(m_a_hi, m_a_lo, m_b_hi, m_b_lo, p);
  };
  // query operand resident in shared memory when it leaves room for at least four list stages
  const uint32_t a_bytes = p.k_blocks * uint32_t(kBM * kBK * 4) * (products >= 2 ? 2u : 1u);
  const bool resident    = products <= 2 && a_bytes + 4u * uint32_t(kBN * kBK * 4) <= kStages * kStageBytes &&
                        tc_resident_ref();
  if (four_by_4) {
    if (products == 1) {
      resident ? launch(coarse_tc_kernel<2, 4, 1, true>) : launch(coarse_tc_kernel<2, 4, 1, false>);
    } else if (products == 2) {
      resident ? launch(coarse_tc_kernel<2, 4, 2, true>) : launch(coarse_tc_kernel<2, 4, 2, false>);
    } else {
      launch(coarse_tc_kernel<2, 4, 3, false>);
    }
  } else {
    if (products == 1) {
      resident ? launch(coarse_tc_kernel<1, 8, 1, true>) : launch(coarse_tc_kernel<1, 8, 1, false>);
    } else if (products == 2) {
      resident ? launch(coarse_tc_kernel<1, 8, 2, true>) : launch(coarse_tc_kernel<1, 8, 2, false>);
    } else {
      launch(coarse_tc_kernel<1, 8, 3, false>);
    }
  }
  CUDA_TRY(cudaGetLastError());

  uint32_t cap     = 2;
  while (cap < 2 * C) { cap <<= 1; }  // room for ties at the selection threshold
  const bool by_maxima  = C * 4 <= n_tiles * 2;  // C small against the number of half tiles
  const size_t fin_smem = size_t(cap) * 8 + size_t(dim_ext) * 4 + size_t(by_maxima ? n_cand / kph : n_cand) * 4;
  // the half-tile-maxima threshold is tight only when C is small against the number of half tiles
  // rows rescored per round: all 64 a query can select if they fit 48 KB of shared memory, else fewer
  uint32_t fin_rows = kFinRows;
  while (fin_rows > 32 && (size_t(dim_ext) + size_t(fin_rows) * (dim_ext + 1)) * 4 > 48 * 1024) { fin_rows /= 2; }
  const size_t fin_small_smem = (size_t(dim_ext) + size_t(fin_rows) * (dim_ext + 1)) * 4;
  if (n_tiles * 2 <= kFinMaxHalfTiles && C <= kFinMaxC && C * 4 <= n_tiles * 2 && fin_small_smem <= 48 * 1024) {
    if (kph == 16) {
      coarse_finish_small_kernel<16><<<n_queries, 256, fin_small_smem, stream>>>(
        cand_key, cand_bnd, n_cand, centers, fq, n_lists, dim_ext, alpha, n_probes, C, cmax, eps_rel, probes,
        scores_out, redo_list, words + 2, fin_rows, words, ext_col, ext_scale, row_scale, down_thr);
    } else {
      coarse_finish_small_kernel<8><<<n_queries, 256, fin_small_smem, stream>>>(
        cand_key, cand_bnd, n_cand, centers, fq, n_lists, dim_ext, alpha, n_probes, C, cmax, eps_rel, probes,
        scores_out, redo_list, words + 2, fin_rows, words, ext_col, ext_scale, row_scale, down_thr);
    }
  } else {
    if (fin_smem > 48 * 1024) { ensure_dynamic_smem(reinterpret_cast<const void*>(coarse_finish_kernel), fin_smem); }
    coarse_finish_kernel<<<n_queries, 256, fin_smem, stream>>>(cand_key, cand_bnd, n_cand, kph, centers, fq,
                                                               n_lists, dim_ext, alpha, n_probes, C, cap,
                                                               cmax, eps_rel, probes, scores_out, redo_list,
                                                               words + 2, words, ext_col, ext_scale, row_scale, down_thr, by_maxima ? 1 : 0);
  }
  uint32_t cap_fb = 2;
  while (cap_fb < n_probes) { cap_fb <<= 1; }
  const size_t fb_smem = size_t(cap_fb) * 8 + size_t(dim_ext) * 4;
  const size_t fs_smem = (size_t(256) * 33 + size_t(kFbGroup) * dim_ext) * 4;
  ensure_dynamic_smem(reinterpret_cast<const void*>(coarse_fallback_scores_kernel), fs_smem);
  coarse_fallback_scores_kernel<<<ceildiv<uint32_t>(n_lists, 256u), 256, fs_smem, stream>>>(
    redo_list, words + 2, centers, fq, n_queries, n_lists, dim_ext, alpha, scratch, kFbSlots, words);
  coarse_fallback_kernel<<<kFbSlots, 256, fb_smem, stream>>>(redo_list, words + 2, centers, fq, n_queries, n_lists,
                                                       dim_ext, alpha, n_probes, cap_fb, scratch, probes,
                                                       scores_out, words + 1, words);
  CUDA_TRY(cudaGetLastError());
  res.launches += 5;
  if (!res.tc_redo_pending) {
    // the error word and how many queries this batch redid exactly: read back without waiting, looked
    // at before a later batch and at the handle's next synchronisation
    if (!res.tc_redo_event) { CUDA_TRY(cudaEventCreateWithFlags(&res.tc_redo_event, cudaEventDisableTiming)); }
    CUDA_TRY(cudaMemcpyAsync(res.pinned + 8, words, 16, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(cudaEventRecord(res.tc_redo_event, stream));
    res.tc_redo_queries  = n_queries;
    res.tc_redo_n_probes = n_probes;
    res.tc_redo_adapts  = !exact_operands && tc_products_ref() == 0;
    res.tc_redo_pending = true;
  }
}

// Reads back the error word and the number of queries redone exactly by the last call that used
// `workspace` (synchronises the stream; used by tests and the benchmark).
void coarse_tc_status(raft::resources& res, const void* workspace, uint32_t n_queries, uint32_t n_lists,
                      uint32_t dim_ext, uint32_t* error, uint32_t* n_fallback)
{
  const uint32_t n_tiles = ceildiv<uint32_t>(n_lists, kBN);
  ws_layout lay;
  lay.add(size_t(n_queries) * dim_ext * 4);
  lay.add(size_t(n_queries) * dim_ext * 4);
  lay.add(size_t(n_queries) * n_tiles * 2 * kMaxKph * 4);
  lay.add(size_t(n_queries) * n_tiles * 4 * 4);
  lay.add(size_t(n_queries) * 4);
  const size_t o = lay.add(256);
  uint32_t h[2]  = {0, 0};
  CUDA_TRY(cudaMemcpyAsync(h, static_cast<const char*>(workspace) + o, 8, cudaMemcpyDeviceToHost, res.stream));
  res.sync();
  *error      = h[0];
  *n_fallback = h[1];
}

}  // namespace cuvs::neighbors::ivf_pq

