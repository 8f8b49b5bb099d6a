// The fine-search kernel: for every (query, probed list) pair build the look-up table in shared
// memory, stream the list's interleaved PQ codes, score every vector and keep the k best in
// registers.  Candidate distances never touch global memory; only k keys per pair are written.
//
// Arithmetic follows the reference's compute_similarity kernel so that results can be compared
// number by number with the CPU oracle:
//   base diff  .. detail/jit_lto_kernels/precompute_base_diff_impl.cuh:14-39
//   LUT        .. detail/jit_lto_kernels/create_lut_impl.cuh:17-79 (fp32 FMA chain over pq_len,
//                 rounded once to the LUT type)
//   8-bit float . ivf_pq_fp_8bit.cuh:31-100
//   score      .. detail/jit_lto_kernels/compute_score_impl.cuh:20-79 (entries summed in subspace
//                 order in the internal distance type)
//
// Execution shape (differs from the reference): a persistent grid of one 1024-thread CTA per SM,
// split into G independent thread groups (G = 8, 4, 2 or 1, as shared memory allows); each group
// pulls pairs from a global counter, owns one LUT and one base-difference vector, and synchronises
// on its own named barrier.  The per-subspace PQ codebook lives where the launch plan puts it:
// in tensor memory (written once per CTA with tcgen05.st, read per thread with tcgen05.ld), in
// shared memory, or in global memory.  The work list holds every query's nearest probe first (so
// that a bound on the k-th best score exists early), then the rest, each segment ordered by list
// so that co-resident groups stream the same bytes out of L2.  LUT entries are computed two at a
// time with packed fp32x2 arithmetic (IEEE round-to-nearest, identical bits to scalar FMA).  Each
// warp scores 32 vectors per step (one 16-byte load per lane per code piece, 512 contiguous bytes
// per warp) and keeps a sorted top-k across its lanes; a per-query bound shared through global
// memory lets later probes discard almost every candidate with one compare, and for L2 metrics a
// lane whose partial sum already exceeds that bound stops its look-ups (checked twice per piece;
// the sum only grows, so no kept candidate is lost).  While warp 0 merges a pair's queues the other
// warps prepare the next pair's base difference; for short lists of the compile-time L2 shapes the
// table is built a code piece at a time and its remainder skipped when no lane survives the first
// piece.  The benchmark shapes (pq_dim, groups, pq_len)
// are instantiated with compile-time trip counts (scan_inst.cu); every other shape runs the
// run-time loops.  scan_glut_kernel is the variant whose table lives in global memory, for tables
// that no shared-memory plan can hold.
#pragma once

#include "topk.cuh"

#include <cuda_fp16.h>

#include <type_traits>

namespace cuvs_b200 {

struct scan_params {
  // index
  const float* pq_centers;
  const float* centers_rot;
  const uint8_t* codes;
  uint32_t pq_dim, pq_len, rot_dim, n_pieces;
  int per_cluster;
  int cosine;
  // batch
  const float* rot_q;           // [n_q, rot_dim]
  const uint4* work;            // [n_pairs][2] descriptors ordered by list: {pair, query, list, size},
                                //   {sample offset, first row lo, first row hi, 0}
  uint32_t n_pairs, n_probes, k;
  uint32_t* query_kth;  // [n_q] ordered-score bound, starts at 0xFFFFFFFF
  uint64_t* out_keys;   // [n_q, n_probes, k]
  float* all_scores;    // store-all mode (KPL == 0): [n_q, max_samples] every score, no top-k
  uint32_t max_samples;
  uint32_t* work_counter;
  const uint32_t* n_work;  // number of work items (non-empty pairs), on the device
  // optional bitset filter over source ids (cpp/src/neighbors/sample_filter.cuh:162-176)
  const int64_t* ids;
  const uint32_t* filter_bits;
  uint64_t filter_nbits;
  // shared memory plan
  uint32_t n_groups, group_threads;
  uint32_t pqc_in_smem, smem_pqc_bytes, smem_group_bytes, lut_bytes, base_bytes, merge_bytes;
  uint32_t base_double;  // base_bytes holds two base-difference buffers
  // codebook in tensor memory: columns allocated (0 = not used), byte offset in shared memory of
  // the word that receives the allocation's address
  uint32_t tmem_cols, tmem_slot_off;
  // host only: whether the launcher may pick an instantiation made for this exact shape
  int allow_fixed_shape;
  // look-up tables too large for shared memory: one table per CTA in global memory
  // ([grid][pq_dim << pq_bits] entries of the table type), used by scan_glut_kernel
  void* lut_global;
};

enum { LUT_F32 = 0, LUT_F16 = 1, LUT_FP8 = 2 };

// ---- packed fp32x2 arithmetic (sm_100) ---------------------------------------------------------
// register-pair packing spelled as mov.b64 so that it costs no shift/or arithmetic
__device__ __forceinline__ uint64_t pack_b32x2(uint32_t lo, uint32_t hi)
{
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo), "r"(hi));
  return v;
}
__device__ __forceinline__ uint64_t pack2(float x, float y)
{
  return pack_b32x2(__float_as_uint(x), __float_as_uint(y));
}
__device__ __forceinline__ float lo2(uint64_t v)
{
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return lo;
}
__device__ __forceinline__ float hi2(uint64_t v)
{
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
  return hi;
}
__device__ __forceinline__ void sts_2xb32(uint32_t a, uint32_t x, uint32_t y)
{
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b)
{
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// a * b: the first term of a sum that starts from +0 (fma(a, a, +0) rounds to the same value, and
// a square is never -0), without materialising a zero register pair
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b)
{
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// ---- 8-bit float, 5 exponent bits (ivf_pq_fp_8bit.cuh) -----------------------------------------
template <bool Signed>
__device__ __forceinline__ uint8_t fp8_encode(float v)
{
  constexpr uint32_t kExpMask = 15u;
  constexpr float kMin        = 1.0f / float(1u << kExpMask);
  constexpr float kMax        = float(1u << (kExpMask + 1u)) * (2.0f - 1.0f / 8.0f);
  float a                     = Signed ? fabsf(v) : v;
  uint8_t u;
  if (a < kMin) {
    u = 0;
  } else if (a >= kMax) {
    u = 0xffu;
  } else {
    u = uint8_t((__float_as_uint(a) + (kExpMask << 23u) - 0x3f800000u) >> 20u);
  }
  if (Signed) { u = uint8_t((u & 0xfeu) | (v < 0 ? 1u : 0u)); }
  return u;
}
template <bool Signed>
__device__ __forceinline__ float fp8_to_float(uint32_t b)
{
  constexpr uint32_t kBase32 = (0x3f800000u | (0x00400000u >> 3)) - (15u << 23);
  uint32_t u                 = Signed ? (b & ~1u) : b;
  uint32_t r                 = kBase32 + (u << 20);
  if (Signed) { r |= (b & 1u) << 31; }
  return __uint_as_float(r);
}
template <bool Signed>
__device__ __forceinline__ __half fp8_to_half(uint32_t b)
{
  constexpr uint32_t kBase16 = (0x3c00u | (0x0200u >> 3)) - (15u << 10);
  uint32_t u                 = Signed ? (b & ~1u) : b;
  uint32_t r                 = (kBase16 + (u << 7)) & 0xffffu;
  if (Signed) { r ^= (b & 1u) << 15; }
  return __ushort_as_half(static_cast<unsigned short>(r));
}

template <int LutKind>
struct lut_elem;
template <> struct lut_elem<LUT_F32> { using type = float; };
template <> struct lut_elem<LUT_F16> { using type = __half; };
template <> struct lut_elem<LUT_FP8> { using type = uint8_t; };

__device__ __forceinline__ void group_bar(int id, int n)
{
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}

// ---- explicit shared-space accesses (32-bit addresses, immediate offsets) ----------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
  return uint32_t(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t lds_b64(uint32_t a)
{
  uint64_t v;
  asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a)
{
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t a)
{
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts_b64(uint32_t a, uint64_t v)
{
  asm volatile("st.shared.b64 [%0], %1;" ::"r"(a), "l"(v) : "memory");
}
__device__ __forceinline__ void sts_b32(uint32_t a, uint32_t v)
{
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_b16(uint32_t a, uint32_t v)
{
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(a), "h"(uint16_t(v)) : "memory");
}
__device__ __forceinline__ uint32_t lds_b32_volatile(uint32_t a)
{
  uint32_t v;
  asm volatile("ld.volatile.shared.b32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
  return v;
}
__device__ __forceinline__ void atoms_min_u32(uint32_t a, uint32_t v)
{
  asm volatile("red.shared.min.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void lds_2xb64(uint32_t a, uint64_t& x, uint64_t& y)
{
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(x), "=l"(y) : "r"(a));
}
__device__ __forceinline__ void sts_b128(uint32_t a, uint64_t x, uint64_t y)
{
  asm volatile("st.shared.v2.b64 [%0], {%1, %2};" ::"r"(a), "l"(x), "l"(y) : "memory");
}
__device__ __forceinline__ uint64_t dup2(float x)
{
  uint64_t v;
  asm("mov.b64 %0, {%1, %1};" : "=l"(v) : "f"(x));
  return v;
}

// LUT of one pair from a codebook resident in shared memory.  A thread owns four adjacent codebook
// entries (b .. b+3) and walks the subspaces with a fixed stride, so all addresses advance by
// constants; per subspace and component it issues one 16-byte codebook load and one broadcast load
// of the pre-duplicated base difference.  LEN > 0 fixes pq_len at compile time.
// Base layout (per rotated dimension): L2 (d, d); inner product (-q, -q, q*c, q*c).
template <int PqBits, int LutKind, bool IsIP, int LEN>
__device__ __forceinline__ void build_lut_smem(uint32_t pqc_a, uint32_t base_a, uint32_t lut_a,
                                               uint32_t pq_dim, uint32_t len_rt, uint32_t gt,
                                               uint32_t gthreads)
{
  constexpr uint32_t kBook  = 1u << PqBits;
  constexpr uint32_t kUPJ   = kBook / 4;  // four-entry units per subspace
  constexpr uint32_t kElem  = LutKind == LUT_F32 ? 4u : (LutKind == LUT_F16 ? 2u : 1u);
  constexpr uint32_t kBaseB = IsIP ? 16u : 8u;
  const uint32_t len      = LEN > 0 ? uint32_t(LEN) : len_rt;
  const uint32_t u        = gt % kUPJ;
  const uint32_t j_first  = gt / kUPJ;
  const uint32_t j_stride = gthreads / kUPJ;
  uint32_t cb             = pqc_a + (j_first * len * kBook + 4u * u) * 4u;
  uint32_t bd             = base_a + j_first * len * kBaseB;
  uint32_t out            = lut_a + (j_first * kBook + 4u * u) * kElem;
  const uint32_t cb_step  = j_stride * len * kBook * 4u;
  const uint32_t bd_step  = j_stride * len * kBaseB;
  const uint32_t out_step = j_stride * kBook * kElem;
  for (uint32_t j = j_first; j < pq_dim; j += j_stride) {
    uint64_t s0 = 0ull, s1 = 0ull;  // entries (b, b+1) and (b+2, b+3), each (+0.0f, +0.0f)
    auto step = [&](uint64_t c0, uint64_t c1, uint64_t x, uint64_t y) {
      if constexpr (!IsIP) {  // x = (d, d)
        const uint64_t e0 = sub2(x, c0);
        const uint64_t e1 = sub2(x, c1);
        s0                = fma2(e0, e0, s0);
        s1                = fma2(e1, e1, s1);
      } else {  // x = (-q, -q), y = (q*c, q*c)
        s0 = sub2(s0, y);
        s1 = sub2(s1, y);
        s0 = fma2(x, c0, s0);
        s1 = fma2(x, c1, s1);
      }
    };
    if constexpr (LEN > 0) {
      uint64_t c0[LEN], c1[LEN], x[LEN], y[LEN];
#pragma unroll
      for (int kk = 0; kk < LEN; kk++) { lds_2xb64(cb + uint32_t(kk) * kBook * 4u, c0[kk], c1[kk]); }
      if constexpr (IsIP) {
#pragma unroll
        for (int kk = 0; kk < LEN; kk++) { lds_2xb64(bd + uint32_t(kk) * 16u, x[kk], y[kk]); }
      } else if constexpr (LEN == 1) {
        x[0] = lds_b64(bd);
      } else {
#pragma unroll
        for (int kk = 0; kk < LEN; kk += 2) { lds_2xb64(bd + uint32_t(kk) * 8u, x[kk], x[kk + 1]); }
      }
#pragma unroll
      for (int kk = 0; kk < LEN; kk++) { step(c0[kk], c1[kk], x[kk], IsIP ? y[kk] : 0ull); }
    } else {
      for (uint32_t kk = 0; kk < len; kk++) {
        uint64_t c0, c1, x, y = 0ull;
        lds_2xb64(cb + kk * kBook * 4u, c0, c1);
        if constexpr (IsIP) {
          lds_2xb64(bd + kk * 16u, x, y);
        } else {
          x = lds_b64(bd + kk * 8u);
        }
        step(c0, c1, x, y);
      }
    }
    if constexpr (LutKind == LUT_F32) {
      sts_b128(out, s0, s1);
    } else if constexpr (LutKind == LUT_F16) {
      const __half2 h0 = __floats2half2_rn(lo2(s0), hi2(s0));
      const __half2 h1 = __floats2half2_rn(lo2(s1), hi2(s1));
      sts_2xb32(out, *reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
    } else {
      sts_b32(out, uint32_t(fp8_encode<IsIP>(lo2(s0))) | (uint32_t(fp8_encode<IsIP>(hi2(s0))) << 8) |
                     (uint32_t(fp8_encode<IsIP>(lo2(s1))) << 16) | (uint32_t(fp8_encode<IsIP>(hi2(s1))) << 24));
    }
    cb += cb_step;
    bd += bd_step;
    out += out_step;
  }
}

// ---- tensor memory (TMEM) as a per-SM store for the codebook -------------------------------------
// Warp w reaches TMEM lanes 32 * (w % 4) .. + 31 (one lane per thread, 32x32b shape); an address is
// (lane << 16) | column.
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_st4(uint32_t taddr, float a, float b, float c, float d)
{
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr),
               "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)),
               "r"(__float_as_uint(d))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[N])
{
  static_assert(N == 4 || N == 8 || N == 16, "4, 8 or 16 columns");
  if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
  } else {
    asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  }
}

// Codebook layout in TMEM (written once per CTA, lane L by the threads with tid % 128 == L, and read
// by every thread from the lane tid % 128).  Lane L serves the four-entry unit u = L % kUPJ of the subspaces
// j = L / kUPJ + m * (128 / kUPJ), m = 0, 1, ...  A group of `gthreads` threads (a multiple of 128)
// gives thread gt the unit gt % kUPJ of subspaces gt / kUPJ + i * gthreads / kUPJ, i.e.
// m = gt / 128 + i * m_stride with m_stride = gthreads / 128; the blocks of one thread's successive
// iterations are stored side by side: block(m) = (m % m_stride) * ipt + m / m_stride, ipt =
// iterations per thread.  A block is 4 * LEN columns: entries 4u .. 4u+3 of component 0, then of
// component 1, ...
__device__ __forceinline__ uint32_t tmem_iters_per_thread(uint32_t pq_dim, uint32_t j_per_m, uint32_t m_stride)
{
  const uint32_t n_m = (pq_dim + j_per_m - 1) / j_per_m;
  return (n_m + m_stride - 1) / m_stride;
}
template <int PqBits, int LEN>
__device__ __forceinline__ void fill_codebook_tmem(uint32_t tmem_lane_a, const float* pq_centers,
                                                   uint32_t pq_dim, uint32_t lane128, uint32_t m_stride,
                                                   uint32_t part, uint32_t n_parts)
{
  constexpr uint32_t kBook  = 1u << PqBits;
  constexpr uint32_t kUPJ   = kBook / 4;
  constexpr uint32_t kJPerM = 128u / kUPJ;
  const uint32_t u          = lane128 % kUPJ;
  const uint32_t ipt        = tmem_iters_per_thread(pq_dim, kJPerM, m_stride);
  // the 128-thread slices of the CTA (every fourth warp reaches the same TMEM lanes) share the blocks
#pragma unroll 4
  for (uint32_t m = part; m < ipt * m_stride; m += n_parts) {
    const uint32_t j     = lane128 / kUPJ + m * kJPerM;
    const uint32_t block = (m % m_stride) * ipt + m / m_stride;
#pragma unroll
    for (int kk = 0; kk < LEN; kk++) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < pq_dim) {
        v = __ldg(reinterpret_cast<const float4*>(pq_centers + (size_t(j) * LEN + kk) * kBook + 4u * u));
      }
      tmem_st4(tmem_lane_a + (block * LEN + uint32_t(kk)) * 4u, v.x, v.y, v.z, v.w);
    }
  }
  tmem_wait_st();
}

// LUT of one pair from the codebook in TMEM: same thread-to-entry assignment and arithmetic as
// build_lut_smem; the codebook operand arrives through tcgen05.ld, 16 columns (4 / LEN subspaces)
// per load, and no longer occupies the shared-memory pipe.
// Columns fetched by one tcgen05.ld of the table builder.  Eight (one subspace at two components
// per codeword) keeps the kernel inside its 64 registers per thread; with sixteen, ten to fourteen
// kernel-lifetime values were spilled and re-read from local memory for every pair, and those loads
// miss L1 (the shared-memory carve-out leaves it almost no room): 1.57 ms against 1.50 ms per launch
// on the 10 M-row workload.
constexpr int kTmemLoadCols = 8;
// I0 / I1 (uniform compile-time shapes only): build the thread's subspaces number I0 .. I1 - 1 of its
// PQD / (GT / units per subspace); I1 < 0 = all.  Subspaces are dealt to threads round robin, so a
// range of iterations is a range of subspaces: the table can be built a code piece at a time.
template <int PqBits, int LutKind, bool IsIP, int LEN, int PQD = 0, int GT = 0, int I0 = 0, int I1 = -1>
__device__ __forceinline__ void build_lut_tmem(uint32_t tmem_lane_a, uint32_t base_a, uint32_t lut_a,
                                               uint32_t pq_dim_rt, uint32_t gt, uint32_t gthreads_rt)
{
  // PQD / GT > 0 fix pq_dim and the threads of a group at compile time (the benchmark shapes): every
  // trip count, stride and offset below is then a constant and the loop is straight-line code
  const uint32_t pq_dim   = PQD > 0 ? uint32_t(PQD) : pq_dim_rt;
  const uint32_t gthreads = GT > 0 ? uint32_t(GT) : gthreads_rt;
  constexpr uint32_t kBook  = 1u << PqBits;
  constexpr uint32_t kUPJ   = kBook / 4;
  constexpr uint32_t kJPerM = 128u / kUPJ;
  constexpr uint32_t kElem  = LutKind == LUT_F32 ? 4u : (LutKind == LUT_F16 ? 2u : 1u);
  constexpr uint32_t kBaseB = IsIP ? 16u : 8u;
  constexpr int kCols       = 4 * LEN;     // columns of one subspace
  constexpr int kLoad       = kTmemLoadCols < kCols ? kCols : kTmemLoadCols;  // columns per load
  constexpr int kPerLoad    = kLoad / kCols;  // subspaces per load
  // every lane of a warp works on the same subspace when a subspace has at least 32 units
  constexpr bool kWarpSameJ = kUPJ >= 32;
  const uint32_t u          = gt % kUPJ;
  const uint32_t j_first    = gt / kUPJ;
  const uint32_t j_stride   = gthreads / kUPJ;
  const uint32_t ipt        = tmem_iters_per_thread(pq_dim, kJPerM, gthreads / 128u);
  // warp-uniform trip count (the tensor-memory loads need the whole warp): a lane whose subspace
  // falls beyond pq_dim computes nothing
  const uint32_t j_warp     = (gt & ~31u) / kUPJ;
  const uint32_t n_iter     = j_warp < pq_dim ? (pq_dim - j_warp + j_stride - 1) / j_stride : 0u;
  uint32_t j                = j_first;
  uint32_t bd               = base_a + j_first * LEN * kBaseB;
  uint32_t out              = lut_a + (j_first * kBook + 4u * u) * kElem;
  uint32_t taddr            = tmem_lane_a + (gt / 128u) * ipt * uint32_t(kCols);
  const uint32_t bd_step    = j_stride * LEN * kBaseB;
  const uint32_t out_step   = j_stride * kBook * kElem;

  // one subspace: sub-iteration T of the 16 columns in `c`
  auto entry = [&](const auto& c, auto tc) {
    constexpr int T = decltype(tc)::value;
    uint64_t s0 = 0ull, s1 = 0ull;  // entries (b, b+1) and (b+2, b+3), each (+0.0f, +0.0f)
    uint64_t x[LEN], y[LEN];
    if constexpr (IsIP) {
#pragma unroll
      for (int kk = 0; kk < LEN; kk++) { lds_2xb64(bd + uint32_t(kk) * 16u, x[kk], y[kk]); }
    } else if constexpr (LEN == 1) {
      x[0] = lds_b64(bd);
    } else {
#pragma unroll
      for (int kk = 0; kk < LEN; kk += 2) { lds_2xb64(bd + uint32_t(kk) * 8u, x[kk], x[kk + 1]); }
    }
#pragma unroll
    for (int kk = 0; kk < LEN; kk++) {
      const uint64_t c0 = pack_b32x2(c[T * kCols + kk * 4 + 0], c[T * kCols + kk * 4 + 1]);
      const uint64_t c1 = pack_b32x2(c[T * kCols + kk * 4 + 2], c[T * kCols + kk * 4 + 3]);
      if constexpr (!IsIP) {  // x = (d, d)
        const uint64_t e0 = sub2(x[kk], c0);
        const uint64_t e1 = sub2(x[kk], c1);
        s0                = kk == 0 ? mul2(e0, e0) : fma2(e0, e0, s0);
        s1                = kk == 0 ? mul2(e1, e1) : fma2(e1, e1, s1);
      } else {  // x = (-q, -q), y = (q*c, q*c)
        s0 = sub2(s0, y[kk]);
        s1 = sub2(s1, y[kk]);
        s0 = fma2(x[kk], c0, s0);
        s1 = fma2(x[kk], c1, s1);
      }
    }
    if constexpr (LutKind == LUT_F32) {
      sts_b128(out, s0, s1);
    } else if constexpr (LutKind == LUT_F16) {
      const __half2 h0 = __floats2half2_rn(lo2(s0), hi2(s0));
      const __half2 h1 = __floats2half2_rn(lo2(s1), hi2(s1));
      sts_2xb32(out, *reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
    } else {
      sts_b32(out, uint32_t(fp8_encode<IsIP>(lo2(s0))) | (uint32_t(fp8_encode<IsIP>(hi2(s0))) << 8) |
                     (uint32_t(fp8_encode<IsIP>(lo2(s1))) << 16) | (uint32_t(fp8_encode<IsIP>(hi2(s1))) << 24));
    }
  };
  auto advance = [&]() {
    j += j_stride;
    bd += bd_step;
    out += out_step;
  };
  // every thread runs the same number of subspaces and none falls beyond pq_dim: no checks at all
  constexpr bool kUniform = PQD > 0 && GT > 0 && (uint32_t(PQD) % ((GT > 0 ? uint32_t(GT) : kUPJ) / kUPJ) == 0u);
  if constexpr (kUniform) {
    constexpr uint32_t kIters = uint32_t(PQD) / (uint32_t(GT) / kUPJ);
    static_assert(kIters % kPerLoad == 0, "whole tensor-memory loads only");
    constexpr uint32_t kBegin = uint32_t(I0);
    constexpr uint32_t kEnd   = I1 < 0 ? kIters : uint32_t(I1);
    static_assert(kBegin % kPerLoad == 0 && kEnd % kPerLoad == 0 && kEnd <= kIters, "whole loads only");
    j += kBegin * j_stride;
    bd += kBegin * bd_step;
    out += kBegin * out_step;
#pragma unroll
    for (uint32_t i = kBegin; i < kEnd; i += kPerLoad) {
      uint32_t c[kLoad];
      tmem_ld<kLoad>(taddr + i / kPerLoad * uint32_t(kLoad), c);
      tmem_wait_ld();
      entry(c, std::integral_constant<int, 0>{});
      advance();
      if constexpr (kPerLoad >= 2) {
        entry(c, std::integral_constant<int, 1>{});
        advance();
      }
      if constexpr (kPerLoad >= 4) {
        entry(c, std::integral_constant<int, 2>{});
        advance();
        entry(c, std::integral_constant<int, 3>{});
        advance();
      }
    }
    return;
  }
  // Whole loads first, without per-subspace checks where the warp shares its subspace; then the rest.
  const uint32_t n_whole = kWarpSameJ ? (n_iter / kPerLoad) * kPerLoad : 0u;
  uint32_t i             = 0;
  for (; i < n_whole; i += kPerLoad, taddr += uint32_t(kLoad)) {
    uint32_t c[kLoad];
    tmem_ld<kLoad>(taddr, c);
    tmem_wait_ld();
    entry(c, std::integral_constant<int, 0>{});
    advance();
    if constexpr (kPerLoad >= 2) {
      entry(c, std::integral_constant<int, 1>{});
      advance();
    }
    if constexpr (kPerLoad >= 4) {
      entry(c, std::integral_constant<int, 2>{});
      advance();
      entry(c, std::integral_constant<int, 3>{});
      advance();
    }
  }
  for (; i < n_iter; i += kPerLoad, taddr += uint32_t(kLoad)) {
    uint32_t c[kLoad];
    tmem_ld<kLoad>(taddr, c);  // may run past this thread's blocks into other columns of the allocation
    tmem_wait_ld();
    if (i < n_iter && (kWarpSameJ || j < pq_dim)) { entry(c, std::integral_constant<int, 0>{}); }
    advance();
    if constexpr (kPerLoad >= 2) {
      if (i + 1u < n_iter && (kWarpSameJ || j < pq_dim)) { entry(c, std::integral_constant<int, 1>{}); }
      advance();
    }
    if constexpr (kPerLoad >= 4) {
      if (i + 2u < n_iter && (kWarpSameJ || j < pq_dim)) { entry(c, std::integral_constant<int, 2>{}); }
      advance();
      if (i + 3u < n_iter && (kWarpSameJ || j < pq_dim)) { entry(c, std::integral_constant<int, 3>{}); }
      advance();
    }
  }
}

// Shared-space loads with an immediate byte offset: [a + OFF].
template <uint32_t OFF>
__device__ __forceinline__ float lds_f32_off(uint32_t a)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(OFF));
  return v;
}
// acc += float(lut[a + OFF]) in one mixed-precision add (the fp16 operand widens exactly, the sum is
// rounded once in fp32: the same value as convert-then-add).
template <uint32_t OFF>
__device__ __forceinline__ void lds_f16_add_f32_off(uint32_t a, float& acc)
{
  asm volatile("{\n\t.reg .b16 h;\n\tld.shared.b16 h, [%1+%2];\n\tadd.rn.f32.f16 %0, h, %0;\n\t}"
               : "+f"(acc)
               : "r"(a), "n"(OFF));
}
template <uint32_t OFF>
__device__ __forceinline__ __half lds_f16_off(uint32_t a)
{
  uint16_t v;
  asm volatile("ld.shared.b16 %0, [%1+%2];" : "=h"(v) : "r"(a), "n"(OFF));
  return __ushort_as_half(v);
}
template <uint32_t OFF>
__device__ __forceinline__ uint32_t lds_u8_off(uint32_t a)
{
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFF));
  return v;
}

// One looked-up entry added to the running score, in the internal distance type.
template <int LutKind, bool OutHalf, bool IsIP>
struct accum {
  using lut_t = typename lut_elem<LutKind>::type;
  float f;
  __half h;
  __device__ __forceinline__ void init()
  {
    f = 0.0f;
    h = __ushort_as_half(0);
  }
  // lut[row][code] lives at shared-space byte address `entry` + OFF
  template <uint32_t OFF>
  __device__ __forceinline__ void add(uint32_t entry)
  {
    if constexpr (!OutHalf) {
      if constexpr (LutKind == LUT_F32) {
        f += lds_f32_off<OFF>(entry);
      } else if constexpr (LutKind == LUT_F16) {
        lds_f16_add_f32_off<OFF>(entry, f);
      } else {
        f += fp8_to_float<IsIP>(lds_u8_off<OFF>(entry));
      }
    } else {
      if constexpr (LutKind == LUT_F16) {
        h = __hadd(h, lds_f16_off<OFF>(entry));
      } else {
        h = __hadd(h, fp8_to_half<IsIP>(lds_u8_off<OFF>(entry)));
      }
    }
  }
  // the running sum (for L2, where every entry is non-negative, a lower bound of the final score)
  __device__ __forceinline__ float partial() const
  {
    if constexpr (!OutHalf) {
      return f;
    } else {
      return __half2float(h);
    }
  }
  __device__ __forceinline__ float result(bool cosine)
  {
    if constexpr (!OutHalf) {
      return cosine ? f + 1.0f : f;
    } else {
      if (cosine) { h = __hadd(h, __float2half(1.0f)); }
      return __half2float(h);
    }
  }
};

// Codes of one 16-byte piece -> LUT lookups.  `row_a` = shared-space address of the LUT row of the
// piece's first subspace; `n_valid` = codes used in this piece.  The row offset of code C is an
// immediate of the load, so a lookup costs: extract, scale-and-add, load, (convert,) add.
template <int PqBits, int LutKind, bool OutHalf, bool IsIP, bool Full, int C, int CEND = 128 / PqBits>
__device__ __forceinline__ void score_codes(accum<LutKind, OutHalf, IsIP>& acc, const uint32_t (&w)[4],
                                            uint32_t row_a, uint32_t n_valid)
{
  constexpr uint32_t kBook = 1u << PqBits;
  constexpr uint32_t kMask = kBook - 1u;
  constexpr int kPerPiece  = 128 / PqBits;
  constexpr uint32_t kElem = LutKind == LUT_F32 ? 4u : (LutKind == LUT_F16 ? 2u : 1u);
  if constexpr (C < kPerPiece && C < CEND) {
    constexpr int bit  = C * PqBits;
    constexpr int word = bit >> 5;
    constexpr int sh   = bit & 31;
    uint32_t code;
    if constexpr (PqBits == 8) {
      code = __byte_perm(w[word], 0u, 0x4440u + uint32_t(sh >> 3));
    } else if constexpr (sh + PqBits <= 32) {
      code = (w[word] >> sh) & kMask;
    } else {
      code = __funnelshift_r(w[word], w[word + 1 > 3 ? 3 : word + 1], sh) & kMask;
    }
    if (Full || uint32_t(C) < n_valid) { acc.template add<uint32_t(C) * kBook * kElem>(row_a + code * kElem); }
    score_codes<PqBits, LutKind, OutHalf, IsIP, Full, C + 1, CEND>(acc, w, row_a, n_valid);
  }
}
template <int PqBits, int LutKind, bool OutHalf, bool IsIP, bool Full>
__device__ __forceinline__ void score_piece(accum<LutKind, OutHalf, IsIP>& acc, const uint4& v,
                                            uint32_t row_a, uint32_t n_valid)
{
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  score_codes<PqBits, LutKind, OutHalf, IsIP, Full, 0>(acc, w, row_a, n_valid);
}
// codes [C0, C1) of a piece
template <int PqBits, int LutKind, bool OutHalf, bool IsIP, bool Full, int C0, int C1>
__device__ __forceinline__ void score_part(accum<LutKind, OutHalf, IsIP>& acc, const uint4& v,
                                           uint32_t row_a, uint32_t n_valid)
{
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  score_codes<PqBits, LutKind, OutHalf, IsIP, Full, C0, C1>(acc, w, row_a, n_valid);
}

// PQD, GT, LEN > 0: pq_dim, threads per group and pq_len fixed at compile time, codebook in tensor
// memory (the shapes of the benchmark configurations; chosen by the launcher when the plan matches).
template <int PqBits, int LutKind, bool OutHalf, bool IsIP, int KPL, int PQD = 0, int GT = 0, int LEN = 0>
__global__ void __launch_bounds__(1024, 1) scan_kernel(const scan_params p)
{
  using lut_t               = typename lut_elem<LutKind>::type;
  constexpr uint32_t kBook  = 1u << PqBits;
  constexpr int kPerPiece   = 128 / PqBits;
  constexpr bool kFixed     = PQD > 0;
  static_assert(!kFixed || (GT > 0 && LEN > 0), "a fixed shape fixes all three");
  extern __shared__ __align__(16) uint8_t smem[];

  const int tid      = threadIdx.x;
  const int gthreads = kFixed ? GT : int(p.group_threads);
  const uint32_t pq_dim   = kFixed ? uint32_t(PQD) : p.pq_dim;
  const uint32_t n_pieces = kFixed ? uint32_t((PQD + kPerPiece - 1) / kPerPiece) : p.n_pieces;
  const uint32_t rot_dim  = kFixed ? uint32_t(PQD * LEN) : p.rot_dim;
  const int g        = tid / gthreads;
  const int gt       = tid - g * gthreads;
  const int gw       = gt >> 5;
  const int lane     = tid & 31;
  const int n_gwarps = gthreads >> 5;
  const int bar_id   = 1 + g;

  float* s_pqc      = reinterpret_cast<float*>(smem);
  // This group's areas, as 32-bit shared-space addresses derived from one register (the offsets are
  // kernel parameters): LUT, base difference, merge buffer, two work-item slots, then the group-wide
  // bound on the k-th best ordered score of the current pair.
  const uint32_t goff    = p.smem_pqc_bytes + uint32_t(g) * p.smem_group_bytes;
  const uint32_t lut_a   = smem_addr(smem) + goff;
  // (recomputed from the parameters where used, so that none of them occupies a register for the
  // life of the kernel)
  // (two base-difference buffers when the plan has room: the warps that idle during the merge of a
  // pair prepare the next pair's vector in the other one)
  const auto s_base_a = [&](uint32_t buf) { return lut_a + p.lut_bytes + (p.base_double ? buf * (p.base_bytes >> 1) : 0u); };
  const auto s_item_a = [&] { return lut_a + p.lut_bytes + p.base_bytes + p.merge_bytes; };
  const auto s_thr_a  = [&] { return s_item_a() + 8u; };

  uint32_t tmem_base = 0;
  if (p.tmem_cols) {
    // per-subspace codebook -> tensor memory, once per CTA
    uint32_t* slot = reinterpret_cast<uint32_t*>(smem + p.tmem_slot_off);
    if (tid < 32) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(slot)),
                   "r"(p.tmem_cols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    tmem_base = *reinterpret_cast<volatile uint32_t*>(slot);
    {
      // lane L of tensor memory is written by the threads with tid % 128 == L
      const uint32_t lane128 = uint32_t(tid) & 127u, part = uint32_t(tid) >> 7, n_parts = blockDim.x >> 7;
      const uint32_t lane_a  = tmem_base + ((lane128 & ~31u) << 16);
      if constexpr (kFixed) {
        fill_codebook_tmem<PqBits, LEN>(lane_a, p.pq_centers, pq_dim, lane128, uint32_t(gthreads) / 128u, part, n_parts);
      } else {
        switch (p.pq_len) {
          case 1: fill_codebook_tmem<PqBits, 1>(lane_a, p.pq_centers, p.pq_dim, lane128, p.group_threads / 128u, part, n_parts); break;
          case 2: fill_codebook_tmem<PqBits, 2>(lane_a, p.pq_centers, p.pq_dim, lane128, p.group_threads / 128u, part, n_parts); break;
          default: fill_codebook_tmem<PqBits, 4>(lane_a, p.pq_centers, p.pq_dim, lane128, p.group_threads / 128u, part, n_parts); break;
        }
      }
    }
    tmem_fence_before();
  }
  if (p.pqc_in_smem) {
    const uint32_t n4 = (p.pq_dim * p.pq_len * kBook) / 4;
    const float4* src = reinterpret_cast<const float4*>(p.pq_centers);
    float4* dst       = reinterpret_cast<float4*>(s_pqc);
    for (uint32_t i = tid; i < n4; i += blockDim.x) { dst[i] = __ldg(src + i); }
  }
  __syncthreads();
  tmem_fence_after();
  // this warp's window into tensor memory: lanes 32 * (warp % 4) .. + 31
  const uint32_t tmem_lane_a = tmem_base + (((uint32_t(tid) >> 5) & 3u) << 21);

  const uint32_t len     = kFixed ? uint32_t(LEN) : p.pq_len;
  const uint32_t k       = p.k;
  constexpr bool kStoreAll = KPL == 0;  // k too large for registers: write every score instead
  warp_topk<(KPL > 0 ? KPL : 1)> queue;

  // Work items are claimed one pair at a time, one claim ahead so that the atomic's latency is
  // hidden (claims of four pairs per atomic measured slower at every work-list length: the tail of
  // the launch is dealt more evenly pair by pair).
  const uint32_t n_work = __ldg(p.n_work);
  constexpr uint32_t claim = 1u;
  if (gt == 0) { sts_b32(s_item_a(), atomicAdd(p.work_counter, claim)); }
  // the base difference of one (query, list): stored pre-duplicated for the packed arithmetic, L2 (d, d),
  // inner product (-q, -q, q*c, q*c); written by threads first, first + step, ...
  const auto write_base = [&](uint32_t base_a, uint32_t q_, uint32_t label_, uint32_t first, uint32_t step) {
    const float* rq = p.rot_q + size_t(q_) * rot_dim;
    const float* c  = p.centers_rot + size_t(label_) * rot_dim;
    for (uint32_t i = first; i < rot_dim; i += step) {
      if constexpr (!IsIP) {
        const float d = __fsub_rn(rq[i], __ldg(c + i));
        sts_b64(base_a + 8u * i, pack2(d, d));
      } else {
        const float qv = rq[i];
        const float y  = __fmul_rn(__ldg(c + i), qv);
        sts_b128(base_a + 16u * i, pack2(-qv, -qv), pack2(y, y));
      }
    }
  };
  // (compiled in only for L2 with k <= 32, where it was measured to pay: the k = 100 and inner-product
  // kernels ran 2-3% slower with the extra code)
  constexpr bool kCanPrefetch = !IsIP && KPL == 1;
  const bool prefetch_base    = kCanPrefetch && p.base_double != 0 && n_gwarps > 1;
  uint32_t cur   = 0;      // buffer that holds (or receives) the current pair's base difference
  bool have_base = false;  // the current pair's base difference and bound were prepared during the last merge
  for (uint32_t it = 0;; it++) {
    group_bar(bar_id, gthreads);
    const uint32_t w = lds_b32_volatile(s_item_a() + 4u * ((it / claim) & 1u)) + (it % claim);
    if (w >= n_work) { break; }
    if (gt == 0 && (it % claim) == 0) {
      sts_b32(s_item_a() + 4u * (((it / claim) + 1u) & 1u), atomicAdd(p.work_counter, claim));
    }
    if (gt == 0) { sts_b32(s_item_a() + 12u, 0u); }  // "some lane survived the first piece" (lazy table build)

    const uint4 d0       = __ldg(p.work + 2 * size_t(w));
    const uint4 d1       = __ldg(p.work + 2 * size_t(w) + 1);
    const uint32_t pair  = d0.x;
    const uint32_t q     = d0.y;
    const uint32_t label = d0.z;
    const uint32_t n     = d0.w;
    const uint32_t sample_offset = d1.x;
    const uint64_t first_row     = (uint64_t(d1.z) << 32) | d1.y;
    uint64_t* out        = p.out_keys + size_t(pair) * k;

    if (n == 0) {
      if constexpr (!kStoreAll) {
        for (uint32_t i = gt; i < k; i += gthreads) { out[i] = kEmptyKey; }
      }
      have_base = false;
      continue;
    }

    // ---- base diff (unless the idle warps of the last merge prepared it) ----
    if (!have_base) {
      if (gt == 0) { sts_b32(s_thr_a(), *reinterpret_cast<volatile uint32_t*>(p.query_kth + q)); }
      write_base(s_base_a(cur), q, label, uint32_t(gt), uint32_t(gthreads));
      group_bar(bar_id, gthreads);
    }

    // The first 16-byte piece of this warp's first group is brought to L2 now, behind the LUT build
    // (a load into registers here would hold four of them through the build); afterwards each piece
    // is requested one piece ahead of its use.
    const uint32_t n_groups = (n + 31u) >> 5;
    const uint4* src = reinterpret_cast<const uint4*>(p.codes + first_row * size_t(n_pieces) * 16u) +
                       size_t(gw) * n_pieces * 32u + lane;
    uint4 nxt = make_uint4(0u, 0u, 0u, 0u);
    if (uint32_t(gw) < n_groups) { asm volatile("prefetch.global.L2 [%0];" ::"l"(src)); }

    // ---- short lists of the compile-time L2 shapes: the table is built a piece at a time ----
    // Rows of the first code piece are built and every vector of the list is scored on that piece
    // alone (partial sums stay in registers, up to kLazyRows groups of 32 rows per warp).  If by then
    // every lane of the group has passed the query's bound -- four pairs in ten on the 96-d benchmark
    // shape -- the other two thirds of the table are never built and nothing is offered to the queues;
    // otherwise the rest is built and the survivors go on.  Same sums in the same order.
    constexpr int kLazyRows = 4;
    constexpr bool kLazyShape = []() {
      // (k <= 32 only: with more keys per lane the extra code costs the long-list kernels 2%)
      if constexpr (kFixed && !IsIP && KPL == 1) {
        constexpr uint32_t js = uint32_t(GT) / (kBook / 4u);  // subspaces built per iteration of a thread
        return js > 0 && uint32_t(PQD) > uint32_t(kPerPiece) && uint32_t(PQD) % js == 0 &&
               uint32_t(kPerPiece) % js == 0;
      } else {
        return false;
      }
    }();
    bool lazy = false;
    if constexpr (kLazyShape) {
      lazy = n_groups <= uint32_t(kLazyRows * n_gwarps) && p.filter_bits == nullptr;
      if (lazy) {
        constexpr uint32_t kIt0    = uint32_t(kPerPiece) / (uint32_t(GT) / (kBook / 4u));
        constexpr uint32_t kPieces = uint32_t((PQD + kPerPiece - 1) / kPerPiece);
        constexpr uint32_t kLast   = uint32_t(PQD) - (kPieces - 1u) * uint32_t(kPerPiece);
        constexpr uint32_t kPieceLutBytes = uint32_t(kPerPiece) * kBook * uint32_t(sizeof(lut_t));
        constexpr int kHalfPiece   = kPerPiece / 2;
        const uint32_t group_stride = uint32_t(n_gwarps) * n_pieces * 32u;  // in 16-byte pieces
        build_lut_tmem<PqBits, LutKind, IsIP, LEN, PQD, GT, 0, int(kIt0)>(tmem_lane_a, s_base_a(cur), lut_a, pq_dim,
                                                                          gt, gthreads);
        uint4 v0[kLazyRows];
#pragma unroll
        for (int r = 0; r < kLazyRows; r++) {
          v0[r] = make_uint4(0u, 0u, 0u, 0u);
          if (uint32_t(gw + r * n_gwarps) < n_groups) { v0[r] = __ldg(src + size_t(r) * group_stride); }
        }
        group_bar(bar_id, gthreads);
        queue.init(int(k));
        const float stop_at = ordered_to_float(lds_b32_volatile(s_thr_a()));  // NaN = no bound yet
        accum<LutKind, OutHalf, IsIP> acc[kLazyRows];
        bool alv[kLazyRows];
        bool any = false;
#pragma unroll
        for (int r = 0; r < kLazyRows; r++) {
          acc[r].init();
          alv[r] = uint32_t(gw + r * n_gwarps) < n_groups;
          if (alv[r]) { score_part<PqBits, LutKind, OutHalf, IsIP, true, 0, kHalfPiece>(acc[r], v0[r], lut_a, 0); }
          alv[r] = alv[r] && !(acc[r].partial() > stop_at);
          if (alv[r]) { score_part<PqBits, LutKind, OutHalf, IsIP, true, kHalfPiece, kPerPiece>(acc[r], v0[r], lut_a, 0); }
          alv[r] = alv[r] && !(acc[r].partial() > stop_at);
          any    = any || alv[r];
        }
        if (__any_sync(kFullMask, any) && lane == 0) { sts_b32(s_item_a() + 12u, 1u); }
        group_bar(bar_id, gthreads);
        if (lds_b32_volatile(s_item_a() + 12u) != 0u) {
          build_lut_tmem<PqBits, LutKind, IsIP, LEN, PQD, GT, int(kIt0), -1>(tmem_lane_a, s_base_a(cur), lut_a, pq_dim,
                                                                             gt, gthreads);
          group_bar(bar_id, gthreads);
#pragma unroll
          for (int r = 0; r < kLazyRows; r++) {
            const uint32_t gi = uint32_t(gw + r * n_gwarps);
            if (gi >= n_groups) { continue; }
            if (__any_sync(kFullMask, alv[r])) {
#pragma unroll
              for (uint32_t c = 1; c < kPieces; c++) {
                const uint4 v     = __ldg(src + size_t(r) * group_stride + c * 32u);
                const uint32_t la = lut_a + c * kPieceLutBytes;
                if (c + 1 < kPieces || kLast == uint32_t(kPerPiece)) {
                  if (alv[r]) { score_part<PqBits, LutKind, OutHalf, IsIP, true, 0, kHalfPiece>(acc[r], v, la, 0); }
                  alv[r] = alv[r] && !(acc[r].partial() > stop_at);
                  if (alv[r]) { score_part<PqBits, LutKind, OutHalf, IsIP, true, kHalfPiece, kPerPiece>(acc[r], v, la, 0); }
                } else {
                  if (alv[r]) { score_part<PqBits, LutKind, OutHalf, IsIP, false, 0, kHalfPiece>(acc[r], v, la, kLast); }
                  alv[r] = alv[r] && !(acc[r].partial() > stop_at);
                  if (alv[r]) { score_part<PqBits, LutKind, OutHalf, IsIP, false, kHalfPiece, kPerPiece>(acc[r], v, la, kLast); }
                }
                if (c + 1 < kPieces) { alv[r] = alv[r] && !(acc[r].partial() > stop_at); }
              }
            }
            // a lane that stopped early holds a partial sum above the bound: rejected below like any other
            const float score  = acc[r].result(p.cosine != 0);
            const uint32_t row = gi * 32u + lane;
            const uint32_t ord = float_to_ordered(score);
            const uint64_t key = (uint64_t(ord) << 32) | (sample_offset + row);
            const uint32_t thr = lds_b32_volatile(s_thr_a());
            const uint64_t before = queue.kth();
            queue.offer(key, row < n && alv[r] && ord <= thr);
            if (queue.kth() != before && lane == 0) { atoms_min_u32(s_thr_a(), uint32_t(queue.kth() >> 32)); }
          }
        }
      }
    }

    if (!lazy) {
    // ---- LUT ----
    if constexpr (kFixed) {
      build_lut_tmem<PqBits, LutKind, IsIP, LEN, PQD, GT>(tmem_lane_a, s_base_a(cur), lut_a, pq_dim, gt, gthreads);
    } else if (p.tmem_cols) {
      const uint32_t base_a = s_base_a(cur);
      switch (len) {
        case 1: build_lut_tmem<PqBits, LutKind, IsIP, 1>(tmem_lane_a, base_a, lut_a, p.pq_dim, gt, gthreads); break;
        case 2: build_lut_tmem<PqBits, LutKind, IsIP, 2>(tmem_lane_a, base_a, lut_a, p.pq_dim, gt, gthreads); break;
        default: build_lut_tmem<PqBits, LutKind, IsIP, 4>(tmem_lane_a, base_a, lut_a, p.pq_dim, gt, gthreads); break;
      }
    } else if (p.pqc_in_smem) {
      const uint32_t pqc_a = smem_addr(s_pqc), base_a = s_base_a(cur);
      switch (len) {
        case 1: build_lut_smem<PqBits, LutKind, IsIP, 1>(pqc_a, base_a, lut_a, p.pq_dim, len, gt, gthreads); break;
        case 2: build_lut_smem<PqBits, LutKind, IsIP, 2>(pqc_a, base_a, lut_a, p.pq_dim, len, gt, gthreads); break;
        case 4: build_lut_smem<PqBits, LutKind, IsIP, 4>(pqc_a, base_a, lut_a, p.pq_dim, len, gt, gthreads); break;
        default: build_lut_smem<PqBits, LutKind, IsIP, 0>(pqc_a, base_a, lut_a, p.pq_dim, len, gt, gthreads);
      }
    } else {
      // codebook read from global memory (PER_CLUSTER, or a per-subspace codebook too large for
      // shared memory): same arithmetic, generic addressing
      constexpr uint32_t kPairs = kBook / 2;
      lut_t* s_lut        = reinterpret_cast<lut_t*>(smem + goff);
      const float* s_base = reinterpret_cast<const float*>(smem + goff + p.lut_bytes +
                                                          (p.base_double ? cur * (p.base_bytes >> 1) : 0u));
      const float* pqc = p.per_cluster ? p.pq_centers + size_t(label) * len * kBook : p.pq_centers;
      const uint32_t b        = (uint32_t(gt) % kPairs) * 2u;
      const uint32_t j_first  = uint32_t(gt) / kPairs;
      const uint32_t j_stride = uint32_t(gthreads) / kPairs;
      const uint32_t cb_step  = p.per_cluster ? 0u : len * kBook;
      const float* cb         = pqc + b + j_first * cb_step;
      const uint64_t* bd      = reinterpret_cast<const uint64_t*>(s_base) + j_first * len * (IsIP ? 2u : 1u);
      uint32_t e2             = j_first * kPairs + (uint32_t(gt) % kPairs);
      for (uint32_t j = j_first; j < p.pq_dim; j += j_stride) {
        uint64_t score = 0ull;
        for (uint32_t kk = 0; kk < len; kk++) {
          const float2 pq    = __ldg(reinterpret_cast<const float2*>(cb + kk * kBook));
          const uint64_t pq2 = pack2(pq.x, pq.y);
          if constexpr (!IsIP) {
            const uint64_t dif = sub2(bd[kk], pq2);
            score              = fma2(dif, dif, score);
          } else {
            score = sub2(score, bd[2 * kk + 1]);
            score = fma2(bd[2 * kk], pq2, score);
          }
        }
        if constexpr (LutKind == LUT_F32) {
          reinterpret_cast<float2*>(s_lut)[e2] = make_float2(lo2(score), hi2(score));
        } else if constexpr (LutKind == LUT_F16) {
          reinterpret_cast<__half2*>(s_lut)[e2] = __floats2half2_rn(lo2(score), hi2(score));
        } else {
          reinterpret_cast<uint16_t*>(s_lut)[e2] =
            uint16_t(fp8_encode<IsIP>(lo2(score))) | (uint16_t(fp8_encode<IsIP>(hi2(score))) << 8);
        }
        cb += j_stride * cb_step;
        bd += j_stride * len * (IsIP ? 2u : 1u);
        e2 += j_stride * kPairs;
      }
    }
    group_bar(bar_id, gthreads);

    // ---- scan ----
    queue.init(int(k));
    if (uint32_t(gw) < n_groups) { nxt = __ldg(src); }
    {
      const uint32_t lut_base_a   = lut_a;
      const uint32_t group_stride = uint32_t(n_gwarps) * n_pieces * 32u;  // in 16-byte pieces
      constexpr uint32_t kPieceLutBytes = uint32_t(kPerPiece) * kBook * uint32_t(sizeof(lut_t));
      // L2 early stop (compute_score_impl.cuh:70-71 of the reference): table entries are non-negative,
      // so a running sum already above the bound on the query's k-th best can only end above it -- the
      // lane stops looking up (its final value is rejected by the same bound below).  Fewer active
      // lanes per look-up means fewer bank-conflict replays, the kernel's limiter.
      constexpr bool kEarlyStop = !IsIP && !kStoreAll;
      for (uint32_t gi = gw; gi < n_groups; gi += n_gwarps, src += group_stride) {
        accum<LutKind, OutHalf, IsIP> acc;
        acc.init();
        [[maybe_unused]] float stop_at = 0.0f;
        [[maybe_unused]] bool alive    = true;
        if constexpr (kEarlyStop) { stop_at = ordered_to_float(lds_b32_volatile(s_thr_a())); }  // NaN = no bound yet
        if constexpr (kFixed) {
          // the pieces of a vector, unrolled: table rows at constant offsets, the next piece (or the
          // first of this warp's next 32 rows) requested before the current one is looked up
          constexpr uint32_t kPieces = uint32_t((PQD + kPerPiece - 1) / kPerPiece);
          constexpr uint32_t kLast   = uint32_t(PQD) - (kPieces - 1u) * uint32_t(kPerPiece);
#pragma unroll
          for (uint32_t c = 0; c < kPieces; c++) {
            const uint4 v = nxt;
            if (c + 1 < kPieces) {
              nxt = __ldg(src + (c + 1) * 32u);
            } else if (gi + n_gwarps < n_groups) {
              nxt = __ldg(src + group_stride);
            }
            if constexpr (kEarlyStop) {
              // two halves per piece, the bound checked after each
              constexpr int kHalfPiece = kPerPiece / 2;
              if (c + 1 < kPieces || kLast == uint32_t(kPerPiece)) {
                if (alive) { score_part<PqBits, LutKind, OutHalf, IsIP, true, 0, kHalfPiece>(acc, v, lut_base_a + c * kPieceLutBytes, 0); }
                alive = alive && !(acc.partial() > stop_at);
                if (alive) { score_part<PqBits, LutKind, OutHalf, IsIP, true, kHalfPiece, kPerPiece>(acc, v, lut_base_a + c * kPieceLutBytes, 0); }
              } else {
                if (alive) { score_part<PqBits, LutKind, OutHalf, IsIP, false, 0, kHalfPiece>(acc, v, lut_base_a + c * kPieceLutBytes, kLast); }
                alive = alive && !(acc.partial() > stop_at);
                if (alive) { score_part<PqBits, LutKind, OutHalf, IsIP, false, kHalfPiece, kPerPiece>(acc, v, lut_base_a + c * kPieceLutBytes, kLast); }
              }
              if (c + 1 < kPieces) { alive = alive && !(acc.partial() > stop_at); }
            } else {
              if (c + 1 < kPieces || kLast == uint32_t(kPerPiece)) {
                score_piece<PqBits, LutKind, OutHalf, IsIP, true>(acc, v, lut_base_a + c * kPieceLutBytes, 0);
              } else {
                score_piece<PqBits, LutKind, OutHalf, IsIP, false>(acc, v, lut_base_a + c * kPieceLutBytes, kLast);
              }
            }
          }
        } else {
          uint32_t row_a = lut_base_a;
          uint32_t j0    = 0;
          for (uint32_t c = 0; c < n_pieces; c++, j0 += kPerPiece, row_a += kPieceLutBytes) {
            const uint4 v = nxt;
            if (c + 1 < n_pieces) {
              nxt = __ldg(src + (c + 1) * 32u);
            } else if (gi + n_gwarps < n_groups) {
              nxt = __ldg(src + group_stride);
            }
            if (!kEarlyStop || alive) {
              if (j0 + kPerPiece <= pq_dim) {
                score_piece<PqBits, LutKind, OutHalf, IsIP, true>(acc, v, row_a, 0);
              } else {
                score_piece<PqBits, LutKind, OutHalf, IsIP, false>(acc, v, row_a, pq_dim - j0);
              }
            }
            if constexpr (kEarlyStop) { alive = alive && !(acc.partial() > stop_at); }
          }
        }
        const float score    = acc.result(p.cosine != 0);
        const uint32_t row   = gi * 32u + lane;
        bool valid           = row < n;
        if (p.filter_bits != nullptr && valid) {
          const int64_t id = p.ids[first_row + row];
          valid = id >= 0 && uint64_t(id) < p.filter_nbits && ((p.filter_bits[id >> 5] >> (id & 31)) & 1u);
        }
        if constexpr (kStoreAll) {
          if (valid) { p.all_scores[size_t(q) * p.max_samples + sample_offset + row] = score; }
        } else {
          const uint32_t ord   = float_to_ordered(score);
          const uint64_t key   = (uint64_t(ord) << 32) | (sample_offset + row);
          // s_thr never exceeds the final k-th best score of the query, so nothing wanted is lost
          const uint32_t thr   = lds_b32_volatile(s_thr_a());
          const uint64_t before = queue.kth();
          queue.offer(key, valid && ord <= thr);
          if (queue.kth() != before && lane == 0) { atoms_min_u32(s_thr_a(), uint32_t(queue.kth() >> 32)); }
        }
      }
    }

    }  // !lazy

    if constexpr (!kStoreAll) {
    // ---- merge the warps' queues, write k keys ----
    uint64_t* s_merge = reinterpret_cast<uint64_t*>(smem + goff + p.lut_bytes + p.base_bytes);
    queue.store(s_merge + size_t(gw) * k, int(k));
    group_bar(bar_id, gthreads);
    // While warp 0 merges, the other warps prepare the next pair: its base difference into the other
    // buffer and the query's bound (every warp has finished scanning, so the bound's slot is free).  The
    // next work item was claimed after the barrier at the top of this iteration.
    have_base = false;
    if constexpr (kCanPrefetch) {
    if (prefetch_base) {
      const uint32_t w_next = lds_b32_volatile(s_item_a() + 4u * ((it + 1u) & 1u));
      if (w_next < n_work) {
        have_base = true;
        cur ^= 1u;
        if (gw != 0) {
          const uint4 nd = __ldg(p.work + 2 * size_t(w_next));
          if (gt == 32) { sts_b32(s_thr_a(), *reinterpret_cast<volatile uint32_t*>(p.query_kth + nd.y)); }
          write_base(s_base_a(cur), nd.y, nd.z, uint32_t(gt) - 32u, uint32_t(gthreads) - 32u);
        }
      }
    }
    }
    if (gw == 0) {
      const uint32_t others = uint32_t(n_gwarps - 1) * k;
      for (uint32_t t0 = 0; t0 < others; t0 += 32) {
        const uint32_t t = t0 + lane;
        uint64_t key     = t < others ? s_merge[k + t] : kEmptyKey;
        queue.offer(key, t < others);
      }
      queue.store(out, int(k));
      const uint32_t kth_score = uint32_t(queue.kth() >> 32);
      if (lane == 0 && kth_score != kEmptyScore) { atomicMin(p.query_kth + q, kth_score); }
    }
    }
    // the barrier at the top of the loop orders warp 0's reads of s_merge before the next writes
  }
  if (p.tmem_cols) {
    tmem_fence_before();
    __syncthreads();
    if (tid < 32) {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                   : "memory");
    }
  }
}

// ---- look-up table in global memory -------------------------------------------------------------
// The variant for tables that do not fit shared memory (the reference's third kernel,
// ivf_pq_compute_similarity_impl.cuh:441-460, conf_no_smem_lut): one 256-thread CTA per pair at a time,
// its table in a slice of a global scratch buffer (written and read through L1 / L2), base differences
// and the merge buffer in shared memory.  Same arithmetic and same result as scan_kernel -- scalar
// fused multiply-adds in the order of the reference's chain, one rounding to the table type, entries
// summed in subspace order, the same 64-bit keys -- without its tuning: this is the rare path.
template <int PqBits, int LutKind, bool OutHalf, bool IsIP, int KPL>
__global__ void __launch_bounds__(256) scan_glut_kernel(const scan_params p)
{
  using lut_t              = typename lut_elem<LutKind>::type;
  constexpr uint32_t kBook = 1u << PqBits;
  constexpr uint32_t kMask = kBook - 1u;
  constexpr int kPerPiece  = 128 / PqBits;
  constexpr bool kStoreAll = KPL == 0;
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_base     = reinterpret_cast<float*>(smem);                         // [rot_dim] or [rot_dim][2]
  uint64_t* s_merge = reinterpret_cast<uint64_t*>(smem + p.base_bytes);       // [8 warps][k]
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lut_size = p.pq_dim << PqBits;
  lut_t* lut = static_cast<lut_t*>(p.lut_global) + size_t(blockIdx.x) * lut_size;
  const uint32_t n_work = *p.n_work;
  const uint32_t k      = p.k;
  const uint32_t len    = p.pq_len;
  warp_topk<(KPL > 0 ? KPL : 1)> queue;

  for (uint32_t w = blockIdx.x; w < n_work; w += gridDim.x) {
    const uint4 d0       = p.work[2 * size_t(w)];
    const uint4 d1       = p.work[2 * size_t(w) + 1];
    const uint32_t pair  = d0.x, q = d0.y, label = d0.z, n = d0.w;
    const uint32_t sample_offset = d1.x;
    const uint64_t first_row     = (uint64_t(d1.z) << 32) | d1.y;
    __syncthreads();  // the previous pair's table and merge buffer are no longer read
    {
      const float* rq = p.rot_q + size_t(q) * p.rot_dim;
      const float* c  = p.centers_rot + size_t(label) * p.rot_dim;
      for (uint32_t i = tid; i < p.rot_dim; i += 256) {
        if constexpr (!IsIP) {
          s_base[i] = __fsub_rn(rq[i], c[i]);
        } else {
          s_base[2 * i]     = rq[i];
          s_base[2 * i + 1] = __fmul_rn(c[i], rq[i]);
        }
      }
    }
    __syncthreads();
    {
      const float* pqc0 = p.per_cluster ? p.pq_centers + size_t(label) * len * kBook : p.pq_centers;
      for (uint32_t e = tid; e < lut_size; e += 256) {
        const uint32_t j = e >> PqBits, b = e & kMask;
        const float* pqc = pqc0 + (p.per_cluster ? size_t(0) : size_t(j) * len * kBook) + b;
        float score      = 0.0f;
        for (uint32_t kk = 0; kk < len; kk++) {
          const float pq_c = pqc[size_t(kk) * kBook];
          const uint32_t d = j * len + kk;
          if constexpr (!IsIP) {
            const float diff = __fsub_rn(s_base[d], pq_c);
            score            = __fmaf_rn(diff, diff, score);
          } else {
            score = __fsub_rn(score, s_base[2 * d + 1]);
            score = __fmaf_rn(-s_base[2 * d], pq_c, score);
          }
        }
        if constexpr (LutKind == LUT_F32) {
          lut[e] = score;
        } else if constexpr (LutKind == LUT_F16) {
          lut[e] = __float2half_rn(score);
        } else {
          lut[e] = fp8_encode<IsIP>(score);
        }
      }
    }
    __syncthreads();  // block-wide visibility of the table written to global memory
    const uint32_t thr0 = kStoreAll ? 0u : *reinterpret_cast<volatile uint32_t*>(p.query_kth + q);
    queue.init(int(k));
    const uint32_t n_groups = (n + 31u) >> 5;
    const uint4* src = reinterpret_cast<const uint4*>(p.codes + first_row * size_t(p.n_pieces) * 16u);
    for (uint32_t gi = warp; gi < n_groups; gi += 8) {
      float f  = 0.0f;
      __half h = __ushort_as_half(0);
      uint32_t j = 0;
      for (uint32_t c = 0; c < p.n_pieces; c++) {
        const uint4 v       = src[(size_t(gi) * p.n_pieces + c) * 32u + lane];
        const uint32_t wd[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int cc = 0; cc < kPerPiece; cc++, j++) {
          if (j < p.pq_dim) {
            const int bit = cc * PqBits, word = bit >> 5, sh = bit & 31;
            uint32_t code = wd[word] >> sh;
            if (sh + PqBits > 32) { code |= wd[word + 1 > 3 ? 3 : word + 1] << (32 - sh); }
            code &= kMask;
            const lut_t entry = lut[size_t(j) * kBook + code];
            if constexpr (!OutHalf) {
              if constexpr (LutKind == LUT_F32) {
                f = __fadd_rn(f, entry);
              } else if constexpr (LutKind == LUT_F16) {
                f = __fadd_rn(f, __half2float(entry));
              } else {
                f = __fadd_rn(f, fp8_to_float<IsIP>(entry));
              }
            } else {
              if constexpr (LutKind == LUT_F16) {
                h = __hadd(h, entry);
              } else if constexpr (LutKind == LUT_FP8) {
                h = __hadd(h, fp8_to_half<IsIP>(entry));
              }
            }
          }
        }
      }
      float score;
      if constexpr (!OutHalf) {
        score = p.cosine ? __fadd_rn(f, 1.0f) : f;
      } else {
        if (p.cosine) { h = __hadd(h, __float2half(1.0f)); }
        score = __half2float(h);
      }
      const uint32_t row = gi * 32u + lane;
      bool valid         = row < n;
      if (p.filter_bits != nullptr && valid) {
        const int64_t id = p.ids[first_row + row];
        valid = id >= 0 && uint64_t(id) < p.filter_nbits && ((p.filter_bits[id >> 5] >> (id & 31)) & 1u);
      }
      if constexpr (kStoreAll) {
        if (valid) { p.all_scores[size_t(q) * p.max_samples + sample_offset + row] = score; }
      } else {
        const uint32_t ord = float_to_ordered(score);
        queue.offer((uint64_t(ord) << 32) | (sample_offset + row), valid && ord <= thr0);
      }
    }
    if constexpr (!kStoreAll) {
      queue.store(s_merge + size_t(warp) * k, int(k));
      __syncthreads();
      if (warp == 0) {
        const uint32_t others = 7u * k;
        for (uint32_t t0 = 0; t0 < others; t0 += 32) {
          const uint32_t t = t0 + lane;
          queue.offer(t < others ? s_merge[k + t] : kEmptyKey, t < others);
        }
        queue.store(p.out_keys + size_t(pair) * k, int(k));
        const uint32_t kth_score = uint32_t(queue.kth() >> 32);
        if (lane == 0 && kth_score != kEmptyScore) { atomicMin(p.query_kth + q, kth_score); }
      }
    }
  }
}

// Host-side launcher of one instantiation family (defined once per PqBits in scan_inst.cu).
void launch_scan(const scan_params& p, int pq_bits, int lut_kind, bool out_half, bool is_ip,
                 int kpl, int grid, size_t smem_bytes, cudaStream_t stream);
// the variant with the table in global memory (p.lut_global); kpl is 0 (store every score) or 4
void launch_scan_glut(const scan_params& p, int pq_bits, int lut_kind, bool out_half, bool is_ip,
                      int kpl, int grid, size_t smem_bytes, cudaStream_t stream);

}  // namespace cuvs_b200
