// Warp-level top-k on 64-bit keys.
//
// A candidate is one 64-bit key: (order-preserving image of the fp32 score) << 32 | 32-bit payload.
// Smaller key = better candidate; equal scores order by payload, so every selection in the search
// path is a total order and the results do not depend on scheduling.
//
// warp_topk<KPL> keeps the 32*KPL smallest keys seen so far, sorted ascending across the warp:
// position p lives in register a[p / 32] of lane p % 32.  A few candidates are inserted one by
// one (a warp-wide shift); many at once are merged as a sorted batch (bitonic networks).  Callers
// pre-filter against kth() so that, after warm-up, almost no candidate reaches either path.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace cuvs_b200 {

constexpr uint64_t kEmptyKey    = 0xFFFFFFFFFFFFFFFFull;
constexpr uint32_t kEmptyScore  = 0xFFFFFFFFu;
constexpr unsigned kFullMask    = 0xFFFFFFFFu;

// fp32 -> uint32 such that a < b  <=>  ord(a) < ord(b) for all non-NaN values.
__host__ __device__ __forceinline__ uint32_t float_to_ordered(float f)
{
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
#endif
  return u ^ ((u >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__host__ __device__ __forceinline__ float ordered_to_float(uint32_t o)
{
  uint32_t u = o ^ ((o >> 31) ? 0x80000000u : 0xFFFFFFFFu);
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}
__device__ __forceinline__ uint64_t make_key(float score, uint32_t payload)
{
  return (uint64_t(float_to_ordered(score)) << 32) | payload;
}

__device__ __forceinline__ uint64_t shfl_u64(uint64_t v, int src)
{
  uint32_t lo = __shfl_sync(kFullMask, uint32_t(v), src);
  uint32_t hi = __shfl_sync(kFullMask, uint32_t(v >> 32), src);
  return (uint64_t(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t shfl_up_u64(uint64_t v, int d)
{
  uint32_t lo = __shfl_up_sync(kFullMask, uint32_t(v), d);
  uint32_t hi = __shfl_up_sync(kFullMask, uint32_t(v >> 32), d);
  return (uint64_t(hi) << 32) | lo;
}

template <int KPL>
struct warp_topk {
  uint64_t a[KPL];
  uint64_t kth_;  // warp-uniform: key at position k-1
  int k_;

  __device__ __forceinline__ void init(int k)
  {
#pragma unroll
    for (int r = 0; r < KPL; r++) { a[r] = kEmptyKey; }
    kth_ = kEmptyKey;
    k_   = k;
  }
  __device__ __forceinline__ uint64_t kth() const { return kth_; }

  // Insert a warp-uniform key c with c < kth().
  __device__ __forceinline__ void insert(uint64_t c)
  {
    const int lane = threadIdx.x & 31;
    uint64_t carry = 0;  // key preceding this row (last key of the previous row)
#pragma unroll
    for (int r = 0; r < KPL; r++) {
      const uint64_t cur  = a[r];
      uint64_t prev       = shfl_up_u64(cur, 1);
      const uint64_t last = shfl_u64(cur, 31);
      if (lane == 0) { prev = carry; }
      a[r]  = (cur <= c) ? cur : (prev > c ? prev : c);
      carry = last;
    }
    refresh_kth();
  }
  __device__ __forceinline__ void refresh_kth()
  {
    const int pos = k_ - 1;
    uint64_t mine = a[0];
#pragma unroll
    for (int r = 1; r < KPL; r++) {
      if ((pos >> 5) == r) { mine = a[r]; }
    }
    kth_ = shfl_u64(mine, pos & 31);
  }

  // Bitonic merge step over the 32 lanes of one register: v holds a bitonic sequence -> ascending.
  static __device__ __forceinline__ uint64_t bitonic_finish(uint64_t v)
  {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 16; j > 0; j >>= 1) {
      const uint64_t o = shfl_u64(v, lane ^ j);
      v                = ((lane & j) == 0) ? (o < v ? o : v) : (o > v ? o : v);
    }
    return v;
  }

  // Merge a whole batch (one key per lane, kEmptyKey where there is none) into the queue: sort the
  // batch across the warp, then row by row split (row, batch) into the 32 smallest (stay in the
  // row) and the 32 largest (carried to the next row).
  __device__ __forceinline__ void merge_batch(uint64_t b)
  {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
        const uint64_t o    = shfl_u64(b, lane ^ j);
        const bool keep_min = ((lane & j) == 0) == ((lane & k) == 0);
        b                   = keep_min ? (o < b ? o : b) : (o > b ? o : b);
      }
    }
#pragma unroll
    for (int r = 0; r < KPL; r++) {
      const uint64_t rev = shfl_u64(b, 31 - lane);  // descending
      // ascending row against descending batch: element-wise min / max are both bitonic and hold
      // the 32 smallest / 32 largest keys of the union
      const uint64_t lo = a[r] < rev ? a[r] : rev;
      const uint64_t hi = a[r] < rev ? rev : a[r];
      a[r]              = bitonic_finish(lo);
      if (r + 1 < KPL) { b = bitonic_finish(hi); }
    }
    refresh_kth();
  }

  // Offer one key per lane (valid lanes only); keys >= kth() are dropped.
  __device__ __forceinline__ void offer(uint64_t key, bool valid)
  {
    const bool pass = valid && key < kth_;
    unsigned m      = __ballot_sync(kFullMask, pass);
    if (m == 0) { return; }
    if (__popc(m) > 2 + 2 * KPL) {
      merge_batch(pass ? key : kEmptyKey);
      return;
    }
    while (m) {
      int src = __ffs(m) - 1;
      m &= m - 1;
      uint64_t c = shfl_u64(key, src);
      if (c < kth_) { insert(c); }
    }
  }

  // Sorted position of register r on this lane.
  static __device__ __forceinline__ uint32_t position(int r) { return uint32_t(r) * 32u + (threadIdx.x & 31); }

  // Store the first n sorted keys to dst[0..n).
  __device__ __forceinline__ void store(uint64_t* dst, int n) const
  {
#pragma unroll
    for (int r = 0; r < KPL; r++) {
      const int p = int(position(r));
      if (p < n) { dst[p] = a[r]; }
    }
  }
};

}  // namespace cuvs_b200
