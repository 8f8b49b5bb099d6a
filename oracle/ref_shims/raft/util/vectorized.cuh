// Shim: N values of T that can also be moved as one aligned block (raft::TxN_t): `io_t` is the
// block type, `val.data[i]` the i-th value, `vectorized_data()` the address of the block.
#pragma once
#include <cstdint>
namespace raft {
template <typename T, int N>
struct TxN_t {
  struct alignas(sizeof(T) * N) io_t {
    T v[N];
  };
  using math_t               = T;
  static constexpr int Ratio = N;
  union {
    io_t internal;
    math_t data[N];
  } val;
#ifdef __CUDACC__
  __host__ __device__
#endif
  io_t* vectorized_data()
  {
    return &val.internal;
  }
};
}  // namespace raft
