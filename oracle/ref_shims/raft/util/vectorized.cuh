// Shim: a 16-byte plain vector type for TxN_t<uint8_t, 16>::io_t.
#pragma once
#include <cstdint>
namespace raft {
template <typename T, int N>
struct TxN_t {
  struct alignas(16) io_t {
    T v[N];
  };
};
}  // namespace raft
