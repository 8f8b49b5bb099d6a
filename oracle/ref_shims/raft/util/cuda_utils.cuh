// Shim: the host/device inline marker used by the pinned headers, the kernel marker and two small
// integer helpers with the meaning their names state.
#pragma once
#include <cstddef>
#include <type_traits>
#ifndef HDI
#ifdef __CUDACC__
#define HDI inline __host__ __device__
#else
#define HDI inline
#endif
#endif
#ifndef RAFT_KERNEL
#define RAFT_KERNEL static __global__ void
#endif
namespace raft {
constexpr int WarpSize = 32;
template <typename T>
constexpr HDI T div_rounding_up_unsafe(T a, T b)
{
  return (a + b - 1) / b;
}
// true when a value of From may not be representable in To
template <typename From, typename To>
constexpr bool is_narrowing_v =
  sizeof(To) < sizeof(From) || (std::is_signed_v<From> && !std::is_signed_v<To>) ||
  (sizeof(To) == sizeof(From) && std::is_signed_v<To> != std::is_signed_v<From>);
}  // namespace raft
