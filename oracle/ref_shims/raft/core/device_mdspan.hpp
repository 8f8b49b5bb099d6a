// Shim: raft's mdspan aliases mapped onto libcu++'s mdspan (row-major = layout_right).
#pragma once
#include <cuda/std/mdspan>
namespace raft {
using cuda::std::dynamic_extent;
using cuda::std::extents;
using row_major = cuda::std::layout_right;
template <typename T, typename E, typename L = row_major>
using device_mdspan = cuda::std::mdspan<T, E, L>;
}  // namespace raft
