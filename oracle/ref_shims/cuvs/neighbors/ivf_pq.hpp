// Shim standing in for the reference's public header when single headers of its search path are
// compiled for the oracle pins.  Only the declarations those headers use are restated here
// (codebook kind, group size, piece size, extents of an interleaved list:
// cpp/include/cuvs/neighbors/ivf_pq.hpp:34-37, 222-247).
#pragma once
#include <cstdint>
#include <raft/core/device_mdspan.hpp>
namespace cuvs::neighbors::ivf_pq {
enum class codebook_gen { PER_SUBSPACE = 0, PER_CLUSTER = 1 };
constexpr static uint32_t kIndexGroupSize   = 32;
constexpr static uint32_t kIndexGroupVecLen = 16;
template <typename SizeT, typename IdxT>
struct list_spec_interleaved {
  using list_extents = raft::
    extents<SizeT, raft::dynamic_extent, raft::dynamic_extent, kIndexGroupSize, kIndexGroupVecLen>;
};
}  // namespace cuvs::neighbors::ivf_pq
