// Shim standing in for the reference's public header when its fp_8bit and code-packing headers are
// compiled on the host for the oracle pin.  Only the three declarations those headers use are
// restated here (group size, piece size, extents of an interleaved list:
// cpp/include/cuvs/neighbors/ivf_pq.hpp:222-247).
#pragma once
#include <cstdint>
#include <raft/core/device_mdspan.hpp>
namespace cuvs::neighbors::ivf_pq {
constexpr static uint32_t kIndexGroupSize   = 32;
constexpr static uint32_t kIndexGroupVecLen = 16;
template <typename SizeT, typename IdxT>
struct list_spec_interleaved {
  using list_extents = raft::
    extents<SizeT, raft::dynamic_extent, raft::dynamic_extent, kIndexGroupSize, kIndexGroupVecLen>;
};
}  // namespace cuvs::neighbors::ivf_pq
