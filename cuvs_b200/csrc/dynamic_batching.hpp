// Dynamic batching front-end: many host threads submit small searches, the runner gathers them into
// batches for the upstream IVF-PQ index.
//
// Mirrors cuvs::neighbors::dynamic_batching of the reference
// (cpp/include/cuvs/neighbors/dynamic_batching.hpp: index_params :39-81, search_params :83-92,
// index :140-190, search :228-...; implementation cpp/src/neighbors/detail/dynamic_batching.cuh):
// same parameters, same contract (k fixed at construction, requests of any size from any number of
// threads, each request answered exactly as a direct upstream search would answer it).
//
// Different inside: the reference couples its threads through lock-free queues and device-side
// spinning kernels that wait for late queries.  Here nothing on the GPU ever waits for the host:
// a batch is closed on the host (full, or `dispatch_timeout_ms` after its first request), the
// dispatching thread makes the queue's stream wait for the contributors' input copies
// (events), launches one upstream search, and the contributors copy their rows out behind an event.
// `conservative_dispatch` is accepted; both settings behave conservatively in the reference's sense.
#pragma once

#include "ivf_pq.hpp"

#include <memory>

namespace cuvs::neighbors::dynamic_batching {

struct index_params {
  int64_t k                  = 10;
  int64_t max_batch_size     = 100;
  size_t n_queues            = 3;
  bool conservative_dispatch = false;
};

struct search_params {
  double dispatch_timeout_ms = 1.0;
};

namespace detail {
class batch_runner;
}

template <typename T, typename IdxT>
struct index {
  std::shared_ptr<detail::batch_runner> runner;
  // `upstream_index` must outlive this object; `upstream_params` are copied.
  index(raft::resources& res, const index_params& params, const ivf_pq::index<int64_t>& upstream_index,
        const ivf_pq::search_params& upstream_params);
};

// queries [n, dim] fp32, neighbors [n, k] i64, distances [n, k] fp32, device memory; work is ordered
// on res.stream like a direct search (the call itself blocks the host until its batch is dispatched).
void search(raft::resources& res, const search_params& params, const index<float, int64_t>& idx,
            const float* queries, uint32_t n_queries, int64_t* neighbors, float* distances);

// the same with the shapes of the caller's tensors checked against the index and k
void search_checked(raft::resources& res, const search_params& params, const index<float, int64_t>& idx,
                    const float* queries, uint32_t n_queries, uint32_t dim, uint32_t k, int64_t* neighbors,
                    float* distances);

// test hook, host side only: the next upstream search of this index throws instead of running (every
// request of that batch then reports the error; the queue stays usable)
void fail_next_upstream_search(const index<float, int64_t>& idx);

// counters for tests: batches dispatched, rows searched
void stats(const index<float, int64_t>& idx, uint64_t* n_batches, uint64_t* n_rows);

}  // namespace cuvs::neighbors::dynamic_batching
