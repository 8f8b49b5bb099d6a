// Multi-GPU IVF-PQ: the host side of the reference's single-node multi-GPU layer
// (cpp/src/neighbors/mg/snmg.cuh, cpp/include/cuvs/neighbors/common.hpp:1843-1900 for the modes,
// cpp/include/cuvs/neighbors/ivf_pq.hpp:2180-2520 for the entry points) re-designed around list
// sharding.
//
// Three kinds of multi-GPU index exist here:
//   REPLICATED ............ every rank holds the whole index (reference semantics: the query batch is
//                           split between the ranks, no exchange);
//   SHARDED, by rows ...... every rank holds an independent index over a slice of the rows with ids
//                           local to the slice (what the reference builds and writes to files); every
//                           rank searches the whole batch, ids are translated, parts are merged;
//   SHARDED, by list ...... this engine's own: one global coarse model replicated on every rank, each
//                           inverted list stored on exactly one rank.  Probe selection is shared by
//                           query slice (one all-gather of n_q * n_probes * 4 bytes), every rank scans
//                           the probes it owns for the whole batch, the per-rank top-k blocks (ids
//                           already global) are all-gathered (12 * n_q * k bytes per rank) and merged.
//                           Total work is that of one GPU (n_probes lists per query in all, not per
//                           rank) and the result equals the single-GPU search.
//
// Two ways to drive it:
//   one process per GPU ... `rank_comm` + `search_rank`: ONE call per batch enqueues the whole step
//                           (probe slice -> all-gather -> scan -> all-gather -> merge) on the handle's
//                           stream, on buffers sized once per communicator; the scan is two launches
//                           (nearest-probe pairs, then the rest) with a min-reduction of the per-query
//                           bounds on the k-th best score between them, so that every rank prunes with
//                           what all ranks have found;
//   one process, all GPUs . `snmg_resources` + `mg_index` + `search`: the reference's shape (host
//                           tensors in and out), one host thread issuing the same step on every device
//                           with the collectives grouped.
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library loads without it.
#pragma once

#include "ivf_pq.hpp"

#include <memory>
#include <string>
#include <vector>

struct ncclComm;

namespace cuvs::neighbors::mg {

using ivf_pq::elem_t;
using ivf_pq::index;

enum class distribution_mode { REPLICATED = 0, SHARDED = 1 };           // common.hpp:1843-1848
enum class replicated_search_mode { LOAD_BALANCER = 0, ROUND_ROBIN = 1 };  // common.hpp:1851-1856
enum class sharded_merge_mode { MERGE_ON_ROOT_RANK = 0, TREE_MERGE = 1 };   // common.hpp:1859-1864
enum class shard_kind { BY_ROWS = 0, BY_LIST = 1 };

struct search_params : ivf_pq::search_params {
  replicated_search_mode search_mode = replicated_search_mode::LOAD_BALANCER;
  // accepted for interface compatibility: both values run the one gather + merge of this engine
  sharded_merge_mode merge_mode = sharded_merge_mode::TREE_MERGE;
  int64_t n_rows_per_batch      = int64_t(1) << 20;
};

struct nccl_unique_id {
  char bytes[128];
};
void make_unique_id(nccl_unique_id* id);

// One rank's end of the exchanges: communicator and grow-only device buffers.
class rank_comm {
 public:
  // joins the communicator described by `id` (blocks until all ranks have joined)
  rank_comm(const nccl_unique_id& id, int rank, int n_ranks);
  // adopts a communicator made elsewhere (not destroyed with this object)
  rank_comm(ncclComm* comm, int rank, int n_ranks);
  ~rank_comm();
  rank_comm(const rank_comm&)            = delete;
  rank_comm& operator=(const rank_comm&) = delete;

  int rank() const { return rank_; }
  int n_ranks() const { return n_ranks_; }
  ncclComm* comm() const { return comm_; }

  // the phases of one list-sharded batch; each enqueues on res.stream and returns
  void select(raft::resources& res, const ivf_pq::search_params& p, const index<int64_t>& shard,
              const void* queries, elem_t qtype, uint32_t nq, uint32_t k);
  void gather_probes(cudaStream_t stream);
  // `exchange_bounds` (one process per GPU only: it issues a collective of its own): the ranks share
  // their per-query bounds between the nearest-probe pairs and the rest
  void scan(raft::resources& res, const ivf_pq::search_params& p, const index<int64_t>& shard,
            const void* queries, elem_t qtype, bool exchange_bounds = false);
  void gather_results(cudaStream_t stream);
  void merge(raft::resources& res, bool select_min, int64_t* neighbors, float* distances);
  // The same two phases with the merge shared out by query slice: every rank receives only its own
  // slice of every rank's block (send/receive pairs, 1/n_ranks of the all-gather's bytes), merges that
  // slice, and the merged slices are all-gathered.  Off unless asked for: on four GPUs it measured no
  // faster than the whole-block all-gather (the blocks are a few MB; two collectives cost what one saves).
  void exchange_slices(cudaStream_t stream);
  void merge_slice_and_gather(raft::resources& res, bool select_min, int64_t* neighbors, float* distances);
  // 0 / 2 = one all-gather of whole blocks, every rank merges everything (the default); 1 = by slice
  void set_merge_mode(int mode) { merge_mode_ = mode; }
  bool merge_by_slice() const { return merge_mode_ == 1; }
  // by-rows shards: plain search of the whole batch into this rank's block, ids += id_offset
  void search_rows(raft::resources& res, const ivf_pq::search_params& p, const index<int64_t>& part,
                   const void* queries, elem_t qtype, uint32_t nq, uint32_t k, int64_t id_offset);

  // Stage times of the one-call step (search_rank), taken only while the handle's stage timing is on:
  // {probe slice, all-gather of the probes, scan of the owned lists, all-gather of the result blocks,
  // merge} in milliseconds, summed over `batches` calls since the last reset.
  void stats(double ms[5], uint64_t* batches, bool reset);
  void mark(raft::resources& res, int i);

  // staging area for host queries of the single-process driver (grow-only)
  void* query_buffer(size_t bytes);
  float* out_distances(size_t n);
  int64_t* out_neighbors(size_t n);

 private:
  void reserve(uint32_t nq, uint32_t n_probes, uint32_t k);
  ncclComm* comm_ = nullptr;
  bool owns_      = false;
  int rank_ = 0, n_ranks_ = 1;
  int merge_mode_ = 0;
  // state of the batch in flight
  uint32_t nq_ = 0, k_ = 0, n_probes_ = 0, slice_ = 0;
  size_t block_bytes_ = 0, ids_bytes_ = 0;
  ivf_pq::dev_array<uint32_t> probes_;  // [n_ranks * slice, n_probes]
  ivf_pq::dev_array<uint8_t> blocks_;   // [n_ranks][ids i64 [nq, k] | distances f32 [nq, k]]
  ivf_pq::dev_array<uint8_t> parts_;    // [n_ranks][ids i64 [slice, k] | distances f32 [slice, k]] of this rank's slice
  ivf_pq::dev_array<uint8_t> queries_;
  ivf_pq::dev_array<float> out_d_;
  ivf_pq::dev_array<int64_t> out_i_;
  struct marks {
    cudaEvent_t e[6];
  };
  std::vector<marks> pending_;
  double stage_ms_[5]    = {0, 0, 0, 0, 0};
  uint64_t stat_batches_ = 0;
};

// The whole list-sharded batch for one rank (one process per GPU): asynchronous on res.stream.
void search_rank(raft::resources& res, rank_comm& comm, const ivf_pq::search_params& params,
                 const index<int64_t>& shard, const void* queries, elem_t qtype, uint32_t nq, uint32_t k,
                 int64_t* neighbors, float* distances);

// ---- one process, all GPUs ----------------------------------------------------------------------
// raft::device_resources_snmg of the reference: the root rank's handle plus one handle, stream and
// communicator per device.
struct snmg_resources : cuvs_b200::resources {
  explicit snmg_resources(const std::vector<int>& device_ids);  // empty = every visible device
  ~snmg_resources();
  int n_ranks() const { return int(devices.size()); }
  std::vector<int> devices;
  std::vector<std::unique_ptr<cuvs_b200::resources>> rank_res;
  std::vector<std::unique_ptr<rank_comm>> comms;
  std::vector<ncclComm*> raw_comms;
  std::vector<cudaStream_t> streams;
};

struct mg_index {
  distribution_mode mode = distribution_mode::SHARDED;
  shard_kind kind        = shard_kind::BY_LIST;
  std::vector<std::unique_ptr<index<int64_t>>> parts;  // one per rank, on that rank's device
  std::vector<int64_t> id_offsets;                     // by-rows shards: rows held by earlier ranks
  int64_t size() const;
};

// mg build (ivf_pq.hpp:2180-2260): host dataset.  SHARDED builds one global index on the root rank and
// deals its lists out; REPLICATED builds once and copies.
void build(snmg_resources& clique, const ivf_pq::index_params& params, distribution_mode mode,
           const void* dataset, elem_t dtype, int64_t n_rows, uint32_t dim, mg_index* out);
void extend(snmg_resources& clique, mg_index* idx, const void* new_vectors, elem_t dtype, int64_t n_rows,
            const int64_t* new_indices);
// host queries, host outputs (ivf_pq.hpp:2328-2440)
void search(snmg_resources& clique, const mg_index& idx, const search_params& params, const void* queries,
            elem_t qtype, int64_t n_queries, uint32_t k, int64_t* neighbors, float* distances);
// files: the reference's multi-GPU format (snmg.cuh:60-91, 780-805).  A by-list index is written as a
// REPLICATED file (one merged stream per rank), which the reference loads as such.
void serialize(snmg_resources& clique, const mg_index& idx, const std::string& filename, const char* dtype_string);
void deserialize(snmg_resources& clique, const std::string& filename, mg_index* out);
// distribute (snmg.cuh:48-58): a single-GPU index file replicated on every rank ...
void distribute(snmg_resources& clique, const std::string& filename, mg_index* out);
// ... or dealt out by inverted list (this engine's sharding)
void distribute_by_list(snmg_resources& clique, const std::string& filename, mg_index* out);

}  // namespace cuvs::neighbors::mg
