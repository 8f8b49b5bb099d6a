/*
 * Multi-GPU IVF-PQ.
 *
 * Part 1 -- the reference's interface (c/include/cuvs/neighbors/mg_ivf_pq.h, mg_common.h): one process
 * drives all GPUs of a node through a multi-GPU resources handle (cuvsMultiGpuResourcesCreate); index
 * parameters carry a distribution mode, search parameters a replicated-search mode, a merge mode and a
 * batch size; datasets, queries and results are host tensors.  Same names, structs, defaults and checks.
 * What differs inside: a SHARDED index built here is sharded by inverted list, not by rows -- one
 * global coarse model on every GPU, every list on exactly one GPU -- so a search probes n_probes lists
 * in all (not n_probes per GPU) and returns what a single-GPU search of the whole index returns.
 * Row-sharded and replicated index files written by the reference load and search with the reference's
 * semantics.
 *
 * Part 2 -- one process per GPU (no counterpart in the reference): every rank holds an ordinary
 * cuvsIvfPqIndex_t with the global coarse model and the lists it owns, joins an NCCL communicator, and
 * ONE call per batch (cuvsMultiGpuIvfPqSearchRank) enqueues the whole step on the handle's stream:
 * probes of this rank's slice of the batch -> all-gather -> scan of the owned lists -> all-gather of the
 * per-rank top-k blocks -> merge.  The building blocks of that step are exported too.
 */
#ifndef CUVS_B200_MG_IVF_PQ_H_
#define CUVS_B200_MG_IVF_PQ_H_

#include "cuvs_ivf_pq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------------
 * Part 1: the reference's single-process interface
 * --------------------------------------------------------------------------------------------- */

/* c/include/cuvs/neighbors/mg_common.h:24-29 */
typedef enum {
  CUVS_NEIGHBORS_MG_REPLICATED = 0,
  CUVS_NEIGHBORS_MG_SHARDED    = 1
} cuvsMultiGpuDistributionMode;
/* c/include/cuvs/neighbors/mg_common.h:34-39 */
typedef enum {
  CUVS_NEIGHBORS_MG_LOAD_BALANCER = 0,
  CUVS_NEIGHBORS_MG_ROUND_ROBIN   = 1
} cuvsMultiGpuReplicatedSearchMode;
/* c/include/cuvs/neighbors/mg_common.h:44-49 -- accepted; both values run this engine's one
 * all-gather + merge */
typedef enum {
  CUVS_NEIGHBORS_MG_MERGE_ON_ROOT_RANK = 0,
  CUVS_NEIGHBORS_MG_TREE_MERGE         = 1
} cuvsMultiGpuShardedMergeMode;

/* c/include/cuvs/neighbors/mg_ivf_pq.h:29-34 */
struct cuvsMultiGpuIvfPqIndexParams {
  cuvsIvfPqIndexParams_t base_params;
  cuvsMultiGpuDistributionMode mode;
};
typedef struct cuvsMultiGpuIvfPqIndexParams* cuvsMultiGpuIvfPqIndexParams_t;
/* c/include/cuvs/neighbors/mg_ivf_pq.h:45 (defaults: base defaults, mode SHARDED) */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqIndexParamsCreate(cuvsMultiGpuIvfPqIndexParams_t* index_params);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:53 */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqIndexParamsDestroy(cuvsMultiGpuIvfPqIndexParams_t index_params);

/* c/include/cuvs/neighbors/mg_ivf_pq.h:69-78 */
struct cuvsMultiGpuIvfPqSearchParams {
  cuvsIvfPqSearchParams_t base_params;
  cuvsMultiGpuReplicatedSearchMode search_mode;
  cuvsMultiGpuShardedMergeMode merge_mode;
  int64_t n_rows_per_batch;
};
typedef struct cuvsMultiGpuIvfPqSearchParams* cuvsMultiGpuIvfPqSearchParams_t;
/* c/include/cuvs/neighbors/mg_ivf_pq.h:88 (defaults: LOAD_BALANCER, TREE_MERGE, 1 << 20 rows per batch) */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSearchParamsCreate(cuvsMultiGpuIvfPqSearchParams_t* params);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:96 */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSearchParamsDestroy(cuvsMultiGpuIvfPqSearchParams_t params);

/* c/include/cuvs/neighbors/mg_ivf_pq.h:111-116 */
typedef struct {
  uintptr_t addr;
  DLDataType dtype;
} cuvsMultiGpuIvfPqIndex;
typedef cuvsMultiGpuIvfPqIndex* cuvsMultiGpuIvfPqIndex_t;
/* c/include/cuvs/neighbors/mg_ivf_pq.h:124 */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqIndexCreate(cuvsMultiGpuIvfPqIndex_t* index);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:132 */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqIndexDestroy(cuvsMultiGpuIvfPqIndex_t index);

/* c/include/cuvs/neighbors/mg_ivf_pq.h:153 -- dataset: host tensor f32/f16/i8/u8 [n_rows, dim].  One
 * global index is built on the root rank and dealt out: by list (SHARDED) or whole (REPLICATED). */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqBuild(cuvsResources_t res,
                                               cuvsMultiGpuIvfPqIndexParams_t params,
                                               DLManagedTensor* dataset_tensor,
                                               cuvsMultiGpuIvfPqIndex_t index);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:177 -- queries, neighbors (int64), distances (f32): host tensors */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSearch(cuvsResources_t res,
                                                cuvsMultiGpuIvfPqSearchParams_t params,
                                                cuvsMultiGpuIvfPqIndex_t index,
                                                DLManagedTensor* queries_tensor,
                                                DLManagedTensor* neighbors_tensor,
                                                DLManagedTensor* distances_tensor);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:202 -- new_indices_tensor may be NULL */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqExtend(cuvsResources_t res,
                                                cuvsMultiGpuIvfPqIndex_t index,
                                                DLManagedTensor* new_vectors_tensor,
                                                DLManagedTensor* new_indices_tensor);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:224 -- the reference's multi-GPU file format; a list-sharded
 * index is written as a REPLICATED file (the merged index once per rank) */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSerialize(cuvsResources_t res,
                                                   cuvsMultiGpuIvfPqIndex_t index,
                                                   const char* filename);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:245 -- REPLICATED or row-SHARDED files of the reference */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqDeserialize(cuvsResources_t res,
                                                     const char* filename,
                                                     cuvsMultiGpuIvfPqIndex_t index);
/* c/include/cuvs/neighbors/mg_ivf_pq.h:266 -- a single-GPU index file replicated on every GPU */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqDistribute(cuvsResources_t res,
                                                    const char* filename,
                                                    cuvsMultiGpuIvfPqIndex_t index);
/* No counterpart in the reference: a single-GPU index file dealt out by inverted list (lists in order
 * of descending size, each to the GPU holding the fewest rows so far). */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqDistributeByList(cuvsResources_t res,
                                                          const char* filename,
                                                          cuvsMultiGpuIvfPqIndex_t index);

/* ---------------------------------------------------------------------------------------------
 * Part 2: one process per GPU (no counterpart in the reference)
 * --------------------------------------------------------------------------------------------- */

/* An NCCL unique id (128 bytes), made by one rank and handed to the others by the host framework. */
typedef struct {
  char bytes[128];
} cuvsMultiGpuCommId;
typedef struct cuvsMultiGpuRankCommOpaque* cuvsMultiGpuRankComm_t;
CUVS_EXPORT cuvsError_t cuvsMultiGpuCommIdCreate(cuvsMultiGpuCommId* id);
/* Joins the communicator (collective: returns when all n_ranks ranks have called it).  The device of
 * `res` must be current.  Exchange buffers are sized on first use and then kept. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuRankCommCreate(cuvsResources_t res,
                                                   const cuvsMultiGpuCommId* id,
                                                   int rank,
                                                   int n_ranks,
                                                   cuvsMultiGpuRankComm_t* comm);
/* Same around an existing ncclComm_t (not destroyed with the object). */
CUVS_EXPORT cuvsError_t cuvsMultiGpuRankCommAdopt(void* nccl_comm,
                                                  int rank,
                                                  int n_ranks,
                                                  cuvsMultiGpuRankComm_t* comm);
CUVS_EXPORT cuvsError_t cuvsMultiGpuRankCommDestroy(cuvsMultiGpuRankComm_t comm);
/* The list-sharded search of one batch, called by every rank with the same queries (device tensors):
 * probes of this rank's slice -> all-gather -> scan of the lists this rank holds -> all-gather of the
 * per-rank blocks -> merge.  Asynchronous on the handle's stream; every rank gets the whole result,
 * equal to cuvsIvfPqSearch on the unsharded index. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSearchRank(cuvsResources_t res,
                                                    cuvsMultiGpuRankComm_t comm,
                                                    cuvsIvfPqSearchParams_t search_params,
                                                    cuvsIvfPqIndex_t shard,
                                                    DLManagedTensor* queries,
                                                    DLManagedTensor* neighbors,
                                                    DLManagedTensor* distances);
/* Stage times of cuvsMultiGpuIvfPqSearchRank calls made while the handle's stage timing was on
 * (cuvsB200StatsEnable): stage_ms[5] = {probe slice, all-gather of the probes, scan of the owned lists,
 * all-gather of the result blocks, merge}, milliseconds summed over *batches calls.  Waits for the calls
 * it reports on. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuRankCommStats(cuvsMultiGpuRankComm_t comm,
                                                  double* stage_ms,
                                                  uint64_t* batches,
                                                  bool reset);
/* How cuvsMultiGpuIvfPqSearchRank exchanges and merges the per-rank results: 0 or 2 = one all-gather of
 * the whole blocks, every rank merges everything (the default); 1 = by slice: every rank receives and
 * merges only its own slice of the queries (send/receive pairs), the merged slices are all-gathered.
 * The result is the same either way; every rank of a communicator must use the same mode. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuRankCommSetMergeMode(cuvsMultiGpuRankComm_t comm, int mode);
/* The rule that deals lists to ranks: owners[l] for list sizes given on the host. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqListOwners(const uint32_t* list_sizes,
                                                    uint32_t n_lists,
                                                    int n_ranks,
                                                    int32_t* owners);

/* Stands in for cuvsMultiGpuIvfPqDistribute (c/include/cuvs/neighbors/mg_ivf_pq.h:266;
 * cpp/src/neighbors/mg/snmg.cuh:48-58) in a one-process-per-GPU deployment: loads a single-GPU
 * index file (format version 4) and keeps the payload of the lists owned by `rank` only (the rule of
 * cuvsMultiGpuIvfPqListOwners); the payload of the other lists is skipped in the file, never read. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqDistributeShard(cuvsResources_t res,
                                                         const char* filename,
                                                         int rank,
                                                         int n_ranks,
                                                         cuvsIvfPqIndex_t index);

/* Stands in for cuvsMultiGpuIvfPqDeserialize (c/include/cuvs/neighbors/mg_ivf_pq.h:245;
 * cpp/src/neighbors/mg/snmg.cuh:60-91) in a one-process-per-GPU deployment: reads the index of `rank`
 * out of a multi-GPU index file written by the reference's cuvsMultiGpuIvfPqSerialize (dtype string,
 * distribution mode, number of ranks, one index stream per rank; the streams of the other ranks are
 * stepped over).  n_ranks must equal the number stored in the file.  mode receives 0 (REPLICATED:
 * every rank holds the whole index) or 1 (SHARDED by rows); id_offset receives the number of rows
 * held by the ranks before this one -- what the reference adds to this rank's neighbour ids when it
 * merges (snmg.cuh:351-355) -- or 0 when replicated. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqDeserializeRank(cuvsResources_t res,
                                                         const char* filename,
                                                         int rank,
                                                         int n_ranks,
                                                         cuvsIvfPqIndex_t index,
                                                         int* mode,
                                                         int64_t* id_offset);

/* Counterpart of cuvsMultiGpuIvfPqSerialize (mg_ivf_pq.h:224; snmg.cuh:780-805) for indexes that live
 * in this process: writes `n_ranks` indexes as one multi-GPU index file of the reference's format.
 * dataset_dtype is the element type the reference records in the file's first four bytes. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSerializeRanks(cuvsResources_t res,
                                                        const char* filename,
                                                        int mode,
                                                        DLDataType dataset_dtype,
                                                        cuvsIvfPqIndex_t* indexes,
                                                        int n_ranks);

/* Stands in for the merge step of the sharded search (cpp/src/neighbors/mg/snmg.cuh:349-392 calling
 * knn_merge_parts, cpp/src/neighbors/detail/knn_merge_parts.cuh:24-170): part_distances f32 and
 * part_neighbors i64 are [n_parts, n_queries, k] device tensors; distances / neighbors are
 * [n_queries, k].  select_min = true keeps the smallest distances (L2, cosine), false the largest
 * (inner product).  Entries whose neighbour is INT64_MAX are ignored.  Each part must be row-major;
 * the parts themselves may lie apart (DLPack strides {s, k, 1} with s >= n_queries * k), e.g. as
 * views into one buffer that an all-gather filled with a block of ids and distances per rank. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqMergeParts(cuvsResources_t res,
                                                    DLManagedTensor* part_distances,
                                                    DLManagedTensor* part_neighbors,
                                                    DLManagedTensor* distances,
                                                    DLManagedTensor* neighbors,
                                                    bool select_min);

/* Probe selection alone (the coarse stage of cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:61-168), so
 * that ranks can share it: each rank selects the probes of a slice of the query batch, the slices are
 * all-gathered, and every rank then scans its own lists for the whole batch with
 * cuvsMultiGpuIvfPqSearchWithProbes.  queries f32/f16/i8/u8 [n, dim]; probes u32 [n, n_probes]
 * (device), ascending by (score, list id).  Asynchronous on the handle's stream. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSelectProbes(cuvsResources_t res,
                                                      cuvsIvfPqIndex_t index,
                                                      DLManagedTensor* queries,
                                                      DLManagedTensor* probes);

/* cuvsIvfPqSearch (c/include/cuvs/neighbors/ivf_pq.h:536) with the probes given instead of selected:
 * probes u32 [n_queries, n_probes] (device); search_params->n_probes must equal probes.shape[1]. */
CUVS_EXPORT cuvsError_t cuvsMultiGpuIvfPqSearchWithProbes(cuvsResources_t res,
                                                          cuvsIvfPqSearchParams_t search_params,
                                                          cuvsIvfPqIndex_t index,
                                                          DLManagedTensor* queries,
                                                          DLManagedTensor* probes,
                                                          DLManagedTensor* neighbors,
                                                          DLManagedTensor* distances);

#ifdef __cplusplus
}
#endif
#endif
