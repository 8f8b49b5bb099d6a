/*
 * Dynamic batching in front of an IVF-PQ index: many host threads submit small searches, the library
 * gathers them into batches for the upstream index.
 *
 * The reference offers this as C++ only (cpp/include/cuvs/neighbors/dynamic_batching.hpp:
 * index_params :39-81, search_params :83-92, index :140-190, search :228 ff.); it has no C
 * interface there.  These entry points expose the same parameters and contract over the C ABI:
 * k is fixed at construction, requests of any size may come from any number of host threads (one
 * resources handle per thread), and every request is answered exactly as a direct cuvsIvfPqSearch
 * with the upstream parameters would answer it.
 */
#ifndef CUVS_B200_DYNAMIC_BATCHING_H_
#define CUVS_B200_DYNAMIC_BATCHING_H_

#include "cuvs_ivf_pq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* dynamic_batching.hpp:39-81 */
struct cuvsDynamicBatchingIndexParams {
  int64_t k;                  /* neighbours per query, fixed for the life of the index */
  int64_t max_batch_size;     /* largest batch handed to the upstream index (reference default 100) */
  size_t n_queues;            /* independent batches in flight, each with its own stream (default 3) */
  bool conservative_dispatch; /* accepted; a batch is always closed on the host before it is searched */
};
typedef struct cuvsDynamicBatchingIndexParams* cuvsDynamicBatchingIndexParams_t;

typedef struct {
  uintptr_t addr;
} cuvsDynamicBatchingIndex;
typedef cuvsDynamicBatchingIndex* cuvsDynamicBatchingIndex_t;

CUVS_EXPORT cuvsError_t cuvsDynamicBatchingIndexParamsCreate(cuvsDynamicBatchingIndexParams_t* params);
CUVS_EXPORT cuvsError_t cuvsDynamicBatchingIndexParamsDestroy(cuvsDynamicBatchingIndexParams_t params);

/* dynamic_batching.hpp:140-190 -- wraps `upstream`, which must outlive the wrapper; the upstream
 * search parameters are copied. */
CUVS_EXPORT cuvsError_t cuvsDynamicBatchingIndexCreate(cuvsResources_t res,
                                                       cuvsDynamicBatchingIndexParams_t params,
                                                       cuvsIvfPqIndex_t upstream,
                                                       cuvsIvfPqSearchParams_t upstream_params,
                                                       cuvsDynamicBatchingIndex_t* index);
CUVS_EXPORT cuvsError_t cuvsDynamicBatchingIndexDestroy(cuvsDynamicBatchingIndex_t index);

/* dynamic_batching.hpp:228 ff. -- queries f32 [n, dim], neighbors i64 [n, k], distances f32 [n, k],
 * device memory.  Blocks the calling thread until the request's batch has been dispatched (at most
 * dispatch_timeout_ms after the batch's first request, reference default 1.0); the result copies are
 * ordered on the stream of `res`. */
CUVS_EXPORT cuvsError_t cuvsDynamicBatchingSearch(cuvsResources_t res,
                                                  cuvsDynamicBatchingIndex_t index,
                                                  double dispatch_timeout_ms,
                                                  DLManagedTensor* queries,
                                                  DLManagedTensor* neighbors,
                                                  DLManagedTensor* distances);

/* Counters for tests: upstream searches launched and rows they carried. */
CUVS_EXPORT cuvsError_t cuvsDynamicBatchingStats(cuvsDynamicBatchingIndex_t index,
                                                 uint64_t* n_batches,
                                                 uint64_t* n_rows);

/* Test hook, host side only (no counterpart in the reference): the next upstream search of this index
 * fails before it runs.  Every request gathered into that batch returns CUVS_ERROR with the reason; the
 * queue stays usable. */
CUVS_EXPORT cuvsError_t cuvsDynamicBatchingFailNext(cuvsDynamicBatchingIndex_t index);

#ifdef __cplusplus
}
#endif
#endif
