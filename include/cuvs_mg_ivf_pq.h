/*
 * List-sharded multi-GPU IVF-PQ, one process per GPU.
 *
 * The reference's multi-GPU layer (c/include/cuvs/neighbors/mg_ivf_pq.h, cpp/src/neighbors/mg/snmg.cuh)
 * drives all GPUs from one process with one OpenMP thread per rank.  Here every rank is its own
 * process holding an ordinary cuvsIvfPqIndex_t that contains the global coarse model and the
 * inverted lists this rank owns (list l belongs to rank l % n_ranks; the others are empty).  Every
 * rank runs the ordinary cuvsIvfPqSearch on the whole query batch -- probe selection is global and
 * identical everywhere, a rank only scans the probes it owns -- and the per-rank top-k lists, which
 * already carry global ids, are exchanged by the host framework (NCCL all-gather) and merged with
 * cuvsMultiGpuIvfPqMergeParts.  The union of the ranks' candidates is exactly the single-GPU
 * candidate set, so the merged result equals the single-GPU search.
 */
#ifndef CUVS_B200_MG_IVF_PQ_H_
#define CUVS_B200_MG_IVF_PQ_H_

#include "cuvs_ivf_pq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Stands in for cuvsMultiGpuIvfPqDistribute (c/include/cuvs/neighbors/mg_ivf_pq.h:266;
 * cpp/src/neighbors/mg/snmg.cuh:48-58) in a one-process-per-GPU deployment: loads a single-GPU
 * index file (format version 4) and keeps the payload of the lists owned by `rank` only; the
 * payload of the other lists is skipped in the file, never read. */
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
