/*
 * Refinement of approximate neighbours with exact distances.
 * Replaces: c/include/cuvs/neighbors/refine.h:60 (cuvsRefine) of the reference.
 */
#ifndef CUVS_B200_REFINE_H_
#define CUVS_B200_REFINE_H_

#include "cuvs_core_c_api.h"
#include "cuvs_distance.h"

#ifdef __cplusplus
extern "C" {
#endif

/* c/include/cuvs/neighbors/refine.h:60 -- dataset and queries f32/f16/i8/u8 (same type),
 * candidates i64 [n_queries, n_candidates], indices i64 [n_queries, k], distances f32
 * [n_queries, k], all device-accessible; k = indices.shape[1] <= n_candidates.  Returns the k
 * candidates with the best exact distance, best first. */
CUVS_EXPORT cuvsError_t cuvsRefine(cuvsResources_t res,
                                   DLManagedTensor* dataset,
                                   DLManagedTensor* queries,
                                   DLManagedTensor* candidates,
                                   cuvsDistanceType metric,
                                   DLManagedTensor* indices,
                                   DLManagedTensor* distances);

#ifdef __cplusplus
}
#endif
#endif
