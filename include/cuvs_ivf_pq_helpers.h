/*
 * Single-list helpers of the IVF-PQ index: read, write, decode, extend and erase the rows of one
 * list (cluster) without going through classification.
 *
 * The reference offers these as C++ only (cpp/include/cuvs/neighbors/ivf_pq.hpp, namespace
 * cuvs::neighbors::ivf_pq::helpers: codepacker::unpack_list_data :2818 and :2854,
 * codepacker::pack_list_data :2739, codepacker::pack_contiguous_list_data :2782,
 * codepacker::reconstruct_list_data :2932-3002, codepacker::extend_list_with_codes :3035,
 * codepacker::extend_list_with_contiguous_codes :3074, codepacker::extend_list :3109-3123,
 * erase_list :3144, reset_index :3166); its C interface has only
 * cuvsIvfPqIndexUnpackContiguousListData.  These entry points expose the same operations, with the
 * same argument meaning, over the C ABI.  All tensors are device tensors.
 */
#ifndef CUVS_B200_IVF_PQ_HELPERS_H_
#define CUVS_B200_IVF_PQ_HELPERS_H_

#include "cuvs_ivf_pq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* out_codes u8 [n_rows, pq_dim], one code per byte, of list rows [offset, offset + n_rows); with
 * `in_cluster_indices` (u32 [n_rows], may be NULL) the rows at those positions instead. */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersUnpackListData(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                       DLManagedTensor* out_codes, uint32_t label,
                                                       uint32_t offset,
                                                       DLManagedTensor* in_cluster_indices);

/* Overwrite list rows [offset, offset + n_rows): codes u8 [n_rows, pq_dim], one code per byte.
 * Nothing is allocated; the rows must exist. */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersPackListData(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                     DLManagedTensor* codes, uint32_t label,
                                                     uint32_t offset);

/* Same with bit-packed rows: codes u8 [n_rows, ceil(pq_dim * pq_bits / 8)]. */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersPackContiguousListData(cuvsResources_t res,
                                                               cuvsIvfPqIndex_t index,
                                                               DLManagedTensor* codes, uint32_t label,
                                                               uint32_t offset);

/* Decode list rows into the input space: out_vectors [n_rows, dim] of f32, f16, i8 or u8.  Rows
 * [offset, offset + n_rows), or those named by `in_cluster_indices` (u32 [n_rows], may be NULL). */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersReconstructListData(cuvsResources_t res,
                                                            cuvsIvfPqIndex_t index,
                                                            DLManagedTensor* out_vectors,
                                                            uint32_t label, uint32_t offset,
                                                            DLManagedTensor* in_cluster_indices);

/* Append rows to one list.  new_codes u8 [n_rows, pq_dim] (one code per byte), or
 * [n_rows, ceil(pq_dim * pq_bits / 8)] when `contiguous`; new_indices i64 [n_rows]. */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersExtendListWithCodes(cuvsResources_t res,
                                                            cuvsIvfPqIndex_t index,
                                                            DLManagedTensor* new_codes,
                                                            DLManagedTensor* new_indices,
                                                            uint32_t label, bool contiguous);

/* Encode new_vectors [n_rows, dim] (f32, f16, i8 or u8) against list `label` and append them. */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersExtendList(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                   DLManagedTensor* new_vectors,
                                                   DLManagedTensor* new_indices, uint32_t label);

/* Remove every row of one list / of all lists; the trained model stays. */
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersEraseList(cuvsResources_t res, cuvsIvfPqIndex_t index,
                                                  uint32_t label);
CUVS_EXPORT cuvsError_t cuvsIvfPqHelpersResetIndex(cuvsResources_t res, cuvsIvfPqIndex_t index);

#ifdef __cplusplus
}
#endif
#endif
