/*
 * IVF-PQ C interface of the B200-native engine.
 *
 * Drop-in for c/include/cuvs/neighbors/ivf_pq.h of the reference: same type names, struct layouts,
 * entry-point names, argument order and error convention, so that a language binding written
 * against the reference (Python/Cython, Go cgo, Rust bindgen, Java Panama) binds to this library
 * unchanged.  Each declaration cites the reference declaration it replaces.
 *
 * Tensors cross the interface as DLManagedTensor*.  Search inputs and outputs must be
 * device-accessible, row-major and compact (c/src/core/detail/interop.hpp:75-139).
 * Calls enqueue work on the stream of the resources handle and return; the caller synchronises with
 * cuvsStreamSync().
 */
#ifndef CUVS_B200_IVF_PQ_H_
#define CUVS_B200_IVF_PQ_H_

#include "cuvs_core_c_api.h"
#include "cuvs_distance.h"

#ifdef __cplusplus
extern "C" {
#endif

/* c/include/cuvs/neighbors/ivf_pq.h:28 */
enum cuvsIvfPqCodebookGen {
  CUVS_IVF_PQ_CODEBOOK_GEN_PER_SUBSPACE = 0,
  CUVS_IVF_PQ_CODEBOOK_GEN_PER_CLUSTER  = 1,
};

/* c/include/cuvs/neighbors/ivf_pq.h:37 */
enum cuvsIvfPqListLayout {
  CUVS_IVF_PQ_LIST_LAYOUT_FLAT        = 0,
  CUVS_IVF_PQ_LIST_LAYOUT_INTERLEAVED = 1,
};

/* c/include/cuvs/neighbors/ivf_pq.h:46 -- same fields, same order */
struct cuvsIvfPqIndexParams {
  cuvsDistanceType metric;
  float metric_arg;
  bool add_data_on_build;
  uint32_t n_lists;
  uint32_t kmeans_n_iters;
  double kmeans_trainset_fraction;
  uint32_t pq_bits; /* 4..8 */
  uint32_t pq_dim;  /* 0 = choose from dim */
  enum cuvsIvfPqCodebookGen codebook_kind;
  bool force_random_rotation;
  bool conservative_memory_allocation;
  uint32_t max_train_points_per_pq_code;
  enum cuvsIvfPqListLayout codes_layout;
};
/* c/include/cuvs/neighbors/ivf_pq.h:138 */
typedef struct cuvsIvfPqIndexParams* cuvsIvfPqIndexParams_t;

/* c/include/cuvs/neighbors/ivf_pq.h:146 (defaults: c/src/neighbors/ivf_pq.cpp:348-363) */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexParamsCreate(cuvsIvfPqIndexParams_t* index_params);
/* c/include/cuvs/neighbors/ivf_pq.h:154 */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexParamsDestroy(cuvsIvfPqIndexParams_t index_params);

/* c/include/cuvs/neighbors/ivf_pq.h:167 -- same fields, same order */
struct cuvsIvfPqSearchParams {
  uint32_t n_probes;
  cudaDataType_t lut_dtype;               /* CUDA_R_32F, CUDA_R_16F or CUDA_R_8U */
  cudaDataType_t internal_distance_dtype; /* CUDA_R_32F or CUDA_R_16F */
  cudaDataType_t coarse_search_dtype;     /* CUDA_R_32F */
  uint32_t max_internal_batch_size;
  double preferred_shmem_carveout;
};
/* c/include/cuvs/neighbors/ivf_pq.h:221 */
typedef struct cuvsIvfPqSearchParams* cuvsIvfPqSearchParams_t;

/* c/include/cuvs/neighbors/ivf_pq.h:229 (defaults: c/src/neighbors/ivf_pq.cpp:371-379) */
CUVS_EXPORT cuvsError_t cuvsIvfPqSearchParamsCreate(cuvsIvfPqSearchParams_t* params);
/* c/include/cuvs/neighbors/ivf_pq.h:237 */
CUVS_EXPORT cuvsError_t cuvsIvfPqSearchParamsDestroy(cuvsIvfPqSearchParams_t params);

/* c/include/cuvs/neighbors/ivf_pq.h:250 */
typedef struct {
  uintptr_t addr;
  DLDataType dtype;
} cuvsIvfPqIndex;
/* c/include/cuvs/neighbors/ivf_pq.h:255 */
typedef cuvsIvfPqIndex* cuvsIvfPqIndex_t;

/* c/include/cuvs/neighbors/ivf_pq.h:263 */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexCreate(cuvsIvfPqIndex_t* index);
/* c/include/cuvs/neighbors/ivf_pq.h:270 */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexDestroy(cuvsIvfPqIndex_t index);

/* c/include/cuvs/neighbors/ivf_pq.h:273-289 -- scalar getters */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetNLists(cuvsIvfPqIndex_t index, int64_t* n_lists);
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetDim(cuvsIvfPqIndex_t index, int64_t* dim);
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetSize(cuvsIvfPqIndex_t index, int64_t* size);
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetPqDim(cuvsIvfPqIndex_t index, int64_t* pq_dim);
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetPqBits(cuvsIvfPqIndex_t index, int64_t* pq_bits);
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetPqLen(cuvsIvfPqIndex_t index, int64_t* pq_len);

/* Tensor getters return non-owning device views; the `shape`/`strides` arrays are freed by the
 * tensor's deleter (c/src/core/detail/interop.hpp:143-174). */
/* c/include/cuvs/neighbors/ivf_pq.h:298 -- [n_lists, dim] view with row stride dim_ext */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetCenters(cuvsIvfPqIndex_t index, DLManagedTensor* centers);
/* c/include/cuvs/neighbors/ivf_pq.h:311 -- [n_lists, dim_ext] */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetCentersPadded(cuvsIvfPqIndex_t index,
                                                       DLManagedTensor* centers);
/* c/include/cuvs/neighbors/ivf_pq.h:323 -- [pq_dim | n_lists, pq_len, 1 << pq_bits] */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetPqCenters(cuvsIvfPqIndex_t index,
                                                   DLManagedTensor* pq_centers);
/* c/include/cuvs/neighbors/ivf_pq.h:333 -- [n_lists, rot_dim] */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetCentersRot(cuvsIvfPqIndex_t index,
                                                    DLManagedTensor* centers_rot);
/* c/include/cuvs/neighbors/ivf_pq.h:344 -- [rot_dim, dim] */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetRotationMatrix(cuvsIvfPqIndex_t index,
                                                        DLManagedTensor* rotation_matrix);
/* c/include/cuvs/neighbors/ivf_pq.h:354 -- u32 [n_lists] */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetListSizes(cuvsIvfPqIndex_t index,
                                                   DLManagedTensor* list_sizes);
/* c/include/cuvs/neighbors/ivf_pq.h:373 -- bit-packed codes u8 [n_rows, ceil(pq_dim*pq_bits/8)] of
 * rows [offset, offset + n_rows) of one list */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexUnpackContiguousListData(cuvsResources_t res,
                                                               cuvsIvfPqIndex_t index,
                                                               DLManagedTensor* out_codes,
                                                               uint32_t label,
                                                               uint32_t offset);
/* c/include/cuvs/neighbors/ivf_pq.h:388 -- i64 [list size] source ids of one list */
CUVS_EXPORT cuvsError_t cuvsIvfPqIndexGetListIndices(cuvsIvfPqIndex_t index,
                                                     uint32_t label,
                                                     DLManagedTensor* out_labels);

/* c/include/cuvs/neighbors/ivf_pq.h:442 -- dataset f32/f16/i8/u8 [n_rows, dim], host or device */
CUVS_EXPORT cuvsError_t cuvsIvfPqBuild(cuvsResources_t res,
                                       cuvsIvfPqIndexParams_t params,
                                       DLManagedTensor* dataset,
                                       cuvsIvfPqIndex_t index);
/* c/include/cuvs/neighbors/ivf_pq.h:476 -- index over given centers/codebooks, no vectors yet */
CUVS_EXPORT cuvsError_t cuvsIvfPqBuildPrecomputed(cuvsResources_t res,
                                                  cuvsIvfPqIndexParams_t params,
                                                  uint32_t dim,
                                                  DLManagedTensor* pq_centers,
                                                  DLManagedTensor* centers,
                                                  DLManagedTensor* centers_rot,
                                                  DLManagedTensor* rotation_matrix,
                                                  cuvsIvfPqIndex_t index);
/* c/include/cuvs/neighbors/ivf_pq.h:536 -- THE HOT CALL (c/src/neighbors/ivf_pq.cpp:303-345):
 * queries f32/f16/i8/u8 [n_q, dim]; neighbors i64 [n_q, k]; distances f32 [n_q, k]; k is taken
 * from neighbors.shape[1]. */
CUVS_EXPORT cuvsError_t cuvsIvfPqSearch(cuvsResources_t res,
                                        cuvsIvfPqSearchParams_t search_params,
                                        cuvsIvfPqIndex_t index,
                                        DLManagedTensor* queries,
                                        DLManagedTensor* neighbors,
                                        DLManagedTensor* distances);
/* c/include/cuvs/neighbors/common.h:25-47 -- filter handle shared by the reference's search calls */
enum cuvsFilterType { NO_FILTER = 0, BITSET = 1, BITMAP = 2 };
typedef struct {
  uintptr_t addr; /* BITSET: DLManagedTensor* of uint32 words on the device, bit i = source id i allowed */
  enum cuvsFilterType type;
} cuvsFilter;

/* The reference's C entry takes no filter; its C++ search does (cpp/include/cuvs/neighbors/ivf_pq.hpp,
 * overload with cuvs::neighbors::filtering::base_filter; device side
 * cpp/src/neighbors/sample_filter.cuh:162-176).  This entry exposes that overload with the
 * cuvsFilter convention the reference uses for its other indexes: NO_FILTER or BITSET. */
CUVS_EXPORT cuvsError_t cuvsIvfPqSearchWithFilter(cuvsResources_t res,
                                                  cuvsIvfPqSearchParams_t search_params,
                                                  cuvsIvfPqIndex_t index,
                                                  DLManagedTensor* queries,
                                                  DLManagedTensor* neighbors,
                                                  DLManagedTensor* distances,
                                                  cuvsFilter filter);

/* c/include/cuvs/neighbors/ivf_pq.h:570 -- writes the reference's file format, version 4 */
CUVS_EXPORT cuvsError_t cuvsIvfPqSerialize(cuvsResources_t res,
                                           const char* filename,
                                           cuvsIvfPqIndex_t index);
/* c/include/cuvs/neighbors/ivf_pq.h:581 -- loads files written by the reference unchanged */
CUVS_EXPORT cuvsError_t cuvsIvfPqDeserialize(cuvsResources_t res,
                                             const char* filename,
                                             cuvsIvfPqIndex_t index);
/* c/include/cuvs/neighbors/ivf_pq.h:599 -- new_indices may be NULL on an empty index */
CUVS_EXPORT cuvsError_t cuvsIvfPqExtend(cuvsResources_t res,
                                        DLManagedTensor* new_vectors,
                                        DLManagedTensor* new_indices,
                                        cuvsIvfPqIndex_t index);
/* c/include/cuvs/neighbors/ivf_pq.h:621 -- labels u32 [n] and bit-packed codes u8 [n, ceil(pq_dim*pq_bits/8)] */
CUVS_EXPORT cuvsError_t cuvsIvfPqTransform(cuvsResources_t res,
                                           cuvsIvfPqIndex_t index,
                                           DLManagedTensor* input_dataset,
                                           DLManagedTensor* output_labels,
                                           DLManagedTensor* output_dataset);

/* No counterpart in the reference.  Nearest-list labels (u32 [n]) of up to 65,536 vectors
 * (f32/f16/i8/u8 [n, dim], device-accessible) computed WITHOUT any allocation: for callers that may
 * not call cudaMalloc while serving (all device memory pre-claimed by a framework allocator, a
 * thread that must avoid cudaMalloc's driver lock and implicit sync, a sandboxed plug-in).  The
 * kernel's scratch is a fixed 512 KiB __device__ array inside the library, shared by all calls:
 * larger batches are rejected, calls must not overlap on the GPU, and the first call on a device
 * (which resolves the array's address) should precede any stream capture.  Labels equal those of
 * cuvsIvfPqTransform.  CosineExpanded indexes are not supported. */
CUVS_EXPORT cuvsError_t cuvsIvfPqPredictNoAlloc(cuvsResources_t res,
                                                cuvsIvfPqIndex_t index,
                                                DLManagedTensor* vectors,
                                                DLManagedTensor* labels);

#ifdef __cplusplus
}
#endif
#endif
