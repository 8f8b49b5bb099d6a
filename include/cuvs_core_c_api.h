/*
 * Core handles of the C interface: error convention, resources (device, stream, workspace).
 * Replaces the subset of c/include/cuvs/core/c_api.h of the reference that callers of the IVF-PQ
 * path use; every entry point cites the declaration it stands in for.
 *
 * Error convention (c/src/core/exceptions.hpp:17-33): every entry point returns CUVS_SUCCESS or
 * CUVS_ERROR; on error the message is kept in thread-local storage and read with
 * cuvsGetLastErrorText(); a successful call clears it.  No exception crosses this interface.
 */
#ifndef CUVS_B200_CORE_C_API_H_
#define CUVS_B200_CORE_C_API_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include <dlpack/dlpack.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CUVS_EXPORT
#define CUVS_EXPORT __attribute__((visibility("default")))
#endif

/* The reference header pulls cudaStream_t and cudaDataType_t from <cuda_runtime.h>; callers that do
 * not include the CUDA headers get layout-compatible declarations here. */
#if !defined(__CUDA_RUNTIME_H__) && !defined(__DRIVER_TYPES_H__)
typedef struct CUstream_st* cudaStream_t;
#endif
#if !defined(__LIBRARY_TYPES_H__) && !defined(CUDART_VERSION)
typedef enum cudaDataType_t {
  CUDA_R_32F = 0,
  CUDA_R_16F = 2,
  CUDA_R_8I  = 3,
  CUDA_R_8U  = 8
} cudaDataType_t;
#endif

/* c/include/cuvs/core/c_api.h:27 */
typedef enum { CUVS_ERROR = 0, CUVS_SUCCESS = 1 } cuvsError_t;

/* c/include/cuvs/core/c_api.h:32 */
CUVS_EXPORT const char* cuvsGetLastErrorText(void);
/* c/include/cuvs/core/c_api.h:38 */
CUVS_EXPORT void cuvsSetLastErrorText(const char* error);

/* c/include/cuvs/core/c_api.h:80 -- opaque handle: device id, stream, grow-only workspace */
typedef uintptr_t cuvsResources_t;

/* c/include/cuvs/core/c_api.h:88 */
CUVS_EXPORT cuvsError_t cuvsResourcesCreate(cuvsResources_t* res);
/* c/include/cuvs/core/c_api.h:123 */
CUVS_EXPORT cuvsError_t cuvsResourcesDestroy(cuvsResources_t res);
/* c/include/cuvs/core/c_api.h:133 */
CUVS_EXPORT cuvsError_t cuvsStreamSet(cuvsResources_t res, cudaStream_t stream);
/* c/include/cuvs/core/c_api.h:142 */
CUVS_EXPORT cuvsError_t cuvsStreamGet(cuvsResources_t res, cudaStream_t* stream);
/* c/include/cuvs/core/c_api.h:150 */
CUVS_EXPORT cuvsError_t cuvsStreamSync(cuvsResources_t res);
/* c/include/cuvs/core/c_api.h:159 */
CUVS_EXPORT cuvsError_t cuvsDeviceIdGet(cuvsResources_t res, int* device_id);
/* c/include/cuvs/core/c_api.h:175 -- pre-sizes the workspace so that search allocates nothing */
CUVS_EXPORT cuvsError_t cuvsResourcesSetWorkspacePool(cuvsResources_t res, size_t initial_size_bytes);
/* c/include/cuvs/core/c_api.h:185 -- the multi-GPU handle (raft::device_resources_snmg in the
 * reference): the root rank's handle plus one handle, stream and NCCL communicator per visible device.
 * It is accepted wherever a cuvsResources_t is (it then acts as the root rank's handle). */
CUVS_EXPORT cuvsError_t cuvsMultiGpuResourcesCreate(cuvsResources_t* res);
/* c/include/cuvs/core/c_api.h:195 -- device_ids: int32 host tensor [n] */
CUVS_EXPORT cuvsError_t cuvsMultiGpuResourcesCreateWithDeviceIds(cuvsResources_t* res,
                                                                 DLManagedTensor* device_ids);
/* c/include/cuvs/core/c_api.h:204 */
CUVS_EXPORT cuvsError_t cuvsMultiGpuResourcesDestroy(cuvsResources_t res);
/* c/include/cuvs/core/c_api.h:213 -- this engine keeps one grow-only workspace per rank instead of a
 * pool: the call reserves that share of each device's free memory for it */
CUVS_EXPORT cuvsError_t cuvsMultiGpuResourcesSetMemoryPool(cuvsResources_t res, int percent_of_free_memory);
/* c/include/cuvs/core/c_api.h:230 -- plain cudaMalloc on the handle's device */
CUVS_EXPORT cuvsError_t cuvsRMMAlloc(cuvsResources_t res, void** ptr, size_t bytes);
/* c/include/cuvs/core/c_api.h:240 */
CUVS_EXPORT cuvsError_t cuvsRMMFree(cuvsResources_t res, void* ptr, size_t bytes);
/* c/include/cuvs/core/c_api.h:301 -- reports the version of the interface this library mirrors */
CUVS_EXPORT cuvsError_t cuvsVersionGet(uint16_t* major, uint16_t* minor, uint16_t* patch);

#ifdef __cplusplus
}
#endif
#endif
