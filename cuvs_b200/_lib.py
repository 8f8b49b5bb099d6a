"""ctypes binding of ``libcuvs_b200.so`` -- the only way Python reaches the engine.

The structures below restate the C declarations of ``include/cuvs_ivf_pq.h`` and
``include/dlpack/dlpack.h``.  There is no fallback: if the library is missing or cannot be loaded,
importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcuvs_b200.so")

CUVS_ERROR, CUVS_SUCCESS = 0, 1

# DLPack ------------------------------------------------------------------------------------------
kDLCPU, kDLCUDA, kDLCUDAHost, kDLCUDAManaged = 1, 2, 3, 13
kDLInt, kDLUInt, kDLFloat = 0, 1, 2


class DLDevice(C.Structure):
    _fields_ = [("device_type", C.c_int), ("device_id", C.c_int32)]


class DLDataType(C.Structure):
    _fields_ = [("code", C.c_uint8), ("bits", C.c_uint8), ("lanes", C.c_uint16)]


class DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device", DLDevice), ("ndim", C.c_int32),
                ("dtype", DLDataType), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("byte_offset", C.c_uint64)]


class DLManagedTensor(C.Structure):
    pass


DLManagedTensor._fields_ = [("dl_tensor", DLTensor), ("manager_ctx", C.c_void_p),
                            ("deleter", C.CFUNCTYPE(None, C.POINTER(DLManagedTensor)))]


# params ------------------------------------------------------------------------------------------
class IndexParamsStruct(C.Structure):
    _fields_ = [("metric", C.c_int), ("metric_arg", C.c_float), ("add_data_on_build", C.c_bool),
                ("n_lists", C.c_uint32), ("kmeans_n_iters", C.c_uint32),
                ("kmeans_trainset_fraction", C.c_double), ("pq_bits", C.c_uint32),
                ("pq_dim", C.c_uint32), ("codebook_kind", C.c_int),
                ("force_random_rotation", C.c_bool), ("conservative_memory_allocation", C.c_bool),
                ("max_train_points_per_pq_code", C.c_uint32), ("codes_layout", C.c_int)]


class SearchParamsStruct(C.Structure):
    _fields_ = [("n_probes", C.c_uint32), ("lut_dtype", C.c_int),
                ("internal_distance_dtype", C.c_int), ("coarse_search_dtype", C.c_int),
                ("max_internal_batch_size", C.c_uint32), ("preferred_shmem_carveout", C.c_double)]


class FilterStruct(C.Structure):
    _fields_ = [("addr", C.c_size_t), ("type", C.c_int)]


class DynamicBatchingIndexParamsStruct(C.Structure):
    _fields_ = [("k", C.c_int64), ("max_batch_size", C.c_int64), ("n_queues", C.c_size_t),
                ("conservative_dispatch", C.c_bool)]


class DynamicBatchingIndexStruct(C.Structure):
    _fields_ = [("addr", C.c_size_t)]


class IndexStruct(C.Structure):
    _fields_ = [("addr", C.c_size_t), ("dtype", DLDataType)]


class MgIndexParamsStruct(C.Structure):
    _fields_ = [("base_params", C.POINTER(IndexParamsStruct)), ("mode", C.c_int)]


class MgSearchParamsStruct(C.Structure):
    _fields_ = [("base_params", C.POINTER(SearchParamsStruct)), ("search_mode", C.c_int),
                ("merge_mode", C.c_int), ("n_rows_per_batch", C.c_int64)]


class CommId(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * 128)]


class SearchStats(C.Structure):
    _fields_ = [("prep_ms", C.c_double), ("coarse_ms", C.c_double), ("sort_ms", C.c_double),
                ("scan_ms", C.c_double), ("merge_ms", C.c_double), ("batches", C.c_uint64),
                ("pairs", C.c_uint64), ("scan_groups", C.c_uint64), ("unique_groups", C.c_uint64),
                ("launches", C.c_uint64)]


_P = C.POINTER

# every entry point declared in include/*.h: name -> argument types
SIGNATURES = {
    "cuvsResourcesCreate": [_P(C.c_size_t)],
    "cuvsResourcesDestroy": [C.c_size_t],
    "cuvsStreamSet": [C.c_size_t, C.c_void_p],
    "cuvsStreamGet": [C.c_size_t, _P(C.c_void_p)],
    "cuvsStreamSync": [C.c_size_t],
    "cuvsDeviceIdGet": [C.c_size_t, _P(C.c_int)],
    "cuvsResourcesSetWorkspacePool": [C.c_size_t, C.c_size_t],
    "cuvsRMMAlloc": [C.c_size_t, _P(C.c_void_p), C.c_size_t],
    "cuvsRMMFree": [C.c_size_t, C.c_void_p, C.c_size_t],
    "cuvsVersionGet": [_P(C.c_uint16), _P(C.c_uint16), _P(C.c_uint16)],
    "cuvsIvfPqIndexParamsCreate": [_P(_P(IndexParamsStruct))],
    "cuvsIvfPqIndexParamsDestroy": [_P(IndexParamsStruct)],
    "cuvsIvfPqSearchParamsCreate": [_P(_P(SearchParamsStruct))],
    "cuvsIvfPqSearchParamsDestroy": [_P(SearchParamsStruct)],
    "cuvsIvfPqIndexCreate": [_P(_P(IndexStruct))],
    "cuvsIvfPqIndexDestroy": [_P(IndexStruct)],
    "cuvsIvfPqIndexGetNLists": [_P(IndexStruct), _P(C.c_int64)],
    "cuvsIvfPqIndexGetDim": [_P(IndexStruct), _P(C.c_int64)],
    "cuvsIvfPqIndexGetSize": [_P(IndexStruct), _P(C.c_int64)],
    "cuvsIvfPqIndexGetPqDim": [_P(IndexStruct), _P(C.c_int64)],
    "cuvsIvfPqIndexGetPqBits": [_P(IndexStruct), _P(C.c_int64)],
    "cuvsIvfPqIndexGetPqLen": [_P(IndexStruct), _P(C.c_int64)],
    "cuvsIvfPqIndexGetCenters": [_P(IndexStruct), _P(DLManagedTensor)],
    "cuvsIvfPqIndexGetCentersPadded": [_P(IndexStruct), _P(DLManagedTensor)],
    "cuvsIvfPqIndexGetPqCenters": [_P(IndexStruct), _P(DLManagedTensor)],
    "cuvsIvfPqIndexGetCentersRot": [_P(IndexStruct), _P(DLManagedTensor)],
    "cuvsIvfPqIndexGetRotationMatrix": [_P(IndexStruct), _P(DLManagedTensor)],
    "cuvsIvfPqIndexGetListSizes": [_P(IndexStruct), _P(DLManagedTensor)],
    "cuvsIvfPqIndexUnpackContiguousListData": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor),
                                               C.c_uint32, C.c_uint32],
    "cuvsIvfPqIndexGetListIndices": [_P(IndexStruct), C.c_uint32, _P(DLManagedTensor)],
    "cuvsIvfPqBuild": [C.c_size_t, _P(IndexParamsStruct), _P(DLManagedTensor), _P(IndexStruct)],
    "cuvsIvfPqBuildPrecomputed": [C.c_size_t, _P(IndexParamsStruct), C.c_uint32,
                                  _P(DLManagedTensor), _P(DLManagedTensor), _P(DLManagedTensor),
                                  _P(DLManagedTensor), _P(IndexStruct)],
    "cuvsIvfPqSearch": [C.c_size_t, _P(SearchParamsStruct), _P(IndexStruct), _P(DLManagedTensor),
                        _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsIvfPqSearchWithFilter": [C.c_size_t, _P(SearchParamsStruct), _P(IndexStruct),
                                  _P(DLManagedTensor), _P(DLManagedTensor), _P(DLManagedTensor),
                                  FilterStruct],
    "cuvsIvfPqSerialize": [C.c_size_t, C.c_char_p, _P(IndexStruct)],
    "cuvsIvfPqDeserialize": [C.c_size_t, C.c_char_p, _P(IndexStruct)],
    "cuvsIvfPqExtend": [C.c_size_t, _P(DLManagedTensor), _P(DLManagedTensor), _P(IndexStruct)],
    "cuvsIvfPqHelpersUnpackListData": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor), C.c_uint32,
                                       C.c_uint32, _P(DLManagedTensor)],
    "cuvsIvfPqHelpersPackListData": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor), C.c_uint32,
                                     C.c_uint32],
    "cuvsIvfPqHelpersPackContiguousListData": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor),
                                               C.c_uint32, C.c_uint32],
    "cuvsIvfPqHelpersReconstructListData": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor),
                                            C.c_uint32, C.c_uint32, _P(DLManagedTensor)],
    "cuvsIvfPqHelpersExtendListWithCodes": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor),
                                            _P(DLManagedTensor), C.c_uint32, C.c_bool],
    "cuvsIvfPqHelpersExtendList": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor),
                                   _P(DLManagedTensor), C.c_uint32],
    "cuvsIvfPqHelpersEraseList": [C.c_size_t, _P(IndexStruct), C.c_uint32],
    "cuvsIvfPqHelpersResetIndex": [C.c_size_t, _P(IndexStruct)],
    "cuvsMultiGpuIvfPqDistributeShard": [C.c_size_t, C.c_char_p, C.c_int, C.c_int, _P(IndexStruct)],
    "cuvsMultiGpuIvfPqMergeParts": [C.c_size_t, _P(DLManagedTensor), _P(DLManagedTensor),
                                    _P(DLManagedTensor), _P(DLManagedTensor), C.c_bool],
    "cuvsMultiGpuIvfPqSelectProbes": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsMultiGpuIvfPqSearchWithProbes": [C.c_size_t, _P(SearchParamsStruct), _P(IndexStruct),
                                          _P(DLManagedTensor), _P(DLManagedTensor), _P(DLManagedTensor),
                                          _P(DLManagedTensor)],
    "cuvsB200CoarseSelect": [C.c_size_t, C.c_void_p, _P(DLManagedTensor), _P(DLManagedTensor),
                             _P(DLManagedTensor), C.c_int, _P(C.c_uint32)],
    "cuvsB200SetCoarseMode": [C.c_int],
    "cuvsB200SetScanCodebookHome": [C.c_int],
    "cuvsB200CoarseTimeouts": [C.c_size_t, _P(C.c_uint64)],
    "cuvsB200SetCoarseWaitTest": [C.c_uint32, C.c_uint32],
    "cuvsB200StatsEnable": [C.c_size_t, C.c_bool],
    "cuvsB200StatsGet": [C.c_size_t, _P(SearchStats), C.c_bool],
    "cuvsIvfPqPredictNoAlloc": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsDynamicBatchingIndexParamsCreate": [_P(_P(DynamicBatchingIndexParamsStruct))],
    "cuvsDynamicBatchingIndexParamsDestroy": [_P(DynamicBatchingIndexParamsStruct)],
    "cuvsDynamicBatchingIndexCreate": [C.c_size_t, _P(DynamicBatchingIndexParamsStruct), _P(IndexStruct),
                                       _P(SearchParamsStruct), _P(_P(DynamicBatchingIndexStruct))],
    "cuvsDynamicBatchingIndexDestroy": [_P(DynamicBatchingIndexStruct)],
    "cuvsDynamicBatchingSearch": [C.c_size_t, _P(DynamicBatchingIndexStruct), C.c_double,
                                  _P(DLManagedTensor), _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsDynamicBatchingFailNext": [_P(DynamicBatchingIndexStruct)],
    "cuvsDynamicBatchingStats": [_P(DynamicBatchingIndexStruct), _P(C.c_uint64), _P(C.c_uint64)],
    "cuvsMultiGpuIvfPqDeserializeRank": [C.c_size_t, C.c_char_p, C.c_int, C.c_int, _P(IndexStruct), _P(C.c_int),
                                         _P(C.c_int64)],
    "cuvsMultiGpuIvfPqSerializeRanks": [C.c_size_t, C.c_char_p, C.c_int, DLDataType, _P(_P(IndexStruct)),
                                        C.c_int],
    "cuvsRefine": [C.c_size_t, _P(DLManagedTensor), _P(DLManagedTensor), _P(DLManagedTensor), C.c_int,
                   _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsIvfPqTransform": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor), _P(DLManagedTensor),
                           _P(DLManagedTensor)],
    "cuvsMultiGpuResourcesCreate": [_P(C.c_size_t)],
    "cuvsMultiGpuResourcesCreateWithDeviceIds": [_P(C.c_size_t), _P(DLManagedTensor)],
    "cuvsMultiGpuResourcesDestroy": [C.c_size_t],
    "cuvsMultiGpuResourcesSetMemoryPool": [C.c_size_t, C.c_int],
    "cuvsMultiGpuIvfPqIndexParamsCreate": [_P(_P(MgIndexParamsStruct))],
    "cuvsMultiGpuIvfPqIndexParamsDestroy": [_P(MgIndexParamsStruct)],
    "cuvsMultiGpuIvfPqSearchParamsCreate": [_P(_P(MgSearchParamsStruct))],
    "cuvsMultiGpuIvfPqSearchParamsDestroy": [_P(MgSearchParamsStruct)],
    "cuvsMultiGpuIvfPqIndexCreate": [_P(_P(IndexStruct))],
    "cuvsMultiGpuIvfPqIndexDestroy": [_P(IndexStruct)],
    "cuvsMultiGpuIvfPqBuild": [C.c_size_t, _P(MgIndexParamsStruct), _P(DLManagedTensor), _P(IndexStruct)],
    "cuvsMultiGpuIvfPqSearch": [C.c_size_t, _P(MgSearchParamsStruct), _P(IndexStruct), _P(DLManagedTensor),
                                _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsMultiGpuIvfPqExtend": [C.c_size_t, _P(IndexStruct), _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsMultiGpuIvfPqSerialize": [C.c_size_t, _P(IndexStruct), C.c_char_p],
    "cuvsMultiGpuIvfPqDeserialize": [C.c_size_t, C.c_char_p, _P(IndexStruct)],
    "cuvsMultiGpuIvfPqDistribute": [C.c_size_t, C.c_char_p, _P(IndexStruct)],
    "cuvsMultiGpuIvfPqDistributeByList": [C.c_size_t, C.c_char_p, _P(IndexStruct)],
    "cuvsMultiGpuCommIdCreate": [_P(CommId)],
    "cuvsMultiGpuRankCommCreate": [C.c_size_t, _P(CommId), C.c_int, C.c_int, _P(C.c_void_p)],
    "cuvsMultiGpuRankCommAdopt": [C.c_void_p, C.c_int, C.c_int, _P(C.c_void_p)],
    "cuvsMultiGpuRankCommDestroy": [C.c_void_p],
    "cuvsMultiGpuIvfPqSearchRank": [C.c_size_t, C.c_void_p, _P(SearchParamsStruct), _P(IndexStruct),
                                    _P(DLManagedTensor), _P(DLManagedTensor), _P(DLManagedTensor)],
    "cuvsMultiGpuRankCommStats": [C.c_void_p, _P(C.c_double), _P(C.c_uint64), C.c_bool],
    "cuvsMultiGpuRankCommSetMergeMode": [C.c_void_p, C.c_int],
    "cuvsMultiGpuIvfPqListOwners": [_P(C.c_uint32), C.c_uint32, C.c_int, _P(C.c_int32)],
}

_lib = None


class CuvsError(RuntimeError):
    """Raised when an entry point returns CUVS_ERROR; carries cuvsGetLastErrorText()."""


def load():
    """Load the shared library and declare every entry point.  Fails loudly when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python cuvs_b200/_build.py` "
            "(or __graft_entry__.build()).  There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    lib.cuvsGetLastErrorText.restype = C.c_char_p
    lib.cuvsGetLastErrorText.argtypes = []
    lib.cuvsSetLastErrorText.restype = None
    lib.cuvsSetLastErrorText.argtypes = [C.c_char_p]
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != CUVS_SUCCESS:
        txt = load().cuvsGetLastErrorText()
        raise CuvsError(txt.decode() if txt else "unknown error")
