"""Mirror of the reference's ``cuvs.neighbors.mg.ivf_pq`` module
(python/cuvs/cuvs/neighbors/mg/ivf_pq/ivf_pq.pyx): one process drives all GPUs of a node through a
multi-GPU resources handle; datasets, queries and results are host (numpy) arrays.  Same names and
arguments -- ``IndexParams(distribution_mode=...)`` :56-103, ``build`` :130, ``SearchParams(search_mode,
merge_mode, n_rows_per_batch)`` :193-273, ``search`` :276, ``extend`` :386, ``save`` :459, ``load`` :497,
``distribute`` :531 -- as thin ctypes calls into the C interface (``cuvsMultiGpuIvfPq*``).

A ``sharded`` index built here is sharded by inverted list: one global coarse model on every GPU, each
list on exactly one GPU, so a search returns what the single-GPU search of the whole index returns.
``distribute_by_list`` (no counterpart in the reference) deals a single-GPU index file out that way.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from . import ivf_pq as _single
from .common import DLTensorRef

_MODES = {"replicated": 0, "sharded": 1}
_SEARCH_MODES = {"load_balancer": 0, "round_robin": 1}
_MERGE_MODES = {"merge_on_root_rank": 0, "tree_merge": 1}


class MultiGpuResources:
    """``cuvs.common.MultiGpuResources``: owns the multi-GPU handle (one stream, workspace and NCCL
    communicator per device)."""

    def __init__(self, device_ids=None):
        self._lib = L.load()
        h = C.c_size_t(0)
        if device_ids is None:
            L.check(self._lib.cuvsMultiGpuResourcesCreate(C.byref(h)))
        else:
            ids = np.ascontiguousarray(device_ids, dtype=np.int32)
            ref = DLTensorRef(ids.view(np.int32))
            L.check(self._lib.cuvsMultiGpuResourcesCreateWithDeviceIds(C.byref(h), ref.ref()))
        self.handle = h.value

    def set_memory_pool(self, percent_of_free_memory: int):
        L.check(self._lib.cuvsMultiGpuResourcesSetMemoryPool(self.handle, C.c_int(percent_of_free_memory)))

    def __del__(self):
        try:
            if getattr(self, "handle", 0):
                self._lib.cuvsMultiGpuResourcesDestroy(self.handle)
                self.handle = 0
        except Exception:
            pass


class IndexParams(_single.IndexParams):
    def __init__(self, *, distribution_mode="sharded", **kwargs):
        super().__init__(**kwargs)
        if distribution_mode not in _MODES:
            raise ValueError("distribution_mode must be 'replicated' or 'sharded'")
        self._mg = L.MgIndexParamsStruct(self._p, _MODES[distribution_mode])

    @property
    def distribution_mode(self):
        return "sharded" if self._mg.mode == 1 else "replicated"


class SearchParams(_single.SearchParams):
    def __init__(self, *, search_mode="load_balancer", merge_mode="tree_merge", n_rows_per_batch=1 << 20,
                 **kwargs):
        super().__init__(**kwargs)
        self._mg = L.MgSearchParamsStruct(self._p, _SEARCH_MODES[search_mode], _MERGE_MODES[merge_mode],
                                          n_rows_per_batch)


class Index:
    def __init__(self):
        self._lib = L.load()
        self._h = C.POINTER(L.IndexStruct)()
        L.check(self._lib.cuvsMultiGpuIvfPqIndexCreate(C.byref(self._h)))

    @property
    def trained(self):
        return bool(self._h.contents.addr)

    def __del__(self):
        try:
            if self._h:
                self._lib.cuvsMultiGpuIvfPqIndexDestroy(self._h)
                self._h = None
        except Exception:
            pass

    def __repr__(self):
        return "Index(type=MultiGpuIvfPq)"


def _np(a, what):
    if not isinstance(a, np.ndarray):
        raise TypeError(f"{what} must be a host (numpy) array")
    return np.ascontiguousarray(a)


def build(index_params: IndexParams, dataset, resources: MultiGpuResources) -> Index:
    idx = Index()
    ref = DLTensorRef(_np(dataset, "dataset"))
    L.check(L.load().cuvsMultiGpuIvfPqBuild(resources.handle, C.byref(index_params._mg), ref.ref(), idx._h))
    return idx


def search(search_params: SearchParams, index: Index, queries, k, neighbors=None, distances=None,
           resources: MultiGpuResources | None = None):
    """Returns ``(distances, neighbors)`` as numpy arrays [n_queries, k]."""
    if not index.trained:
        raise ValueError("Index needs to be built before calling search.")
    q = _np(queries, "queries")
    n = q.shape[0]
    neighbors = np.empty((n, k), dtype=np.int64) if neighbors is None else neighbors
    distances = np.empty((n, k), dtype=np.float32) if distances is None else distances
    a, b, c = DLTensorRef(q), DLTensorRef(neighbors), DLTensorRef(distances)
    L.check(L.load().cuvsMultiGpuIvfPqSearch(resources.handle, C.byref(search_params._mg), index._h, a.ref(),
                                             b.ref(), c.ref()))
    return distances, neighbors


def extend(index: Index, new_vectors, new_indices=None, resources: MultiGpuResources | None = None) -> Index:
    v = DLTensorRef(_np(new_vectors, "new_vectors"))
    i = DLTensorRef(_np(new_indices, "new_indices").astype(np.int64, copy=False)) if new_indices is not None else None
    L.check(L.load().cuvsMultiGpuIvfPqExtend(resources.handle, index._h, v.ref(), i.ref() if i else None))
    return index


def save(index: Index, filename: str, resources: MultiGpuResources | None = None) -> None:
    L.check(L.load().cuvsMultiGpuIvfPqSerialize(resources.handle, index._h, filename.encode()))


def load(filename: str, resources: MultiGpuResources | None = None) -> Index:
    idx = Index()
    L.check(L.load().cuvsMultiGpuIvfPqDeserialize(resources.handle, filename.encode(), idx._h))
    return idx


def distribute(filename: str, resources: MultiGpuResources | None = None) -> Index:
    idx = Index()
    L.check(L.load().cuvsMultiGpuIvfPqDistribute(resources.handle, filename.encode(), idx._h))
    return idx


def distribute_by_list(filename: str, resources: MultiGpuResources | None = None) -> Index:
    idx = Index()
    L.check(L.load().cuvsMultiGpuIvfPqDistributeByList(resources.handle, filename.encode(), idx._h))
    return idx
