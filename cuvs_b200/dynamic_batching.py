"""Dynamic batching in front of an IVF-PQ index: many host threads submit small searches, the library
gathers them into batches for the upstream index.

Mirrors ``cuvs::neighbors::dynamic_batching`` of the reference
(cpp/include/cuvs/neighbors/dynamic_batching.hpp; C++ only there, no Python module): same
parameters, same contract -- every request is answered exactly as a direct upstream search would."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from . import ivf_pq
from .common import DLTensorRef, Resources, default_resources


class Index:
    """``Index(upstream, search_params, k, max_batch_size=100, n_queues=3)``; ``upstream`` (an
    :class:`cuvs_b200.ivf_pq.Index`) must outlive this object."""

    def __init__(self, upstream: ivf_pq.Index, search_params: ivf_pq.SearchParams, k: int,
                 max_batch_size: int = 100, n_queues: int = 3, conservative_dispatch: bool = False,
                 resources: Resources | None = None):
        lib = L.load()
        res = resources or default_resources()
        p = C.POINTER(L.DynamicBatchingIndexParamsStruct)()
        L.check(lib.cuvsDynamicBatchingIndexParamsCreate(C.byref(p)))
        try:
            p.contents.k = k
            p.contents.max_batch_size = max_batch_size
            p.contents.n_queues = n_queues
            p.contents.conservative_dispatch = conservative_dispatch
            self._h = C.POINTER(L.DynamicBatchingIndexStruct)()
            L.check(lib.cuvsDynamicBatchingIndexCreate(res.handle, p, upstream._h, search_params._p,
                                                       C.byref(self._h)))
        finally:
            lib.cuvsDynamicBatchingIndexParamsDestroy(p)
        self._upstream = upstream          # keeps the upstream index alive
        self.k = k

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            L.load().cuvsDynamicBatchingIndexDestroy(h)
            self._h = None

    def fail_next(self):
        """Test hook (host side): the next upstream search of this index fails before it runs."""
        L.check(L.load().cuvsDynamicBatchingFailNext(self._h))

    def stats(self):
        """(upstream searches launched, rows they carried)."""
        a, b = C.c_uint64(), C.c_uint64()
        L.check(L.load().cuvsDynamicBatchingStats(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value


def search(index: Index, queries, neighbors=None, distances=None, dispatch_timeout_ms: float = 1.0,
           resources: Resources | None = None, sync: bool = True):
    """One request (any number of rows) from the calling thread; use one ``Resources`` per thread.
    Returns ``(distances, neighbors)``."""
    res = resources or default_resources()
    res.use_current_stream()
    n = queries.shape[0]
    if neighbors is None:
        neighbors = torch.empty((n, index.k), dtype=torch.int64, device=queries.device)
    if distances is None:
        distances = torch.empty((n, index.k), dtype=torch.float32, device=queries.device)
    q, nb, ds = DLTensorRef(queries), DLTensorRef(neighbors), DLTensorRef(distances)
    L.check(L.load().cuvsDynamicBatchingSearch(res.handle, index._h, C.c_double(dispatch_timeout_ms),
                                               q.ref(), nb.ref(), ds.ref()))
    if sync:
        res.sync()
    return distances, neighbors
