"""Mirror of the reference's ``cuvs.neighbors.refine`` (python/cuvs/cuvs/neighbors/refine/refine.pyx):
re-rank candidate neighbours with exact distances on the original vectors."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from .common import DLTensorRef, Resources, default_resources
from .ivf_pq import _METRICS


def refine(dataset, queries, candidates, k=None, metric="sqeuclidean", indices=None, distances=None,
           resources: Resources | None = None, sync: bool = True):
    """Returns ``(distances, indices)`` of the k best candidates per query by exact distance."""
    res = resources or default_resources()
    res.use_current_stream()
    n = queries.shape[0]
    if k is None:
        if indices is None:
            raise ValueError("Argument k must be specified if both indices and distances arg is None")
        k = indices.shape[1]
    if indices is None:
        indices = torch.empty((n, k), dtype=torch.int64, device="cuda")
    if distances is None:
        distances = torch.empty((n, k), dtype=torch.float32, device="cuda")
    if metric not in _METRICS:
        raise ValueError(f"metric {metric!r} not supported")
    a, b, c, d, e = (DLTensorRef(t) for t in (dataset, queries, candidates, indices, distances))
    L.check(L.load().cuvsRefine(res.handle, a.ref(), b.ref(), c.ref(), C.c_int(_METRICS[metric]),
                                d.ref(), e.ref()))
    if sync:
        res.sync()
    return distances, indices
