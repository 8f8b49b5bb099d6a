"""Single-list helpers of the IVF-PQ index, the Python face of the reference's
``cuvs::neighbors::ivf_pq::helpers`` namespace (cpp/include/cuvs/neighbors/ivf_pq.hpp:2564-3166):
read, overwrite, decode, extend and erase the rows of one list without classification.  Same names
and argument meaning as the C++ functions; all arrays are torch CUDA tensors.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib as L
from .common import DLTensorRef, Resources, default_resources
from .ivf_pq import Index

_TORCH = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16,
          np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8}


def _res(resources):
    res = resources or default_resources()
    res.use_current_stream()
    return res


def _list_size(index: Index, label: int) -> int:
    return int(index.list_sizes[label].item())


def _rows(index, label, n_rows, offset, in_cluster_indices):
    if in_cluster_indices is not None:
        return int(in_cluster_indices.shape[0]), DLTensorRef(in_cluster_indices)
    return (n_rows if n_rows else _list_size(index, label) - offset), None


def unpack_list_data(index: Index, label: int, offset: int = 0, n_rows: int = 0,
                     in_cluster_indices=None, out_codes=None, resources: Resources | None = None):
    """Codes of list rows, one per byte: u8 [n_rows, pq_dim] (ivf_pq.hpp:2818, :2854)."""
    res = _res(resources)
    n, ind = _rows(index, label, n_rows, offset, in_cluster_indices)
    if out_codes is None:
        out_codes = torch.empty((n, index.pq_dim), dtype=torch.uint8, device="cuda")
    out = DLTensorRef(out_codes)
    L.check(L.load().cuvsIvfPqHelpersUnpackListData(res.handle, index._h, out.ref(), C.c_uint32(label),
                                                    C.c_uint32(offset), ind.ref() if ind else None))
    res.sync()
    return out_codes


def pack_list_data(index: Index, codes, label: int, offset: int = 0,
                   resources: Resources | None = None) -> None:
    """Overwrite rows [offset, offset + n) of a list with codes u8 [n, pq_dim] (ivf_pq.hpp:2739)."""
    res = _res(resources)
    c = DLTensorRef(codes)
    L.check(L.load().cuvsIvfPqHelpersPackListData(res.handle, index._h, c.ref(), C.c_uint32(label),
                                                  C.c_uint32(offset)))
    res.sync()


def pack_contiguous_list_data(index: Index, codes, label: int, offset: int = 0,
                              resources: Resources | None = None) -> None:
    """Same with bit-packed rows u8 [n, ceil(pq_dim * pq_bits / 8)] (ivf_pq.hpp:2782)."""
    res = _res(resources)
    c = DLTensorRef(codes)
    L.check(L.load().cuvsIvfPqHelpersPackContiguousListData(res.handle, index._h, c.ref(),
                                                            C.c_uint32(label), C.c_uint32(offset)))
    res.sync()


def reconstruct_list_data(index: Index, label: int, offset: int = 0, n_rows: int = 0,
                          in_cluster_indices=None, dtype=np.float32, out_vectors=None,
                          resources: Resources | None = None):
    """Decoded vectors [n_rows, dim] of list rows (ivf_pq.hpp:2932-3002)."""
    res = _res(resources)
    n, ind = _rows(index, label, n_rows, offset, in_cluster_indices)
    if out_vectors is None:
        out_vectors = torch.empty((n, index.dim), dtype=_TORCH[np.dtype(dtype)], device="cuda")
    out = DLTensorRef(out_vectors)
    L.check(L.load().cuvsIvfPqHelpersReconstructListData(res.handle, index._h, out.ref(),
                                                         C.c_uint32(label), C.c_uint32(offset),
                                                         ind.ref() if ind else None))
    res.sync()
    return out_vectors


def extend_list_with_codes(index: Index, new_codes, new_indices, label: int,
                           resources: Resources | None = None) -> None:
    """Append rows given as codes u8 [n, pq_dim] with their source ids (ivf_pq.hpp:3035)."""
    res = _res(resources)
    a, b = DLTensorRef(new_codes), DLTensorRef(new_indices)
    L.check(L.load().cuvsIvfPqHelpersExtendListWithCodes(res.handle, index._h, a.ref(), b.ref(),
                                                         C.c_uint32(label), False))


def extend_list_with_contiguous_codes(index: Index, new_codes, new_indices, label: int,
                                      resources: Resources | None = None) -> None:
    """Append rows given as bit-packed codes (ivf_pq.hpp:3074)."""
    res = _res(resources)
    a, b = DLTensorRef(new_codes), DLTensorRef(new_indices)
    L.check(L.load().cuvsIvfPqHelpersExtendListWithCodes(res.handle, index._h, a.ref(), b.ref(),
                                                         C.c_uint32(label), True))


def extend_list(index: Index, new_vectors, new_indices, label: int,
                resources: Resources | None = None) -> None:
    """Encode vectors against list `label` and append them (ivf_pq.hpp:3109-3123)."""
    res = _res(resources)
    a, b = DLTensorRef(new_vectors), DLTensorRef(new_indices)
    L.check(L.load().cuvsIvfPqHelpersExtendList(res.handle, index._h, a.ref(), b.ref(),
                                                C.c_uint32(label)))


def erase_list(index: Index, label: int, resources: Resources | None = None) -> None:
    """Remove every row of one list (ivf_pq.hpp:3144)."""
    L.check(L.load().cuvsIvfPqHelpersEraseList(_res(resources).handle, index._h, C.c_uint32(label)))


def reset_index(index: Index, resources: Resources | None = None) -> None:
    """Remove every row of every list; the trained model stays (ivf_pq.hpp:3166)."""
    L.check(L.load().cuvsIvfPqHelpersResetIndex(_res(resources).handle, index._h))
