"""Python mirror of the reference's ``cuvs.neighbors.ivf_pq`` module
(python/cuvs/cuvs/neighbors/ivf_pq/ivf_pq.pyx): the same names, arguments and defaults
(``IndexParams`` :134-147, ``SearchParams`` :704-707, ``build`` :477, ``search`` :745, ``save`` :843,
``load`` :880, ``extend`` :913, ``transform`` :987), implemented as thin ctypes calls into the C
interface of this engine.  Device arrays are torch CUDA tensors; host arrays are numpy arrays.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib as L
from .common import DLTensorRef, Resources, default_resources, view_to_torch

_METRICS = {"sqeuclidean": 0, "euclidean": 1, "cosine": 2, "inner_product": 6}
_METRIC_NAMES = {v: k for k, v in _METRICS.items()}
_CUDA_DTYPE = {np.dtype(np.float32): 0, np.dtype(np.float16): 2, np.dtype(np.int8): 3,
               np.dtype(np.uint8): 8}
_CODEBOOK = {"subspace": 0, "cluster": 1}


def _cuda_dtype(dt, allowed):
    code = _CUDA_DTYPE.get(np.dtype(dt))
    if code is None or np.dtype(dt) not in [np.dtype(a) for a in allowed]:
        raise ValueError(f"dtype {dt} is not supported here; supported: {allowed}")
    return code


class IndexParams:
    """Parameters to build the index (ivf_pq.pyx:40-236)."""

    def __init__(self, *, n_lists=1024, metric="sqeuclidean", metric_arg=2.0, kmeans_n_iters=20,
                 kmeans_trainset_fraction=0.5, pq_bits=8, pq_dim=0, codebook_kind="subspace",
                 force_random_rotation=False, add_data_on_build=True,
                 conservative_memory_allocation=False, max_train_points_per_pq_code=256,
                 codes_layout="interleaved"):
        lib = L.load()
        self._p = C.POINTER(L.IndexParamsStruct)()
        L.check(lib.cuvsIvfPqIndexParamsCreate(C.byref(self._p)))
        p = self._p.contents
        if metric not in _METRICS:
            raise ValueError(f"metric {metric!r} not supported; one of {sorted(_METRICS)}")
        if codebook_kind not in _CODEBOOK:
            raise ValueError("Incorrect codebook kind %s" % codebook_kind)
        p.metric = _METRICS[metric]
        p.metric_arg = metric_arg
        p.add_data_on_build = add_data_on_build
        p.n_lists = n_lists
        p.kmeans_n_iters = kmeans_n_iters
        p.kmeans_trainset_fraction = kmeans_trainset_fraction
        p.pq_bits = pq_bits
        p.pq_dim = pq_dim
        p.codebook_kind = _CODEBOOK[codebook_kind]
        p.force_random_rotation = force_random_rotation
        p.conservative_memory_allocation = conservative_memory_allocation
        p.max_train_points_per_pq_code = max_train_points_per_pq_code
        if codes_layout not in ("flat", "interleaved"):
            raise ValueError("codes_layout must be 'flat' or 'interleaved'")
        p.codes_layout = 0 if codes_layout == "flat" else 1

    def __del__(self):
        try:
            L.load().cuvsIvfPqIndexParamsDestroy(self._p)
        except Exception:
            pass

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        v = getattr(self._p.contents, name)
        if name == "metric":
            return _METRIC_NAMES[v]
        if name == "codebook_kind":
            return "subspace" if v == 0 else "cluster"
        return v


class SearchParams:
    """Parameters of a search (ivf_pq.pyx:667-741)."""

    def __init__(self, *, n_probes=20, lut_dtype=np.float32, internal_distance_dtype=np.float32,
                 coarse_search_dtype=np.float32, max_internal_batch_size=4096):
        lib = L.load()
        self._p = C.POINTER(L.SearchParamsStruct)()
        L.check(lib.cuvsIvfPqSearchParamsCreate(C.byref(self._p)))
        p = self._p.contents
        p.n_probes = n_probes
        p.lut_dtype = _cuda_dtype(lut_dtype, [np.float32, np.float16, np.uint8])
        p.internal_distance_dtype = _cuda_dtype(internal_distance_dtype, [np.float32, np.float16])
        p.coarse_search_dtype = _cuda_dtype(coarse_search_dtype, [np.float32, np.float16, np.int8])
        p.max_internal_batch_size = max_internal_batch_size

    def __del__(self):
        try:
            L.load().cuvsIvfPqSearchParamsDestroy(self._p)
        except Exception:
            pass

    @property
    def n_probes(self):
        return self._p.contents.n_probes

    @property
    def max_internal_batch_size(self):
        return self._p.contents.max_internal_batch_size


class Index:
    """IVF-PQ index handle (ivf_pq.pyx:239-475)."""

    def __init__(self):
        self._lib = L.load()
        self._h = C.POINTER(L.IndexStruct)()
        L.check(self._lib.cuvsIvfPqIndexCreate(C.byref(self._h)))

    def __del__(self):
        try:
            if self._h:
                self._lib.cuvsIvfPqIndexDestroy(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def trained(self):
        return bool(self._h.contents.addr)

    def _scalar(self, fn):
        v = C.c_int64(0)
        L.check(fn(self._h, C.byref(v)))
        return v.value

    @property
    def n_lists(self):
        return self._scalar(self._lib.cuvsIvfPqIndexGetNLists)

    @property
    def dim(self):
        return self._scalar(self._lib.cuvsIvfPqIndexGetDim)

    @property
    def pq_dim(self):
        return self._scalar(self._lib.cuvsIvfPqIndexGetPqDim)

    @property
    def pq_len(self):
        return self._scalar(self._lib.cuvsIvfPqIndexGetPqLen)

    @property
    def pq_bits(self):
        return self._scalar(self._lib.cuvsIvfPqIndexGetPqBits)

    def __len__(self):
        return self._scalar(self._lib.cuvsIvfPqIndexGetSize)

    def _tensor(self, fn, *args):
        mt = L.DLManagedTensor()
        L.check(fn(self._h, *args, C.byref(mt)))
        return view_to_torch(mt)

    @property
    def centers(self):
        return self._tensor(self._lib.cuvsIvfPqIndexGetCenters)

    @property
    def centers_padded(self):
        return self._tensor(self._lib.cuvsIvfPqIndexGetCentersPadded)

    @property
    def pq_centers(self):
        return self._tensor(self._lib.cuvsIvfPqIndexGetPqCenters)

    @property
    def centers_rot(self):
        return self._tensor(self._lib.cuvsIvfPqIndexGetCentersRot)

    @property
    def rotation_matrix(self):
        return self._tensor(self._lib.cuvsIvfPqIndexGetRotationMatrix)

    @property
    def list_sizes(self):
        return self._tensor(self._lib.cuvsIvfPqIndexGetListSizes)

    def list_indices(self, label, n_rows=0):
        out = self._tensor(self._lib.cuvsIvfPqIndexGetListIndices, C.c_uint32(label))
        return out[:n_rows] if n_rows else out

    def list_data(self, label, n_rows=0, offset=0, out_codes=None, resources=None):
        """Bit-packed codes of rows [offset, offset + n_rows) of one list."""
        res = resources or default_resources()
        res.use_current_stream()
        if n_rows == 0:
            n_rows = int(self.list_sizes[label].item()) - offset
        nbytes = (self.pq_dim * self.pq_bits + 7) // 8
        if out_codes is None:
            out_codes = torch.empty((n_rows, nbytes), dtype=torch.uint8, device="cuda")
        ref = DLTensorRef(out_codes)
        L.check(self._lib.cuvsIvfPqIndexUnpackContiguousListData(
            res.handle, self._h, ref.ref(), C.c_uint32(label), C.c_uint32(offset)))
        res.sync()
        return out_codes

    def __repr__(self):
        if not self.trained:
            return "Index(type=IvfPq, untrained)"
        return (f"Index(type=IvfPq, size={len(self)}, dim={self.dim}, pq_dim={self.pq_dim}, "
                f"pq_bits={self.pq_bits}, n_lists={self.n_lists})")


def _res(resources):
    res = resources or default_resources()
    res.use_current_stream()
    return res


def build(index_params: IndexParams, dataset, resources: Resources | None = None) -> Index:
    """Build the index from a [n_rows, dim] f32/f16/i8/u8 dataset on host or device."""
    res = _res(resources)
    idx = Index()
    ref = DLTensorRef(dataset)
    L.check(L.load().cuvsIvfPqBuild(res.handle, index_params._p, ref.ref(), idx._h))
    res.sync()
    return idx


def build_precomputed(index_params: IndexParams, dim, pq_centers, centers, centers_rot,
                      rotation_matrix, resources: Resources | None = None) -> Index:
    res = _res(resources)
    idx = Index()
    refs = [DLTensorRef(t) for t in (pq_centers, centers, centers_rot, rotation_matrix)]
    L.check(L.load().cuvsIvfPqBuildPrecomputed(res.handle, index_params._p, C.c_uint32(dim),
                                               *[r.ref() for r in refs], idx._h))
    res.sync()
    return idx


def search(search_params: SearchParams, index: Index, queries, k, neighbors=None, distances=None,
           resources: Resources | None = None, sync: bool = True, filter=None):
    """Returns ``(distances, neighbors)`` -- f32 and i64 device tensors of shape [n_queries, k].

    ``filter``: optional uint32 device tensor, the reference's bitset filter -- the vector with
    source id ``i`` may be returned only if bit ``i`` (bit ``i % 32`` of word ``i // 32``) is set."""
    if not index.trained:
        raise ValueError("Index needs to be built before calling search.")
    res = _res(resources)
    n = queries.shape[0]
    if neighbors is None:
        neighbors = torch.empty((n, k), dtype=torch.int64, device="cuda")
    if distances is None:
        distances = torch.empty((n, k), dtype=torch.float32, device="cuda")
    q, nb, ds = DLTensorRef(queries), DLTensorRef(neighbors), DLTensorRef(distances)
    if filter is None:
        L.check(L.load().cuvsIvfPqSearch(res.handle, search_params._p, index._h, q.ref(), nb.ref(),
                                         ds.ref()))
    else:
        fb = DLTensorRef(filter)
        f = L.FilterStruct(C.addressof(fb.managed), 1)   # BITSET
        L.check(L.load().cuvsIvfPqSearchWithFilter(res.handle, search_params._p, index._h, q.ref(),
                                                   nb.ref(), ds.ref(), f))
    if sync:
        res.sync()
    return distances, neighbors


def save(filename: str, index: Index, include_dataset: bool = True,
         resources: Resources | None = None) -> None:
    res = _res(resources)
    L.check(L.load().cuvsIvfPqSerialize(res.handle, filename.encode(), index._h))


def load(filename: str, resources: Resources | None = None) -> Index:
    res = _res(resources)
    idx = Index()
    L.check(L.load().cuvsIvfPqDeserialize(res.handle, filename.encode(), idx._h))
    return idx


def extend(index: Index, new_vectors, new_indices, resources: Resources | None = None) -> Index:
    res = _res(resources)
    v = DLTensorRef(new_vectors)
    i = DLTensorRef(new_indices) if new_indices is not None else None
    L.check(L.load().cuvsIvfPqExtend(res.handle, v.ref(), i.ref() if i else None, index._h))
    res.sync()
    return index


def transform(index: Index, input_dataset, output_labels=None, output_dataset=None,
              resources: Resources | None = None):
    """Labels (u32 [n]) and bit-packed PQ codes (u8 [n, ceil(pq_dim*pq_bits/8)]) of vectors."""
    res = _res(resources)
    n = input_dataset.shape[0]
    nbytes = (index.pq_dim * index.pq_bits + 7) // 8
    if output_labels is None:
        output_labels = torch.empty((n,), dtype=torch.uint32, device="cuda")
    if output_dataset is None:
        output_dataset = torch.empty((n, nbytes), dtype=torch.uint8, device="cuda")
    a, b, c = DLTensorRef(input_dataset), DLTensorRef(output_labels), DLTensorRef(output_dataset)
    L.check(L.load().cuvsIvfPqTransform(res.handle, index._h, a.ref(), b.ref(), c.ref()))
    res.sync()
    return output_labels, output_dataset
