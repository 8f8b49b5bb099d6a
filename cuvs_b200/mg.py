"""List-sharded multi-GPU IVF-PQ search, one process per GPU.

Every rank holds the global coarse model and the inverted lists it owns (lists are dealt in order of
descending size, each to the rank holding the fewest rows so far: ``list_owners``).  ``search`` is ONE
call into the C++ host side (``cuvsMultiGpuIvfPqSearchRank``), which enqueues the whole step on the
handle's stream: probes of this rank's slice of the batch -> NCCL all-gather -> scan of the owned lists
for the whole batch -> all-gather of the per-rank top-k blocks (ids already global) -> merge.  The
merged result equals the single-GPU search on the unsharded index.  ``torch.distributed`` is used only
to hand the NCCL id to the other ranks when the communicator is made.

Reference behaviour this replaces: sharded search with merge in
cpp/src/neighbors/mg/snmg.cuh:249-561 (one process, one OpenMP thread per GPU, ncclSend/ncclRecv to
the root, knn_merge_parts); index distribution in snmg.cuh:48-58.  The single-process interface of the
reference (``cuvsMultiGpuIvfPqSearch`` and friends) is mirrored by ``cuvs_b200.mg_ivf_pq``.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib as L
from . import ivf_pq
from .common import DLTensorRef, Resources, default_resources


def list_owners(list_sizes, n_ranks: int):
    """Owner rank of every inverted list (the rule of the C++ shard loader), as a list of ints."""
    import numpy as np
    sizes = np.ascontiguousarray(np.asarray(list_sizes), dtype=np.uint32)
    owners = np.zeros(sizes.shape[0], dtype=np.int32)
    L.check(L.load().cuvsMultiGpuIvfPqListOwners(sizes.ctypes.data_as(C.POINTER(C.c_uint32)),
                                                 C.c_uint32(sizes.shape[0]), C.c_int(n_ranks),
                                                 owners.ctypes.data_as(C.POINTER(C.c_int32))))
    return owners.tolist()


class RankComm:
    """This rank's end of the exchanges of the list-sharded search: an NCCL communicator of its own
    (made from an id that rank 0 creates and the process group hands round) plus the exchange buffers
    the C++ side sizes once and keeps."""

    def __init__(self, group=None, resources: Resources | None = None):
        self._lib = L.load()
        self.rank, self.n_ranks = _rank_world(group)
        res = resources or default_resources()
        cid = L.CommId()
        if self.n_ranks > 1:
            box = [None]
            if self.rank == 0:
                L.check(self._lib.cuvsMultiGpuCommIdCreate(C.byref(cid)))
                box[0] = C.string_at(C.addressof(cid), 128)     # all 128 bytes, NULs included
            dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0,
                                       group=group)
            C.memmove(C.byref(cid), box[0], 128)
        self.handle = C.c_void_p()
        if self.n_ranks > 1:
            L.check(self._lib.cuvsMultiGpuRankCommCreate(res.handle, C.byref(cid), C.c_int(self.rank),
                                                         C.c_int(self.n_ranks), C.byref(self.handle)))
        else:
            L.check(self._lib.cuvsMultiGpuRankCommAdopt(None, 0, 1, C.byref(self.handle)))

    def set_merge_mode(self, mode: int):
        """0 or 2 = one all-gather of whole blocks, every rank merges everything (the default); 1 = the
        merge shared out by query slice.  Same result; same mode on every rank."""
        L.check(self._lib.cuvsMultiGpuRankCommSetMergeMode(self.handle, C.c_int(mode)))

    def stats(self, reset: bool = True):
        """Per-call stage times in ms of the searches made while the handle's stage timing was on:
        dict(select, gather_probes, scan, gather_results, merge, batches)."""
        ms = (C.c_double * 5)()
        n = C.c_uint64(0)
        L.check(self._lib.cuvsMultiGpuRankCommStats(self.handle, ms, C.byref(n), C.c_bool(reset)))
        b = max(1, n.value)
        names = ("select_ms", "gather_probes_ms", "scan_ms", "gather_results_ms", "merge_ms")
        out = {k: ms[i] / b for i, k in enumerate(names)}
        out["batches"] = n.value
        return out

    def __del__(self):
        try:
            if getattr(self, "handle", None):
                self._lib.cuvsMultiGpuRankCommDestroy(self.handle)
                self.handle = None
        except Exception:
            pass


_default_comm = {}


def default_comm(group=None) -> RankComm:
    key = (torch.cuda.current_device(), id(group))
    c = _default_comm.get(key)
    if c is None:
        c = _default_comm[key] = RankComm(group)
    return c


def _rank_world(group=None):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def load_shard(filename: str, rank: int | None = None, n_ranks: int | None = None,
               resources: Resources | None = None, group=None) -> ivf_pq.Index:
    """Load this rank's shard of a single-GPU index file (lists owned by other ranks are skipped)."""
    r, w = _rank_world(group)
    rank = r if rank is None else rank
    n_ranks = w if n_ranks is None else n_ranks
    res = resources or default_resources()
    res.use_current_stream()
    idx = ivf_pq.Index()
    L.check(L.load().cuvsMultiGpuIvfPqDistributeShard(res.handle, filename.encode(), C.c_int(rank),
                                                      C.c_int(n_ranks), idx._h))
    return idx


REPLICATED, SHARDED = 0, 1      # cuvs::neighbors::distribution_mode (common.hpp:1843-1848)


def load_reference_mg(filename: str, rank: int | None = None, n_ranks: int | None = None,
                      resources: Resources | None = None, group=None):
    """This rank's index out of a multi-GPU index file written by the reference
    (``cuvsMultiGpuIvfPqSerialize``).  Returns ``(index, mode, id_offset)``: ``mode`` is
    ``REPLICATED`` or ``SHARDED`` (by rows), ``id_offset`` what has to be added to this rank's
    neighbour ids in sharded mode."""
    r, w = _rank_world(group)
    rank = r if rank is None else rank
    n_ranks = w if n_ranks is None else n_ranks
    res = resources or default_resources()
    res.use_current_stream()
    idx = ivf_pq.Index()
    mode, off = C.c_int(), C.c_int64()
    L.check(L.load().cuvsMultiGpuIvfPqDeserializeRank(res.handle, filename.encode(), C.c_int(rank),
                                                      C.c_int(n_ranks), idx._h, C.byref(mode), C.byref(off)))
    return idx, mode.value, off.value


def save_reference_mg(filename: str, indexes, mode: int, dataset_dtype=torch.float32,
                      resources: Resources | None = None):
    """Write ``indexes`` (one per rank, all in this process) as one multi-GPU index file of the
    reference's format."""
    res = resources or default_resources()
    code_bits = {torch.float32: (2, 32), torch.float16: (2, 16), torch.int8: (0, 8), torch.uint8: (1, 8)}
    code, bits = code_bits[dataset_dtype]
    arr = (C.POINTER(L.IndexStruct) * len(indexes))(*[ix._h for ix in indexes])
    L.check(L.load().cuvsMultiGpuIvfPqSerializeRanks(res.handle, filename.encode(), C.c_int(mode),
                                                     L.DLDataType(code, bits, 1), arr, C.c_int(len(indexes))))


def translate_ids(neighbors: torch.Tensor, id_offset: int) -> torch.Tensor:
    """Local ids of a row shard -> global ids (missing results, INT64_MAX, stay as they are)."""
    if id_offset == 0:
        return neighbors
    missing = neighbors == torch.iinfo(torch.int64).max
    return torch.where(missing, neighbors, neighbors + id_offset)


def search_reference_mg(search_params: ivf_pq.SearchParams, index: ivf_pq.Index, mode: int, id_offset: int,
                        queries, k: int, group=None, resources: Resources | None = None, sync: bool = True,
                        metric: str = "sqeuclidean"):
    """Search an index loaded with :func:`load_reference_mg`, with the reference's semantics
    (cpp/src/neighbors/mg/snmg.cuh:249-561): SHARDED -- every rank searches its own rows for the whole
    batch, ids are made global, the per-rank lists are merged; REPLICATED -- the batch is split between
    the ranks and the slices are gathered.  Every rank passes the same queries and gets the result."""
    res = resources or default_resources()
    rank, w = _rank_world(group)
    if mode == SHARDED:
        d, i = ivf_pq.search(search_params, index, queries, k, resources=res, sync=False)
        i = translate_ids(i, id_offset)
        if w == 1:
            if sync:
                res.sync()
            return d, i
        part_d, part_i = gather_parts(d, i, group)
        # larger is better for inner product, smaller otherwise (snmg.cuh:263: is_min_close(metric))
        return merge_parts(part_d, part_i, metric != "inner_product", res, sync)
    n = queries.shape[0]
    if w == 1:
        return ivf_pq.search(search_params, index, queries, k, resources=res, sync=sync)
    s = -(-n // w)
    lo, hi = min(n, rank * s), min(n, (rank + 1) * s)
    mine_d = torch.zeros((s, k), dtype=torch.float32, device=queries.device)
    mine_i = torch.zeros((s, k), dtype=torch.int64, device=queries.device)
    if hi > lo:
        d, i = ivf_pq.search(search_params, index, queries[lo:hi].contiguous(), k, resources=res, sync=False)
        mine_d[: hi - lo], mine_i[: hi - lo] = d, i
    all_d = torch.empty((w * s, k), dtype=torch.float32, device=queries.device)
    all_i = torch.empty((w * s, k), dtype=torch.int64, device=queries.device)
    dist.all_gather_into_tensor(all_d, mine_d, group=group)
    dist.all_gather_into_tensor(all_i, mine_i, group=group)
    if sync:
        res.sync()
    return all_d[:n], all_i[:n]


def gather_parts(local_d: torch.Tensor, local_i: torch.Tensor, group=None):
    """All-gather the per-rank results: returns ([R, n, k] distances, [R, n, k] ids)."""
    _, w = _rank_world(group)
    if w == 1:
        return local_d.unsqueeze(0), local_i.unsqueeze(0)
    n, k = local_d.shape
    # concatenated along dim 0 (the form both NCCL and gloo accept), viewed as [R, n, k]
    part_d = torch.empty((w * n, k), dtype=local_d.dtype, device=local_d.device)
    part_i = torch.empty((w * n, k), dtype=local_i.dtype, device=local_i.device)
    dist.all_gather_into_tensor(part_d, local_d.contiguous(), group=group)
    dist.all_gather_into_tensor(part_i, local_i.contiguous(), group=group)
    return part_d.view(w, n, k), part_i.view(w, n, k)


def merge_parts(part_d: torch.Tensor, part_i: torch.Tensor, select_min: bool = True,
                resources: Resources | None = None, sync: bool = True):
    """Merge [R, n, k] per-part results into [n, k] on the GPU (cuvsMultiGpuIvfPqMergeParts)."""
    res = resources or default_resources()
    res.use_current_stream()
    _, n, k = part_d.shape
    out_d = torch.empty((n, k), dtype=torch.float32, device=part_d.device)
    out_i = torch.empty((n, k), dtype=torch.int64, device=part_d.device)
    # the parts may be views into one gathered buffer: row-major each, any stride between them
    a, b = DLTensorRef(part_d, strided=True), DLTensorRef(part_i, strided=True)
    c, d = DLTensorRef(out_d), DLTensorRef(out_i)
    L.check(L.load().cuvsMultiGpuIvfPqMergeParts(res.handle, a.ref(), b.ref(), c.ref(), d.ref(),
                                                 C.c_bool(select_min)))
    if sync:
        res.sync()
    return out_d, out_i


def select_probes(shard: ivf_pq.Index, queries, n_probes: int, resources: Resources | None = None,
                  out=None):
    """Probes of `queries` (u32 [n, n_probes], ascending by (score, list id)); asynchronous.
    `out`: optional destination (contiguous u32 [n, n_probes])."""
    res = resources or default_resources()
    res.use_current_stream()
    probes = out if out is not None else \
        torch.empty((queries.shape[0], n_probes), dtype=torch.uint32, device=queries.device)
    if queries.shape[0]:
        q, p = DLTensorRef(queries), DLTensorRef(probes)
        L.check(L.load().cuvsMultiGpuIvfPqSelectProbes(res.handle, shard._h, q.ref(), p.ref()))
    return probes


def search_with_probes(search_params: ivf_pq.SearchParams, shard: ivf_pq.Index, queries, probes,
                       k: int, resources: Resources | None = None, sync: bool = True, out=None):
    """Fine search of this rank's lists for given probes; `out` = optional (distances, neighbors)."""
    res = resources or default_resources()
    res.use_current_stream()
    n = queries.shape[0]
    if out is not None:
        d, i = out
    else:
        d = torch.empty((n, k), dtype=torch.float32, device=queries.device)
        i = torch.empty((n, k), dtype=torch.int64, device=queries.device)
    a, b, c, e = DLTensorRef(queries), DLTensorRef(probes.contiguous()), DLTensorRef(i), DLTensorRef(d)
    L.check(L.load().cuvsMultiGpuIvfPqSearchWithProbes(res.handle, search_params._p, shard._h, a.ref(),
                                                       b.ref(), c.ref(), e.ref()))
    if sync:
        res.sync()
    return d, i


def search(search_params: ivf_pq.SearchParams, shard: ivf_pq.Index, queries, k: int,
           group=None, resources: Resources | None = None, sync: bool = True, comm: RankComm | None = None,
           out=None):
    """Sharded search: every rank passes the same queries (device tensor) and gets the same merged
    result ``(distances, neighbors)``.  One call into the C++ step (see the module text); whether the
    smallest or the largest distances win follows from the index metric.  ``out``: optional
    ``(distances, neighbors)`` to fill."""
    res = resources or default_resources()
    res.use_current_stream()
    comm = comm or default_comm(group)
    n = queries.shape[0]
    if out is not None:
        d, i = out
    else:
        d = torch.empty((n, k), dtype=torch.float32, device=queries.device)
        i = torch.empty((n, k), dtype=torch.int64, device=queries.device)
    a, b, c = DLTensorRef(queries), DLTensorRef(i), DLTensorRef(d)
    L.check(L.load().cuvsMultiGpuIvfPqSearchRank(res.handle, comm.handle, search_params._p, shard._h, a.ref(),
                                                 b.ref(), c.ref()))
    if sync:
        res.sync()
    return d, i
