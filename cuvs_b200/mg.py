"""List-sharded multi-GPU IVF-PQ search, one process per GPU over ``torch.distributed``.

Every rank holds the global coarse model and the inverted lists it owns (list ``l`` belongs to rank
``l % n_ranks``).  A search runs the ordinary single-GPU search on every rank for the whole query
batch -- the probes chosen are identical on every rank, a rank scans only the ones it owns -- then
all-gathers the per-rank top-k (``n_queries * k * 12`` bytes per rank, ids already global) and
merges them on the GPU.  The merged result equals the single-GPU search on the unsharded index.

Reference behaviour this replaces: sharded search with merge in
cpp/src/neighbors/mg/snmg.cuh:249-561 (one process, one OpenMP thread per GPU, ncclSend/ncclRecv to
the root, knn_merge_parts); index distribution in snmg.cuh:48-58.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib as L
from . import ivf_pq
from .common import DLTensorRef, Resources, default_resources


def shard_of_list(label: int, n_ranks: int) -> int:
    """Owner rank of an inverted list (same rule as the C++ loader)."""
    return int(label) % int(n_ranks)


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
                        queries, k: int, select_min: bool = True, group=None,
                        resources: Resources | None = None, sync: bool = True):
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
        return merge_parts(part_d, part_i, select_min, res, sync)
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


def shared_probes(shard: ivf_pq.Index, queries, n_probes: int, group=None,
                  resources: Resources | None = None):
    """Probe selection shared between the ranks: rank r selects the probes of the r-th slice of the
    batch (the global coarse model is replicated, so every rank would choose the same lists), the
    slices are all-gathered (n_queries * n_probes * 4 bytes in total)."""
    rank, w = _rank_world(group)
    n = queries.shape[0]
    if w == 1:
        return select_probes(shard, queries, n_probes, resources)
    s = -(-n // w)
    lo, hi = min(n, rank * s), min(n, (rank + 1) * s)
    every = torch.empty((w * s, n_probes), dtype=torch.uint32, device=queries.device)
    if _in_place_gather(group):
        # this rank's slice is written where the gather wants it and gathered in place (rows past
        # n exist only as padding of the last slice and are never read)
        if hi > lo:
            select_probes(shard, queries[lo:hi], n_probes, resources, out=every[lo:hi])
        mine = every[rank * s:(rank + 1) * s]
    else:
        mine = torch.zeros((s, n_probes), dtype=torch.uint32, device=queries.device)
        if hi > lo:
            mine[: hi - lo] = select_probes(shard, queries[lo:hi], n_probes, resources)
    # NCCL has no uint32: exchange the same bytes as int32
    dist.all_gather_into_tensor(every.view(torch.int32), mine.view(torch.int32), group=group)
    return every[:n]


def _in_place_gather(group=None) -> bool:
    """NCCL gathers in place when a rank's input is its own slot of the output."""
    return dist.get_backend(group) == "nccl"


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
           select_min: bool = True, group=None, resources: Resources | None = None,
           sync: bool = True):
    """Sharded search: every rank passes the same queries and gets the same merged result.
    Probe selection is split between the ranks by query slice, the code scan by inverted list."""
    res = resources or default_resources()
    _, w = _rank_world(group)
    if w == 1:
        return ivf_pq.search(search_params, shard, queries, k, resources=res, sync=sync)
    n_probes = min(search_params.n_probes, shard.n_lists)
    probes = shared_probes(shard, queries, n_probes, group, res)
    n = queries.shape[0]
    nk = n * k
    if _in_place_gather(group) and nk % 2 == 0 and nk > 0:
        # one exchange for ids and distances: every rank's block is [n*k int64 ids | n*k f32
        # distances], written by the search straight into this rank's slot of the gathered buffer
        rank = dist.get_rank(group)
        blocks = torch.empty((w, nk * 12), dtype=torch.uint8, device=queries.device)
        part_i = blocks[:, :nk * 8].view(torch.int64).view(w, n, k)
        part_d = blocks[:, nk * 8:].view(torch.float32).view(w, n, k)
        search_with_probes(search_params, shard, queries, probes, k, res, sync=False,
                           out=(part_d[rank], part_i[rank]))
        dist.all_gather_into_tensor(blocks, blocks[rank], group=group)
        return merge_parts(part_d, part_i, select_min, res, sync)
    d, i = search_with_probes(search_params, shard, queries, probes, k, res, sync=False)
    part_d, part_i = gather_parts(d, i, group)
    return merge_parts(part_d, part_i, select_min, res, sync)
