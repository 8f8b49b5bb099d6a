"""CPU test (gloo, world size 2) of the list-sharded search logic: ownership rule, gather layout and
the claim that merging per-shard results reproduces the unsharded search.  The per-shard searches
and the merge are done by the oracle here (this is host-logic coverage; the CUDA merge kernel has its
own GPU test)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import make_mixture


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _merge_numpy(part_d, part_i, k):
    """Same contract as cuvsMultiGpuIvfPqMergeParts (select_min): smallest k, out-of-bounds ignored."""
    r, n, _ = part_d.shape
    d = np.transpose(part_d, (1, 0, 2)).reshape(n, -1)
    i = np.transpose(part_i, (1, 0, 2)).reshape(n, -1)
    d = np.where(i == np.iinfo(np.int64).max, np.inf, d)
    o = np.argsort(d, axis=1, kind="stable")[:, :k]
    return np.take_along_axis(d, o, 1), np.take_along_axis(i, o, 1)


def _worker(rank, world, port, path, q, k, n_probes, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cuvs_b200 import mg
    from oracle import oracle as O
    ix = O.OracleIndex.load(path)
    # keep the lists this rank owns (the rule of the C++ shard loader)
    owners = mg.list_owners(ix.list_sizes, world)
    for l in range(ix.n_lists):
        if owners[l] != rank:
            ix.list_sizes[l] = 0
            ix.list_codes[l] = np.zeros(0, np.uint8)
            ix.list_ids[l] = np.zeros(0, np.int64)
    ix._flat = None
    d, i = O.search(ix, q, k, n_probes=n_probes)
    part_d, part_i = mg.gather_parts(torch.from_numpy(d), torch.from_numpy(i))
    assert part_d.shape == (world, q.shape[0], k)
    md, mi = _merge_numpy(part_d.numpy(), part_i.numpy(), k)
    if rank == 0:
        np.save(out + "_d.npy", md)
        np.save(out + "_i.npy", mi)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_search_equals_unsharded(oracle_mod, small_l2, tmp_path):
    O = oracle_mod
    q, k, p = small_l2["q"][:40], 10, 8
    out = str(tmp_path / "merged")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, small_l2["path"], q, k, p, out), nprocs=2, join=True)
    md, mi = np.load(out + "_d.npy"), np.load(out + "_i.npy")
    d, i = O.search(small_l2["ix"], q, k, n_probes=p)
    assert (mi == i).all()
    assert (md.view(np.uint32) == d.view(np.uint32)).all()


def test_ownership_rule():
    """Lists are dealt in order of descending size, each to the rank holding the fewest rows so far:
    equal sizes come out round-robin, skewed sizes come out balanced."""
    from cuvs_b200 import mg
    owners = mg.list_owners([100] * 64, 8)
    assert owners[:9] == [0, 1, 2, 3, 4, 5, 6, 7, 0]
    assert all(owners.count(r) == 8 for r in range(8))
    rng = np.random.default_rng(0)
    sizes = (rng.pareto(1.5, 5000) * 300).astype(np.uint32)       # heavy-tailed list sizes
    owners = np.array(mg.list_owners(sizes, 8))
    load = np.array([sizes[owners == r].sum() for r in range(8)], dtype=np.float64)
    assert load.max() <= max(load.mean() * 1.01, float(sizes.max()))
    naive = np.array([sizes[np.arange(5000) % 8 == r].sum() for r in range(8)], dtype=np.float64)
    assert load.max() - load.min() <= naive.max() - naive.min()
    assert mg.list_owners([5, 0, 7], 1) == [0, 0, 0]
