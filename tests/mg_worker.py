"""Rank program of tests/test_mg_gpu.py (launched with torch.distributed.run): the list-sharded search
over NCCL must give, on every rank, exactly the single-GPU result."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    path, qpath = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from cuvs_b200 import ivf_pq, mg
    q = torch.from_numpy(np.load(qpath)).cuda()
    for suffix, lut_cases in (("", ((10, 8, np.float32), (40, 24, np.float16), (100, 12, np.uint8), (200, 16, np.float32))),
                              (".ip", ((10, 8, np.float32), (150, 10, np.float16)))):
        full = ivf_pq.load(path + suffix)
        shard = mg.load_shard(path + suffix)
        assert int(shard.list_sizes.sum().item()) < int(full.list_sizes.sum().item())
        for k, p, lut in lut_cases:
            sp = ivf_pq.SearchParams(n_probes=p, lut_dtype=lut)
            d0, i0 = ivf_pq.search(sp, full, q, k)
            for rep in range(2):          # the second call reuses the exchange buffers
                d1, i1 = mg.search(sp, shard, q, k)
                # distances bit for bit; ids wherever the distance is not shared with a neighbour in the
                # row or with the k-th place (the merge orders equal distances by part, the single-GPU
                # path by position in the probed lists)
                assert (d0.view(torch.int32) == d1.view(torch.int32)).all(), (rank, k, p, suffix)
                tied = torch.zeros_like(i0, dtype=torch.bool)
                tied[:, 1:] |= d0[:, 1:] == d0[:, :-1]
                tied[:, :-1] |= d0[:, :-1] == d0[:, 1:]
                tied |= d0 == d0[:, -1:]
                assert ((i0 == i1) | tied).all(), (rank, k, p, suffix)
                assert tied.float().mean().item() < 0.2, (rank, k, p, suffix)
        # the merge shared out by query slice (optional mode) gives the same result,
        # also when the batch does not divide evenly and for k beyond the register merge
        comm = mg.default_comm()
        comm.set_merge_mode(1)
        for k, p, nq in ((10, 8, q.shape[0]), (40, 12, q.shape[0] - 1), (200, 16, 7)):
            sp = ivf_pq.SearchParams(n_probes=p)
            qs = q[:nq].contiguous()
            d0, i0 = ivf_pq.search(sp, full, qs, k)
            d1, i1 = mg.search(sp, shard, qs, k)
            assert (d0.view(torch.int32) == d1.view(torch.int32)).all(), ("slice merge", rank, k, suffix)
            tied = torch.zeros_like(i0, dtype=torch.bool)
            tied[:, 1:] |= d0[:, 1:] == d0[:, :-1]
            tied[:, :-1] |= d0[:, :-1] == d0[:, 1:]
            tied |= d0 == d0[:, -1:]
            assert ((i0 == i1) | tied).all(), ("slice merge ids", rank, k, suffix)
        comm.set_merge_mode(0)
        # int8 coarse search: the shared probe selection honours coarse_search_dtype
        if suffix == "":
            sp = ivf_pq.SearchParams(n_probes=8, coarse_search_dtype=np.int8)
            d0, i0 = ivf_pq.search(sp, full, q, 10)
            d1, i1 = mg.search(sp, shard, q, 10)
            assert (d0.view(torch.int32) == d1.view(torch.int32)).all(), "int8 coarse"
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("MG_OK", world)


if __name__ == "__main__":
    try:
        main()
    except BaseException:  # noqa: BLE001 - the launcher swallows child tracebacks; keep ours
        import traceback
        with open(sys.argv[3] + "." + os.environ.get("RANK", "x"), "w") as f:
            traceback.print_exc(file=f)
        raise
