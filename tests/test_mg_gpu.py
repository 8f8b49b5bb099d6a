"""List-sharded search over NCCL on two GPUs of one box (skipped where fewer are visible): every rank
gets exactly the single-GPU result."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_two_ranks_over_nccl_equal_the_single_gpu_search(oracle_mod, tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    x = make_mixture(12000, 48, 64, 0.2, seed=9)
    q = make_mixture(300, 48, 64, 0.2, seed=10)
    ix = oracle_mod.build_index(x, 96, pq_dim=24, pq_bits=8, kmeans_iters=3, seed=0)
    path, qpath = str(tmp_path / "mg.ivfpq"), str(tmp_path / "q.npy")
    ix.save(path)
    # the same data as an inner-product index: there the LARGEST distances win the merge
    oracle_mod.build_index(x, 96, pq_dim=24, pq_bits=8, metric=oracle_mod.InnerProduct, kmeans_iters=3,
                           seed=0).save(path + ".ip")
    np.save(qpath, q)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mg_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", worker, path, qpath,
                        str(tmp_path / "trace")],
                       env=env, capture_output=True, text=True, timeout=600)
    traces = "".join(open(tmp_path / f).read() for f in sorted(os.listdir(tmp_path)) if f.startswith("trace."))
    assert r.returncode == 0, traces or (r.stdout[-2000:] + r.stderr[-2000:])
    assert "MG_OK 2" in r.stdout
