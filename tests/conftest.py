import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def make_mixture(n, dim, n_centers, sigma, seed, dtype=np.float32, lo=-1.0, hi=1.0):
    """Seeded Gaussian-mixture data, the shape of the benchmark configurations in miniature."""
    rng = np.random.default_rng(seed)
    cent = rng.uniform(lo, hi, size=(n_centers, dim)).astype(np.float32)
    x = cent[rng.integers(0, n_centers, size=n)] + sigma * rng.standard_normal((n, dim)).astype(np.float32)
    if dtype == np.uint8:
        return np.clip(np.rint(x), 0, 255).astype(np.uint8)
    if dtype == np.int8:
        return np.clip(np.rint(x), -128, 127).astype(np.int8)
    return x.astype(dtype)


@pytest.fixture(scope="session")
def oracle_mod():
    from oracle import oracle as O
    O.lib()
    return O


@pytest.fixture(scope="session")
def small_l2(oracle_mod, tmp_path_factory):
    """4000 x 32 fp32, 32 lists, pq 16 x 8 bits, L2 -- with its serialized file."""
    O = oracle_mod
    x = make_mixture(4000, 32, 40, 0.15, seed=0)
    q = make_mixture(100, 32, 40, 0.15, seed=1)
    ix = O.build_index(x, 32, pq_dim=16, pq_bits=8, kmeans_iters=4, seed=0)
    path = str(tmp_path_factory.mktemp("ix") / "small_l2.ivfpq")
    ix.save(path)
    return {"x": x, "q": q, "ix": ix, "path": path}
