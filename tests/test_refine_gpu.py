"""GPU tests of cuvsRefine (exact re-ranking of candidates) against a float64 numpy statement,
in the spirit of the reference's cpp/tests/neighbors/refine.cu (candidates from brute force with
extra noise, refined result must equal the exact top-k)."""
import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def exact_refine(x, q, cand, k, metric):
    x64, q64 = x.astype(np.float64), q.astype(np.float64)
    out_i = np.zeros((q.shape[0], k), np.int64)
    out_d = np.zeros((q.shape[0], k), np.float64)
    for r in range(q.shape[0]):
        c = cand[r]
        v = x64[c]
        if metric == "inner_product":
            s = -(v @ q64[r])
        elif metric == "cosine":
            s = 1.0 - (v @ q64[r]) / (np.linalg.norm(v, axis=1) * np.linalg.norm(q64[r]))
        else:
            s = ((v - q64[r]) ** 2).sum(1)
        o = np.argsort(s, kind="stable")[:k]
        out_i[r] = c[o]
        out_d[r] = s[o]
    if metric == "inner_product":
        out_d = -out_d
    if metric == "euclidean":
        out_d = np.sqrt(out_d)
    return out_d, out_i


@pytest.mark.parametrize("metric", ["sqeuclidean", "euclidean", "inner_product", "cosine"])
@pytest.mark.parametrize("dtype", [np.float32, np.uint8])
def test_refine_matches_exact_reranking(metric, dtype):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import refine
    if dtype == np.uint8:
        x = make_mixture(5000, 48, 20, 15.0, 1, np.uint8, 20, 200)
        q = make_mixture(200, 48, 20, 15.0, 2, np.uint8, 20, 200)
    else:
        x = make_mixture(5000, 48, 20, 0.3, 1)
        q = make_mixture(200, 48, 20, 0.3, 2)
    rng = np.random.default_rng(3)
    cand = np.stack([rng.choice(5000, size=64, replace=False) for _ in range(200)]).astype(np.int64)
    k = 10
    d, i = refine(torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(cand).cuda(),
                  k=k, metric=metric)
    d, i = d.cpu().numpy(), i.cpu().numpy()
    ed, ei = exact_refine(x, q, cand, k, metric)
    same = (i == ei).all(axis=1)
    assert same.mean() > 0.99            # rows may differ only at fp32-level ties
    assert np.allclose(d[same], ed[same], rtol=2e-5, atol=1e-5)


def test_refine_ignores_missing_candidates_and_checks_arguments():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import refine
    from cuvs_b200._lib import CuvsError
    x = make_mixture(1000, 16, 8, 0.3, 4)
    q = make_mixture(8, 16, 8, 0.3, 5)
    cand = np.tile(np.arange(12, dtype=np.int64), (8, 1))
    cand[:, 5:] = np.iinfo(np.int64).max            # only 5 real candidates per query
    d, i = refine(torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(cand).cuda(), k=8)
    i, d = i.cpu().numpy(), d.cpu().numpy()
    assert (np.sort(i[:, :5], axis=1) == np.arange(5)).all()
    assert (i[:, 5:] == np.iinfo(np.int64).max).all() and np.isinf(d[:, 5:]).all()
    with pytest.raises(CuvsError, match="cannot be smaller than k"):
        refine(torch.from_numpy(x).cuda(), torch.from_numpy(q).cuda(), torch.from_numpy(cand[:, :4].copy()).cuda(), k=8)
