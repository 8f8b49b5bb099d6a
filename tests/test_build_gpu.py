"""GPU tests of index construction through the C interface: recall against exact brute force (the
reference's own criterion, cpp/tests/neighbors/ann_ivf_pq.cuh:639-689) and, because the oracle
searches any index obeying the data contract, id-level parity on the GPU-built index too."""
import numpy as np
import pytest

from conftest import make_mixture
from test_search_gpu import LUT, assert_parity, gpu_search

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ivf():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    return ivf_pq


def min_recall(n_probes, n_lists, compression_ratio):
    """cpp/tests/neighbors/ann_ivf_pq.cuh:639-656."""
    from math import erfc
    p = n_probes / n_lists
    return min(erfc(0.05 * compression_ratio / max(p, 0.5)), p)


@pytest.mark.parametrize("host", [False, True])
def test_build_search_recall_and_parity(ivf, oracle_mod, tmp_path, host):
    O = oracle_mod
    x = make_mixture(20000, 64, 64, 0.15, seed=10)
    q = make_mixture(256, 64, 64, 0.15, seed=11)
    params = ivf.IndexParams(n_lists=64, pq_dim=32, pq_bits=8, kmeans_n_iters=10,
                             kmeans_trainset_fraction=1.0)
    g = ivf.build(params, x if host else torch.from_numpy(x).cuda())
    assert len(g) == 20000 and g.n_lists == 64 and g.pq_dim == 32
    sizes = g.list_sizes.cpu().numpy()
    assert sizes.sum() == 20000
    k, p = 32, 16
    d, i = gpu_search(ivf, g, q, k, p)
    gt_d, gt_i = O.brute_force(x, q, k)
    rec = O.recall(i, gt_i)
    cr = 64 * 4 / 32
    assert rec >= min_recall(p, 64, cr) * 0.98, rec
    assert rec > 0.8, rec
    assert (i >= 0).all() and (i < 20000).all()
    assert all(len(set(r.tolist())) == k for r in i)      # no duplicates
    # same index through the file format into the oracle: id-level parity
    path = str(tmp_path / "gpu_built.ivfpq")
    ivf.save(path, g)
    ix = O.OracleIndex.load(path)
    do, io = O.search(ix, q, k, n_probes=p)
    assert_parity(d, i, do, io, 1e-5)
    assert abs(O.recall(io, gt_i) - rec) <= 0.002


@pytest.mark.parametrize("bits,kind,metric", [(4, "subspace", "sqeuclidean"), (6, "cluster", "sqeuclidean"),
                                              (8, "subspace", "inner_product"), (5, "subspace", "cosine"),
                                              (8, "cluster", "euclidean")])
def test_build_variants(ivf, oracle_mod, tmp_path, bits, kind, metric):
    O = oracle_mod
    x = make_mixture(8000, 40, 40, 0.2, seed=20)
    q = make_mixture(100, 40, 40, 0.2, seed=21)
    params = ivf.IndexParams(n_lists=32, pq_dim=40, pq_bits=bits, codebook_kind=kind, metric=metric,
                             kmeans_n_iters=8, kmeans_trainset_fraction=1.0)
    g = ivf.build(params, torch.from_numpy(x).cuda())
    mcode = {"sqeuclidean": 0, "euclidean": 1, "cosine": 2, "inner_product": 6}[metric]
    d, i = gpu_search(ivf, g, q, 10, 16)
    gt_d, gt_i = O.brute_force(x, q, 10, mcode)
    rec = O.recall(i, gt_i)
    assert rec > (0.5 if bits < 6 else 0.7), rec
    path = str(tmp_path / "v.ivfpq")
    ivf.save(path, g)
    ix = O.OracleIndex.load(path)
    do, io = O.search(ix, q, 10, n_probes=16)
    assert_parity(d, i, do, io, 1e-5)


def test_random_rotation_build(ivf, oracle_mod):
    x = make_mixture(6000, 30, 30, 0.2, seed=30)
    q = make_mixture(64, 30, 30, 0.2, seed=31)
    g = ivf.build(ivf.IndexParams(n_lists=16, pq_dim=8, kmeans_n_iters=5, force_random_rotation=True),
                  torch.from_numpy(x).cuda())
    R = g.rotation_matrix.cpu().numpy().astype(np.float64)
    assert R.shape == (32, 30)
    assert np.allclose(R.T @ R, np.eye(30), atol=1e-5)      # orthonormal columns
    d, i = gpu_search(ivf, g, q, 10, 16)
    gt_d, gt_i = oracle_mod.brute_force(x, q, 10)
    assert oracle_mod.recall(i, gt_i) > 0.4


def test_extend_and_ids(ivf, oracle_mod):
    O = oracle_mod
    x = make_mixture(9000, 32, 32, 0.15, seed=40)
    q = make_mixture(64, 32, 32, 0.15, seed=41)
    params = ivf.IndexParams(n_lists=32, pq_dim=16, kmeans_n_iters=6, add_data_on_build=False,
                             kmeans_trainset_fraction=1.0)
    xd = torch.from_numpy(x).cuda()
    g = ivf.build(params, xd)
    assert len(g) == 0
    ids = np.arange(9000, dtype=np.int64) + 100000
    ivf.extend(g, xd[:3000], torch.from_numpy(ids[:3000]).cuda())
    ivf.extend(g, xd[3000:], torch.from_numpy(ids[3000:]).cuda())
    assert len(g) == 9000
    d, i = gpu_search(ivf, g, q, 10, 32)
    assert (i >= 100000).all() and (i < 109000).all()
    gt_d, gt_i = O.brute_force(x, q, 10)
    assert O.recall(i - 100000, gt_i) > 0.7
    # one-shot build places the same vectors: same neighbour sets as the two-step extend
    g2 = ivf.build(ivf.IndexParams(n_lists=32, pq_dim=16, kmeans_n_iters=6,
                                   kmeans_trainset_fraction=1.0), xd)
    d2, i2 = gpu_search(ivf, g2, q, 10, 32)
    assert np.mean([len(set(a - 100000) & set(b)) / 10 for a, b in zip(i, i2)]) > 0.99
    from cuvs_b200._lib import CuvsError
    with pytest.raises(CuvsError, match="must pass data indices"):
        ivf.extend(g, xd[:10], None)


def test_lists_are_balanced_on_skewed_data(ivf):
    """Balanced k-means (the reference's adjust_centers step, cpp/src/cluster/detail/kmeans_balanced.cuh:616-720):
    on a mixture whose components differ 50-fold in weight, no list ends far above the mean size and few
    end far below it.  Plain Lloyd leaves the heavy components in a few huge lists."""
    import torch
    rng = np.random.default_rng(5)
    n, dim, n_comp, n_lists = 200_000, 32, 48, 1024
    cent = rng.uniform(-1.0, 1.0, size=(n_comp, dim)).astype(np.float32)
    w = np.geomspace(1.0, 50.0, n_comp)
    comp = rng.choice(n_comp, size=n, p=w / w.sum())
    x = (cent[comp] + 0.2 * rng.standard_normal((n, dim))).astype(np.float32)
    g = ivf.build(ivf.IndexParams(n_lists=n_lists, pq_dim=16, kmeans_n_iters=12, kmeans_trainset_fraction=0.5),
                  torch.from_numpy(x).cuda())
    sizes = g.list_sizes.to(torch.int64).cpu().numpy()
    assert sizes.sum() == n
    mean = n / n_lists
    print(f"list sizes: max {sizes.max() / mean:.2f} x mean, {np.mean(sizes < mean / 4):.3f} below a quarter of it")
    assert sizes.max() <= 4.0 * mean
    assert np.mean(sizes < mean / 4) <= 0.05


def test_transform_equals_stored_codes(ivf):
    """python/cuvs/cuvs/tests/test_ivf_pq.py test_transform: codes of `transform` equal what build stored."""
    x = make_mixture(4000, 32, 32, 0.15, seed=50)
    xd = torch.from_numpy(x).cuda()
    g = ivf.build(ivf.IndexParams(n_lists=16, pq_dim=16, pq_bits=6, kmeans_n_iters=5), xd)
    labels, codes = ivf.transform(g, xd)
    labels, codes = labels.cpu().numpy().astype(np.int64), codes.cpu().numpy()
    for l in (0, 7, 15):
        stored_ids = g.list_indices(l).cpu().numpy()
        stored = g.list_data(l).cpu().numpy()
        assert (labels[stored_ids] == l).all()
        assert (codes[stored_ids] == stored).all()


def test_flat_codes_layout_builds_extends_and_round_trips_but_is_not_searched(oracle_mod, tmp_path):
    """codes_layout = FLAT (list_spec_flat, cpp/include/cuvs/neighbors/ivf_pq.hpp:308-360): every vector's
    codes are one bit-packed row.  Such an index is built, extended, written, read and unpacked; its rows
    are the rows `unpack_contiguous_list_data` gives for the interleaved index of the same build; the
    search refuses it with the reference's message (ivf_pq_search.cuh:915-917)."""
    import torch
    from cuvs_b200 import ivf_pq
    from cuvs_b200._lib import CuvsError
    O = oracle_mod
    x = make_mixture(5000, 40, 30, 0.2, seed=21)
    xd = torch.from_numpy(x).cuda()
    kw = dict(n_lists=20, pq_dim=20, pq_bits=6, kmeans_n_iters=4)
    # one trained model, two empty indexes made from it (two independent trainings need not agree to the
    # last bit: the k-means sums are accumulated with atomics), filled by the same two extend calls
    model = ivf_pq.build(ivf_pq.IndexParams(add_data_on_build=False, **kw), xd[:4000])
    parts = (model.pq_centers, model.centers, model.centers_rot, model.rotation_matrix)
    inter = ivf_pq.build_precomputed(ivf_pq.IndexParams(**kw), 40, *parts)
    flat = ivf_pq.build_precomputed(ivf_pq.IndexParams(codes_layout="flat", **kw), 40, *parts)
    for index in (inter, flat):
        ivf_pq.extend(index, xd[:4000], torch.arange(0, 4000, device="cuda"))
        ivf_pq.extend(index, xd[4000:], torch.arange(4000, 5000, device="cuda"))
    assert len(flat) == 5000 and (flat.list_sizes == inter.list_sizes).all()
    for l in (0, 7, 19):
        assert (flat.list_data(l) == inter.list_data(l)).all()
        assert (flat.list_indices(l) == inter.list_indices(l)).all()
    # file: the layout scalar and per-list [size, bytes_per_vector] records
    path = str(tmp_path / "flat.ivfpq")
    ivf_pq.save(path, flat)
    ix = O.OracleIndex.load(path)
    assert ix.codes_layout == 0 and ix.size == 5000
    for l in (0, 7, 19):
        n = int(ix.list_sizes[l])
        assert ix.list_codes[l].shape == (n, 15)
        assert (ix.list_codes[l] == flat.list_data(l).cpu().numpy()).all()
    ix.save(str(tmp_path / "flat2.ivfpq"))
    assert open(path, "rb").read() == open(str(tmp_path / "flat2.ivfpq"), "rb").read()
    back = ivf_pq.load(path)
    assert (back.list_data(7) == flat.list_data(7)).all()
    with pytest.raises(CuvsError, match="FLAT layout is not supported"):
        ivf_pq.search(ivf_pq.SearchParams(n_probes=4), back, xd[:8].contiguous(), 5)
