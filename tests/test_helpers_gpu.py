"""GPU tests of the single-list helpers (the reference's ivf_pq::helpers namespace) through the C
interface.  Codes, list bytes and ids are compared bit for bit with the CPU oracle's statement of
the list layout; decoded vectors within a stated tolerance (the reference's own test compares
reconstructed vectors with the encoder input through a loose norm bound,
cpp/tests/neighbors/ann_ivf_pq.cuh:268-330, and packs/unpacks through the same helpers :332-440)."""
import numpy as np
import pytest

from conftest import make_mixture
from test_search_gpu import assert_parity, gpu_search

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import helpers, ivf_pq
    return ivf_pq, helpers


def build_small(ivf, bits=8, kind="subspace", pq_dim=20, dim=40, n=6000, force_rot=False):
    x = make_mixture(n, dim, 24, 0.2, seed=40 + bits)
    params = ivf.IndexParams(n_lists=24, pq_dim=pq_dim, pq_bits=bits, codebook_kind=kind,
                             kmeans_n_iters=6, kmeans_trainset_fraction=1.0,
                             force_random_rotation=force_rot)
    return x, ivf.build(params, torch.from_numpy(x).cuda())


def to_oracle(ivf, O, g, tmp_path, name="h.ivfpq"):
    path = str(tmp_path / name)
    ivf.save(path, g)
    return O.OracleIndex.load(path)


def biggest_list(g):
    sizes = g.list_sizes.cpu().numpy()
    return int(sizes.argmax()), int(sizes.max())


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
def test_unpack_list_data_matches_the_layout(mods, oracle_mod, tmp_path, bits):
    ivf, H = mods
    O = oracle_mod
    # pq_bits * pq_dim must be a multiple of 8; 22 and 24 leave a partly filled last 16-byte piece
    _, g = build_small(ivf, bits=bits, pq_dim={4: 22, 5: 24, 6: 20, 7: 24, 8: 21}[bits])
    ix = to_oracle(ivf, O, g, tmp_path)
    label, n = biggest_list(g)
    want = O.unpack_list(ix.list_codes[label], n, ix.pq_dim, bits)
    got = H.unpack_list_data(g, label).cpu().numpy()
    assert got.shape == (n, g.pq_dim) and (got == want).all()
    # a window, and rows picked by position
    got = H.unpack_list_data(g, label, offset=37, n_rows=45).cpu().numpy()
    assert (got == want[37:82]).all()
    rows = np.random.default_rng(1).integers(0, n, 50).astype(np.uint32)
    got = H.unpack_list_data(g, label, in_cluster_indices=torch.from_numpy(rows).cuda()).cpu().numpy()
    assert (got == want[rows]).all()
    # the bit-packed form of the same rows
    flat = g.list_data(label).cpu().numpy()
    assert (flat == O.pack_contiguous(want, bits)).all()


@pytest.mark.parametrize("bits", [4, 5, 7, 8])
def test_pack_list_data_writes_the_layout(mods, oracle_mod, tmp_path, bits):
    ivf, H = mods
    O = oracle_mod
    _, g = build_small(ivf, bits=bits, pq_dim={4: 18, 5: 24, 7: 24, 8: 19}[bits])
    label, n = biggest_list(g)
    before = H.unpack_list_data(g, label).cpu().numpy()
    rng = np.random.default_rng(bits)
    new = rng.integers(0, 1 << bits, (60, g.pq_dim)).astype(np.uint8)
    H.pack_list_data(g, torch.from_numpy(new).cuda(), label, offset=33)
    want = before.copy()
    want[33:93] = new
    assert (H.unpack_list_data(g, label).cpu().numpy() == want).all()
    # list bytes as the file holds them: exactly the oracle's packing (padding bits stay zero)
    ix = to_oracle(ivf, O, g, tmp_path)
    assert (ix.list_codes[label].reshape(-1) == O.pack_list(want, bits).reshape(-1)).all()
    # the bit-packed writer produces the same bytes
    newer = rng.integers(0, 1 << bits, (41, g.pq_dim)).astype(np.uint8)
    H.pack_contiguous_list_data(g, torch.from_numpy(O.pack_contiguous(newer, bits)).cuda(), label, offset=2)
    want[2:43] = newer
    assert (H.unpack_list_data(g, label).cpu().numpy() == want).all()
    ix = to_oracle(ivf, O, g, tmp_path, "h2.ivfpq")
    assert (ix.list_codes[label].reshape(-1) == O.pack_list(want, bits).reshape(-1)).all()
    # other lists are untouched
    other = (label + 1) % g.n_lists
    ix0 = to_oracle(ivf, O, g, tmp_path, "h3.ivfpq")
    m = int(g.list_sizes[other].item())
    assert (H.unpack_list_data(g, other).cpu().numpy()
            == O.unpack_list(ix0.list_codes[other], m, ix0.pq_dim, bits)).all()


@pytest.mark.parametrize("bits,kind,force_rot", [(8, "subspace", False), (4, "cluster", False),
                                                 (6, "subspace", True)])
def test_reconstruct_list_data(mods, oracle_mod, tmp_path, bits, kind, force_rot):
    ivf, H = mods
    O = oracle_mod
    x, g = build_small(ivf, bits=bits, kind=kind, pq_dim=20, dim=40, force_rot=force_rot)
    ix = to_oracle(ivf, O, g, tmp_path)
    label, n = biggest_list(g)
    want = O.reconstruct_list(ix, label, np.arange(n))
    got = H.reconstruct_list_data(g, label).cpu().numpy()
    # fp32 sum of rot_dim products against a float64 sum: 1e-5 of the vector scale
    tol = 1e-5 * max(1.0, float(np.abs(want).max()))
    assert got.shape == (n, g.dim) and np.abs(got - want).max() <= tol
    rows = np.random.default_rng(2).integers(0, n, 33).astype(np.uint32)
    got_rows = H.reconstruct_list_data(g, label, in_cluster_indices=torch.from_numpy(rows).cuda()).cpu().numpy()
    assert (got_rows == got[rows]).all()
    assert (H.reconstruct_list_data(g, label, offset=5, n_rows=17).cpu().numpy() == got[5:22]).all()
    # the decoded vectors approximate what was encoded (the reference's criterion is a norm bound)
    ids = g.list_indices(label).cpu().numpy()[:n]
    err = np.linalg.norm(got - x[ids], axis=1) / np.linalg.norm(x[ids], axis=1)
    assert np.median(err) < (0.2 if bits >= 6 else 0.35), np.median(err)
    # other output types are the reference's mapping of the same fp32 values
    for dt in (np.float16, np.int8, np.uint8):
        out = H.reconstruct_list_data(g, label, dtype=dt).cpu().numpy()
        # int8 clamps out-of-range values; uint8 is compared on the values its range holds
        same = np.ones_like(got, dtype=bool) if dt != np.uint8 else (got >= 0.0) & (got < 0.99)
        assert (out[same] == O.map_from_float(got, dt)[same]).all()


def test_extend_list_with_codes_and_search_parity(mods, oracle_mod, tmp_path):
    ivf, H = mods
    O = oracle_mod
    x, g = build_small(ivf, bits=8, pq_dim=20)
    q = make_mixture(64, 40, 24, 0.2, seed=77)
    label, n = biggest_list(g)
    small = int(g.list_sizes.cpu().numpy().argmin())
    codes = H.unpack_list_data(g, label, n_rows=50)
    size0 = len(g)
    ids_a = torch.arange(100000, 100050, dtype=torch.int64, device="cuda")
    H.extend_list_with_codes(g, codes, ids_a, small)
    packed = g.list_data(label, n_rows=30, offset=50)
    ids_b = torch.arange(200000, 200030, dtype=torch.int64, device="cuda")
    H.extend_list_with_contiguous_codes(g, packed, ids_b, small)
    assert len(g) == size0 + 80
    m = int(g.list_sizes[small].item())
    got = H.unpack_list_data(g, small).cpu().numpy()
    assert (got[m - 80:m - 30] == codes.cpu().numpy()).all()
    assert (got[m - 30:] == H.unpack_list_data(g, label, offset=50, n_rows=30).cpu().numpy()).all()
    ids = g.list_indices(small).cpu().numpy()[:m]
    assert (ids[m - 80:m - 30] == ids_a.cpu().numpy()).all() and (ids[m - 30:] == ids_b.cpu().numpy()).all()
    # the changed index still searches exactly as the oracle searches its file
    ix = to_oracle(ivf, O, g, tmp_path)
    assert ix.size == size0 + 80
    d, i = gpu_search(ivf, g, q, 10, 24)
    do, io = O.search(ix, q, 10, n_probes=24)
    assert_parity(d, i, do, io, 1e-5)


@pytest.mark.parametrize("dtype", [np.float32, np.int8])
def test_extend_list_encodes_like_build(mods, dtype):
    ivf, H = mods
    x = make_mixture(5000, 32, 16, 0.2, seed=90)
    if dtype == np.int8:
        x = np.clip(np.round(x * 100), -127, 127).astype(np.int8)
    g = ivf.build(ivf.IndexParams(n_lists=16, pq_dim=16, pq_bits=6, kmeans_n_iters=6,
                                  kmeans_trainset_fraction=1.0), torch.from_numpy(x).cuda())
    label, n = biggest_list(g)
    codes = H.unpack_list_data(g, label).cpu().numpy()
    ids = g.list_indices(label)[:n].clone()
    H.erase_list(g, label)
    assert int(g.list_sizes[label].item()) == 0 and len(g) == 5000 - n
    # the same vectors, forced into the same list, get the same codes and keep their ids
    vecs = torch.from_numpy(x).cuda()[ids]
    H.extend_list(g, vecs[: n // 2].contiguous(), ids[: n // 2].contiguous(), label)
    H.extend_list(g, vecs[n // 2:].contiguous(), ids[n // 2:].contiguous(), label)
    assert len(g) == 5000 and int(g.list_sizes[label].item()) == n
    assert (H.unpack_list_data(g, label).cpu().numpy() == codes).all()
    assert (g.list_indices(label)[:n] == ids).all()


def test_erase_list_and_reset_index(mods, oracle_mod, tmp_path):
    ivf, H = mods
    O = oracle_mod
    x, g = build_small(ivf, bits=8, pq_dim=20)
    q = make_mixture(64, 40, 24, 0.2, seed=78)
    label, n = biggest_list(g)
    gone = set(g.list_indices(label).cpu().numpy()[:n].tolist())
    H.erase_list(g, label)
    assert len(g) == 6000 - n and int(g.list_sizes[label].item()) == 0
    d, i = gpu_search(ivf, g, q, 10, 24)
    assert not (set(i.reshape(-1).tolist()) & gone)
    ix = to_oracle(ivf, O, g, tmp_path)
    do, io = O.search(ix, q, 10, n_probes=24)
    assert_parity(d, i, do, io, 1e-5)
    H.reset_index(g)
    assert len(g) == 0 and int(g.list_sizes.sum().item()) == 0
    # the model is still there: the emptied index can be filled again
    ivf.extend(g, torch.from_numpy(x).cuda(), torch.arange(6000, dtype=torch.int64, device="cuda"))
    assert len(g) == 6000


def test_row_ranges_are_checked(mods):
    ivf, H = mods
    from cuvs_b200._lib import CuvsError
    _, g = build_small(ivf, bits=8, pq_dim=20)
    label, n = biggest_list(g)
    with pytest.raises(CuvsError, match="not bigger than the cluster size"):
        H.unpack_list_data(g, label, offset=n - 3, n_rows=4)
    with pytest.raises(CuvsError, match="not bigger than the cluster size"):
        H.reconstruct_list_data(g, label, offset=1, n_rows=n)
    with pytest.raises(CuvsError, match="not bigger than the cluster size"):
        H.pack_list_data(g, torch.zeros((4, 20), dtype=torch.uint8, device="cuda"), label, offset=n - 3)
    with pytest.raises(CuvsError, match="out of range"):
        H.erase_list(g, g.n_lists)
    with pytest.raises(CuvsError, match="pq_dim columns"):
        H.pack_list_data(g, torch.zeros((4, 19), dtype=torch.uint8, device="cuda"), label)
