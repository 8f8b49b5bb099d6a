"""GPU parity tests: the CUDA search path, called through the C interface (ctypes), against the
CPU oracle on the same serialized index and the same seeded inputs.

Bar: neighbour ids and fp32 distance bits identical to the oracle.  The comparator also accepts a
row that differs only where distances tie within the stated tolerance (relative 1e-5 for an fp32
look-up table, 1e-2 for fp16 / 8-bit tables) and bounds how many rows may do so.
"""
import os

import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

LUT = {"f32": (np.float32, 0), "f16": (np.float16, 2), "fp8": (np.uint8, 8)}


@pytest.fixture(scope="module")
def ivf():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    return ivf_pq


@pytest.fixture(autouse=True, params=["codebook-auto", "codebook-not-in-tmem", "lut-in-global-memory"])
def scan_codebook_home(request, ivf):
    """Every test of this module runs three times: with the fine-search kernel keeping the per-subspace
    codebook in tensor memory wherever it fits (the default), with tensor memory ruled out (codebook in
    shared or global memory), and with the variant for look-up tables too large for shared memory
    (one table per CTA in global memory) forced on every shape."""
    from cuvs_b200 import _lib as L
    L.check(L.load().cuvsB200SetScanCodebookHome(
        {"codebook-auto": 0, "codebook-not-in-tmem": 1, "lut-in-global-memory": 3}[request.param]))
    yield
    L.check(L.load().cuvsB200SetScanCodebookHome(0))


def assert_parity(d_gpu, i_gpu, d_orc, i_orc, rel_tol, max_tie_rows=0.01):
    d_gpu, i_gpu = np.asarray(d_gpu), np.asarray(i_gpu)
    assert d_gpu.shape == d_orc.shape and i_gpu.shape == i_orc.shape
    same_ids = (i_gpu == i_orc).all(axis=1)
    n_bad = 0
    for r in np.nonzero(~same_ids)[0]:
        # rows may differ only inside runs of tied distances (ids swapped or replaced at a tie)
        og = dict(zip(i_orc[r].tolist(), d_orc[r].tolist()))
        kth = d_orc[r][-1]
        for idv, dv in zip(i_gpu[r].tolist(), d_gpu[r].tolist()):
            ref = og.get(idv, kth)
            assert abs(dv - ref) <= rel_tol * max(abs(ref), 1e-30) + 1e-30, (r, idv, dv, ref)
        n_bad += 1
    assert n_bad <= max_tie_rows * len(same_ids), f"{n_bad} rows differ (ties)"
    m = same_ids
    a, b = d_gpu[m], d_orc[m]
    fin = np.isfinite(b)
    assert (np.isfinite(a) == fin).all()
    assert (a[fin].view(np.uint32) == b[fin].view(np.uint32)).all(), \
        f"max rel diff {np.max(np.abs(a[fin] - b[fin]) / np.maximum(np.abs(b[fin]), 1e-30))}"


def gpu_search(ivf, index, q, k, n_probes, lut="f32", internal="f32", batch=4096):
    sp = ivf.SearchParams(n_probes=n_probes, lut_dtype=LUT[lut][0],
                          internal_distance_dtype=LUT[internal][0], max_internal_batch_size=batch)
    qd = torch.from_numpy(np.ascontiguousarray(q)).cuda()
    d, i = ivf.search(sp, index, qd, k)
    return d.cpu().numpy(), i.cpu().numpy()


def build_case(O, tmp_path, name, n=3000, dim=32, n_lists=24, pq_dim=16, pq_bits=8, metric=0,
               kind=0, force_rot=False, dtype=np.float32, seed=0, nq=64):
    if dtype in (np.uint8, np.int8):
        lo, hi, sigma = (20, 200, 12.0) if dtype == np.uint8 else (-90, 90, 12.0)
        x = make_mixture(n, dim, 30, sigma, seed, dtype, lo, hi)
        q = make_mixture(nq, dim, 30, sigma, seed + 1, dtype, lo, hi)
    else:
        x = make_mixture(n, dim, 30, 0.15, seed, dtype)
        q = make_mixture(nq, dim, 30, 0.15, seed + 1, dtype)
    ix = O.build_index(x, n_lists, pq_dim=pq_dim, pq_bits=pq_bits, metric=metric,
                       codebook_kind=kind, force_random_rotation=force_rot, kmeans_iters=3, seed=seed)
    path = str(tmp_path / f"{name}.ivfpq")
    ix.save(path)
    return x, q, ix, path


# ------------------------------------------------------------------------------------------------
def test_deserialize_matches_oracle_arrays(ivf, oracle_mod, small_l2):
    ix = small_l2["ix"]
    g = ivf.load(small_l2["path"])
    assert (g.n_lists, g.dim, g.pq_dim, g.pq_bits, g.pq_len, len(g)) == \
        (ix.n_lists, ix.dim, ix.pq_dim, ix.pq_bits, ix.pq_len, ix.size)
    assert (g.centers_padded.cpu().numpy() == ix.centers).all()
    assert (g.centers.cpu().numpy() == ix.centers[:, :ix.dim]).all()
    assert (g.pq_centers.cpu().numpy() == ix.pq_centers).all()
    assert (g.centers_rot.cpu().numpy() == ix.centers_rot).all()
    assert (g.rotation_matrix.cpu().numpy() == ix.rotation).all()
    assert (g.list_sizes.cpu().numpy().astype(np.uint32) == ix.list_sizes).all()
    for l in (0, 5, ix.n_lists - 1):
        n = int(ix.list_sizes[l])
        assert (g.list_indices(l).cpu().numpy() == ix.list_ids[l][:n]).all()
        if n:
            flat = g.list_data(l).cpu().numpy()
            codes = oracle_mod.unpack_list(ix.list_codes[l], n, ix.pq_dim, ix.pq_bits)
            assert (flat == codes).all()   # pq_bits = 8: one byte per code


def test_search_parity_fp32(ivf, oracle_mod, small_l2):
    g = ivf.load(small_l2["path"])
    for k, p in ((10, 8), (1, 1), (32, 32), (5, 1000)):
        d, i = gpu_search(ivf, g, small_l2["q"], k, p)
        do, io = oracle_mod.search(small_l2["ix"], small_l2["q"], k, n_probes=p)
        assert_parity(d, i, do, io, 1e-5, max_tie_rows=0.0)


@pytest.mark.parametrize("lut,internal", [("f16", "f32"), ("fp8", "f32"), ("f16", "f16"), ("fp8", "f16")])
def test_search_parity_lut_dtypes(ivf, oracle_mod, small_l2, lut, internal):
    g = ivf.load(small_l2["path"])
    d, i = gpu_search(ivf, g, small_l2["q"], 10, 8, lut, internal)
    do, io = oracle_mod.search(small_l2["ix"], small_l2["q"], 10, n_probes=8,
                               lut_dtype=LUT[lut][1], internal_dtype=LUT[internal][1])
    assert_parity(d, i, do, io, 1e-2)


@pytest.mark.parametrize("bits,pq_dim", [(4, 16), (5, 8), (6, 12), (7, 8), (8, 19)])
def test_search_parity_pq_bits(ivf, oracle_mod, tmp_path, bits, pq_dim):
    x, q, ix, path = build_case(oracle_mod, tmp_path, f"b{bits}", dim=38 if pq_dim == 19 else 32,
                                pq_dim=pq_dim, pq_bits=bits)
    g = ivf.load(path)
    for lut in ("f32", "fp8"):
        d, i = gpu_search(ivf, g, q, 10, 6, lut)
        do, io = oracle_mod.search(ix, q, 10, n_probes=6, lut_dtype=LUT[lut][1])
        assert_parity(d, i, do, io, 1e-5 if lut == "f32" else 1e-2)


@pytest.mark.parametrize("metric", [0, 1, 6, 2])
@pytest.mark.parametrize("kind", [0, 1])
def test_search_parity_metrics_and_codebooks(ivf, oracle_mod, tmp_path, metric, kind):
    x, q, ix, path = build_case(oracle_mod, tmp_path, f"m{metric}k{kind}", metric=metric, kind=kind,
                                n=2000, n_lists=16)
    g = ivf.load(path)
    for lut in ("f32", "f16", "fp8"):
        d, i = gpu_search(ivf, g, q, 10, 5, lut)
        do, io = oracle_mod.search(ix, q, 10, n_probes=5, lut_dtype=LUT[lut][1])
        assert_parity(d, i, do, io, 1e-5 if lut == "f32" else 1e-2)


def test_search_parity_random_rotation_and_padding(ivf, oracle_mod, tmp_path):
    # dim 30 with pq_dim 8 -> pq_len 4, rot_dim 32 != dim: a real rotation matrix
    x, q, ix, path = build_case(oracle_mod, tmp_path, "rot", dim=30, pq_dim=8, force_rot=True)
    assert ix.rot_dim == 32
    g = ivf.load(path)
    d, i = gpu_search(ivf, g, q, 10, 6)
    do, io = oracle_mod.search(ix, q, 10, n_probes=6)
    assert_parity(d, i, do, io, 1e-5)


@pytest.mark.parametrize("dtype", [np.uint8, np.int8, np.float16])
def test_search_parity_element_types(ivf, oracle_mod, tmp_path, dtype):
    x, q, ix, path = build_case(oracle_mod, tmp_path, f"t{np.dtype(dtype).name}", dtype=dtype)
    g = ivf.load(path)
    d, i = gpu_search(ivf, g, q, 10, 6, "fp8" if dtype != np.float16 else "f16")
    do, io = oracle_mod.search(ix, q, 10, n_probes=6,
                               lut_dtype=8 if dtype != np.float16 else 2)
    assert_parity(d, i, do, io, 1e-2)
    if dtype == np.uint8:   # distances come back in the units of the source data
        gt_d, gt_i = oracle_mod.brute_force(x, q, 10)
        assert np.median(d[:, 0] / (gt_d[:, 0] * 65536.0 + 1e-9)) == pytest.approx(1.0, rel=0.5)


@pytest.mark.parametrize("k", [1, 31, 32, 33, 64, 65, 100, 128])
def test_search_parity_k_boundaries(ivf, oracle_mod, small_l2, k):
    g = ivf.load(small_l2["path"])
    d, i = gpu_search(ivf, g, small_l2["q"][:32], k, 6, "f16")
    do, io = oracle_mod.search(small_l2["ix"], small_l2["q"][:32], k, n_probes=6, lut_dtype=2)
    assert_parity(d, i, do, io, 1e-2)


def test_ragged_and_empty_lists(ivf, oracle_mod, tmp_path):
    """List sizes 0, 1, 31, 32, 33 and a query batch of one."""
    O = oracle_mod
    x, q, ix, path = build_case(O, tmp_path, "ragged", n=600, n_lists=8, nq=16)
    # rebuild the lists by hand with the wanted sizes
    sizes = [0, 1, 31, 32, 33, 0, 64, 97]
    rng = np.random.default_rng(0)
    codes, ids, nxt = [], [], 0
    for s in sizes:
        c = rng.integers(0, 256, size=(s, ix.pq_dim), dtype=np.uint8)
        codes.append(O.pack_list(c, 8) if s else np.zeros(0, np.uint8))
        ids.append(np.arange(nxt, nxt + s, dtype=np.int64) * 3 + 7)
        nxt += s
    ix.list_sizes = np.array(sizes, dtype=np.uint32)
    ix.list_codes, ix.list_ids, ix._flat = codes, ids, None
    ix.save(path)
    g = ivf.load(path)
    for nq in (1, 16):
        for p in (1, 3, 8):
            d, i = gpu_search(ivf, g, q[:nq], 20, p)
            do, io = O.search(ix, q[:nq], 20, n_probes=p)
            assert_parity(d, i, do, io, 1e-5)
            assert ((i == O.OUT_OF_BOUNDS) == (io == O.OUT_OF_BOUNDS)).all()


def test_internal_batching_does_not_change_results(ivf, oracle_mod, small_l2):
    g = ivf.load(small_l2["path"])
    d1, i1 = gpu_search(ivf, g, small_l2["q"], 10, 8, batch=4096)
    d2, i2 = gpu_search(ivf, g, small_l2["q"], 10, 8, batch=7)
    assert (i1 == i2).all() and (d1.view(np.uint32) == d2.view(np.uint32)).all()


def test_serialize_round_trip_is_byte_identical(ivf, oracle_mod, small_l2, tmp_path):
    g = ivf.load(small_l2["path"])
    out = str(tmp_path / "resaved.ivfpq")
    ivf.save(out, g)
    assert open(out, "rb").read() == open(small_l2["path"], "rb").read()
    ix2 = oracle_mod.OracleIndex.load(out)
    assert (ix2.list_sizes == small_l2["ix"].list_sizes).all()


def test_argument_errors_mirror_the_reference(ivf, small_l2):
    from cuvs_b200._lib import CuvsError
    g = ivf.load(small_l2["path"])
    q = torch.from_numpy(small_l2["q"]).cuda()
    with pytest.raises(CuvsError, match="Number of query dimensions"):
        ivf.search(ivf.SearchParams(), g, q[:, :16].contiguous(), 5)
    with pytest.raises(CuvsError, match="must not be larger"):
        ivf.search(ivf.SearchParams(), g, q, 128, neighbors=torch.empty((100, len(g) + 1), dtype=torch.int64, device="cuda"),
                   distances=torch.empty((100, len(g) + 1), device="cuda"))
    with pytest.raises(CuvsError, match="n_probes"):
        ivf.search(ivf.SearchParams(n_probes=0), g, q, 5)
    with pytest.raises(CuvsError, match="lut_dtype / internal_distance_dtype"):
        ivf.search(ivf.SearchParams(lut_dtype=np.float32, internal_distance_dtype=np.float16), g, q, 5)
    with pytest.raises(CuvsError, match="neighbors should be of type int64_t"):
        ivf.search(ivf.SearchParams(), g, q, 5, neighbors=torch.empty((100, 5), dtype=torch.int32, device="cuda"))
    with pytest.raises(CuvsError, match="device compatible"):
        ivf.search(ivf.SearchParams(), g, small_l2["q"], 5)
    with pytest.raises(CuvsError, match="Cannot open file"):
        ivf.load("/nonexistent/file.ivfpq")


def test_truncated_file_is_rejected(ivf, small_l2, tmp_path):
    from cuvs_b200._lib import CuvsError
    blob = open(small_l2["path"], "rb").read()
    for cut in (10, 700, len(blob) // 2, len(blob) - 9):
        p = str(tmp_path / f"cut{cut}.ivfpq")
        open(p, "wb").write(blob[:cut])
        with pytest.raises(CuvsError):
            ivf.load(p)
    p = str(tmp_path / "badver.ivfpq")
    import struct
    off = 10 + struct.unpack("<H", blob[8:10])[0]      # payload of the first record (the version)
    assert blob[off] == 4
    open(p, "wb").write(blob[:off] + bytes([5]) + blob[off + 1:])
    with pytest.raises(CuvsError, match="serialization version mismatch"):
        ivf.load(p)


def test_list_sharded_search_merges_to_the_unsharded_result(ivf, oracle_mod, small_l2):
    """Both shards of a 2-way list sharding on one GPU: shard loader + merge kernel."""
    from cuvs_b200 import mg
    q = torch.from_numpy(small_l2["q"]).cuda()
    full = ivf.load(small_l2["path"])
    sp = ivf.SearchParams(n_probes=8)
    d_full, i_full = ivf.search(sp, full, q, 10)
    parts = []
    sizes = []
    for r in range(2):
        shard = mg.load_shard(small_l2["path"], r, 2)
        sizes.append(shard.list_sizes.cpu().numpy())
        parts.append(ivf.search(sp, shard, q, 10))
    ref_sizes = small_l2["ix"].list_sizes
    owner = np.array(mg.list_owners(ref_sizes, 2))
    for r in range(2):
        assert (sizes[r][owner == r] == ref_sizes[owner == r]).all() and (sizes[r][owner != r] == 0).all()
    assert abs(int(sizes[0].sum()) - int(sizes[1].sum())) <= int(ref_sizes.max())
    pd = torch.stack([p[0] for p in parts])
    pi = torch.stack([p[1] for p in parts])
    d, i = mg.merge_parts(pd, pi, True)
    assert (i == i_full).all()
    assert (d.view(torch.int32) == d_full.view(torch.int32)).all()
    # select_max on negated distances gives the same ids (the inner-product direction)
    d2, i2 = mg.merge_parts(-pd, pi, False)
    assert (i2 == i_full).all()


def test_a_shard_with_fewer_rows_than_k_is_searched_and_padded(ivf, small_l2):
    """One rank of a many-way list sharding holds fewer rows than k.  The sharded entry must not refuse
    it (an error on one rank alone would leave the others waiting in a collective): the rank returns what
    it has and pads; the merge over all ranks equals the unsharded result."""
    from cuvs_b200 import mg
    q = torch.from_numpy(small_l2["q"][:50]).cuda()
    full = ivf.load(small_l2["path"])
    n_ranks, k = 16, 300
    sp = ivf.SearchParams(n_probes=int(full.n_lists))
    d_full, i_full = ivf.search(sp, full, q, k)
    probes = mg.select_probes(full, q, int(full.n_lists))
    parts = []
    small = 0
    for r in range(n_ranks):
        shard = mg.load_shard(small_l2["path"], r, n_ranks)
        small += int(shard.list_sizes.to(torch.int64).sum().item()) < k
        parts.append(mg.search_with_probes(sp, shard, q, probes, k))
    assert small > 0, "the case needs at least one shard smaller than k"
    d, i = mg.merge_parts(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]), True)
    assert (d.view(torch.int32) == d_full.view(torch.int32)).all()
    # ids equal except inside runs of equal distances (the merge orders those by id)
    tie = torch.zeros_like(i, dtype=torch.bool)
    eq = d[:, 1:] == d[:, :-1]
    tie[:, 1:] |= eq
    tie[:, :-1] |= eq
    assert ((i == i_full) | tie).all()


# ------------------------------------------------------------------------------------------------
# probe selection stage alone: exact SIMT path, tensor-core path and the oracle must agree
# ------------------------------------------------------------------------------------------------
def coarse_select(index, q, n_probes, mode):
    import ctypes as C
    from cuvs_b200 import _lib as L
    from cuvs_b200.common import DLTensorRef, default_resources
    res = default_resources()
    res.use_current_stream()
    qd = torch.from_numpy(np.ascontiguousarray(q)).cuda()
    probes = torch.empty((q.shape[0], n_probes), dtype=torch.uint32, device="cuda")
    scores = torch.empty((q.shape[0], n_probes), dtype=torch.float32, device="cuda")
    status = (C.c_uint32 * 2)()
    a, b, c = DLTensorRef(qd), DLTensorRef(probes), DLTensorRef(scores)
    L.check(L.load().cuvsB200CoarseSelect(res.handle, C.cast(index._h, C.c_void_p), a.ref(), b.ref(),
                                          c.ref(), mode, status))
    return probes.cpu().numpy().astype(np.uint32), scores.cpu().numpy(), (status[0], status[1])


@pytest.fixture(scope="module")
def many_lists(ivf):
    """120,000 x 64 fp32 in 8,192 lists (enough lists for the tensor-core path)."""
    x = make_mixture(120000, 64, 512, 0.25, seed=70)
    g = ivf.build(ivf.IndexParams(n_lists=8192, pq_dim=32, kmeans_n_iters=3,
                                  kmeans_trainset_fraction=0.5), torch.from_numpy(x).cuda())
    return x, g


@pytest.mark.parametrize("nq,n_probes", [(1, 1), (7, 20), (128, 32), (300, 40), (1000, 20), (500, 64)])
def test_coarse_tensor_core_path_equals_exact_path(ivf, oracle_mod, many_lists, tmp_path, nq, n_probes):
    x, g = many_lists
    q = make_mixture(nq, 64, 512, 0.25, seed=71 + nq)
    p1, s1, st1 = coarse_select(g, q, n_probes, 1)
    p2, s2, st2 = coarse_select(g, q, n_probes, 2)
    assert st2[0] == 0, "device-side wait timed out"
    assert (p1 == p2).all()
    assert (s1.view(np.uint32) == s2.view(np.uint32)).all()
    print(f"exact-path fallbacks: {st2[1]} of {nq}")
    assert st2[1] <= max(1, nq // 20), f"{st2[1]} of {nq} queries fell back to the exact path"
    # and both equal the oracle's selection on the same model
    path = str(tmp_path / "many.ivfpq")
    ivf.save(path, g)
    ix = oracle_mod.OracleIndex.load(path)
    fq, _ = oracle_mod.prepare_queries(ix, q)
    po, so = oracle_mod.select_clusters(ix, fq, n_probes)
    assert (po == p1).all()
    assert (so.view(np.uint32) == s1.view(np.uint32)).all()


def test_coarse_tensor_core_path_with_more_than_512_half_tiles(ivf):
    """70,000 lists: the finish kernel that takes its threshold from the half-tile maxima and re-reads
    only the qualifying half tiles' keys; probes and scores equal the exact path's."""
    x = make_mixture(140000, 32, 4096, 0.3, seed=90)
    g = ivf.build(ivf.IndexParams(n_lists=70000, pq_dim=16, kmeans_n_iters=2,
                                  kmeans_trainset_fraction=1.0), torch.from_numpy(x).cuda())
    q = make_mixture(600, 32, 4096, 0.3, seed=91)
    for n_probes in (20, 100):
        p1, s1, _ = coarse_select(g, q, n_probes, 1)
        p2, s2, st = coarse_select(g, q, n_probes, 2)
        assert st[0] == 0
        assert (p1 == p2).all() and (s1.view(np.uint32) == s2.view(np.uint32)).all()
        assert st[1] <= len(q) // 20


def test_search_is_identical_under_both_coarse_paths(ivf, many_lists):
    from cuvs_b200 import _lib as L
    x, g = many_lists
    q = make_mixture(500, 64, 512, 0.25, seed=80)
    lib = L.load()
    try:
        L.check(lib.cuvsB200SetCoarseMode(1))
        d1, i1 = gpu_search(ivf, g, q, 10, 24, "f16")
        L.check(lib.cuvsB200SetCoarseMode(2))
        d2, i2 = gpu_search(ivf, g, q, 10, 24, "f16")
    finally:
        L.check(lib.cuvsB200SetCoarseMode(0))
    assert (i1 == i2).all() and (d1.view(np.uint32) == d2.view(np.uint32)).all()


@pytest.mark.parametrize("mode", [11, 12, 13, 21, 22])
def test_coarse_tensor_core_products_all_give_the_exact_probes(ivf, many_lists, mode):
    """The tensor-core coarse GEMM may issue 1, 2 or 3 products of the TF32 operand split per K step
    (a handle starts with 2 and raises the number if too many queries need the exact redo); the guard
    widens its error bound accordingly, so the probes and their scores equal the exact path's.
    Modes 11 and 12 keep the query tile resident in shared memory on this shape, 21 and 22 stream
    both operands."""
    from cuvs_b200 import _lib as L
    x, g = many_lists
    q = make_mixture(700, 64, 512, 0.25, seed=81)
    lib = L.load()
    try:
        p1, s1, _ = coarse_select(g, q, 20, 1)
        L.check(lib.cuvsB200SetCoarseMode(mode))
        p2, s2, st = coarse_select(g, q, 20, 2)
    finally:
        L.check(lib.cuvsB200SetCoarseMode(0))
    assert st[0] == 0
    assert (p1 == p2).all() and (s1.view(np.uint32) == s2.view(np.uint32)).all()
    assert st[1] <= len(q) // 20          # the exact redo stays the exception


def test_a_wait_that_runs_out_is_reported_and_the_probes_stay_exact(ivf, many_lists):
    """Every wait in the tensor-core coarse kernel is bounded.  Here one operand stage is never filled
    and the limit is shortened to a few milliseconds: the kernel gives up, sets its error word and
    returns; the stages behind it recompute every query of the batch exactly; the handle counts the
    event; the search result is the one of a healthy run; the GPU keeps answering."""
    import ctypes as C
    from cuvs_b200 import _lib as L
    from cuvs_b200.common import default_resources
    x, g = many_lists
    q = make_mixture(300, 64, 512, 0.25, seed=90)
    lib = L.load()
    res = default_resources()
    n0 = C.c_uint64(0)
    p1, s1, _ = coarse_select(g, q, 20, 1)
    d1, i1 = gpu_search(ivf, g, q, 10, 20, "f16")
    L.check(lib.cuvsStreamSync(res.handle))
    L.check(lib.cuvsB200CoarseTimeouts(res.handle, C.byref(n0)))
    try:
        L.check(lib.cuvsB200SetCoarseWaitTest(4000, 2))
        p2, s2, st = coarse_select(g, q, 20, 2)
        assert st[0] == 1, "the kernel should have reported the wait that ran out"
        assert st[1] == len(q), "every query of the batch is redone exactly"
        assert (p1 == p2).all() and (s1.view(np.uint32) == s2.view(np.uint32)).all()
        d2, i2 = gpu_search(ivf, g, q, 10, 20, "f16")
    finally:
        L.check(lib.cuvsB200SetCoarseWaitTest(0, 0))
    assert (i1 == i2).all() and (d1.view(np.uint32) == d2.view(np.uint32)).all()
    L.check(lib.cuvsStreamSync(res.handle))
    n1 = C.c_uint64(0)
    L.check(lib.cuvsB200CoarseTimeouts(res.handle, C.byref(n1)))
    assert n1.value > n0.value
    # and a healthy run afterwards
    p3, s3, st3 = coarse_select(g, q, 20, 2)
    assert st3[0] == 0 and (p3 == p1).all()
    with pytest.raises(L.CuvsError, match="spin_limit"):
        L.check(lib.cuvsB200SetCoarseWaitTest(10, 0))


@pytest.mark.parametrize("k,lut,internal", [(129, "f32", "f32"), (200, "f16", "f32"), (513, "fp8", "f16")])
def test_search_parity_large_k_store_all_path(ivf, oracle_mod, small_l2, k, lut, internal):
    """k > 128 switches to the mode where the scan stores every score and a selection follows
    (the reference's non-fused kernel, cpp/tests/neighbors/ann_ivf_pq.cuh var_k cases)."""
    g = ivf.load(small_l2["path"])
    q = small_l2["q"][:48]
    for p in (6, 32):
        d, i = gpu_search(ivf, g, q, k, p, lut, internal)
        do, io = oracle_mod.search(small_l2["ix"], q, k, n_probes=p, lut_dtype=LUT[lut][1],
                                   internal_dtype=LUT[internal][1])
        assert_parity(d, i, do, io, 1e-5 if lut == "f32" else 1e-2, max_tie_rows=0.05)
        assert ((i == oracle_mod.OUT_OF_BOUNDS) == (io == oracle_mod.OUT_OF_BOUNDS)).all()


def test_search_with_given_probes_equals_plain_search(ivf, many_lists):
    """The two halves of the shared probe selection: select_probes then search_with_probes."""
    from cuvs_b200 import mg
    x, g = many_lists
    q = torch.from_numpy(make_mixture(333, 64, 512, 0.25, seed=90)).cuda()
    sp = ivf.SearchParams(n_probes=24, lut_dtype=np.float16)
    d0, i0 = ivf.search(sp, g, q, 10)
    probes = torch.cat([mg.select_probes(g, q[:100], 24), mg.select_probes(g, q[100:], 24)])
    d1, i1 = mg.search_with_probes(sp, g, q, probes, 10)
    assert (i0 == i1).all() and (d0.view(torch.int32) == d1.view(torch.int32)).all()


def test_bitset_filter_parity(ivf, oracle_mod, small_l2):
    """cpp/tests/neighbors/ann_ivf_pq.cuh:724-876: a bitset removes ids from the search; here a
    random third of the ids plus the first 300, checked id-for-id against the filtered oracle."""
    O = oracle_mod
    ix, q = small_l2["ix"], small_l2["q"]
    n = ix.size
    rng = np.random.default_rng(11)
    allowed = rng.random(n) > 0.33
    allowed[:300] = False
    words = np.zeros((n + 31) // 32, dtype=np.uint32)
    idx = np.nonzero(allowed)[0]
    np.bitwise_or.at(words, idx // 32, (np.uint32(1) << (idx % 32).astype(np.uint32)))
    g = ivf.load(small_l2["path"])
    qd = torch.from_numpy(q).cuda()
    fd = torch.from_numpy(words.view(np.int32)).cuda().view(torch.uint32)
    for k, p, lut in ((10, 8, "f32"), (40, 32, "fp8"), (200, 16, "f16")):
        sp = ivf.SearchParams(n_probes=p, lut_dtype=LUT[lut][0])
        d, i = ivf.search(sp, g, qd, k, filter=fd)
        d, i = d.cpu().numpy(), i.cpu().numpy()
        do, io = O.search(ix, q, k, n_probes=p, lut_dtype=LUT[lut][1], bitset=words)
        assert_parity(d, i, do, io, 1e-5 if lut == "f32" else 1e-2, max_tie_rows=0.05)
        found = i[i != O.OUT_OF_BOUNDS]
        assert allowed[found].all()


def test_a_table_larger_than_shared_memory_goes_to_global_memory(ivf, oracle_mod, tmp_path):
    """pq_dim 256 x 8 bits with an fp32 table is 256 KB: no shared-memory plan exists, the search takes
    the variant with the table in global memory (the reference's conf_no_smem_lut) and still equals
    the oracle."""
    O = oracle_mod
    x, q, ix, path = build_case(O, tmp_path, "wide", n=2500, dim=256, n_lists=16, pq_dim=256, pq_bits=8, nq=40)
    g = ivf.load(path)
    for k, p in ((10, 6), (150, 16)):
        d, i = gpu_search(ivf, g, q, k, p, "f32")
        do, io = O.search(ix, q, k, n_probes=p)
        assert_parity(d, i, do, io, 1e-5)
