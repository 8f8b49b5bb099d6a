"""GPU parity tests of the search with coarse_search_dtype = CUDA_R_8I (the reference's int8 coarse
search, cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:171-256 with the operands of
cpp/src/neighbors/ivf_pq_index.cu:624-738): int8 images of centers, rotation matrix and queries,
int32 coarse scores, rotated queries (R8 q8) / 128^2.  Everything up to the probes is integer
arithmetic, so the bar is the usual one: ids and fp32 distance bits identical to the CPU oracle on
the same serialized index (equal int32 coarse scores are ordered by list id on both sides; the
reference's selection leaves that order open)."""
import numpy as np
import pytest

from conftest import make_mixture
from test_search_gpu import LUT, assert_parity, build_case

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def ivf():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    return ivf_pq


def gpu_search_i8(ivf, index, q, k, n_probes, lut="f32", internal="f32", batch=4096):
    sp = ivf.SearchParams(n_probes=n_probes, lut_dtype=LUT[lut][0], internal_distance_dtype=LUT[internal][0],
                          coarse_search_dtype=np.int8, max_internal_batch_size=batch)
    d, i = ivf.search(sp, index, torch.from_numpy(np.ascontiguousarray(q)).cuda(), k)
    return d.cpu().numpy(), i.cpu().numpy()


@pytest.mark.parametrize("metric,dtype,dim,force_rot", [
    (0, np.float32, 32, False),    # L2, 16 spare int8 columns
    (0, np.float32, 30, True),     # 2 spare columns, random rotation
    (1, np.float32, 47, False),    # sqrt L2, 17 spare columns
    (6, np.float32, 32, False),    # inner product (the norm columns still enter the score)
    (2, np.float32, 40, True),     # cosine
    (0, np.int8, 32, False),
    (0, np.uint8, 32, True),
])
def test_int8_coarse_search_parity(ivf, oracle_mod, tmp_path, metric, dtype, dim, force_rot):
    O = oracle_mod
    pq_dim = 16 if dim != 47 else 24
    x, q, ix, path = build_case(O, tmp_path, "i8", n=4000, dim=dim, n_lists=40, pq_dim=pq_dim,
                                metric=metric, force_rot=force_rot, dtype=dtype, seed=5, nq=96)
    g = ivf.load(path)
    for k, p, lut in ((10, 8, "f32"), (5, 40, "f16"), (33, 3, "fp8")):
        d, i = gpu_search_i8(ivf, g, q, k, p, lut)
        do, io = O.search_int8_coarse(ix, q, k, n_probes=p, lut_dtype=LUT[lut][1])
        assert_parity(d, i, do, io, 1e-5 if lut == "f32" else 1e-2)
    # internal batching does not change the result
    d1, i1 = gpu_search_i8(ivf, g, q, 10, 8, batch=7)
    d2, i2 = gpu_search_i8(ivf, g, q, 10, 8)
    assert (i1 == i2).all() and (d1.view(np.uint32) == d2.view(np.uint32)).all()


def test_int8_coarse_on_the_tensor_core_path(ivf, oracle_mod, tmp_path):
    """Enough lists for the tcgen05 coarse GEMM: its single TF32 product of the integer operands must
    give the int32 scores exactly (no query may need the exact redo for a wrong reason), and the
    SIMT path the same probes."""
    from cuvs_b200 import _lib as L
    O = oracle_mod
    x = (make_mixture(60000, 48, 256, 0.25, seed=90) * 0.5).astype(np.float32)
    q = (make_mixture(300, 48, 256, 0.25, seed=91) * 0.5).astype(np.float32)
    g = ivf.build(ivf.IndexParams(n_lists=4096, pq_dim=24, kmeans_n_iters=3, kmeans_trainset_fraction=0.5),
                  torch.from_numpy(x).cuda())
    path = str(tmp_path / "i8_many.ivfpq")
    ivf.save(path, g)
    ix = O.OracleIndex.load(path)
    do, io = O.search_int8_coarse(ix, q, 10, n_probes=20, lut_dtype=LUT["f16"][1])
    lib = L.load()
    try:
        for mode in (2, 1, 0):
            L.check(lib.cuvsB200SetCoarseMode(mode))
            d, i = gpu_search_i8(ivf, g, q, 10, 20, "f16")
            assert_parity(d, i, do, io, 1e-2)
    finally:
        L.check(lib.cuvsB200SetCoarseMode(0))
    # the int8 coarse search is an approximation of the fp32 one: recall stays close
    gt_d, gt_i = O.brute_force(x, q, 10)
    sp = ivf.SearchParams(n_probes=20, lut_dtype=np.float16)
    _, i32 = ivf.search(sp, g, torch.from_numpy(q).cuda(), 10)
    r8, r32 = O.recall(i, gt_i), O.recall(i32.cpu().numpy(), gt_i)
    assert r8 >= r32 - 0.05, (r8, r32)


def test_int8_coarse_with_half_queries(ivf, oracle_mod, tmp_path):
    O = oracle_mod
    x, q, ix, path = build_case(O, tmp_path, "i8h", n=4000, dim=32, n_lists=40, pq_dim=16, dtype=np.float16,
                                seed=7, nq=64)
    g = ivf.load(path)
    d, i = gpu_search_i8(ivf, g, q, 10, 8)
    do, io = O.search_int8_coarse(ix, q, 10, n_probes=8)
    assert_parity(d, i, do, io, 1e-5)

