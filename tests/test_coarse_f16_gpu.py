"""GPU parity tests of the search with coarse_search_dtype = CUDA_R_16F (the reference's half-precision
coarse search, cpp/src/neighbors/ivf_pq/ivf_pq_search.cuh:259-340 and :996-1025): queries, centers and
rotation matrix rounded to half precision, half-precision coarse scores.  The reference leaves the
accumulation of its library GEMMs and the order of equal scores open; the rule implemented and
restated by the oracle is: fp32 fused multiply-adds over ascending k on the half-rounded operands,
the scaled sum rounded once to half, probes ordered by (half score, list id).  Bar: ids and fp32
distance bits identical to the oracle; recall within 0.002 of the fp32 coarse search."""
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


def gpu_search_h(ivf, index, q, k, n_probes, lut="f32", coarse=np.float16, batch=4096):
    sp = ivf.SearchParams(n_probes=n_probes, lut_dtype=LUT[lut][0], coarse_search_dtype=coarse,
                          max_internal_batch_size=batch)
    d, i = ivf.search(sp, index, torch.from_numpy(np.ascontiguousarray(q)).cuda(), k)
    return d.cpu().numpy(), i.cpu().numpy()


@pytest.mark.parametrize("metric,dtype,dim,force_rot", [
    (0, np.float32, 32, False), (0, np.float32, 30, True), (1, np.float16, 32, False),
    (6, np.float32, 32, False), (2, np.float32, 40, True), (0, np.int8, 32, False), (0, np.uint8, 32, True),
])
def test_f16_coarse_search_parity(ivf, oracle_mod, tmp_path, metric, dtype, dim, force_rot):
    O = oracle_mod
    x, q, ix, path = build_case(O, tmp_path, "h", n=4000, dim=dim, n_lists=40, pq_dim=16 if dim != 30 else 15,
                                metric=metric, force_rot=force_rot, dtype=dtype, seed=6, nq=96)
    g = ivf.load(path)
    for k, p, lut in ((10, 8, "f32"), (5, 40, "f16"), (33, 3, "fp8")):
        d, i = gpu_search_h(ivf, g, q, k, p, lut)
        do, io = O.search_f16_coarse(ix, q, k, n_probes=p, lut_dtype=LUT[lut][1])
        assert_parity(d, i, do, io, 1e-5 if lut == "f32" else 1e-2)
    d1, i1 = gpu_search_h(ivf, g, q, 10, 8, batch=7)
    d2, i2 = gpu_search_h(ivf, g, q, 10, 8)
    assert (i1 == i2).all() and (d1.view(np.uint32) == d2.view(np.uint32)).all()


def test_f16_coarse_search_recall_is_that_of_the_fp32_coarse_search(ivf, oracle_mod):
    O = oracle_mod
    x = make_mixture(60000, 64, 300, 0.25, seed=11)
    q = make_mixture(2000, 64, 300, 0.25, seed=12)
    g = ivf.build(ivf.IndexParams(n_lists=3000, pq_dim=32, kmeans_n_iters=4, kmeans_trainset_fraction=0.5),
                  torch.from_numpy(x).cuda())
    _, truth = O.brute_force(x, q, 10)
    rec = {}
    for name, dt in (("f32", np.float32), ("f16", np.float16)):
        _, i = gpu_search_h(ivf, g, q, 10, 12, "f16", coarse=dt)
        rec[name] = O.recall(i, truth)
    assert abs(rec["f16"] - rec["f32"]) <= 0.002, rec
