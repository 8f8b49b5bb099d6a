"""GPU test of cuvsIvfPqPredictNoAlloc, the entry point for callers that cannot allocate device
memory while they run (memory fully pre-claimed by a host framework, threads that must not take
cudaMalloc's driver lock, sandboxed plug-ins).  Its scratch is a fixed array inside the library, so
the test calls it twice in a row -- the second call sees the first call's leftovers -- and checks
both results, through the C interface, against the labels of the regular cuvsIvfPqTransform.
Collected last on purpose: a stop-at-first-failure run has then exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def predict_no_alloc(index, vectors):
    from cuvs_b200 import _lib as L
    from cuvs_b200.common import DLTensorRef, default_resources
    res = default_resources()
    res.use_current_stream()
    labels = torch.empty((vectors.shape[0],), dtype=torch.uint32, device="cuda")
    v, l = DLTensorRef(vectors), DLTensorRef(labels)
    L.check(L.load().cuvsIvfPqPredictNoAlloc(res.handle, index._h, v.ref(), l.ref()))
    res.sync()
    return labels.cpu().numpy().astype(np.int64)


def test_predict_no_alloc_matches_transform_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    from cuvs_b200._lib import CuvsError
    x = make_mixture(6000, 40, 48, 0.2, seed=60)
    xd = torch.from_numpy(x).cuda()
    index = ivf_pq.build(ivf_pq.IndexParams(n_lists=100, pq_dim=20, kmeans_n_iters=5), xd)
    a = torch.from_numpy(make_mixture(5000, 40, 48, 0.2, seed=61)).cuda()
    b = torch.from_numpy(make_mixture(777, 40, 48, 0.2, seed=62)).cuda()
    want_a = ivf_pq.transform(index, a)[0].cpu().numpy().astype(np.int64)
    want_b = ivf_pq.transform(index, b)[0].cpu().numpy().astype(np.int64)
    got_a = predict_no_alloc(index, a)       # first call: resolves the scratch address
    got_b = predict_no_alloc(index, b)       # second call: scratch holds the first call's values
    assert (got_a == want_a).all()
    assert (got_b == want_b).all()
    assert (predict_no_alloc(index, a) == want_a).all()
    # other element types go through the same entry point
    h = a.half()
    assert (predict_no_alloc(index, h) == ivf_pq.transform(index, h)[0].cpu().numpy()).all()
    # sizes beyond the fixed scratch are refused with a clear message
    big = torch.zeros((65537, 40), dtype=torch.float32, device="cuda")
    with pytest.raises(CuvsError, match="at most 65536 rows"):
        predict_no_alloc(index, big)
    assert predict_no_alloc(index, a[:0]).shape == (0,)
