"""Dynamic batching front-end (cpp/tests/neighbors/dynamic_batching.cuh of the reference: single
queries submitted from many threads must get the answers of a direct upstream search)."""
import threading

import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def setup(oracle_mod, tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    x = make_mixture(20000, 64, 64, 0.2, seed=5)
    q = make_mixture(600, 64, 64, 0.2, seed=6)
    ix = oracle_mod.build_index(x, 128, pq_dim=32, pq_bits=8, kmeans_iters=3, seed=0)
    path = str(tmp_path_factory.mktemp("db") / "db.ivfpq")
    ix.save(path)
    g = ivf_pq.load(path)
    sp = ivf_pq.SearchParams(n_probes=16, lut_dtype=np.float16)
    qd = torch.from_numpy(q).cuda()
    d, i = ivf_pq.search(sp, g, qd, 10)
    return g, sp, qd, d.cpu().numpy(), i.cpu().numpy()


@pytest.mark.parametrize("max_batch,n_queues,n_threads,rows", [(64, 3, 32, 1), (4, 1, 16, 1), (100, 2, 8, 7),
                                                                 (16, 3, 12, 40)])
def test_threads_get_the_answers_of_a_direct_search(setup, max_batch, n_queues, n_threads, rows):
    from cuvs_b200 import dynamic_batching as db
    from cuvs_b200.common import Resources
    g, sp, qd, d_ref, i_ref = setup
    index = db.Index(g, sp, k=10, max_batch_size=max_batch, n_queues=n_queues)
    nq = qd.shape[0]
    out_d = torch.zeros((nq, 10), dtype=torch.float32, device="cuda")
    out_i = torch.zeros((nq, 10), dtype=torch.int64, device="cuda")
    errors = []
    starts = list(range(0, nq, rows))

    def worker(t):
        try:
            torch.cuda.set_device(0)
            res = Resources()                       # one handle per host thread
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                res.use_current_stream()
                for s in starts[t::n_threads]:
                    e = min(nq, s + rows)
                    db.search(index, qd[s:e], out_i[s:e], out_d[s:e], dispatch_timeout_ms=0.5,
                              resources=res, sync=False)
                res.sync()
        except Exception as exc:                    # noqa: BLE001 - reported by the main thread
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(n_threads)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout=120)
    assert not errors, errors
    assert not any(th.is_alive() for th in threads)
    torch.cuda.synchronize()
    assert (out_i.cpu().numpy() == i_ref).all()
    assert (out_d.cpu().numpy().view(np.uint32) == d_ref.view(np.uint32)).all()
    n_batches, n_rows = index.stats()
    assert n_rows == nq
    assert n_batches >= -(-nq // max_batch)
    if rows == 1 and n_threads >= 8 * max(1, max_batch // 16):
        assert n_batches < nq                       # requests really were gathered


def test_a_request_larger_than_the_batch_is_split(setup):
    from cuvs_b200 import dynamic_batching as db
    g, sp, qd, d_ref, i_ref = setup
    index = db.Index(g, sp, k=10, max_batch_size=32, n_queues=2)
    d, i = db.search(index, qd[:150], dispatch_timeout_ms=0.1)
    assert (i.cpu().numpy() == i_ref[:150]).all()
    assert (d.cpu().numpy().view(np.uint32) == d_ref[:150].view(np.uint32)).all()
    assert index.stats() == (5, 150)


def test_argument_errors(setup):
    from cuvs_b200 import dynamic_batching as db
    from cuvs_b200 import _lib as L
    g, sp, qd, _, _ = setup
    index = db.Index(g, sp, k=10)
    with pytest.raises(L.CuvsError, match="k is fixed"):
        db.search(index, qd[:4], torch.empty((4, 5), dtype=torch.int64, device="cuda"),
                  torch.empty((4, 5), dtype=torch.float32, device="cuda"))
    with pytest.raises(L.CuvsError, match="query dimensions"):
        db.search(index, qd[:4, :32].contiguous())
    with pytest.raises(L.CuvsError, match="max_batch_size"):
        db.Index(g, sp, k=10, max_batch_size=0)


def test_a_failed_upstream_search_fails_its_whole_batch_and_nobody_hangs(setup):
    """The dispatcher thread's upstream search fails (injected on the host): every request gathered
    into that batch gets the error, no thread is left waiting, and the next batch is served."""
    import threading
    from cuvs_b200 import dynamic_batching as db
    from cuvs_b200 import _lib as L
    from cuvs_b200.common import Resources
    g, sp, qd, d_ref, i_ref = setup
    index = db.Index(g, sp, k=10, max_batch_size=8, n_queues=1)
    index.fail_next()
    outcome = [None] * 8

    def worker(t):
        res = Resources()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            res.use_current_stream()
            try:
                db.search(index, qd[t:t + 1], dispatch_timeout_ms=2000.0, resources=res)
                outcome[t] = "ok"
            except L.CuvsError as exc:
                outcome[t] = str(exc)

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(8)]
    for th in threads:
        th.start()
    for th in threads:
        th.join(timeout=60)
    assert not any(th.is_alive() for th in threads), "a caller is still waiting"
    assert all(o is not None and "injected" in o for o in outcome), outcome
    # the queue is usable again
    d, i = db.search(index, qd[:8], dispatch_timeout_ms=0.1)
    assert (i.cpu().numpy() == i_ref[:8]).all()


def test_upstream_parameters_are_checked_when_the_index_is_made(setup):
    from cuvs_b200 import dynamic_batching as db
    from cuvs_b200 import ivf_pq
    from cuvs_b200 import _lib as L
    g, _, _, _, _ = setup
    bad = ivf_pq.SearchParams(n_probes=4, lut_dtype=np.float32, internal_distance_dtype=np.float16)
    with pytest.raises(L.CuvsError, match="lut_dtype / internal_distance_dtype"):
        db.Index(g, bad, k=10)
