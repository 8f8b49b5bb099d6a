"""The reference's single-process multi-GPU interface (cuvsMultiGpuIvfPq*) on every GPU that is visible
(one on a one-GPU box: the same code path with a clique of one; two or more exercise the NCCL
exchanges): list-sharded, replicated and row-sharded indexes give the single-GPU result."""
import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def env(oracle_mod, tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq, mg_ivf_pq
    d = tmp_path_factory.mktemp("snmg")
    x = make_mixture(9000, 40, 50, 0.2, seed=3)
    q = make_mixture(257, 40, 50, 0.2, seed=4)
    out = {}
    for name, metric in (("l2", oracle_mod.L2Expanded), ("ip", oracle_mod.InnerProduct)):
        ix = oracle_mod.build_index(x, 70, pq_dim=20, pq_bits=8, metric=metric, kmeans_iters=3, seed=1)
        out[name] = str(d / f"{name}.ivfpq")
        ix.save(out[name])
    res = mg_ivf_pq.MultiGpuResources()
    return dict(x=x, q=q, files=out, res=res, ivf=ivf_pq, mg=mg_ivf_pq, dir=d, n_gpus=torch.cuda.device_count())


def _single(env, name, k, p, lut=np.float32):
    ivf = env["ivf"]
    g = ivf.load(env["files"][name])
    d, i = ivf.search(ivf.SearchParams(n_probes=p, lut_dtype=lut), g, torch.from_numpy(env["q"]).cuda(), k)
    return d.cpu().numpy(), i.cpu().numpy()


def _same(d0, i0, d1, i1):
    assert (d0.view(np.uint32) == d1.view(np.uint32)).all()
    tied = np.zeros_like(i0, dtype=bool)
    tied[:, 1:] |= d0[:, 1:] == d0[:, :-1]
    tied[:, :-1] |= d0[:, :-1] == d0[:, 1:]
    tied |= d0 == d0[:, -1:]
    assert ((i0 == i1) | tied).all()


@pytest.mark.parametrize("name,k,p", [("l2", 10, 8), ("l2", 200, 12), ("ip", 10, 8), ("ip", 150, 9)])
def test_list_sharded_index_equals_the_single_gpu_search(env, name, k, p):
    mg = env["mg"]
    index = mg.distribute_by_list(env["files"][name], env["res"])
    for rows_per_batch in (1 << 20, 100):
        sp = mg.SearchParams(n_probes=p, n_rows_per_batch=rows_per_batch, merge_mode="merge_on_root_rank")
        d, i = mg.search(sp, index, env["q"], k, resources=env["res"])
        _same(*_single(env, name, k, p), d, i)


def test_replicated_index_and_both_search_modes(env):
    mg = env["mg"]
    index = mg.distribute(env["files"]["l2"], env["res"])
    want = _single(env, "l2", 10, 8)
    for mode in ("load_balancer", "round_robin"):
        sp = mg.SearchParams(n_probes=8, search_mode=mode, n_rows_per_batch=64)
        d, i = mg.search(sp, index, env["q"], 10, resources=env["res"])
        assert (i == want[1]).all() and (d.view(np.uint32) == want[0].view(np.uint32)).all()


def test_build_extend_save_load(env, oracle_mod):
    mg, ivf = env["mg"], env["ivf"]
    x, q = env["x"], env["q"]
    ip = mg.IndexParams(n_lists=64, pq_dim=20, kmeans_n_iters=5, distribution_mode="sharded")
    assert ip.distribution_mode == "sharded"
    index = mg.build(ip, x[:6000], env["res"])
    sp = mg.SearchParams(n_probes=16)
    d, i = mg.search(sp, index, q, 10, resources=env["res"])
    _, truth = oracle_mod.brute_force(x[:6000], q, 10)
    r0 = oracle_mod.recall(i, truth)
    assert r0 > 0.5 and (i < 6000).all()
    # new rows: ids default to old size + position; every row lands on the GPU that holds its list
    mg.extend(index, x[6000:], None, resources=env["res"])
    d, i = mg.search(sp, index, q, 10, resources=env["res"])
    _, truth = oracle_mod.brute_force(x, q, 10)
    assert oracle_mod.recall(i, truth) > 0.5 and i.max() >= 6000 and (i < 9000).all()
    # written as a multi-GPU file of the reference's format (the merged index once per rank) and read back
    path = str(env["dir"] / "built.mg")
    mg.save(index, path, resources=env["res"])
    back = mg.load(path, resources=env["res"])
    d2, i2 = mg.search(sp, back, q, 10, resources=env["res"])
    _same(d, i, d2, i2)
    # its first stream is an ordinary single-GPU index of the whole data
    from oracle import oracle as O
    import io
    blob = open(path, "rb").read()
    f = io.BytesIO(blob[4:])
    assert int(O.read_record(f)) == 0 and int(O.read_record(f)) == env["n_gpus"]
    whole = O.OracleIndex.load(f)
    assert whole.size == 9000
    with pytest.raises(Exception, match="host"):
        mg.search(sp, index, torch.from_numpy(q).cuda(), 10, resources=env["res"])


def test_errors(env):
    from cuvs_b200 import _lib as L
    from cuvs_b200.common import default_resources
    mg = env["mg"]
    index = mg.Index()
    with pytest.raises(ValueError):
        mg.search(mg.SearchParams(), index, env["q"], 5, resources=env["res"])
    with pytest.raises(L.CuvsError, match="multi-GPU resources handle"):
        mg.distribute(env["files"]["l2"], default_resources())
    with pytest.raises(L.CuvsError, match="Cannot open file"):
        mg.distribute_by_list(str(env["dir"] / "missing"), env["res"])
