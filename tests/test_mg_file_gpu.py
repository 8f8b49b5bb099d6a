"""Multi-GPU index files of the reference's format (cpp/src/neighbors/mg/snmg.cuh:60-91, 780-805): each
rank's index read back by one process per GPU (here: one process, the ranks in turn), row-sharded
search with id translation and merge against the CPU oracle, replicated mode, writer round trip."""
import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def mgfile(oracle_mod, tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    O = oracle_mod
    x = make_mixture(9000, 32, 40, 0.2, seed=21)
    q = make_mixture(80, 32, 40, 0.2, seed=22)
    cuts = [0, 3500, 6200, 9000]       # three unequal row shards
    parts = [O.build_index(x[a:b], 20, pq_dim=16, pq_bits=8, kmeans_iters=3, seed=r)
             for r, (a, b) in enumerate(zip(cuts[:-1], cuts[1:]))]
    d = tmp_path_factory.mktemp("mgfile")
    sharded = str(d / "sharded.mg")
    O.save_mg(sharded, O.SHARDED, parts)
    replicated = str(d / "replicated.mg")
    O.save_mg(replicated, O.REPLICATED, [parts[0], parts[0]])
    return dict(O=O, q=q, parts=parts, cuts=cuts, sharded=sharded, replicated=replicated, dir=d)


def test_row_sharded_file_search_matches_the_oracle(mgfile):
    from cuvs_b200 import ivf_pq, mg
    O, q, parts, cuts = mgfile["O"], mgfile["q"], mgfile["parts"], mgfile["cuts"]
    k, n_probes = 10, 6
    sp = ivf_pq.SearchParams(n_probes=n_probes)
    qd = torch.from_numpy(q).cuda()
    ds, ids, ref = [], [], []
    for r in range(3):
        index, mode, off = mg.load_reference_mg(mgfile["sharded"], r, 3)
        assert mode == mg.SHARDED and off == cuts[r] and len(index) == cuts[r + 1] - cuts[r]
        d, i = ivf_pq.search(sp, index, qd, k)
        do, io = O.search(parts[r], q, k, n_probes=n_probes)
        assert (i.cpu().numpy() == io).all() and (d.cpu().numpy().view(np.uint32) == do.view(np.uint32)).all()
        ds.append(d)
        ids.append(mg.translate_ids(i, off))
        ref.append((do, np.where(io == O.OUT_OF_BOUNDS, io, io + off)))
    d, i = mg.merge_parts(torch.stack(ds), torch.stack(ids), True)
    d, i = d.cpu().numpy(), i.cpu().numpy()
    # the reference's merge on the CPU: k smallest of the 3k candidates per query
    all_d = np.concatenate([r[0] for r in ref], axis=1)
    all_i = np.concatenate([r[1] for r in ref], axis=1)
    order = np.lexsort((all_i, all_d), axis=1)[:, :k]
    want_d = np.take_along_axis(all_d, order, axis=1)
    want_i = np.take_along_axis(all_i, order, axis=1)
    assert (d.view(np.uint32) == want_d.view(np.uint32)).all()
    tied = np.zeros_like(i, dtype=bool)
    tied[:, 1:] |= want_d[:, 1:] == want_d[:, :-1]
    tied[:, :-1] |= want_d[:, :-1] == want_d[:, 1:]
    assert ((i == want_i) | tied).all()
    assert (i < 9000).all() and (i[:, 0] >= 0).all()
    # the same through the one-call wrapper (world size 1: rank 0's shard alone)
    index, mode, off = mg.load_reference_mg(mgfile["sharded"], 1, 3)
    d1, i1 = mg.search_reference_mg(sp, index, mode, off, qd, k)
    assert (i1.cpu().numpy() == ref[1][1]).all()


def test_replicated_file_gives_every_rank_the_whole_index(mgfile):
    from cuvs_b200 import ivf_pq, mg
    O, q, parts = mgfile["O"], mgfile["q"], mgfile["parts"]
    qd = torch.from_numpy(q).cuda()
    sp = ivf_pq.SearchParams(n_probes=5)
    do, io = O.search(parts[0], q, 7, n_probes=5)
    for r in range(2):
        index, mode, off = mg.load_reference_mg(mgfile["replicated"], r, 2)
        assert mode == mg.REPLICATED and off == 0 and len(index) == parts[0].size
        d, i = mg.search_reference_mg(sp, index, mode, off, qd, 7)
        assert (i.cpu().numpy() == io).all()


def test_writer_is_byte_identical_to_the_oracle_writer_and_errors_mirror_the_reference(mgfile):
    from cuvs_b200 import _lib as L
    from cuvs_b200 import mg
    shards = [mg.load_reference_mg(mgfile["sharded"], r, 3)[0] for r in range(3)]
    out = str(mgfile["dir"] / "rewritten.mg")
    mg.save_reference_mg(out, shards, mg.SHARDED)
    assert open(out, "rb").read() == open(mgfile["sharded"], "rb").read()
    with pytest.raises(L.CuvsError, match="Serialized index has 3 ranks whereas NCCL clique has 2 ranks"):
        mg.load_reference_mg(mgfile["sharded"], 0, 2)
    with pytest.raises(L.CuvsError, match="Cannot open file"):
        mg.load_reference_mg(str(mgfile["dir"] / "missing.mg"), 0, 3)
    blob = open(mgfile["sharded"], "rb").read()
    cut = str(mgfile["dir"] / "cut.mg")
    open(cut, "wb").write(blob[: len(blob) * 2 // 3])
    with pytest.raises(L.CuvsError):
        mg.load_reference_mg(cut, 2, 3)
