"""Properties that do not depend on size, checked on a configuration-2-shaped index too large for the
CPU oracle (400,000 x 96 fp32, 2,000 lists, pq 48 x 8 bits, built on the GPU): order and validity of
the results, recall against exact brute force, invariance under internal batching, list sharding
and the choice of kernels, self-retrieval of database vectors."""
import numpy as np
import pytest

from conftest import make_mixture

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

N, DIM, LISTS, K = 400_000, 96, 2000, 10


@pytest.fixture(scope="module")
def big(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    g = torch.Generator(device="cuda").manual_seed(3)
    centers = torch.randn((1024, DIM), generator=g, device="cuda")
    centers /= centers.norm(dim=1, keepdim=True)
    scale = torch.exp(torch.empty((1024, 1), device="cuda").uniform_(np.log(0.05), np.log(0.5), generator=g))

    def draw(n):
        c = torch.randint(0, 1024, (n,), generator=g, device="cuda")
        x = centers[c] + scale[c] * torch.randn((n, DIM), generator=g, device="cuda") / np.sqrt(DIM)
        return (x / x.norm(dim=1, keepdim=True)).contiguous()

    x, q = draw(N), draw(2000)
    params = ivf_pq.IndexParams(n_lists=LISTS, pq_dim=48, pq_bits=8, kmeans_n_iters=8,
                                kmeans_trainset_fraction=0.2)
    index = ivf_pq.build(params, x)
    path = str(tmp_path_factory.mktemp("big") / "big.ivfpq")
    ivf_pq.save(path, index)
    # exact neighbours
    truth = torch.empty((q.shape[0], K), dtype=torch.int64, device="cuda")
    for s in range(0, q.shape[0], 500):
        d = torch.cdist(q[s:s + 500], x)
        truth[s:s + 500] = d.topk(K, dim=1, largest=False).indices
    return dict(ivf=ivf_pq, index=index, x=x, q=q, truth=truth, path=path)


def recall(found, truth):
    hit = (found.unsqueeze(2) == truth.unsqueeze(1)).any(dim=2).sum().item()
    return hit / truth.numel()


def test_rows_are_sorted_valid_and_free_of_duplicates(big):
    ivf = big["ivf"]
    sp = ivf.SearchParams(n_probes=30, lut_dtype=np.float16)
    d, i = ivf.search(sp, big["index"], big["q"], 50)
    assert (d[:, 1:] >= d[:, :-1]).all()
    assert (i >= 0).all() and (i < N).all()
    srt = i.sort(dim=1).values
    assert (srt[:, 1:] != srt[:, :-1]).all()


def test_recall_grows_with_probes_and_refinement_reaches_the_target(big):
    from cuvs_b200 import refine
    ivf = big["ivf"]
    rec = []
    for p in (5, 20, 80):
        sp = ivf.SearchParams(n_probes=p, lut_dtype=np.float16)
        _, i = ivf.search(sp, big["index"], big["q"], K)
        rec.append(recall(i, big["truth"]))
    assert rec[0] <= rec[1] + 0.005 and rec[1] <= rec[2] + 0.005
    assert rec[2] > 0.6
    sp = ivf.SearchParams(n_probes=80, lut_dtype=np.float16)
    _, cand = ivf.search(sp, big["index"], big["q"], 4 * K)
    d, i = refine(big["x"], big["q"], cand, k=K)
    assert recall(i, big["truth"]) >= 0.95
    # refined distances are the exact squared distances of the returned ids
    exact = ((big["q"].unsqueeze(1) - big["x"][i]) ** 2).sum(dim=2)
    assert torch.allclose(d, exact, rtol=1e-4, atol=1e-6)


def test_internal_batching_and_kernel_choices_do_not_change_a_bit(big):
    from cuvs_b200 import _lib as L
    ivf = big["ivf"]
    lib = L.load()
    q = big["q"]
    base = ivf.search(ivf.SearchParams(n_probes=20, lut_dtype=np.float16), big["index"], q, K)
    small = ivf.search(ivf.SearchParams(n_probes=20, lut_dtype=np.float16, max_internal_batch_size=333),
                       big["index"], q, K)
    assert (base[1] == small[1]).all() and (base[0].view(torch.int32) == small[0].view(torch.int32)).all()
    try:
        for coarse, home in ((1, 0), (13, 1), (11, 0)):
            L.check(lib.cuvsB200SetCoarseMode(coarse))
            L.check(lib.cuvsB200SetScanCodebookHome(home))
            other = ivf.search(ivf.SearchParams(n_probes=20, lut_dtype=np.float16), big["index"], q, K)
            assert (base[1] == other[1]).all()
            assert (base[0].view(torch.int32) == other[0].view(torch.int32)).all()
    finally:
        L.check(lib.cuvsB200SetCoarseMode(0))
        L.check(lib.cuvsB200SetScanCodebookHome(0))


def test_three_list_shards_merge_to_the_unsharded_result(big):
    from cuvs_b200 import mg
    ivf = big["ivf"]
    q = big["q"]
    sp = ivf.SearchParams(n_probes=20, lut_dtype=np.float16)
    d_full, i_full = ivf.search(sp, big["index"], q, K)
    probes = mg.select_probes(big["index"], q, 20)
    parts = []
    total = 0
    for r in range(3):
        shard = mg.load_shard(big["path"], r, 3)
        total += int(shard.list_sizes.sum().item())
        parts.append(mg.search_with_probes(sp, shard, q, probes, K))
    assert total == N
    d, i = mg.merge_parts(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]), True)
    # distances bit for bit; ids wherever the distance is not shared with a neighbour in the row or
    # with the k-th place (the merge orders equal distances by id, the one-index search by position
    # in the probed lists, and f16 look-up tables do produce equal distances)
    assert (d.view(torch.int32) == d_full.view(torch.int32)).all()
    tied = torch.zeros_like(i, dtype=torch.bool)
    tied[:, 1:] |= d[:, 1:] == d[:, :-1]
    tied[:, :-1] |= d[:, :-1] == d[:, 1:]
    tied |= d == d[:, -1:]
    assert ((i == i_full) | tied).all()
    assert tied[:, :-1].float().mean().item() < 0.05      # the k-th place always counts as tied


def test_database_vectors_find_themselves(big):
    ivf = big["ivf"]
    rows = torch.arange(0, N, N // 1000, device="cuda")[:1000]
    sp = ivf.SearchParams(n_probes=10, lut_dtype=np.float32)
    _, i = ivf.search(sp, big["index"], big["x"][rows].contiguous(), 5)
    assert ((i == rows.unsqueeze(1)).any(dim=1).float().mean().item()) >= 0.95
