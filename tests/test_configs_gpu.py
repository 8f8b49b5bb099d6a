"""Id-level parity against the CPU oracle on the shapes of the five benchmark configurations:
configuration 1 exactly (it is small), the others as miniatures that keep what makes each one
different for the kernels -- configuration 2: dim 96, pq 48 x 8, fp16 table, fp32 internal distances,
short lists; 3: uint8 data, pq 64 x 8, 8-bit table, k = 100, lists of a few thousand rows; 4: int8
data, same table, k = 10, longer lists, many probes; 5: fp16 data, inner product, dim 768,
pq 384 x 4 (twelve 16-byte pieces per vector), fp16 table.  Indexes are built on the GPU, written to
a file, and the oracle searches the same file.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from test_search_gpu import assert_parity  # noqa: E402


@pytest.fixture(scope="module")
def ivf():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cuvs_b200 import ivf_pq
    return ivf_pq


def _mixture(n, dim, n_comp, seed, kind):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if kind == "cfg1":       # centres uniform in [-1, 1]^dim, sigma 0.15
        c = torch.rand((n_comp, dim), generator=g, device="cuda") * 2 - 1
        draw = lambda m: c[torch.randint(0, n_comp, (m,), generator=g, device="cuda")] + \
            0.15 * torch.randn((m, dim), generator=g, device="cuda")
    elif kind == "deep":     # L2-normalised anisotropic mixture
        c = torch.randn((n_comp, dim), generator=g, device="cuda")
        s = torch.exp(torch.empty((n_comp, dim), device="cuda").uniform_(np.log(0.05), np.log(0.5), generator=g))
        s = s * c.norm(dim=1, keepdim=True) / np.sqrt(dim)

        def draw(m):
            i = torch.randint(0, n_comp, (m,), generator=g, device="cuda")
            return torch.nn.functional.normalize(c[i] + s[i] * torch.randn((m, dim), generator=g, device="cuda"), dim=1)
    elif kind == "u8":       # values in [0, 255], mass skewed towards 0-40
        c = torch.rand((n_comp, dim), generator=g, device="cuda") * 60 + \
            torch.empty((n_comp, dim), device="cuda").exponential_(1 / 20.0, generator=g)
        draw = lambda m: (c[torch.randint(0, n_comp, (m,), generator=g, device="cuda")] +
                          12 * torch.randn((m, dim), generator=g, device="cuda")).round().clamp(0, 255).to(torch.uint8)
    elif kind == "i8":       # centres uniform in [-100, 100], sigma 12, clipped
        c = torch.rand((n_comp, dim), generator=g, device="cuda") * 200 - 100
        draw = lambda m: (c[torch.randint(0, n_comp, (m,), generator=g, device="cuda")] +
                          12 * torch.randn((m, dim), generator=g, device="cuda")).round().clamp(-128, 127).to(torch.int8)
    else:                    # unit vectors around unit centres, mean cosine to the centre about 0.8
        c = torch.nn.functional.normalize(torch.randn((n_comp, dim), generator=g, device="cuda"), dim=1)

        def draw(m):
            i = torch.randint(0, n_comp, (m,), generator=g, device="cuda")
            x = c[i] + (0.75 / np.sqrt(dim)) * torch.randn((m, dim), generator=g, device="cuda")
            return torch.nn.functional.normalize(x, dim=1).to(torch.float16)
    return draw(n).contiguous(), draw


def _run(ivf, O, tmp_path, x, q, index_params, search_kw, k, tol, n_oracle):
    index = ivf.build(index_params, x)
    path = str(tmp_path / "cfg.ivfpq")
    ivf.save(path, index)
    sp = ivf.SearchParams(**search_kw)
    d, i = ivf.search(sp, index, q, k)
    ix = O.OracleIndex.load(path)
    lut = {np.float32: O.CUDA_R_32F, np.float16: O.CUDA_R_16F, np.uint8: O.CUDA_R_8U}[search_kw["lut_dtype"]]
    qh = q[:n_oracle].cpu().numpy()
    do, io = O.search(ix, qh, k, n_probes=search_kw["n_probes"], lut_dtype=lut)
    assert_parity(d[:n_oracle].cpu().numpy(), i[:n_oracle].cpu().numpy(), do, io, tol)
    return index, d, i


def test_configuration_1_exact(ivf, oracle_mod, tmp_path):
    x, draw = _mixture(100_000, 128, 1024, 0, "cfg1")
    q = draw(1000).contiguous()
    ip = ivf.IndexParams(n_lists=1024, pq_dim=64, pq_bits=8, kmeans_trainset_fraction=0.5, kmeans_n_iters=10)
    _, _, i = _run(ivf, oracle_mod, tmp_path, x, q, ip,
                   dict(n_probes=32, lut_dtype=np.float32, max_internal_batch_size=1000), 10, 1e-5, 1000)
    # sanity of the configuration itself: recall against exact search
    dist = torch.cdist(q, x)
    truth = dist.topk(10, dim=1, largest=False).indices
    rec = (i.unsqueeze(2) == truth.unsqueeze(1)).any(2).float().sum().item() / truth.numel()
    assert rec > 0.5, rec


def test_configuration_2_shape(ivf, oracle_mod, tmp_path):
    x, draw = _mixture(400_000, 96, 1024, 1, "deep")
    q = draw(4000).contiguous()
    ip = ivf.IndexParams(n_lists=2000, pq_dim=48, pq_bits=8, kmeans_trainset_fraction=0.2, kmeans_n_iters=8)
    _run(ivf, oracle_mod, tmp_path, x, q, ip,
         dict(n_probes=20, lut_dtype=np.float16, max_internal_batch_size=4000), 10, 1e-2, 300)


def test_configuration_3_miniature(ivf, oracle_mod, tmp_path):
    x, draw = _mixture(300_000, 128, 512, 2, "u8")
    q = draw(2000).contiguous()
    ip = ivf.IndexParams(n_lists=150, pq_dim=64, pq_bits=8, kmeans_trainset_fraction=0.2, kmeans_n_iters=8)
    _run(ivf, oracle_mod, tmp_path, x, q, ip,
         dict(n_probes=16, lut_dtype=np.uint8, max_internal_batch_size=2000), 100, 1e-2, 150)


def test_configuration_4_miniature(ivf, oracle_mod, tmp_path):
    x, draw = _mixture(300_000, 128, 512, 3, "i8")
    q = draw(2000).contiguous()
    ip = ivf.IndexParams(n_lists=80, pq_dim=64, pq_bits=8, kmeans_trainset_fraction=0.2, kmeans_n_iters=8)
    _run(ivf, oracle_mod, tmp_path, x, q, ip,
         dict(n_probes=32, lut_dtype=np.uint8, max_internal_batch_size=2000), 10, 1e-2, 100)


def test_configuration_5_miniature(ivf, oracle_mod, tmp_path):
    x, draw = _mixture(40_000, 768, 256, 4, "vmf")
    q = draw(1000).contiguous()
    ip = ivf.IndexParams(n_lists=128, metric="inner_product", pq_dim=384, pq_bits=4,
                         kmeans_trainset_fraction=0.5, kmeans_n_iters=8)
    kw = dict(n_probes=25, lut_dtype=np.float16, max_internal_batch_size=1000)
    index, d, i = _run(ivf, oracle_mod, tmp_path, x, q, ip, kw, 10, 1e-2, 120)
    # the configuration's latency batches (1 and 10 queries) take the small-batch path of the search:
    # same bits as the same queries inside the large batch
    for nq in (1, 10):
        d2, i2 = ivf.search(ivf.SearchParams(**kw), index, q[:nq].contiguous(), 10)
        assert (i2 == i[:nq]).all() and (d2.view(torch.int32) == d[:nq].view(torch.int32)).all()
