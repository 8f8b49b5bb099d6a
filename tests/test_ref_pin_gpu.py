"""GPU tests that pin the arithmetic to the reference's own code.

oracle/_ref/libref_pin_dev.so is the reference's scoring code -- base differences, look-up table,
code unpack + score, cosine increment, 8-bit float, value mappings, distance and neighbour
post-processing -- compiled unmodified by nvcc from the reference checkout (oracle/ref_pin_dev.cu).
Here it runs on the device next to the C oracle and next to the product's search, on the same
seeded miniature indexes, and everything is compared bit for bit:
    reference code == C oracle          (tables, scores, mappings, post-processing)
    reference code == product search    (every distance of every vector, through the C interface)
The same reference outputs are stored in tests/golden/ref_dev.npz for the CPU tests.
"""
import importlib.util
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

HERE = os.path.dirname(os.path.abspath(__file__))


def _gen():
    spec = importlib.util.spec_from_file_location("make_golden_dev", os.path.join(HERE, "golden", "make_golden_dev.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


@pytest.fixture(scope="module")
def R():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import refdev
    if refdev.load() is None:
        pytest.skip("oracle/_ref/libref_pin_dev.so was not built (no reference checkout at build time)")
    return refdev


@pytest.fixture(scope="module")
def gen():
    return _gen()


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("case", range(13))
def test_reference_tables_and_scores_equal_oracle_and_product(R, gen, oracle_mod, tmp_path, case):
    O = oracle_mod
    from cuvs_b200 import ivf_pq
    bits, pq_dim, pq_len, metric, kind = gen.CASES[case]
    ix, c = gen.make_case(case, bits, pq_dim, pq_len, metric, kind)
    is_ip = metric in (O.InnerProduct, O.CosineExpanded)
    n_lists = ix.n_lists
    path = str(tmp_path / "case.ivfpq")
    ix.save(path)
    g = ivf_pq.load(path)
    q = c["queries"]
    qd = torch.from_numpy(q).cuda()
    rq = c["pair_query"][::n_lists]
    id_to_pos = {}
    for l in range(n_lists):
        for r, idv in enumerate(ix.list_ids[l][:int(ix.list_sizes[l])].tolist()):
            id_to_pos[idv] = (l, r)
    diff_precomp = 0
    for lut_dtype, out_half in gen.COMBOS:
        internal = O.CUDA_R_16F if out_half else O.CUDA_R_32F
        ref = {}
        for precomp in (1, 0):
            ref[precomp] = R.pairs(is_ip, metric == O.CosineExpanded, bool(precomp), kind == O.PER_CLUSTER, bits,
                                   pq_dim, pq_len, c["pair_query"], c["pair_label"], c["centers_rot"],
                                   c["pq_centers"], c["codes"], c["code_off"], c["list_sizes"], lut_dtype, out_half)
        lut_ref, sc_ref = ref[1]
        # the reference's other variant (base differences not precomputed) may contract q * c into the
        # subtraction for inner product; for L2 both variants are the same arithmetic
        if not is_ip:
            assert (ref[0][0].view(np.uint8) == lut_ref.view(np.uint8)).all()
        else:
            diff_precomp += int((ref[0][0].view(np.uint8) != lut_ref.view(np.uint8)).sum())
        # reference == oracle: tables and per-vector scores
        for p in range(c["pair_label"].shape[0]):
            label = int(c["pair_label"][p])
            lut_o = O.build_lut(ix, label, c["pair_query"][p], lut_dtype)
            assert (lut_o.view(np.uint8) == lut_ref[p].view(np.uint8)).all(), (lut_dtype, p)
            s_o = O.pair_scores(ix, label, c["pair_query"][p], lut_dtype, internal)
            n = int(ix.list_sizes[label])
            assert (_bits(s_o) == _bits(sc_ref[p, :n])).all(), (lut_dtype, out_half, p)
        # reference == product: every vector's distance, both top-k modes of the scan kernel
        lut_np = {O.CUDA_R_32F: np.float32, O.CUDA_R_16F: np.float16, O.CUDA_R_8U: np.uint8}[lut_dtype]
        for k in (min(ix.size, 100), ix.size):
            sp = ivf_pq.SearchParams(n_probes=n_lists, lut_dtype=lut_np,
                                     internal_distance_dtype=np.float16 if out_half else np.float32)
            d, i = ivf_pq.search(sp, g, qd, k)
            d, i = d.cpu().numpy(), i.cpu().numpy()
            for qi in range(q.shape[0]):
                exp_raw = np.array([sc_ref[qi * n_lists + id_to_pos[idv][0], id_to_pos[idv][1]] for idv in i[qi].tolist()],
                                   dtype=np.float32)
                exp = R.postprocess_distances(exp_raw, metric, 1.0, metric != O.CosineExpanded)
                assert (_bits(exp) == _bits(d[qi])).all(), (lut_dtype, out_half, k, qi)
                assert (_bits(O.postprocess(exp_raw, metric, 1.0)) == _bits(exp)).all()
                if k == ix.size:
                    assert sorted(i[qi].tolist()) == sorted(id_to_pos)
    print(f"case {case}: table bytes that differ between the reference's two base-difference variants: {diff_precomp}")


def test_reference_value_types_equal_oracle(R, oracle_mod):
    O = oracle_mod
    L = O.lib()
    rng = np.random.default_rng(5)
    vals = (rng.standard_normal(20000) * 10.0 ** rng.integers(-7, 6, 20000)).astype(np.float32)
    for sg in (0, 1):
        enc, d32, d16 = R.fp8(vals, bool(sg))
        mine = np.array([L.orc_fp8_encode(float(v), sg) for v in vals], dtype=np.uint8)
        assert (mine == enc).all()
        a32, a16 = R.fp8_decode(np.arange(256, dtype=np.uint8), bool(sg))
        o32 = np.array([L.orc_fp8_decode(b, sg) for b in range(256)], dtype=np.float32)
        o16 = np.array([L.orc_fp8_decode_half(b, sg) for b in range(256)], dtype=np.uint16)
        assert (_bits(o32) == _bits(a32)).all()
        fin = np.isfinite(a16.view(np.float16))
        assert (o16[fin] == a16[fin]).all()
    u8 = np.arange(256).astype(np.uint8)
    i8 = np.arange(-128, 128).astype(np.int8)
    f16 = (rng.uniform(-2, 2, 3000)).astype(np.float16)
    for arr in (u8, i8, f16):
        assert (_bits(R.mapping(arr, np.float32)) == _bits(O.map_to_float(arr))).all()


def test_reference_postprocessing_equals_oracle(R, oracle_mod):
    O = oracle_mod
    rng = np.random.default_rng(9)
    sc = np.abs(rng.standard_normal((8, 32))).astype(np.float32) * 5
    sc[0, :3] = (0.0, np.inf, 1e-30)
    for metric in (O.L2Expanded, O.L2SqrtExpanded, O.CosineExpanded, O.InnerProduct):
        for scale in (1.0, 128.0, 256.0):
            src = -sc if metric == O.InnerProduct else sc
            for in_place in (True, False):
                ref = R.postprocess_distances(src, metric, scale, metric != O.CosineExpanded, in_place)
                assert (_bits(ref) == _bits(O.postprocess(src, metric, scale))).all(), (metric, scale)
