"""CPU tests of the oracle: pinned against the reference-generated golden vectors, the file format
against numpy, and end-to-end sanity against exact brute force."""
import ctypes as C
import io
import os

import numpy as np
import pytest

from conftest import make_mixture

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_pin.npz")


def test_fp8_matches_reference_golden(oracle_mod):
    O = oracle_mod
    g = np.load(GOLDEN)
    L = O.lib()
    for sg in (0, 1):
        enc = np.array([L.orc_fp8_encode(float(v), sg) for v in g["fp8_inputs"]], dtype=np.uint8)
        assert (enc == g[f"fp8_encode_s{sg}"]).all()
        dec = np.array([L.orc_fp8_decode(b, sg) for b in range(256)], dtype=np.float32)
        assert (dec.view(np.uint32) == g[f"fp8_decode_s{sg}"].view(np.uint32)).all()
        dech = np.array([L.orc_fp8_decode_half(b, sg) for b in range(256)], dtype=np.uint16)
        ref = g[f"fp8_decode_half_s{sg}"]
        # codes whose value exceeds the fp16 range decode to NaN patterns; compare the rest bit-exactly
        finite = np.isfinite(ref.view(np.float16))
        assert (dech[finite] == ref[finite]).all()
        assert np.isnan(dech[~finite].view(np.float16)).all()


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
def test_code_layout_matches_reference_golden(oracle_mod, bits):
    O = oracle_mod
    g = np.load(GOLDEN)
    codes, packed = g[f"pack_codes_b{bits}"], g[f"pack_list_b{bits}"]
    n, pq_dim = codes.shape
    assert (O.pack_list(codes, bits).reshape(-1) == packed).all()
    assert (O.pack_list_numpy(codes, bits).reshape(-1) == packed).all()
    assert (O.unpack_list(packed, n, pq_dim, bits) == codes).all()


def test_reference_pin_library_when_present(oracle_mod):
    """Where oracle/_ref was built from the reference checkout, compare against it live."""
    O = oracle_mod
    so = os.path.join(os.path.dirname(O.__file__), "_ref", "libref_pin.so")
    if not os.path.exists(so):
        pytest.skip("oracle/_ref/libref_pin.so not built here")
    ref = C.CDLL(so)
    ref.ref_fp8_encode.restype = C.c_uint8
    ref.ref_fp8_encode.argtypes = [C.c_float, C.c_int]
    L = O.lib()
    rng = np.random.default_rng(5)
    vals = (rng.standard_normal(4000) * 10.0 ** rng.integers(-7, 6, 4000)).astype(np.float32)
    for sg in (0, 1):
        for v in vals:
            assert L.orc_fp8_encode(float(v), sg) == ref.ref_fp8_encode(float(v), sg)


def test_half_conversion_is_round_to_nearest_even(oracle_mod):
    L = oracle_mod.lib()
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 5, 20000)).astype(np.float32)
    x = np.concatenate([x, np.array([65504, 65519.9, 65520, 6e-8, 2.98e-8, 2.99e-8, 0, -0.0], np.float32)])
    mine = np.array([L.orc_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16).view(np.uint16)
    assert (mine == ref).all()


def test_file_records_are_valid_npy(oracle_mod, small_l2):
    """Every record of a serialized index loads with numpy's own .npy reader."""
    O = oracle_mod
    with open(small_l2["path"], "rb") as f:
        recs = []
        while True:
            pos = f.tell()
            if not f.read(1):
                break
            f.seek(pos)
            assert pos % 64 == 0 or True
            recs.append(np.load(f, allow_pickle=False))
    ix = small_l2["ix"]
    assert int(recs[0]) == 4 and recs[0].dtype == np.int32
    assert int(recs[1]) == ix.size and recs[1].dtype == np.int64
    assert [int(r) for r in recs[2:5]] == [ix.dim, ix.pq_bits, ix.pq_dim]
    assert recs[10].shape == (ix.pq_dim, ix.pq_len, 1 << ix.pq_bits)
    assert recs[11].shape == (ix.n_lists, ix.dim_ext)
    assert recs[14].dtype == np.uint32 and recs[14].shape == (ix.n_lists,)
    # per list: size, then (codes, ids) when non-empty
    n_nonempty = int((ix.list_sizes > 0).sum())
    assert len(recs) == 15 + ix.n_lists + 2 * n_nonempty


def test_save_load_round_trip(oracle_mod, small_l2):
    O = oracle_mod
    ix = small_l2["ix"]
    ix2 = O.OracleIndex.load(small_l2["path"])
    assert (ix2.list_sizes == ix.list_sizes).all()
    assert (ix2.centers == ix.centers).all() and (ix2.pq_centers == ix.pq_centers).all()
    for a, b in zip(ix.list_codes, ix2.list_codes):
        assert (np.asarray(a).reshape(-1) == np.asarray(b).reshape(-1)).all()
    d1, i1 = O.search(ix, small_l2["q"], 10, n_probes=8)
    d2, i2 = O.search(ix2, small_l2["q"], 10, n_probes=8)
    assert (i1 == i2).all() and (d1 == d2).all()


def test_corrupt_files_are_rejected(oracle_mod, small_l2):
    O = oracle_mod
    blob = open(small_l2["path"], "rb").read()
    with pytest.raises(ValueError):
        O.OracleIndex.load(io.BytesIO(blob[: len(blob) // 2]))
    with pytest.raises(ValueError):
        O.OracleIndex.load(io.BytesIO(b"garbage" + blob))


def test_oracle_recall_and_distances(oracle_mod, small_l2):
    """Probing every list makes IVF exhaustive: PQ distances must track the exact ones."""
    O = oracle_mod
    ix, x, q = small_l2["ix"], small_l2["x"], small_l2["q"]
    gt_d, gt_i = O.brute_force(x, q, 10)
    d, i = O.search(ix, q, 10, n_probes=ix.n_lists)
    assert O.recall(i, gt_i) > 0.75
    assert not (i == O.OUT_OF_BOUNDS).any()
    assert np.all(np.diff(d, axis=1) >= 0)
    # every returned id is unique within its row
    assert all(len(set(r.tolist())) == len(r) for r in i)


@pytest.mark.parametrize("lut,internal", [(0, 0), (2, 0), (8, 0), (2, 2), (8, 2)])
def test_oracle_lut_dtypes_agree(oracle_mod, small_l2, lut, internal):
    O = oracle_mod
    ix, q = small_l2["ix"], small_l2["q"]
    d0, i0 = O.search(ix, q, 10, n_probes=8)
    d, i = O.search(ix, q, 10, n_probes=8, lut_dtype=lut, internal_dtype=internal)
    overlap = np.mean([len(set(a) & set(b)) / 10 for a, b in zip(i, i0)])
    assert overlap > (0.9 if lut != 8 else 0.8)
    assert np.allclose(d[:, 0], d0[:, 0], rtol=0.08, atol=1e-3)


def test_oracle_rejects_invalid_dtype_pair(oracle_mod, small_l2):
    with pytest.raises(ValueError):
        oracle_mod.search(small_l2["ix"], small_l2["q"], 5, lut_dtype=0, internal_dtype=2)


def test_oracle_too_few_candidates_pads_with_out_of_bounds(oracle_mod):
    O = oracle_mod
    x = make_mixture(300, 16, 8, 0.1, seed=4)
    ix = O.build_index(x, 16, pq_dim=8, pq_bits=4, kmeans_iters=3)
    smallest = int(ix.list_sizes.min())
    d, i = O.search(ix, x[:20], 64, n_probes=1)
    assert (i == O.OUT_OF_BOUNDS).any() or smallest >= 64
    missing = i == O.OUT_OF_BOUNDS
    assert np.isinf(d[missing]).all()


@pytest.mark.parametrize("metric", [6, 2, 1])
def test_oracle_other_metrics(oracle_mod, metric):
    O = oracle_mod
    x = make_mixture(2000, 24, 20, 0.2, seed=7)
    q = make_mixture(50, 24, 20, 0.2, seed=8)
    ix = O.build_index(x, 16, pq_dim=12, pq_bits=8, metric=metric, kmeans_iters=3)
    gt_d, gt_i = O.brute_force(x, q, 10, metric)
    d, i = O.search(ix, q, 10, n_probes=16)
    assert O.recall(i, gt_i) > 0.6
    if metric == 6:      # inner product: larger is better, returned descending
        assert np.all(np.diff(d, axis=1) <= 1e-6)
    if metric == 1:      # sqrt of the squared distance
        d2, _ = O.search(O.build_index(x, 16, pq_dim=12, pq_bits=8, metric=0, kmeans_iters=3), q, 10, n_probes=16)
        assert np.allclose(d, np.sqrt(d2), rtol=1e-5)


def test_multi_gpu_index_file_round_trip(oracle_mod, tmp_path):
    """cpp/src/neighbors/mg/snmg.cuh:780-805: dtype string, mode, rank count, one index per rank."""
    O = oracle_mod
    rng = np.random.default_rng(3)
    x = rng.standard_normal((900, 16)).astype(np.float32)
    parts = [O.build_index(x[:500], 8, pq_dim=8, kmeans_iters=2, seed=0),
             O.build_index(x[500:], 8, pq_dim=8, kmeans_iters=2, seed=1)]
    path = str(tmp_path / "mg.bin")
    O.save_mg(path, O.SHARDED, parts)
    blob = open(path, "rb").read()
    assert blob[:4] == b"<f4\x00" and blob[4:10] == b"\x93NUMPY"
    dtype_string, mode, back = O.load_mg(path)
    assert dtype_string == "<f4" and mode == O.SHARDED and len(back) == 2
    for a, b in zip(parts, back):
        assert a.size == b.size and (a.list_sizes == b.list_sizes).all()
        assert (a.centers == b.centers).all() and (a.pq_centers == b.pq_centers).all()
        for l in range(a.n_lists):
            s = int(a.list_sizes[l])
            assert (np.asarray(a.list_ids[l][:s]) == np.asarray(b.list_ids[l][:s])).all()


def test_int8_coarse_search_restatement(oracle_mod):
    """coarse_search_dtype = CUDA_R_8I (ivf_pq_index.cu:661-738, ivf_pq_search.cuh:171-256): the int8
    operands encode 128^2 * (<q, c> - |c|^2 / 2) up to quantisation, so the int32 scores order the
    lists nearly as the fp32 scores do, and the search built on them keeps its recall."""
    O = oracle_mod
    rng = np.random.default_rng(11)
    cent = rng.uniform(-0.6, 0.6, (40, 32)).astype(np.float32)
    x = (cent[rng.integers(0, 40, 5000)] + 0.08 * rng.standard_normal((5000, 32))).astype(np.float32)
    q = (cent[rng.integers(0, 40, 100)] + 0.08 * rng.standard_normal((100, 32))).astype(np.float32)
    ix = O.build_index(x, 48, pq_dim=16, pq_bits=8, kmeans_iters=4)
    c8, r8 = O.int8_operands(ix)
    d8 = c8.shape[1]
    assert d8 == 48 and r8.shape == (ix.rot_dim, ix.dim)          # round_up(32 + 2, 16)
    # the norm slots: z in column dim, round(y) in the m - 1 columns after it, with
    # (m - 1) * (z + 128 * round(y)) ~ 128 * 64 * |c|^2
    m = d8 - ix.dim
    n2 = ix.centers[:, ix.dim].astype(np.float64)
    enc = (m - 1) * (c8[:, ix.dim].astype(np.float64) + 128.0 * c8[:, ix.dim + 1].astype(np.float64))
    assert (c8[:, ix.dim + 1:] == c8[:, ix.dim + 1:ix.dim + 2]).all()
    assert np.abs(enc - 8192.0 * n2).max() <= (m - 1) * 1.0 + 1e-6
    q8, rq = O.prepare_queries_int8(ix, q, r8)
    assert (q8[:, ix.dim] == 1 - m).all() and (q8[:, ix.dim + 1:] == -128).all()
    assert (q8[:, :ix.dim] == np.trunc(q * 128.0).astype(np.int8)).all()
    # int32 scores against the fp32 ones: -2 * 128^2 * (<q,c> - |c|^2/2) = 128^2 * (|c|^2 - 2<q,c>)
    fq, rq32 = O.prepare_queries(ix, q)
    p32, s32, all32 = O.select_clusters(ix, fq, 8, want_all=True)
    p8, s8 = O.select_clusters_int8(ix, c8, q8, 8)
    first = np.take_along_axis(all32, p8[:, :1].astype(np.int64), axis=1)[:, 0]
    assert np.abs(s8[:, 0] / 16384.0 - first).max() < 0.3          # truncation toward zero shrinks the products
    overlap = np.mean([len(set(a) & set(b)) / 8 for a, b in zip(p8.tolist(), p32.tolist())])
    assert overlap > 0.85, overlap
    assert np.abs(rq - rq32).max() < 0.03                          # rotated queries, 1/128 grid
    gt_d, gt_i = O.brute_force(x, q, 10)
    r32 = O.recall(O.search(ix, q, 10, n_probes=8)[1], gt_i)
    r8 = O.recall(O.search_int8_coarse(ix, q, 10, n_probes=8)[1], gt_i)
    assert r8 > r32 - 0.08, (r8, r32)


# ------------------------------------------------------------------------------------------------
# Pins against tests/golden/ref_dev.npz: outputs of the reference's own scoring code (look-up table,
# code unpack + score, cosine increment, 8-bit float, value mappings, distance and neighbour
# post-processing) compiled by nvcc from the reference checkout and run on a B200
# (oracle/ref_pin_dev.cu, generator tests/golden/make_golden_dev.py).
# ------------------------------------------------------------------------------------------------
GOLDEN_DEV = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_dev.npz")


@pytest.fixture(scope="module")
def gdev():
    return np.load(GOLDEN_DEV)


def _index_from_golden(O, g, i):
    bits, pq_dim, pq_len, metric, kind, n_lists = (int(v) for v in g[f"c{i}_meta"])
    dim = pq_dim * pq_len
    sizes = g[f"c{i}_list_sizes"]
    ix = O.OracleIndex(metric, kind, dim, pq_dim, bits, n_lists, g[f"c{i}_pq_centers"],
                       np.zeros((n_lists, O.round_up(dim + 1, 8)), np.float32), g[f"c{i}_centers_rot"],
                       np.eye(dim, dtype=np.float32), sizes)
    codes, off = g[f"c{i}_codes"], g[f"c{i}_code_off"]
    ix.list_codes = [codes[int(off[l]):int(off[l]) + O.list_bytes(int(sizes[l]), pq_dim, bits)].copy()
                     for l in range(n_lists)]
    ix.list_ids = [np.arange(int(s), dtype=np.int64) for s in sizes]
    return ix


@pytest.mark.parametrize("case", range(13))
def test_tables_and_scores_match_reference_golden(oracle_mod, gdev, case):
    import zlib
    O, g = oracle_mod, gdev
    assert case < int(g["n_cases"])
    ix = _index_from_golden(O, g, case)
    pq, pl = g[f"c{case}_pair_query"], g[f"c{case}_pair_label"]
    for lut_dtype, out_half in ((O.CUDA_R_32F, 0), (O.CUDA_R_16F, 0), (O.CUDA_R_16F, 1), (O.CUDA_R_8U, 0),
                                (O.CUDA_R_8U, 1)):
        tag = f"c{case}_t{lut_dtype}_h{out_half}_p1"
        luts = np.stack([O.build_lut(ix, int(pl[p]), pq[p], lut_dtype) for p in range(pl.shape[0])])
        if not out_half:
            raw = np.ascontiguousarray(luts).view(np.uint8)
            assert np.uint32(zlib.crc32(raw.tobytes())) == g[tag + "_lutcrc"]
            if tag + "_lut" in g:
                assert (raw.reshape(-1) == g[tag + "_lut"].reshape(-1)).all()
        ref = g[tag + "_scores"]
        for p in range(pl.shape[0]):
            s = O.pair_scores(ix, int(pl[p]), pq[p], lut_dtype, O.CUDA_R_16F if out_half else O.CUDA_R_32F)
            assert (s.view(np.uint32) == ref[p, :s.size]).all(), (lut_dtype, out_half, p)
        # L2: the reference's variant without precomputed base differences is the same arithmetic
        if ix.metric in (O.L2Expanded, O.L2SqrtExpanded):
            assert (g[f"c{case}_t{lut_dtype}_h{out_half}_p0_scores"] == ref).all()


def test_value_types_match_reference_device_golden(oracle_mod, gdev):
    O, g = oracle_mod, gdev
    L = O.lib()
    for sg in (0, 1):
        enc = np.array([L.orc_fp8_encode(float(v), sg) for v in g["fp8_inputs"]], dtype=np.uint8)
        assert (enc == g[f"fp8_enc_s{sg}"]).all()
        d32 = np.array([L.orc_fp8_decode(b, sg) for b in range(256)], dtype=np.float32)
        assert (d32.view(np.uint32) == g[f"fp8_all32_s{sg}"]).all()
        d16 = np.array([L.orc_fp8_decode_half(b, sg) for b in range(256)], dtype=np.uint16)
        fin = np.isfinite(g[f"fp8_all16_s{sg}"].view(np.float16))
        assert (d16[fin] == g[f"fp8_all16_s{sg}"][fin]).all()
    for name in ("f16", "i8", "u8"):
        assert (O.map_to_float(g[f"map_in_{name}"]).view(np.uint32) == g[f"map_{name}_to_f32"]).all()
    # mapping<int8_t>: fp32 (clamped), uint8 (halved), int8 (identity)
    assert (O.map_from_float(g["map_in_f32"], np.int8) == g["map_f32_to_i8"]).all()
    assert ((g["map_in_u8"] >> 1).astype(np.int8) == g["map_u8_to_i8"]).all()
    assert (g["map_in_i8"] == g["map_i8_to_i8"]).all()


def test_postprocessing_matches_reference_device_golden(oracle_mod, gdev):
    O, g = oracle_mod, gdev
    sc = g["post_in"]
    for metric in (O.L2Expanded, O.L2SqrtExpanded, O.CosineExpanded, O.InnerProduct):
        for scale in (1, 128, 256):
            src = -sc if metric == O.InnerProduct else sc
            mine = O.postprocess(src, metric, float(scale)).view(np.uint32)
            for in_place in (0, 1):
                assert (mine == g[f"post_m{metric}_s{scale}_i{in_place}"]).all(), (metric, scale)
    # sample index -> probe -> source id (find_chunk_ix + postprocess_neighbors_kernel)
    sizes, ids, probes, chunk, samples = (g[k] for k in ("nb_sizes", "nb_ids", "nb_probes", "nb_chunk", "nb_samples"))
    id_off = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    for r in range(samples.shape[0]):
        for c in range(samples.shape[1]):
            s, p = int(samples[r, c]), 0
            while p < probes.shape[1] and chunk[r, p] <= s:
                p += 1
            if p < probes.shape[1]:
                row = s - (int(chunk[r, p - 1]) if p else 0)
                exp = ids[int(id_off[probes[r, p]]) + row]
            else:
                exp = O.OUT_OF_BOUNDS
            assert g["nb_out"][r, c] == exp
