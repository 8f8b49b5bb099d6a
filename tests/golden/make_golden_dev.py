"""Generates tests/golden/ref_dev.npz from the reference's own scoring code run on a GPU.

Needs a CUDA device and oracle/_ref/libref_pin_dev.so (the reference's table / score / mapping /
post-processing code compiled by nvcc from the reference checkout: oracle/ref_pin_dev.cu,
``oracle.build_ref_pin_dev``).  Usage:
    python tests/golden/make_golden_dev.py [output.npz]
For each seeded miniature index (pq_bits 4..8, whole and partial 16-byte code pieces, pq_len 1..4,
L2 / inner product / cosine, per-subspace and per-cluster codebooks) it records the inputs and, from
the reference code, every look-up table in its three storage types and every per-vector score in both
internal distance types, with the base differences precomputed or not; plus value mappings, the 8-bit
float and the distance / neighbour post-processing on seeded inputs.  The fixture travels with the
repository; the CPU tests that read it need neither the reference nor a GPU.
"""
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from oracle import refdev as R  # noqa: E402

# (pq_bits, pq_dim, pq_len, metric, codebook kind)
CASES = [(8, 8, 2, O.L2Expanded, O.PER_SUBSPACE), (8, 24, 1, O.InnerProduct, O.PER_SUBSPACE),
         (8, 16, 3, O.L2Expanded, O.PER_CLUSTER), (8, 8, 4, O.CosineExpanded, O.PER_SUBSPACE),
         (7, 8, 2, O.L2Expanded, O.PER_SUBSPACE), (7, 24, 2, O.InnerProduct, O.PER_CLUSTER),
         (6, 8, 1, O.InnerProduct, O.PER_SUBSPACE), (6, 24, 2, O.L2Expanded, O.PER_SUBSPACE),
         (5, 8, 2, O.L2Expanded, O.PER_CLUSTER), (5, 32, 2, O.CosineExpanded, O.PER_SUBSPACE),
         (4, 8, 3, O.InnerProduct, O.PER_SUBSPACE), (4, 32, 2, O.L2Expanded, O.PER_SUBSPACE),
         (4, 40, 2, O.L2Expanded, O.PER_SUBSPACE)]
COMBOS = [(O.CUDA_R_32F, False), (O.CUDA_R_16F, False), (O.CUDA_R_16F, True), (O.CUDA_R_8U, False),
          (O.CUDA_R_8U, True)]   # (table type, fp16 internal distances)


def make_case(i, bits, pq_dim, pq_len, metric, kind):
    rng = np.random.default_rng(1000 + i)
    dim = pq_dim * pq_len
    n_lists, n = 3, 150
    cent = rng.uniform(-1, 1, (6, dim)).astype(np.float32)
    x = (cent[rng.integers(0, 6, n)] + 0.3 * rng.standard_normal((n, dim))).astype(np.float32)
    q = (cent[rng.integers(0, 6, 2)] + 0.3 * rng.standard_normal((2, dim))).astype(np.float32)
    ix = O.build_index(x, n_lists, pq_dim=pq_dim, pq_bits=bits, metric=metric, codebook_kind=kind,
                       force_random_rotation=bool(i % 2), kmeans_iters=2, seed=i)
    _, rq = O.prepare_queries(ix, q)
    code_off, codes, _, _ = ix.flat()
    pair_q = np.repeat(rq, n_lists, axis=0)
    pair_l = np.tile(np.arange(n_lists, dtype=np.uint32), 2)
    return ix, dict(meta=np.array([bits, pq_dim, pq_len, metric, kind, n_lists], dtype=np.int64),
                    pq_centers=ix.pq_centers, centers_rot=ix.centers_rot, list_sizes=ix.list_sizes,
                    codes=codes, code_off=code_off, pair_query=pair_q, pair_label=pair_l, queries=q)


def main(out_path):
    if R.load() is None:
        raise SystemExit("oracle/_ref/libref_pin_dev.so not found: build it where the reference checkout is")
    out = {"n_cases": np.int64(len(CASES))}
    for i, (bits, pq_dim, pq_len, metric, kind) in enumerate(CASES):
        ix, c = make_case(i, bits, pq_dim, pq_len, metric, kind)
        for key, v in c.items():
            out[f"c{i}_{key}"] = v
        is_ip = metric in (O.InnerProduct, O.CosineExpanded)
        for lut_dtype, out_half in COMBOS:
            for precomp in (1, 0):
                lut, sc = R.pairs(is_ip, metric == O.CosineExpanded, bool(precomp), kind == O.PER_CLUSTER, bits,
                                  pq_dim, pq_len, c["pair_query"], c["pair_label"], c["centers_rot"],
                                  c["pq_centers"], c["codes"], c["code_off"], c["list_sizes"], lut_dtype, out_half)
                tag = f"c{i}_t{lut_dtype}_h{int(out_half)}_p{precomp}"
                if not out_half:
                    # the table itself where it is small, its CRC-32 always
                    raw = np.ascontiguousarray(lut).view(np.uint8)
                    out[tag + "_lutcrc"] = np.uint32(zlib.crc32(raw.tobytes()))
                    if raw.size <= 16384 and precomp:
                        out[tag + "_lut"] = raw
                out[tag + "_scores"] = sc.view(np.uint32)
    rng = np.random.default_rng(77)
    sweep = np.concatenate([rng.standard_normal(400).astype(np.float32) * np.float32(s)
                            for s in (1e-6, 1e-4, 1e-2, 1.0, 1e2, 1e4, 1e6)]
                           + [np.array([0.0, -0.0, 1.0 / 32768, 122880.0, 122879.0, 65536.0, 3.0e-5], np.float32)])
    out["fp8_inputs"] = sweep
    for sg in (0, 1):
        enc, d32, d16 = R.fp8(sweep, bool(sg))
        out[f"fp8_enc_s{sg}"], out[f"fp8_dec32_s{sg}"], out[f"fp8_dec16_s{sg}"] = enc, d32.view(np.uint32), d16
        a32, a16 = R.fp8_decode(np.arange(256, dtype=np.uint8), bool(sg))
        out[f"fp8_all32_s{sg}"], out[f"fp8_all16_s{sg}"] = a32.view(np.uint32), a16
    # value mappings (ann_utils.cuh): to fp32 from every element type, to int8 from every element type
    f32 = np.concatenate([rng.uniform(-1.5, 1.5, 500).astype(np.float32),
                          np.array([1.0, -1.0, 0.9999, 127.4 / 128, 127.6 / 128, -1.004, 2.0, -3.0, 0.0], np.float32)])
    f16 = f32.astype(np.float16)
    i8 = np.arange(-128, 128).astype(np.int8)
    u8 = np.arange(256).astype(np.uint8)
    for name, arr in (("f32", f32), ("f16", f16), ("i8", i8), ("u8", u8)):
        out[f"map_in_{name}"] = arr
        out[f"map_{name}_to_f32"] = R.mapping(arr, np.float32).view(np.uint32)
        out[f"map_{name}_to_i8"] = R.mapping(arr, np.int8)
    # distance post-processing: metric x scaling factor as the search passes them
    # (ivf_pq_search.cuh:658-665: account_for_max_close = metric != cosine; factor 1, 128 or 256)
    sc = np.concatenate([np.abs(rng.standard_normal(60)).astype(np.float32) * 3,
                         np.array([0.0, np.inf, 1e-20, 3.4e38], np.float32)]).reshape(4, 16)
    out["post_in"] = sc
    for metric in (O.L2Expanded, O.L2SqrtExpanded, O.CosineExpanded, O.InnerProduct):
        for scale in (1.0, 128.0, 256.0):
            src = -sc if metric == O.InnerProduct else sc
            for in_place in (1, 0):
                out[f"post_m{metric}_s{int(scale)}_i{in_place}"] = R.postprocess_distances(
                    src, metric, scale, metric != O.CosineExpanded, bool(in_place)).view(np.uint32)
    # neighbour post-processing: sample index -> (probe, row) -> source id
    sizes = np.array([5, 0, 33, 7, 64], dtype=np.uint32)
    id_off = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.uint64)
    ids = rng.permutation(int(sizes.sum()) * 3)[:int(sizes.sum())].astype(np.int64)
    probes = np.array([[4, 0, 2], [1, 3, 0], [2, 1, 1]], dtype=np.uint32)
    chunk = np.cumsum(sizes[probes], axis=1).astype(np.uint32)
    samples = np.stack([rng.integers(0, max(int(chunk[r, -1]) + 4, 1), 12) for r in range(3)]).astype(np.uint32)
    out.update(nb_sizes=sizes, nb_ids=ids, nb_probes=probes, nb_chunk=chunk, nb_samples=samples,
               nb_out=R.postprocess_neighbors(samples, ids, id_off, probes, chunk))
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_dev.npz"))
