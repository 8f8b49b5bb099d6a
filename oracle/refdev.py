"""ctypes access to oracle/_ref/libref_pin_dev.so -- TEST INFRASTRUCTURE ONLY.

The library is the reference's own scoring code (table construction, code unpack + score, 8-bit
float, value mappings, distance / neighbour post-processing) compiled with nvcc from the reference
checkout by ``oracle.build_ref_pin_dev`` (see oracle/ref_pin_dev.cu).  It needs a GPU to run and
exists only where it was built or shipped to; ``load()`` returns None otherwise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libref_pin_dev.so")
_lib = None

LUT_KIND = {0: 0, 2: 1, 8: 2}            # cudaDataType_t of the table -> kind index of the library
LUT_NP = {0: np.float32, 2: np.float16, 8: np.uint8}
ELEM = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.int8): 2, np.dtype(np.uint8): 3}


def load():
    global _lib
    if _lib is None and os.path.exists(_SO):
        _lib = C.CDLL(_SO)
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def pairs(metric_ip: bool, increment: bool, precomp: bool, per_cluster: bool, pq_bits: int, pq_dim: int,
          pq_len: int, pair_query, pair_label, centers_rot, pq_centers, codes, code_off, list_sizes,
          lut_dtype: int, out_half: bool, threads: int = 128):
    """Tables (bytes, [n_pairs, pq_dim << pq_bits] in the table type) and scores ([n_pairs, max_rows]
    fp32; slots past a list's size hold NaN) of the given (query, list) pairs."""
    lib = load()
    pq = np.ascontiguousarray(pair_query, dtype=np.float32)
    pl = np.ascontiguousarray(pair_label, dtype=np.uint32)
    cr = np.ascontiguousarray(centers_rot, dtype=np.float32)
    pc = np.ascontiguousarray(pq_centers, dtype=np.float32)
    cd = np.ascontiguousarray(codes, dtype=np.uint8)
    co = np.ascontiguousarray(code_off, dtype=np.uint64)
    ls = np.ascontiguousarray(list_sizes, dtype=np.uint32)
    n_pairs = pl.shape[0]
    max_rows = max(int(ls.max()), 1)
    lut = np.zeros((n_pairs, pq_dim << pq_bits), dtype=LUT_NP[lut_dtype])
    scores = np.zeros((n_pairs, max_rows), dtype=np.float32)
    rc = lib.refdev_pairs(C.c_int(LUT_KIND[lut_dtype]), C.c_int(int(out_half)), C.c_int(int(metric_ip)),
                          C.c_int(int(increment)), C.c_int(int(precomp)), C.c_uint32(pq_bits),
                          C.c_int(int(per_cluster)), C.c_uint32(pq_dim), C.c_uint32(pq_len),
                          C.c_uint32(n_pairs), _p(pq), _p(pl), C.c_uint32(ls.shape[0]), _p(cr), _p(pc),
                          C.c_uint64(pc.size), _p(cd), C.c_uint64(cd.size), _p(co), _p(ls),
                          C.c_uint32(max_rows), _p(lut), _p(scores), C.c_int(threads))
    if rc != 0:
        raise RuntimeError(f"refdev_pairs failed ({rc})")
    return lut, scores


def fp8(values, signed: bool):
    v = np.ascontiguousarray(values, dtype=np.float32)
    enc = np.zeros(v.size, np.uint8)
    d32 = np.zeros(v.size, np.float32)
    d16 = np.zeros(v.size, np.uint16)
    rc = load().refdev_fp8(_p(v), C.c_uint64(v.size), C.c_int(int(signed)), _p(enc), _p(d32), _p(d16))
    assert rc == 0
    return enc, d32, d16


def fp8_decode(codes, signed: bool):
    b = np.ascontiguousarray(codes, dtype=np.uint8)
    d32 = np.zeros(b.size, np.float32)
    d16 = np.zeros(b.size, np.uint16)
    rc = load().refdev_fp8_decode(_p(b), C.c_uint64(b.size), C.c_int(int(signed)), _p(d32), _p(d16))
    assert rc == 0
    return d32, d16


def mapping(values, dst):
    """mapping<dst>(value) of cpp/src/neighbors/detail/ann_utils.cuh; dst is np.float32 or np.int8."""
    v = np.ascontiguousarray(values)
    out = np.zeros(v.shape, dtype=dst)
    rc = load().refdev_mapping(C.c_int(ELEM[v.dtype]), C.c_int(ELEM[np.dtype(dst)]), _p(v),
                               C.c_uint64(v.size), _p(out))
    assert rc == 0
    return out


def postprocess_distances(scores, metric: int, scale: float, account_for_max_close: bool,
                          in_place: bool = True):
    s = np.ascontiguousarray(scores, dtype=np.float32)
    s2 = s.reshape(s.shape[0], -1) if s.ndim > 1 else s.reshape(1, -1)
    out = np.zeros_like(s2)
    rc = load().refdev_postprocess_distances(_p(s2), _p(out), C.c_uint32(s2.shape[0]), C.c_uint32(s2.shape[1]),
                                             C.c_int(metric), C.c_float(scale),
                                             C.c_int(int(account_for_max_close)), C.c_int(int(in_place)))
    assert rc == 0
    return out.reshape(s.shape)


def postprocess_neighbors(sample_ix, ids, id_off, probes, chunk_indices):
    n_q, k = sample_ix.shape
    si = np.ascontiguousarray(sample_ix, dtype=np.uint32)
    idv = np.ascontiguousarray(ids, dtype=np.int64)
    io = np.ascontiguousarray(id_off, dtype=np.uint64)
    pr = np.ascontiguousarray(probes, dtype=np.uint32)
    ch = np.ascontiguousarray(chunk_indices, dtype=np.uint32)
    out = np.zeros((n_q, k), dtype=np.int64)
    rc = load().refdev_postprocess_neighbors(_p(si), _p(idv), _p(io), C.c_uint32(io.shape[0]),
                                             C.c_uint64(idv.size), _p(pr), _p(ch), C.c_uint32(n_q),
                                             C.c_uint32(pr.shape[1]), C.c_uint32(k), _p(out))
    assert rc == 0
    return out
