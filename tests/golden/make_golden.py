"""Generates tests/golden/ref_pin.npz from the reference's own code.

Run in an environment where the reference checkout is present (its location is the argument, else
the environment variable CUVS_REFERENCE_ROOT, else a `reference` folder beside this repository):
    python tests/golden/make_golden.py [reference_root]
It builds oracle/_ref/libref_pin.so (two reference headers compiled on the host, see
oracle/ref_pin.cpp) and records, for seeded inputs,
  * the reference's 8-bit float: encodings of a float sweep, both decodings of all 256 codes;
  * the reference's interleaved code layout: packed lists for pq_bits 4..8.
The fixture travels with the repository; the tests that read it need neither the reference nor
the pin library.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402


def main(reference_root=None):
    so = O.build_ref_pin(reference_root)
    if so is None:
        raise SystemExit("reference checkout not found; cannot regenerate the golden fixture")
    ref = C.CDLL(so)
    ref.ref_fp8_encode.restype = C.c_uint8
    ref.ref_fp8_encode.argtypes = [C.c_float, C.c_int]
    ref.ref_fp8_decode.restype = C.c_float
    ref.ref_fp8_decode.argtypes = [C.c_uint8, C.c_int]
    ref.ref_fp8_decode_half.restype = C.c_uint16
    ref.ref_fp8_decode_half.argtypes = [C.c_uint8, C.c_int]

    rng = np.random.default_rng(20251125)
    sweep = np.concatenate(
        [rng.standard_normal(512).astype(np.float32) * np.float32(s)
         for s in (1e-6, 1e-4, 1e-2, 1.0, 1e2, 1e4, 1e6)]
        + [np.array([0.0, -0.0, 1.0 / 32768, 122880.0, 122879.0, 65536.0, 3.0e-5, 1.0, 2.0, 0.5],
                    dtype=np.float32)]
        + [np.float32(2.0) ** np.arange(-20, 20, dtype=np.float32)])
    out = {"fp8_inputs": sweep}
    for sg in (0, 1):
        out[f"fp8_encode_s{sg}"] = np.array([ref.ref_fp8_encode(float(v), sg) for v in sweep],
                                            dtype=np.uint8)
        out[f"fp8_decode_s{sg}"] = np.array([ref.ref_fp8_decode(b, sg) for b in range(256)],
                                            dtype=np.float32)
        out[f"fp8_decode_half_s{sg}"] = np.array([ref.ref_fp8_decode_half(b, sg) for b in range(256)],
                                                 dtype=np.uint16)
    for bits, pq_dim in ((4, 22), (5, 8), (6, 20), (7, 24), (8, 37)):
        assert (bits * pq_dim) % 8 == 0
        n = 77
        codes = rng.integers(0, 1 << bits, size=(n, pq_dim), dtype=np.uint8)
        g = (n + 31) // 32
        buf = np.zeros(O.list_bytes(n, pq_dim, bits), dtype=np.uint8)
        rc = ref.ref_pack_list(codes.ctypes.data_as(C.c_void_p), n, pq_dim, bits, 0,
                               buf.ctypes.data_as(C.c_void_p), g)
        assert rc == 0
        back = np.zeros_like(codes)
        ref.ref_unpack_list(buf.ctypes.data_as(C.c_void_p), n, pq_dim, bits, 0,
                            back.ctypes.data_as(C.c_void_p), g)
        assert (back == codes).all()
        out[f"pack_codes_b{bits}"] = codes
        out[f"pack_list_b{bits}"] = buf
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_pin.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(*sys.argv[1:])
