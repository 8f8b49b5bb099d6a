"""CPU oracle for the IVF-PQ search path -- TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  It is used by the tests, by the smoke check
and by the benchmark's timed CPU baseline.  It wraps ``liboracle.so`` (the C restatement of the
reference search arithmetic, see the header of ``ivfpq_oracle.c`` for the file:line map) and adds,
in numpy:

* a reader and a writer for the reference's index file format, version 4
  (cpp/src/neighbors/ivf_pq/ivf_pq_serialize.cuh:41-87 and :124-211,
  cpp/src/neighbors/ivf_list.cuh:108-176): a sequence of NumPy ``.npy`` v1.0 records, scalars being
  0-d arrays.  The record framing follows the published ``.npy`` format; the reader accepts any
  valid v1.0 header.  No file written by the reference itself was available to check against
  (parity unpinned for the framing); each record is checked with ``numpy.lib.format`` instead.
* a small CPU index builder (plain Lloyd k-means; it does not imitate the reference's balanced
  hierarchical k-means -- any index obeying the data contract is searchable), so that fixtures
  exist without the reference;
* exact brute-force k-NN for recall.
"""
from __future__ import annotations

import ctypes as C
import io
import os
import struct
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# metric codes: c/include/cuvs/distance/distance.h
L2Expanded, L2SqrtExpanded, CosineExpanded, InnerProduct = 0, 1, 2, 6
# cudaDataType_t values used by search_params
CUDA_R_32F, CUDA_R_16F, CUDA_R_8U = 0, 2, 8
PER_SUBSPACE, PER_CLUSTER = 0, 1
SERIALIZATION_VERSION = 4
OUT_OF_BOUNDS = np.iinfo(np.int64).max

_QTYPE = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.int8): 2,
          np.dtype(np.uint8): 3}


def build_lib(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile next to this file (gcc, a second or two)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "ivfpq_oracle.c")
    if force or not os.path.exists(so) or (
            os.path.exists(src) and os.path.getmtime(so) < os.path.getmtime(src)):
        env = dict(os.environ)
        env.pop("CC", None)
        env.pop("CXX", None)
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], env=env,
                              stdout=subprocess.DEVNULL)
    return so


def reference_root() -> str | None:
    """The reference checkout, named by the environment variable CUVS_REFERENCE_ROOT or found as a
    `reference` folder beside this repository; None where there is none (e.g. on a GPU box)."""
    cand = os.environ.get("CUVS_REFERENCE_ROOT") or os.path.join(
        os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "cpp", "src", "neighbors", "ivf_pq")) else None


def _make(target: str, ref: str) -> None:
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    subprocess.check_call(["make", "-C", _HERE, target, f"REF={ref}"], env=env, stdout=subprocess.DEVNULL)


def build_ref_pin(root: str | None = None) -> str | None:
    """Compile oracle/_ref/libref_pin.so from two headers of the reference checkout, if present."""
    so = os.path.join(_HERE, "_ref", "libref_pin.so")
    root = root or reference_root()
    if root:
        _make("ref", root)
    return so if os.path.exists(so) else None


def _cut(text: str, start: str, end: str, what: str) -> str:
    a = text.find(start)
    b = text.find(end, a + 1) if a >= 0 else -1
    if a < 0 or b < 0:
        raise RuntimeError(f"reference layout changed: cannot find {what}")
    return text[a:b]


def build_ref_pin_dev(root: str | None = None) -> str | None:
    """Compile oracle/_ref/libref_pin_dev.so (nvcc, sm_100a) from the reference's scoring headers, if
    the checkout is present.  Two of the headers drag in the un-vendored memory libraries, so only the
    parts under test are cut out of them, verbatim, into oracle/_ref/extract/ (untracked):
    `config<>` + `mapping<>` of cpp/src/neighbors/detail/ann_utils.cuh, and kOutOfBoundsRecord,
    find_chunk_ix, postprocess_neighbors and postprocess_distances of cpp/src/neighbors/ivf_common.cuh."""
    so = os.path.join(_HERE, "_ref", "libref_pin_dev.so")
    root = root or reference_root()
    if root:
        ext = os.path.join(_HERE, "_ref", "extract")
        os.makedirs(ext, exist_ok=True)
        ann = open(os.path.join(root, "cpp/src/neighbors/detail/ann_utils.cuh")).read()
        part = _cut(ann, "template <typename T>\nstruct config {};", "/**\n * @brief Sets the first num bytes",
                    "config<> / mapping<> in ann_utils.cuh")
        com = open(os.path.join(root, "cpp/src/neighbors/ivf_common.cuh")).read()
        oob = _cut(com, "template <typename IdxT>\nconstexpr static IdxT kOutOfBoundsRecord", "\n\n",
                   "kOutOfBoundsRecord in ivf_common.cuh")
        post = _cut(com, "__device__ inline auto find_chunk_ix", "/** Update the state of the dependent index",
                    "the post-processing functions in ivf_common.cuh")
        for name, body in (("ann_utils_mapping.inc", part), ("ivf_common_postprocess.inc", oob + "\n\n" + post)):
            path = os.path.join(ext, name)
            if not os.path.exists(path) or open(path).read() != body:
                with open(path, "w") as f:
                    f.write(body)
        _make("refdev", root)
    return so if os.path.exists(so) else None


class _OrcIndex(C.Structure):
    _fields_ = [("metric", C.c_int32), ("codebook_kind", C.c_int32),
                ("n_lists", C.c_uint32), ("dim", C.c_uint32), ("dim_ext", C.c_uint32),
                ("rot_dim", C.c_uint32), ("pq_dim", C.c_uint32), ("pq_len", C.c_uint32),
                ("pq_bits", C.c_uint32), ("_pad", C.c_uint32),
                ("pq_centers", C.c_void_p), ("centers", C.c_void_p), ("centers_rot", C.c_void_p),
                ("rotation", C.c_void_p), ("list_sizes", C.c_void_p), ("code_offsets", C.c_void_p),
                ("codes", C.c_void_p), ("id_offsets", C.c_void_p), ("ids", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_lib())
        _lib.orc_fp8_encode.restype = C.c_uint8
        _lib.orc_fp8_encode.argtypes = [C.c_float, C.c_int]
        _lib.orc_fp8_decode.restype = C.c_float
        _lib.orc_fp8_decode.argtypes = [C.c_uint8, C.c_int]
        _lib.orc_fp8_decode_half.restype = C.c_uint16
        _lib.orc_fp8_decode_half.argtypes = [C.c_uint8, C.c_int]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_list_bytes.restype = C.c_uint64
        _lib.orc_list_bytes.argtypes = [C.c_uint32] * 3
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def n_pieces(pq_dim: int, pq_bits: int) -> int:
    cpp = 128 // pq_bits
    return (pq_dim + cpp - 1) // cpp


def list_bytes(n_rows: int, pq_dim: int, pq_bits: int) -> int:
    return ((n_rows + 31) // 32) * n_pieces(pq_dim, pq_bits) * 512


def calculate_pq_dim(dim: int) -> int:
    """cpp/src/neighbors/ivf_pq_index.cu:611-622."""
    if dim >= 128:
        dim //= 2
    r = dim // 32 * 32
    if r > 0:
        return r
    r = 1
    while (r << 1) <= dim:
        r <<= 1
    return r


# --------------------------------------------------------------------------------------------
# .npy v1.0 records
# --------------------------------------------------------------------------------------------

def _descr(dt: np.dtype) -> str:
    dt = np.dtype(dt)
    if dt == np.bool_:
        return "|u1"   # the reference serialises bool through its unsigned-integer branch
    return dt.str


def write_record(f, arr) -> None:
    """One .npy v1.0 record: magic, version, u16 header length, dict padded with spaces to a
    64-byte multiple and closed by a newline, then the raw little-endian C-order data."""
    arr = np.asarray(arr)
    shape = arr.shape
    if len(shape) == 0:
        shape_s = "()"
    elif len(shape) == 1:
        shape_s = f"({shape[0]},)"
    else:
        shape_s = "(" + ", ".join(str(s) for s in shape) + ")"
    d = f"{{'descr': '{_descr(arr.dtype)}', 'fortran_order': False, 'shape': {shape_s}}}"
    preamble = 6 + 2 + 2 + len(d) + 1
    pad = 64 - preamble % 64
    header = d + " " * pad + "\n"
    f.write(b"\x93NUMPY\x01\x00")
    f.write(struct.pack("<H", len(header)))
    f.write(header.encode("latin1"))
    f.write(np.ascontiguousarray(arr).tobytes())


def read_record(f, expect_dtype=None, expect_shape=None) -> np.ndarray:
    magic = f.read(6)
    if magic != b"\x93NUMPY":
        raise ValueError("bad .npy magic")
    major, minor = f.read(2)
    if major == 1:
        (hlen,) = struct.unpack("<H", f.read(2))
    else:
        (hlen,) = struct.unpack("<I", f.read(4))
    header = f.read(hlen).decode("latin1")
    import ast
    meta = ast.literal_eval(header.strip())
    if meta["fortran_order"]:
        raise ValueError("fortran order not supported")
    dt = np.dtype(meta["descr"])
    shape = tuple(meta["shape"])
    n = int(np.prod(shape, dtype=np.int64)) if shape else 1
    data = f.read(n * dt.itemsize)
    if len(data) != n * dt.itemsize:
        raise ValueError("truncated record")
    arr = np.frombuffer(data, dtype=dt).reshape(shape).copy()
    if expect_dtype is not None and np.dtype(expect_dtype).itemsize != dt.itemsize:
        raise ValueError(f"dtype mismatch: {dt} vs {expect_dtype}")
    if expect_shape is not None and tuple(expect_shape) != shape:
        raise ValueError(f"shape mismatch: {shape} vs {expect_shape}")
    return arr


# --------------------------------------------------------------------------------------------
# multi-GPU index files (cpp/src/neighbors/mg/snmg.cuh:60-91 reader, :780-805 writer): four bytes with
# the numpy dtype string of the dataset type, distribution mode and number of ranks as scalar
# records (C++ int), then one complete index stream per rank.  Parity unpinned for the framing, like
# the single-index format: no file written by the reference was available.
# --------------------------------------------------------------------------------------------
REPLICATED, SHARDED = 0, 1


def save_mg(path, mode: int, indexes, dtype_string: str = "<f4") -> None:
    with open(path, "wb") as f:
        f.write(dtype_string.encode("latin1").ljust(4, b"\0")[:4])
        write_record(f, np.int32(mode))
        write_record(f, np.int32(len(indexes)))
        for ix in indexes:
            ix.save(f)


def load_mg(path):
    """Returns (dtype_string, mode, [OracleIndex per rank])."""
    with open(path, "rb") as f:
        dtype_string = f.read(4).rstrip(b"\0").decode("latin1")
        mode = int(read_record(f))
        n = int(read_record(f))
        return dtype_string, mode, [OracleIndex.load(f) for _ in range(n)]


# --------------------------------------------------------------------------------------------
# index
# --------------------------------------------------------------------------------------------

@dataclass
class OracleIndex:
    metric: int
    codebook_kind: int
    dim: int
    pq_dim: int
    pq_bits: int
    n_lists: int
    pq_centers: np.ndarray      # f32 [pq_dim | n_lists, pq_len, 1 << pq_bits]
    centers: np.ndarray         # f32 [n_lists, dim_ext]
    centers_rot: np.ndarray     # f32 [n_lists, rot_dim]
    rotation: np.ndarray        # f32 [rot_dim, dim]
    list_sizes: np.ndarray      # u32 [n_lists]
    list_codes: list = field(default_factory=list)   # per list u8 [groups, pieces, 32, 16]
    list_ids: list = field(default_factory=list)     # per list i64 [size]
    conservative_memory_allocation: bool = False
    # 1 = INTERLEAVED (searchable); 0 = FLAT: list_codes[l] is u8 [size, ceil(pq_dim * pq_bits / 8)],
    # one bit-packed row per vector (cpp/include/cuvs/neighbors/ivf_pq.hpp:308-360)
    codes_layout: int = 1
    _flat: tuple | None = None

    @property
    def pq_len(self):
        return (self.dim + self.pq_dim - 1) // self.pq_dim

    @property
    def rot_dim(self):
        return self.pq_len * self.pq_dim

    @property
    def dim_ext(self):
        return round_up(self.dim + 1, 8)

    @property
    def size(self):
        return int(self.list_sizes.astype(np.int64).sum())

    # -- flat arrays the C library walks -------------------------------------------------------
    def flat(self):
        if self.codes_layout != 1:
            raise ValueError("IVF-PQ search requires INTERLEAVED codes layout")
        if self._flat is None:
            lb = np.array([list_bytes(int(s), self.pq_dim, self.pq_bits) for s in self.list_sizes],
                          dtype=np.uint64)
            code_off = np.zeros(self.n_lists, dtype=np.uint64)
            code_off[1:] = np.cumsum(lb)[:-1]
            id_off = np.zeros(self.n_lists, dtype=np.uint64)
            id_off[1:] = np.cumsum(self.list_sizes.astype(np.uint64))[:-1]
            codes = np.zeros(int(lb.sum()) + 16, dtype=np.uint8)
            ids = np.zeros(max(self.size, 1), dtype=np.int64)
            for l in range(self.n_lists):
                s = int(self.list_sizes[l])
                if s:
                    codes[int(code_off[l]):int(code_off[l]) + int(lb[l])] = \
                        self.list_codes[l].reshape(-1)[:int(lb[l])]
                    ids[int(id_off[l]):int(id_off[l]) + s] = self.list_ids[l][:s]
            self._flat = (code_off, codes, id_off, ids)
        return self._flat

    def c_struct(self):
        code_off, codes, id_off, ids = self.flat()
        self._keep = [np.ascontiguousarray(a) for a in (
            self.pq_centers, self.centers, self.centers_rot, self.rotation, self.list_sizes)]
        s = _OrcIndex(self.metric, self.codebook_kind, self.n_lists, self.dim, self.dim_ext,
                      self.rot_dim, self.pq_dim, self.pq_len, self.pq_bits, 0,
                      _ptr(self._keep[0]), _ptr(self._keep[1]), _ptr(self._keep[2]),
                      _ptr(self._keep[3]), _ptr(self._keep[4]), _ptr(code_off), _ptr(codes),
                      _ptr(id_off), _ptr(ids))
        return s

    # -- file format v4 ----------------------------------------------------------------------
    def save(self, path_or_file) -> None:
        f = open(path_or_file, "wb") if isinstance(path_or_file, (str, os.PathLike)) else path_or_file
        try:
            write_record(f, np.int32(SERIALIZATION_VERSION))
            write_record(f, np.int64(self.size))
            write_record(f, np.uint32(self.dim))
            write_record(f, np.uint32(self.pq_bits))
            write_record(f, np.uint32(self.pq_dim))
            write_record(f, np.bool_(self.conservative_memory_allocation))
            write_record(f, np.int32(self.metric))
            write_record(f, np.int32(self.codebook_kind))
            write_record(f, np.int32(self.codes_layout))
            write_record(f, np.uint32(self.n_lists))
            write_record(f, self.pq_centers.astype(np.float32))
            write_record(f, self.centers.astype(np.float32))
            write_record(f, self.centers_rot.astype(np.float32))
            write_record(f, self.rotation.astype(np.float32))
            write_record(f, self.list_sizes.astype(np.uint32))
            np_ = n_pieces(self.pq_dim, self.pq_bits)
            for l in range(self.n_lists):
                s = int(self.list_sizes[l])
                write_record(f, np.uint32(s))
                if s == 0:
                    continue
                if self.codes_layout == 0:
                    bpv = (self.pq_dim * self.pq_bits + 7) // 8
                    write_record(f, np.ascontiguousarray(self.list_codes[l], dtype=np.uint8).reshape(s, bpv))
                else:
                    g = (s + 31) // 32
                    write_record(f, self.list_codes[l].reshape(-1)[:g * np_ * 512].reshape(g, np_, 32, 16))
                write_record(f, np.asarray(self.list_ids[l][:s], dtype=np.int64))
        finally:
            if isinstance(path_or_file, (str, os.PathLike)):
                f.close()

    @staticmethod
    def load(path_or_file) -> "OracleIndex":
        f = open(path_or_file, "rb") if isinstance(path_or_file, (str, os.PathLike)) else path_or_file
        try:
            ver = int(read_record(f))
            if ver != SERIALIZATION_VERSION:
                raise ValueError(f"serialization version mismatch {ver} vs {SERIALIZATION_VERSION}")
            n_rows = int(read_record(f))
            dim = int(read_record(f))
            pq_bits = int(read_record(f))
            pq_dim = int(read_record(f))
            cma = bool(read_record(f))
            metric = int(read_record(f))
            kind = int(read_record(f))
            layout = int(read_record(f))
            if layout not in (0, 1):
                raise ValueError(f"invalid list_layout value {layout}")
            n_lists = int(read_record(f))
            pq_centers = read_record(f).astype(np.float32)
            centers = read_record(f).astype(np.float32)
            centers_rot = read_record(f).astype(np.float32)
            rotation = read_record(f).astype(np.float32)
            list_sizes = read_record(f).astype(np.uint32)
            codes, ids = [], []
            for l in range(n_lists):
                s = int(read_record(f))
                if s == 0:
                    codes.append(np.zeros((0,), np.uint8))
                    ids.append(np.zeros((0,), np.int64))
                    continue
                codes.append(read_record(f).astype(np.uint8))
                ids.append(read_record(f).astype(np.int64))
            ix = OracleIndex(metric, kind, dim, pq_dim, pq_bits, n_lists, pq_centers, centers,
                             centers_rot, rotation, list_sizes, codes, ids, cma, layout)
            assert ix.size == n_rows
            return ix
        finally:
            if isinstance(path_or_file, (str, os.PathLike)):
                f.close()


# --------------------------------------------------------------------------------------------
# code packing
# --------------------------------------------------------------------------------------------

def pack_list(codes: np.ndarray, pq_bits: int) -> np.ndarray:
    """[n, pq_dim] one code per byte -> interleaved u8 [groups, pieces, 32, 16]."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    n, pq_dim = codes.shape
    out = np.zeros(list_bytes(n, pq_dim, pq_bits), dtype=np.uint8)
    lib().orc_pack_list(_ptr(codes), C.c_uint32(n), C.c_uint32(pq_dim), C.c_uint32(pq_bits),
                        C.c_uint32(0), _ptr(out))
    return out.reshape(-1, n_pieces(pq_dim, pq_bits), 32, 16)


def unpack_list(data: np.ndarray, n: int, pq_dim: int, pq_bits: int) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.zeros((n, pq_dim), dtype=np.uint8)
    lib().orc_unpack_list(_ptr(data), C.c_uint32(n), C.c_uint32(pq_dim), C.c_uint32(pq_bits),
                          C.c_uint32(0), _ptr(out))
    return out


def pack_list_numpy(codes: np.ndarray, pq_bits: int) -> np.ndarray:
    """Independent numpy statement of the same layout (little-endian bit stream per 16-byte piece)."""
    codes = np.asarray(codes, dtype=np.uint8)
    n, pq_dim = codes.shape
    cpp = 128 // pq_bits
    np_ = n_pieces(pq_dim, pq_bits)
    g = (n + 31) // 32
    out = np.zeros((g, np_, 32, 16), dtype=np.uint8)
    for i in range(n):
        for c in range(np_):
            val = 0
            for k in range(cpp):
                j = c * cpp + k
                if j < pq_dim:
                    val |= int(codes[i, j]) << (k * pq_bits)
            out[i // 32, c, i % 32, :] = np.frombuffer(val.to_bytes(16, "little"), dtype=np.uint8)
    return out


def pack_contiguous(codes: np.ndarray, pq_bits: int) -> np.ndarray:
    """[n, pq_dim] one code per byte -> bit-packed rows u8 [n, ceil(pq_dim * pq_bits / 8)], code j
    at bits [j * pq_bits, (j + 1) * pq_bits) of the row's little-endian bit stream
    (bitfield_view_t over the row, cpp/src/neighbors/ivf_pq/ivf_pq_codepacking.cuh:201-218)."""
    codes = np.asarray(codes, dtype=np.uint8)
    n, pq_dim = codes.shape
    bits = ((codes[:, :, None] >> np.arange(pq_bits, dtype=np.uint8)) & 1).reshape(n, pq_dim * pq_bits)
    pad = (-bits.shape[1]) % 8
    bits = np.concatenate([bits, np.zeros((n, pad), dtype=np.uint8)], axis=1)
    return np.packbits(bits.reshape(n, -1, 8), axis=2, bitorder="little").reshape(n, -1)


def map_from_float(x: np.ndarray, dtype) -> np.ndarray:
    """mapping<T> applied to f32 values (cpp/src/neighbors/detail/ann_utils.cuh:168-217): scale by
    128 (int8, clamped to [-128, 127] first) or 256 (uint8, in-range values only: the conversion of
    the others is whatever the device's float -> integer cast does), then truncation toward zero."""
    dtype = np.dtype(dtype)
    x = np.asarray(x, dtype=np.float32)
    if dtype == np.int8:
        return np.trunc(np.clip(x * np.float32(128.0), -128.0, 127.0)).astype(np.int8)
    if dtype == np.uint8:
        return np.trunc(x * np.float32(256.0)).astype(np.uint8)
    return x.astype(dtype)


def reconstruct_list(ix: "OracleIndex", label: int, rows: np.ndarray) -> np.ndarray:
    """Decoded vectors f32 [len(rows), dim] of rows of one list
    (reconstruct_vectors + the product with the rotation matrix,
    cpp/src/neighbors/ivf_pq/ivf_pq_build.cuh:519-571 and :593-676):
    rotated[i, j, k] = pq_centers[j or label, k, code(i, j)] + centers_rot[label, j, k] in fp32,
    out[i, :] = rotation^T @ rotated[i, :] (the reference calls a library GEMM there, whose summation
    order is not specified; this restatement accumulates in float64 and callers compare with a
    tolerance)."""
    n = int(ix.list_sizes[label])
    codes = unpack_list(ix.list_codes[label], n, ix.pq_dim, ix.pq_bits)[np.asarray(rows, dtype=np.int64)]
    j = np.arange(ix.pq_dim)
    if ix.codebook_kind == 1:
        book = ix.pq_centers[label][None, :, :].repeat(ix.pq_dim, axis=0)    # [pq_dim, len, book]
    else:
        book = ix.pq_centers
    dec = book[j[None, :], :, codes.astype(np.int64)]                        # [n, pq_dim, len]
    rot = dec.astype(np.float32) + ix.centers_rot[label].reshape(1, ix.pq_dim, ix.pq_len)
    rot = rot.reshape(len(codes), ix.rot_dim).astype(np.float32)
    return (rot.astype(np.float64) @ ix.rotation.astype(np.float64)).astype(np.float32)


# --------------------------------------------------------------------------------------------
# search
# --------------------------------------------------------------------------------------------

def map_to_float(x: np.ndarray) -> np.ndarray:
    """mapping<float> of cpp/src/neighbors/detail/ann_utils.cuh:168-199."""
    if x.dtype == np.uint8:
        return x.astype(np.float32) * np.float32(1.0 / 256.0)
    if x.dtype == np.int8:
        return x.astype(np.float32) * np.float32(1.0 / 128.0)
    return x.astype(np.float32)


def prepare_queries(ix: OracleIndex, queries: np.ndarray):
    q = np.ascontiguousarray(queries)
    n_q = q.shape[0]
    fq = np.zeros((n_q, ix.dim_ext), dtype=np.float32)
    rq = np.zeros((n_q, ix.rot_dim), dtype=np.float32)
    s = ix.c_struct()
    lib().orc_prepare_queries(C.byref(s), _ptr(q), C.c_int(_QTYPE[q.dtype]), C.c_uint32(n_q),
                              _ptr(fq), _ptr(rq))
    return fq, rq


def select_clusters(ix: OracleIndex, fq: np.ndarray, n_probes: int, want_all: bool = False):
    n_q = fq.shape[0]
    n_probes = min(n_probes, ix.n_lists)
    probes = np.zeros((n_q, n_probes), dtype=np.uint32)
    scores = np.zeros((n_q, n_probes), dtype=np.float32)
    all_scores = np.zeros((n_q, ix.n_lists), dtype=np.float32) if want_all else None
    s = ix.c_struct()
    lib().orc_select_clusters(C.byref(s), _ptr(fq), C.c_uint32(n_q), C.c_uint32(n_probes),
                              _ptr(probes), _ptr(scores),
                              _ptr(all_scores) if want_all else None)
    return (probes, scores, all_scores) if want_all else (probes, scores)


def int8_operands(ix: OracleIndex):
    """(centers_int8 [n_lists, dim_ext_int8], rotation_int8 [rot_dim, dim]) of the int8 coarse search
    (cpp/src/neighbors/ivf_pq_index.cu:624-738)."""
    d8 = int(lib().orc_dim_ext_int8(C.c_uint32(ix.dim)))
    c8 = np.zeros((ix.n_lists, d8), dtype=np.int8)
    r8 = np.zeros((ix.rot_dim, ix.dim), dtype=np.int8)
    s = ix.c_struct()
    lib().orc_centers_int8(C.byref(s), _ptr(c8))
    lib().orc_rotation_int8(C.byref(s), _ptr(r8))
    return c8, r8


def prepare_queries_int8(ix: OracleIndex, queries: np.ndarray, r8: np.ndarray):
    q = np.ascontiguousarray(queries)
    n_q = q.shape[0]
    d8 = int(lib().orc_dim_ext_int8(C.c_uint32(ix.dim)))
    q8 = np.zeros((n_q, d8), dtype=np.int8)
    rq = np.zeros((n_q, ix.rot_dim), dtype=np.float32)
    s = ix.c_struct()
    lib().orc_prepare_queries_int8(C.byref(s), _ptr(q), C.c_int(_QTYPE[q.dtype]), C.c_uint32(n_q),
                                   _ptr(r8), _ptr(q8), _ptr(rq))
    return q8, rq


def select_clusters_int8(ix: OracleIndex, c8: np.ndarray, q8: np.ndarray, n_probes: int):
    n_q = q8.shape[0]
    n_probes = min(n_probes, ix.n_lists)
    probes = np.zeros((n_q, n_probes), dtype=np.uint32)
    scores = np.zeros((n_q, n_probes), dtype=np.int32)
    s = ix.c_struct()
    lib().orc_select_clusters_int8(C.byref(s), _ptr(c8), _ptr(q8), C.c_uint32(n_q),
                                   C.c_uint32(n_probes), _ptr(probes), _ptr(scores))
    return probes, scores


def search_int8_coarse(ix: OracleIndex, queries: np.ndarray, k: int, n_probes: int = 20,
                       lut_dtype=CUDA_R_32F, internal_dtype=CUDA_R_32F, return_probes=False):
    """search with coarse_search_dtype = CUDA_R_8I (ivf_pq_search.cuh:171-256, :926-1048): int8 images
    of centers, rotation matrix and queries, int32 coarse scores, rotated queries (R8 q8) / 128^2;
    the fine search is the usual one."""
    q = np.ascontiguousarray(queries)
    c8, r8 = int8_operands(ix)
    q8, rq = prepare_queries_int8(ix, q, r8)
    probes, scores = select_clusters_int8(ix, c8, q8, n_probes)
    scale = {np.dtype(np.uint8): 256.0, np.dtype(np.int8): 128.0}.get(q.dtype, 1.0)
    ds, nb, _ = search_probes(ix, rq, probes, k, lut_dtype, internal_dtype, scale)
    return (ds, nb, probes, scores) if return_probes else (ds, nb)


def search_f16_coarse(ix: OracleIndex, queries: np.ndarray, k: int, n_probes: int = 20,
                      lut_dtype=CUDA_R_32F, internal_dtype=CUDA_R_32F, return_probes=False):
    """search with coarse_search_dtype = CUDA_R_16F (ivf_pq_search.cuh:259-340, :996-1025): queries,
    centers and rotation matrix rounded to half precision, half-precision coarse scores ordered by
    (score, list id), rotated queries from the half-rounded operands; the fine search is the usual one."""
    q = np.ascontiguousarray(queries)
    n_q = q.shape[0]
    n_probes = min(n_probes, ix.n_lists)
    fq = np.zeros((n_q, ix.dim_ext), dtype=np.float32)
    rq = np.zeros((n_q, ix.rot_dim), dtype=np.float32)
    s = ix.c_struct()
    lib().orc_prepare_queries_f16(C.byref(s), _ptr(q), C.c_int(_QTYPE[q.dtype]), C.c_uint32(n_q), _ptr(fq), _ptr(rq))
    probes = np.zeros((n_q, n_probes), dtype=np.uint32)
    scores = np.zeros((n_q, n_probes), dtype=np.float32)
    lib().orc_select_clusters_f16(C.byref(s), _ptr(fq), C.c_uint32(n_q), C.c_uint32(n_probes), _ptr(probes),
                                  _ptr(scores))
    scale = {np.dtype(np.uint8): 256.0, np.dtype(np.int8): 128.0}.get(q.dtype, 1.0)
    ds, nb, _ = search_probes(ix, rq, probes, k, lut_dtype, internal_dtype, scale)
    return (ds, nb, probes, scores) if return_probes else (ds, nb)


def build_lut(ix: OracleIndex, label: int, rot_q: np.ndarray, lut_dtype: int) -> np.ndarray:
    n = ix.pq_dim << ix.pq_bits
    dt = {CUDA_R_32F: np.float32, CUDA_R_16F: np.float16, CUDA_R_8U: np.uint8}[lut_dtype]
    out = np.zeros(n, dtype=dt)
    s = ix.c_struct()
    rq = np.ascontiguousarray(rot_q, dtype=np.float32)
    lib().orc_build_lut(C.byref(s), C.c_uint32(label), _ptr(rq), C.c_int(lut_dtype), _ptr(out))
    return out


def pair_scores(ix: OracleIndex, label: int, rot_q: np.ndarray, lut_dtype: int,
                internal_dtype: int = CUDA_R_32F) -> np.ndarray:
    """Internal score of every vector of list `label` for one rotated query, in stored order."""
    out = np.zeros(int(ix.list_sizes[label]), dtype=np.float32)
    s = ix.c_struct()
    rq = np.ascontiguousarray(rot_q, dtype=np.float32)
    rc = lib().orc_pair_scores(C.byref(s), C.c_uint32(label), _ptr(rq), C.c_int(lut_dtype),
                               C.c_int(internal_dtype), _ptr(out))
    if rc != 0:
        raise ValueError("unsupported lut_dtype / internal_distance_dtype combination")
    return out


def postprocess(scores: np.ndarray, metric: int, scale: float = 1.0) -> np.ndarray:
    f = lib().orc_postprocess
    f.restype = C.c_float
    f.argtypes = [C.c_float, C.c_int, C.c_float]
    flat = np.asarray(scores, dtype=np.float32).reshape(-1)
    return np.array([f(float(v), int(metric), float(scale)) for v in flat],
                    dtype=np.float32).reshape(np.shape(scores))


def search_probes(ix: OracleIndex, rot_q, probes, k, lut_dtype=CUDA_R_32F,
                  internal_dtype=CUDA_R_32F, scale=1.0):
    n_q, n_probes = probes.shape
    nb = np.zeros((n_q, k), dtype=np.int64)
    ds = np.zeros((n_q, k), dtype=np.float32)
    raw = np.zeros((n_q, k), dtype=np.float32)
    s = ix.c_struct()
    rq = np.ascontiguousarray(rot_q, dtype=np.float32)
    pr = np.ascontiguousarray(probes, dtype=np.uint32)
    rc = lib().orc_search_probes(C.byref(s), _ptr(rq), _ptr(pr), C.c_uint32(n_q),
                                 C.c_uint32(n_probes), C.c_uint32(k), C.c_int(lut_dtype),
                                 C.c_int(internal_dtype), C.c_float(scale), _ptr(nb), _ptr(ds),
                                 _ptr(raw))
    if rc != 0:
        raise ValueError("unsupported lut_dtype / internal_distance_dtype combination")
    return ds, nb, raw


def search(ix: OracleIndex, queries: np.ndarray, k: int, n_probes: int = 20,
           lut_dtype=CUDA_R_32F, internal_dtype=CUDA_R_32F, return_probes=False, bitset=None):
    """Returns (distances f32 [n_q,k], neighbors i64 [n_q,k]) like the reference's search.
    `bitset` (u32 words, bit i = source id i may be returned) is the reference's bitset filter."""
    q = np.ascontiguousarray(queries)
    if bitset is not None:
        bits = np.ascontiguousarray(bitset, dtype=np.uint32)
        lib().orc_set_filter(_ptr(bits), C.c_uint64(bits.size * 32))
    try:
        return _search(ix, q, k, n_probes, lut_dtype, internal_dtype, return_probes)
    finally:
        if bitset is not None:
            lib().orc_set_filter(None, C.c_uint64(0))


def _search(ix, q, k, n_probes, lut_dtype, internal_dtype, return_probes):
    n_q = q.shape[0]
    if q.shape[1] != ix.dim:
        raise ValueError("Number of query dimensions should equal number of dimensions in the index.")
    n_probes = min(n_probes, ix.n_lists)
    nb = np.zeros((n_q, k), dtype=np.int64)
    ds = np.zeros((n_q, k), dtype=np.float32)
    probes = np.zeros((n_q, n_probes), dtype=np.uint32)
    s = ix.c_struct()
    rc = lib().orc_search(C.byref(s), _ptr(q), C.c_int(_QTYPE[q.dtype]), C.c_uint32(n_q),
                          C.c_uint32(n_probes), C.c_uint32(k), C.c_int(lut_dtype),
                          C.c_int(internal_dtype), _ptr(nb), _ptr(ds), _ptr(probes))
    if rc != 0:
        raise ValueError(f"oracle search failed ({rc})")
    return (ds, nb, probes) if return_probes else (ds, nb)


# --------------------------------------------------------------------------------------------
# CPU builder (fixtures)
# --------------------------------------------------------------------------------------------

def _kmeans(x: np.ndarray, k: int, iters: int, rng: np.random.Generator) -> np.ndarray:
    n = x.shape[0]
    if n >= k:
        c = x[rng.choice(n, size=k, replace=False)].copy()
    else:
        c = np.concatenate([x, x[rng.integers(0, n, size=k - n)] +
                            1e-3 * rng.standard_normal((k - n, x.shape[1])).astype(np.float32)])
    for _ in range(iters):
        lab = _assign(x, c)
        sums = np.zeros_like(c, dtype=np.float64)
        np.add.at(sums, lab, x)
        cnt = np.bincount(lab, minlength=k)
        nz = cnt > 0
        c[nz] = (sums[nz] / cnt[nz, None]).astype(np.float32)
        if (~nz).any():
            c[~nz] = x[rng.integers(0, n, size=int((~nz).sum()))]
    return c.astype(np.float32)


def _assign(x: np.ndarray, c: np.ndarray) -> np.ndarray:
    out = np.empty(x.shape[0], dtype=np.int64)
    cn = (c.astype(np.float64) ** 2).sum(1)
    step = max(1, 4_000_000 // max(1, c.shape[0]))
    for s in range(0, x.shape[0], step):
        xb = x[s:s + step].astype(np.float64)
        d = cn[None, :] - 2.0 * xb @ c.astype(np.float64).T
        out[s:s + step] = d.argmin(1)
    return out


def random_rotation(rot_dim: int, dim: int, rng: np.random.Generator) -> np.ndarray:
    a = rng.standard_normal((rot_dim, rot_dim))
    qm, _ = np.linalg.qr(a)
    return np.ascontiguousarray(qm[:, :dim].astype(np.float32)) if rot_dim >= dim else None


def build_index(dataset: np.ndarray, n_lists: int, pq_dim: int = 0, pq_bits: int = 8,
                metric: int = L2Expanded, codebook_kind: int = PER_SUBSPACE,
                force_random_rotation: bool = False, kmeans_iters: int = 10, seed: int = 0,
                ids: np.ndarray | None = None) -> OracleIndex:
    rng = np.random.default_rng(seed)
    x = map_to_float(np.asarray(dataset))
    n, dim = x.shape
    if metric == CosineExpanded:
        x = x / np.maximum(np.linalg.norm(x, axis=1, keepdims=True), 1e-20).astype(np.float32)
    pq_dim = pq_dim or calculate_pq_dim(dim)
    assert 4 <= pq_bits <= 8 and (pq_bits * pq_dim) % 8 == 0
    pq_len = (dim + pq_dim - 1) // pq_dim
    rot_dim = pq_len * pq_dim
    dim_ext = round_up(dim + 1, 8)
    book = 1 << pq_bits

    cent = _kmeans(x, n_lists, kmeans_iters, rng)
    labels = _assign(x, cent)
    if rot_dim == dim and not force_random_rotation:
        rot = np.eye(dim, dtype=np.float32)
    else:
        rot = random_rotation(rot_dim, dim, rng)
    centers = np.zeros((n_lists, dim_ext), dtype=np.float32)
    centers[:, :dim] = cent
    centers[:, dim] = (cent.astype(np.float64) ** 2).sum(1).astype(np.float32)
    centers_rot = (cent.astype(np.float64) @ rot.astype(np.float64).T).astype(np.float32)

    resid = ((x - cent[labels]).astype(np.float64) @ rot.astype(np.float64).T).astype(np.float32)
    if codebook_kind == PER_SUBSPACE:
        pqc = np.zeros((pq_dim, pq_len, book), dtype=np.float32)
        sub = resid[rng.choice(n, size=min(n, 256 * book), replace=False)]
        for j in range(pq_dim):
            cb = _kmeans(sub[:, j * pq_len:(j + 1) * pq_len], book, 8, rng)
            pqc[j] = cb.T
    else:
        pqc = np.zeros((n_lists, pq_len, book), dtype=np.float32)
        for l in range(n_lists):
            r = resid[labels == l]
            if r.shape[0] == 0:
                r = resid[rng.integers(0, n, size=book)]
            pts = r.reshape(-1, pq_len)
            if pts.shape[0] > 64 * book:
                pts = pts[rng.choice(pts.shape[0], size=64 * book, replace=False)]
            pqc[l] = _kmeans(pts, book, 6, rng).T

    ix = OracleIndex(metric, codebook_kind, dim, pq_dim, pq_bits, n_lists, pqc, centers,
                     centers_rot, rot, np.zeros(n_lists, dtype=np.uint32))
    # encode with the C encoder (same argmin rule as the reference's encoder)
    ix.list_codes = [np.zeros(0, np.uint8)] * n_lists
    ix.list_ids = [np.zeros(0, np.int64)] * n_lists
    s = ix.c_struct()
    codes = np.zeros((n, pq_dim), dtype=np.uint8)
    xl = np.ascontiguousarray(x, dtype=np.float32)
    lab32 = np.ascontiguousarray(labels, dtype=np.uint32)
    lib().orc_encode(C.byref(s), _ptr(xl), _ptr(lab32), C.c_uint32(n), _ptr(codes))
    all_ids = np.arange(n, dtype=np.int64) if ids is None else np.asarray(ids, dtype=np.int64)
    order = np.argsort(labels, kind="stable")
    sizes = np.bincount(labels, minlength=n_lists).astype(np.uint32)
    pos = 0
    lc, li = [], []
    for l in range(n_lists):
        sl = order[pos:pos + int(sizes[l])]
        pos += int(sizes[l])
        if len(sl):
            lc.append(pack_list(codes[sl], pq_bits))
            li.append(all_ids[sl].copy())
        else:
            lc.append(np.zeros(0, np.uint8))
            li.append(np.zeros(0, np.int64))
    ix.list_sizes = sizes
    ix.list_codes = lc
    ix.list_ids = li
    ix._flat = None
    return ix


# --------------------------------------------------------------------------------------------
# exact k-NN and recall
# --------------------------------------------------------------------------------------------

def brute_force(dataset: np.ndarray, queries: np.ndarray, k: int, metric: int = L2Expanded):
    x = map_to_float(np.asarray(dataset)).astype(np.float64)
    q = map_to_float(np.asarray(queries)).astype(np.float64)
    if metric in (L2Expanded, L2SqrtExpanded):
        d = (q ** 2).sum(1)[:, None] + (x ** 2).sum(1)[None, :] - 2.0 * q @ x.T
    elif metric == InnerProduct:
        d = -(q @ x.T)
    else:
        xn = x / np.maximum(np.linalg.norm(x, axis=1, keepdims=True), 1e-30)
        qn = q / np.maximum(np.linalg.norm(q, axis=1, keepdims=True), 1e-30)
        d = 1.0 - qn @ xn.T
    idx = np.argpartition(d, min(k, d.shape[1] - 1), axis=1)[:, :k]
    dd = np.take_along_axis(d, idx, axis=1)
    o = np.argsort(dd, axis=1, kind="stable")
    return np.take_along_axis(dd, o, axis=1), np.take_along_axis(idx, o, axis=1)


def recall(found: np.ndarray, truth: np.ndarray) -> float:
    hits = 0
    for f, t in zip(found, truth):
        hits += len(set(f.tolist()) & set(t.tolist()))
    return hits / truth.size
