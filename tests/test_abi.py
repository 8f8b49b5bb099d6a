"""CPU test of the drop-in boundary: the shared library loads and exports every entry point that
include/*.h declares (no compute is called here)."""
import ctypes as C
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"CUVS_EXPORT\s+[\w\s\*]+?\b(cuvs\w+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_headers_declare_the_reference_entry_points():
    names = declared_symbols()
    for must in ("cuvsIvfPqSearch", "cuvsIvfPqBuild", "cuvsIvfPqExtend", "cuvsIvfPqSerialize",
                 "cuvsIvfPqDeserialize", "cuvsIvfPqTransform", "cuvsIvfPqIndexGetCenters",
                 "cuvsResourcesCreate", "cuvsStreamSync", "cuvsGetLastErrorText"):
        assert must in names
    assert len(names) >= 39


def test_library_exports_every_declared_symbol():
    from cuvs_b200 import _lib
    lib = C.CDLL(_lib.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_ctypes_signatures_cover_the_headers():
    from cuvs_b200 import _lib
    declared = declared_symbols() - {"cuvsGetLastErrorText", "cuvsSetLastErrorText"}
    assert declared <= set(_lib.SIGNATURES), declared - set(_lib.SIGNATURES)


def test_param_defaults_match_the_reference():
    """Defaults of c/src/neighbors/ivf_pq.cpp:348-379; these calls touch no GPU."""
    from cuvs_b200 import _lib
    lib = _lib.load()
    ip = C.POINTER(_lib.IndexParamsStruct)()
    assert lib.cuvsIvfPqIndexParamsCreate(C.byref(ip)) == _lib.CUVS_SUCCESS
    p = ip.contents
    assert (p.metric, p.n_lists, p.kmeans_n_iters, p.pq_bits, p.pq_dim) == (0, 1024, 20, 8, 0)
    assert p.kmeans_trainset_fraction == 0.5 and p.add_data_on_build and p.codes_layout == 1
    assert p.max_train_points_per_pq_code == 256 and p.metric_arg == 2.0
    lib.cuvsIvfPqIndexParamsDestroy(ip)
    sp = C.POINTER(_lib.SearchParamsStruct)()
    assert lib.cuvsIvfPqSearchParamsCreate(C.byref(sp)) == _lib.CUVS_SUCCESS
    s = sp.contents
    assert (s.n_probes, s.lut_dtype, s.internal_distance_dtype, s.coarse_search_dtype) == (20, 0, 0, 0)
    assert s.max_internal_batch_size == 4096 and s.preferred_shmem_carveout == 1.0
    lib.cuvsIvfPqSearchParamsDestroy(sp)


def test_error_text_convention():
    from cuvs_b200 import _lib
    lib = _lib.load()
    lib.cuvsSetLastErrorText(b"boom")
    assert lib.cuvsGetLastErrorText() == b"boom"
    lib.cuvsSetLastErrorText(None)
    assert lib.cuvsGetLastErrorText() is None
    # a failing call (null handle) returns CUVS_ERROR and leaves a message
    out = C.c_int(0)
    assert lib.cuvsDeviceIdGet(C.c_size_t(0), C.byref(out)) == _lib.CUVS_ERROR
    assert b"null resources" in lib.cuvsGetLastErrorText()
    a, b, c = C.c_uint16(0), C.c_uint16(0), C.c_uint16(0)
    assert lib.cuvsVersionGet(C.byref(a), C.byref(b), C.byref(c)) == _lib.CUVS_SUCCESS
    assert (a.value, b.value) == (26, 10)
    assert lib.cuvsGetLastErrorText() is None


def test_tensor_descriptions_carry_strides_only_on_request():
    """A non-contiguous tensor is refused unless the caller says the entry point takes strides (the
    merge of gathered per-rank blocks does); then shape and strides are passed in elements."""
    import pytest
    import torch
    from cuvs_b200.common import DLTensorRef
    block = torch.zeros((3, 40), dtype=torch.float32)
    parts = block[:, 8:32].view(3, 4, 6)                  # three [4, 6] parts, 40 elements apart
    assert not parts.is_contiguous()
    with pytest.raises(ValueError, match="row-major"):
        DLTensorRef(parts)
    ref = DLTensorRef(parts, strided=True)
    t = ref.managed.dl_tensor
    assert [t.shape[i] for i in range(3)] == [3, 4, 6]
    assert [t.strides[i] for i in range(3)] == [40, 6, 1]
    assert t.data == parts.data_ptr()
    whole = DLTensorRef(block)
    assert not whole.managed.dl_tensor.strides            # contiguous: no strides, as before
