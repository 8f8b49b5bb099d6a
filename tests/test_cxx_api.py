"""The C++ interface: a caller translation unit compiled against include/cuvs/neighbors/ivf_pq.hpp alone
and linked to the shared library (CPU test: it compiles and links, so the header is self-contained and the
library exports what it declares), then run on a GPU (GPU test)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cxx", "caller.cpp")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(out_dir):
    gxx = shutil.which("g++")
    if gxx is None or not os.path.isdir(os.path.join(CUDA, "include")):
        pytest.skip("g++ or the CUDA headers are not available")
    exe = os.path.join(out_dir, "caller")
    lib_dir = os.path.join(ROOT, "cuvs_b200")
    cmd = [gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"), SRC,
           "-o", exe, "-L", lib_dir, "-lcuvs_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"]
    env = dict(os.environ)
    env.pop("CXX", None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr[-4000:]
    return exe


def test_caller_compiles_and_links_against_the_public_header(tmp_path):
    assert os.path.exists(_build(str(tmp_path)))


@pytest.mark.gpu
def test_caller_runs(tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    exe = _build(str(tmp_path))
    r = subprocess.run([exe, str(tmp_path / "caller.ivfpq")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CALLER_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
