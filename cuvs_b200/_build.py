"""Compile the CUDA sources of this package into ``libcuvs_b200.so`` (in-tree, next to this file).

Plain nvcc for sm_100a, one object per translation unit, built in parallel and linked once.
Objects are cached under ``csrc/_obj`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(HERE, "libcuvs_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC,
              "-diag-suppress", "177"]

# (source, object name, extra flags)
UNITS = [("resources.cu", "resources.o", []), ("index.cu", "index.o", []),
         ("coarse.cu", "coarse.o", []), ("coarse_tc.cu", "coarse_tc.o", []), ("search.cu", "search.o", []),
         ("build.cu", "build.o", []), ("c_api.cu", "c_api.o", []),
         ("no_alloc.cu", "no_alloc.o", []), ("refine.cu", "refine.o", []),
         ("dynamic_batching.cu", "dynamic_batching.o", []), ("mg.cu", "mg.o", []),
         ("c_api_mg.cu", "c_api_mg.o", [])]
UNITS += [("scan_inst.cu", f"scan_{b}.o", [f"-DPQ_BITS={b}"]) for b in (4, 5, 6, 7, 8)]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _newest_header() -> float:
    t = 0.0
    for root in (CSRC, INCLUDE):
        for dp, _, files in os.walk(root):
            for f in files:
                if f.endswith((".hpp", ".cuh", ".h")):
                    t = max(t, os.path.getmtime(os.path.join(dp, f)))
    return t


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    hdr_t = _newest_header()
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)

    def compile_one(unit):
        src, obj, extra = unit
        src_p, obj_p = os.path.join(CSRC, src), os.path.join(OBJ, obj)
        if (not force and os.path.exists(obj_p)
                and os.path.getmtime(obj_p) > max(os.path.getmtime(src_p), hdr_t)):
            return obj_p, False
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", src_p, "-o", obj_p]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose and r.stderr.strip():
            print(r.stderr, file=sys.stderr)
        return obj_p, True

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, UNITS))
    objs = [o for o, _ in results]
    if force or any(c for _, c in results) or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-ldl"]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
