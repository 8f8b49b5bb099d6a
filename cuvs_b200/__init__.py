"""B200-native IVF-PQ search engine: a drop-in for the ``cuvs::neighbors::ivf_pq`` path.

``cuvs_b200.ivf_pq`` mirrors the reference's Python module of the same name; everything runs
through the C interface of ``libcuvs_b200.so`` (hand-written sm_100a CUDA).  There is no CPU or
library fallback: the module raises at import when the shared library has not been built.
"""
from . import _lib

_lib.load()

from . import ivf_pq  # noqa: E402
from .refine import refine  # noqa: E402
from .common import Resources  # noqa: E402

__all__ = ["ivf_pq", "refine", "Resources"]
