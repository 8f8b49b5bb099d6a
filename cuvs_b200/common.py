"""Resources handle and tensor marshalling shared by the Python mirror of the C interface."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib as L

_TORCH_DL = {torch.float32: (L.kDLFloat, 32), torch.float16: (L.kDLFloat, 16),
             torch.int8: (L.kDLInt, 8), torch.uint8: (L.kDLUInt, 8), torch.int64: (L.kDLInt, 64),
             torch.uint32: (L.kDLUInt, 32), torch.int32: (L.kDLInt, 32)}
_NP_DL = {np.dtype(np.float32): (L.kDLFloat, 32), np.dtype(np.float16): (L.kDLFloat, 16),
          np.dtype(np.int8): (L.kDLInt, 8), np.dtype(np.uint8): (L.kDLUInt, 8),
          np.dtype(np.int64): (L.kDLInt, 64), np.dtype(np.uint32): (L.kDLUInt, 32),
          np.dtype(np.int32): (L.kDLInt, 32)}


class Resources:
    """Mirror of ``cuvs.common.Resources``: owns a ``cuvsResources_t`` bound to the current device.

    Work is enqueued on ``stream`` (default: torch's current stream at call time); ``sync()`` waits
    for it.
    """

    def __init__(self, stream: int | None = None):
        self._lib = L.load()
        h = C.c_size_t(0)
        L.check(self._lib.cuvsResourcesCreate(C.byref(h)))
        self.handle = h.value
        self._fixed_stream = stream
        if stream is not None:
            L.check(self._lib.cuvsStreamSet(self.handle, C.c_void_p(stream)))

    def use_current_stream(self):
        if self._fixed_stream is None:
            s = torch.cuda.current_stream().cuda_stream
            L.check(self._lib.cuvsStreamSet(self.handle, C.c_void_p(s)))

    def sync(self):
        L.check(self._lib.cuvsStreamSync(self.handle))

    def set_workspace_pool(self, nbytes: int):
        L.check(self._lib.cuvsResourcesSetWorkspacePool(self.handle, C.c_size_t(nbytes)))

    def __del__(self):
        try:
            if getattr(self, "handle", 0):
                self._lib.cuvsResourcesDestroy(self.handle)
                self.handle = 0
        except Exception:
            pass


_default_resources = {}


def default_resources() -> Resources:
    dev = torch.cuda.current_device()
    r = _default_resources.get(dev)
    if r is None:
        r = _default_resources[dev] = Resources()
    return r


class DLTensorRef:
    """A DLManagedTensor describing (not owning) a torch tensor or a numpy array."""

    def __init__(self, obj, strided: bool = False):
        """`strided`: describe a non-contiguous torch tensor by its strides (only entry points that
        say so accept one) instead of refusing it."""
        strides = None
        if isinstance(obj, torch.Tensor):
            if not obj.is_contiguous():
                if not strided:
                    raise ValueError("Expected a row-major matrix")
                strides = tuple(obj.stride())
            code, bits = _TORCH_DL[obj.dtype]
            if obj.is_cuda:
                dev = L.DLDevice(L.kDLCUDA, obj.device.index or 0)
            elif obj.is_pinned():
                dev = L.DLDevice(L.kDLCUDAHost, 0)
            else:
                dev = L.DLDevice(L.kDLCPU, 0)
            ptr, shape = obj.data_ptr(), tuple(obj.shape)
        elif isinstance(obj, np.ndarray):
            if not obj.flags.c_contiguous:
                raise ValueError("Expected a row-major matrix")
            code, bits = _NP_DL[obj.dtype]
            dev = L.DLDevice(L.kDLCPU, 0)
            ptr, shape = obj.ctypes.data, tuple(obj.shape)
        else:
            raise TypeError(f"unsupported array type {type(obj)}")
        self._keep = obj
        self._shape = (C.c_int64 * max(1, len(shape)))(*shape)
        self.managed = L.DLManagedTensor()
        t = self.managed.dl_tensor
        t.data = C.c_void_p(ptr)
        t.device = dev
        t.ndim = len(shape)
        t.dtype = L.DLDataType(code, bits, 1)
        t.shape = C.cast(self._shape, C.POINTER(C.c_int64))
        if strides is None:
            t.strides = None
        else:
            self._strides = (C.c_int64 * len(strides))(*strides)
            t.strides = C.cast(self._strides, C.POINTER(C.c_int64))
        t.byte_offset = 0

    def ref(self):
        return C.byref(self.managed)


_TYPESTR = {(L.kDLFloat, 32): "<f4", (L.kDLUInt, 32): "<u4", (L.kDLInt, 64): "<i8",
            (L.kDLUInt, 8): "|u1"}


class _CudaView:
    def __init__(self, ptr, shape, typestr, strides_bytes):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": strides_bytes}


def view_to_torch(mt: L.DLManagedTensor) -> torch.Tensor:
    """Copy a device view returned by a getter into an owning torch tensor, then free the view's
    shape arrays through its deleter."""
    t = mt.dl_tensor
    shape = tuple(int(t.shape[i]) for i in range(t.ndim))
    typestr = _TYPESTR[(t.dtype.code, t.dtype.bits)]
    itemsize = t.dtype.bits // 8
    strides = None
    if t.strides:
        strides = tuple(int(t.strides[i]) * itemsize for i in range(t.ndim))
    n = 1
    for s in shape:
        n *= s
    if n == 0:
        out = torch.empty(shape, dtype={"<f4": torch.float32, "<u4": torch.uint32,
                                        "<i8": torch.int64, "|u1": torch.uint8}[typestr],
                          device="cuda")
    else:
        out = torch.as_tensor(_CudaView(t.data, shape, typestr, strides), device="cuda").clone()
    if mt.deleter:
        mt.deleter(C.pointer(mt))
    return out
