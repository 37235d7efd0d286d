"""``QuarkTensor``: a device buffer with a shape and a dtype string, nothing more.

Mirrors the part of the reference tensor class the hot path touches
(``src/quark/runtime/tensor.py:262-1002``): ``data_ptr()``, ``shape``, ``dtype`` in
{"bf16", "e4m3", "f32", "s32"}, row-major contiguous storage, ``zeros`` / ``empty`` /
``from_numpy`` / ``to_numpy`` / ``borrow`` / ``zero_`` / ``reshape``.  bf16 travels on the host
as ``uint16`` and e4m3 as ``uint8``; ``from_numpy`` narrows f32 to bf16 by truncation exactly as
the reference does (``src/quark/runtime/utils.py:51-58``).  Memory comes from the kernel library
(``qb_malloc``); there is no torch anywhere.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib
from . import stream as _stream

_ITEMSIZE = {"bf16": 2, "e4m3": 1, "f32": 4, "s32": 4}
_CARRIER = {"bf16": np.uint16, "e4m3": np.uint8, "f32": np.float32, "s32": np.int32}
_FROM_NP = {np.dtype("float32"): "f32", np.dtype("uint16"): "bf16", np.dtype("int32"): "s32", np.dtype("uint8"): "e4m3"}


class _Storage:
    """Owns one device allocation; freed when the last tensor viewing it goes away."""

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        _lib.check(_lib.load().qb_malloc(C.byref(p), max(int(nbytes), 16)))
        self.ptr = int(p.value)
        self.nbytes = int(nbytes)
        self.host_writes = 0  # copies and fills issued from the host (a cache's shadow copy notices them)

    def __del__(self):
        try:
            if self.ptr:
                _lib.load().qb_free(C.c_void_p(self.ptr))
                self.ptr = 0
        except Exception:
            pass


class _Borrowed:
    """Foreign memory (``src/quark/runtime/tensor.py:88-163`` ``_BorrowedStorage``): never freed here."""

    def __init__(self, ptr: int, nbytes: int, keepalive=None):
        self.ptr = int(ptr)
        self.nbytes = int(nbytes)
        self.keepalive = keepalive
        self.host_writes = 0


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class QuarkTensor:
    __slots__ = ("_storage", "_offset", "shape", "dtype")

    def __init__(self, storage, shape, dtype: str, offset: int = 0):
        if dtype not in _ITEMSIZE:
            raise TypeError(f"QuarkTensor: unsupported dtype {dtype!r}")
        self._storage = storage
        self._offset = int(offset)
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype

    # ---- construction
    @staticmethod
    def empty(*shape, dtype: str = "bf16") -> "QuarkTensor":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return QuarkTensor(_Storage(_numel(shape) * _ITEMSIZE[dtype]), shape, dtype)

    @staticmethod
    def zeros(*shape, dtype: str = "bf16") -> "QuarkTensor":
        t = QuarkTensor.empty(*shape, dtype=dtype)
        t.zero_()
        return t

    @staticmethod
    def from_numpy(arr, dtype: str | None = None) -> "QuarkTensor":
        arr = np.asarray(arr)
        if dtype is None:
            dtype = _FROM_NP.get(arr.dtype)
            if dtype is None:
                raise ValueError(f"from_numpy: unsupported dtype {arr.dtype}")
        target = np.dtype(_CARRIER[dtype])
        if arr.dtype != target:
            if dtype == "bf16" and arr.dtype == np.float32:
                arr = (np.ascontiguousarray(arr).view(np.uint32) >> np.uint32(16)).astype(np.uint16)
            elif arr.dtype.itemsize == target.itemsize:
                arr = arr.view(target)
            else:
                arr = arr.astype(target)
        arr = np.ascontiguousarray(arr)
        t = QuarkTensor.empty(*arr.shape, dtype=dtype)
        t.copy_from_numpy(arr)
        return t

    @staticmethod
    def borrow(ptr: int, shape, dtype: str, keepalive=None) -> "QuarkTensor":
        return QuarkTensor(_Borrowed(ptr, _numel(shape) * _ITEMSIZE[dtype], keepalive), shape, dtype)

    # ---- introspection
    def data_ptr(self) -> int:
        return self._storage.ptr + self._offset

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        return _numel(self.shape)

    @property
    def nbytes(self) -> int:
        return self.numel * _ITEMSIZE[self.dtype]

    @property
    def quark_dtype(self) -> str:
        return self.dtype

    def __repr__(self) -> str:
        return f"QuarkTensor(shape={self.shape}, dtype={self.dtype!r}, ptr=0x{self.data_ptr():x})"

    # ---- views
    def reshape(self, *shape) -> "QuarkTensor":
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = list(shape)
        if -1 in shape:
            known = _numel([s for s in shape if s != -1])
            shape[shape.index(-1)] = self.numel // max(known, 1)
        if _numel(shape) != self.numel:
            raise ValueError(f"reshape: cannot view {self.shape} as {tuple(shape)}")
        return QuarkTensor(self._storage, shape, self.dtype, self._offset)

    def rows(self, start: int, stop: int) -> "QuarkTensor":
        """Contiguous view of rows ``[start, stop)`` of a rank-2 tensor."""
        if self.ndim != 2 or not (0 <= start <= stop <= self.shape[0]):
            raise ValueError(f"rows({start}, {stop}) on shape {self.shape}")
        pitch = self.shape[1] * _ITEMSIZE[self.dtype]
        return QuarkTensor(self._storage, (stop - start, self.shape[1]), self.dtype, self._offset + start * pitch)

    # ---- data movement (synchronous with respect to the host)
    def zero_(self) -> "QuarkTensor":
        self._storage.host_writes += 1
        _lib.check(_lib.load().qb_memset_async(C.c_void_p(self.data_ptr()), 0, self.nbytes, C.c_void_p(_stream.active_stream())))
        return self

    def copy_from_numpy(self, arr) -> "QuarkTensor":
        arr = np.ascontiguousarray(arr)
        if arr.nbytes != self.nbytes:
            raise ValueError(f"copy_from_numpy: {arr.nbytes} bytes into a tensor of {self.nbytes}")
        self._storage.host_writes += 1
        lib = _lib.load()
        s = C.c_void_p(_stream.active_stream())
        _lib.check(lib.qb_memcpy_async(C.c_void_p(self.data_ptr()), C.c_void_p(arr.ctypes.data), self.nbytes, 0, s))
        _lib.check(lib.qb_stream_sync(s))
        return self

    def copy_from(self, other: "QuarkTensor") -> "QuarkTensor":
        """Device-to-device copy on the active stream (asynchronous)."""
        if other.nbytes != self.nbytes:
            raise ValueError("copy_from: size mismatch")
        self._storage.host_writes += 1
        _lib.check(
            _lib.load().qb_memcpy_async(C.c_void_p(self.data_ptr()), C.c_void_p(other.data_ptr()), self.nbytes, 2, C.c_void_p(_stream.active_stream()))
        )
        return self

    def to_numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=_CARRIER[self.dtype])
        lib = _lib.load()
        s = C.c_void_p(_stream.active_stream())
        _lib.check(lib.qb_memcpy_async(C.c_void_p(out.ctypes.data), C.c_void_p(self.data_ptr()), self.nbytes, 1, s))
        _lib.check(lib.qb_stream_sync(s))
        return out

    def to_bytes(self) -> bytes:
        return self.to_numpy().tobytes()

    def to_f32_numpy(self) -> np.ndarray:
        """Host copy widened to f32 (bf16 by a 16-bit shift, e4m3 through the OCP table)."""
        a = self.to_numpy()
        if self.dtype == "bf16":
            return (a.astype(np.uint32) << np.uint32(16)).view(np.float32)
        if self.dtype == "e4m3":
            return _e4m3_table()[a]
        return a.astype(np.float32)


_E4M3 = None


def _e4m3_table() -> np.ndarray:
    global _E4M3
    if _E4M3 is None:
        b = np.arange(256)
        sign = np.where(b & 0x80, -1.0, 1.0)
        e = (b >> 3) & 0xF
        m = b & 7
        val = np.where(e == 0, (m / 8.0) * 2.0**-6, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7))
        val = np.where((e == 0xF) & (m == 7), np.nan, val)
        _E4M3 = (sign * val).astype(np.float32)
    return _E4M3
