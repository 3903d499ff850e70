"""Device context and device buffers.

``DBuf`` plays the role of the reference's ``_DBuf`` (ancora/model/resident.py:52-94),
``_Buf`` (ancora/optim/adamw.py:51-60) and ``_GpuArray`` (ancora/kernels/loss.py:277-294):
a persistent device allocation exposing ``__cuda_array_interface__`` v3, ``.ptr``,
cheap reshaped views (``view``), row-offset views (``at_pos``), ``to_numpy`` and ``free``.
A failed allocation raises (reference: resident.py:57-59); views must never be freed.
"""
import ctypes as C
import os

import numpy as np

from . import _lib as L

_contexts = {}
_default_device = None


def set_device(device):
    """Selects the GPU used by contexts created without an explicit device."""
    global _default_device
    _default_device = int(device)


def default_device():
    if _default_device is not None:
        return _default_device
    return int(os.environ.get("LOCAL_RANK", "0"))


class Context:
    """One (device, stream) pair plus the library's device workspace."""

    def __init__(self, device=None, stream=None):
        self.device = default_device() if device is None else int(device)
        h = C.c_void_p()
        L.check(L.lib().anc_ctx_create(self.device, C.c_void_p(stream or None), C.byref(h)))
        self.handle = h
        s = C.c_void_p()
        L.check(L.lib().anc_ctx_stream(self.handle, C.byref(s)))
        self.stream = s.value or 0

    def reserve_sms(self, n):
        """SMs the persistent Newton-Schulz kernel leaves free for other streams' kernels."""
        L.check(L.lib().anc_ctx_reserve_sms(self.handle, int(n)))

    def sync(self, stream=None):
        L.check(L.lib().anc_ctx_sync(self.handle, C.c_void_p(stream or None)))

    def status(self):
        code = C.c_uint32()
        L.check(L.lib().anc_ctx_status(self.handle, C.byref(code)))
        return code.value

    def check_status(self):
        code = self.status()
        if code:
            raise L.AncoraError(L.E_DEVICE, f"device status word 0x{code:x} "
                                "(1 TMA wait, 2 MMA wait, 4 epilogue wait ran out; 8 bad table index; "
                                "0x10 a tile's dependency never completed)")

    def flush_l2(self, stream=None):
        L.check(L.lib().anc_flush_l2(self.handle, C.c_void_p(stream or None)))

    def destroy(self):
        if self.handle:
            L.lib().anc_ctx_destroy(self.handle)
            self.handle = None


def get_context(device=None):
    """Process-wide context per device (the reference is one model per process)."""
    d = default_device() if device is None else int(device)
    if d not in _contexts:
        _contexts[d] = Context(d)
    return _contexts[d]


def dev_ptr(obj):
    """Device address of a DBuf, a reference-style buffer (``.ptr`` / ``._ptr``), any
    object with ``__cuda_array_interface__``, or a plain int."""
    if obj is None:
        return None
    if isinstance(obj, int):
        return obj
    for attr in ("ptr", "_ptr"):
        if hasattr(obj, attr):
            return int(getattr(obj, attr))
    cai = getattr(obj, "__cuda_array_interface__", None)
    if cai is not None:
        return int(cai["data"][0])
    raise TypeError(f"cannot take a device pointer from {type(obj).__name__}")


class DBuf:
    def __init__(self, arr, ctx=None):
        arr = np.ascontiguousarray(arr)
        self.ctx = ctx or get_context()
        self.shape, self.dtype, self.nbytes = arr.shape, arr.dtype, arr.nbytes
        p = C.c_void_p()
        L.check(L.lib().anc_malloc(self.ctx.handle, arr.nbytes, C.byref(p)))
        self.ptr = p.value
        self._owner = True
        if arr.nbytes:
            L.check(L.lib().anc_h2d(self.ctx.handle, self.ptr, arr.ctypes.data, arr.nbytes, None, 1))
        self._set_cai()

    def _set_cai(self):
        self.__cuda_array_interface__ = {"shape": tuple(self.shape), "typestr": np.dtype(self.dtype).str,
                                         "data": (int(self.ptr), False), "version": 3}

    @classmethod
    def empty(cls, shape, dtype=np.uint16, ctx=None):
        self = cls.__new__(cls)
        self.ctx = ctx or get_context()
        self.shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        p = C.c_void_p()
        L.check(L.lib().anc_malloc(self.ctx.handle, self.nbytes, C.byref(p)))
        self.ptr = p.value
        self._owner = True
        self._set_cai()
        return self

    @classmethod
    def zeros(cls, shape, dtype=np.uint16, ctx=None):
        self = cls.empty(shape, dtype, ctx)
        if self.nbytes:
            L.check(L.lib().anc_memset(self.ctx.handle, self.ptr, 0, self.nbytes, None))
            self.ctx.sync()
        return self

    def _alias(self, shape, ptr, nbytes, dtype=None):
        v = DBuf.__new__(DBuf)
        v.ctx, v.shape, v.dtype, v.nbytes, v.ptr = self.ctx, tuple(shape), np.dtype(dtype or self.dtype), nbytes, ptr
        v._owner = False
        v._set_cai()
        return v

    def view(self, shape, dtype=None):
        return self._alias(shape, self.ptr, self.nbytes, dtype)

    def at_pos(self, pos):
        """View offset by ``pos`` rows of width ``shape[-1]`` (resident.py:74-87)."""
        if pos == 0:
            return self
        off = pos * self.shape[-1] * np.dtype(self.dtype).itemsize
        return self._alias(self.shape, int(self.ptr) + off, self.nbytes - off)

    def slice_elems(self, start, count, shape=None):
        """View of ``count`` elements starting at flat element ``start``."""
        it = np.dtype(self.dtype).itemsize
        return self._alias(shape or (count,), int(self.ptr) + start * it, count * it)

    def upload(self, arr, stream=None, sync=True):
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes, "upload larger than the buffer"
        L.check(L.lib().anc_h2d(self.ctx.handle, self.ptr, arr.ctypes.data, arr.nbytes,
                                C.c_void_p(stream or None), 1 if sync else 0))

    def to_numpy(self, stream=None):
        out = np.empty(self.shape, self.dtype)
        if out.nbytes:
            L.check(L.lib().anc_d2h(self.ctx.handle, out.ctypes.data, self.ptr, out.nbytes,
                                    C.c_void_p(stream or None), 1))
        return out

    numpy = to_numpy

    def zero_(self, stream=None):
        L.check(L.lib().anc_memset(self.ctx.handle, self.ptr, 0, self.nbytes, C.c_void_p(stream or None)))

    def free(self):
        if not getattr(self, "_owner", False):
            raise RuntimeError("never free a view (only the owning DBuf)")
        if self.ptr:
            L.check(L.lib().anc_free(self.ctx.handle, self.ptr))
            self.ptr = 0


class PinnedArray:
    """Page-locked host memory viewed as a numpy array (staging for host<->device)."""

    def __init__(self, shape, dtype, device=None):
        """device: place the pages on the NUMA node next to that GPU."""
        self.shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        p = C.c_void_p()
        if device is None:
            L.check(L.lib().anc_host_alloc(max(self.nbytes, 1), C.byref(p)))
        else:
            L.check(L.lib().anc_host_alloc_near(int(device), max(self.nbytes, 1), C.byref(p)))
        self.ptr = p.value
        buf = (C.c_char * max(self.nbytes, 1)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype, count=int(np.prod(self.shape, dtype=np.int64))).reshape(self.shape)

    def free(self):
        if self.ptr:
            self.array = None
            L.lib().anc_host_free(self.ptr)
            self.ptr = 0


class Event:
    def __init__(self):
        h = C.c_void_p()
        L.check(L.lib().anc_event_create(C.byref(h)))
        self.handle = h

    def record(self, stream):
        L.check(L.lib().anc_event_record(self.handle, C.c_void_p(stream or None)))

    def sync(self):
        L.check(L.lib().anc_event_sync(self.handle))

    def elapsed_ms(self, later):
        ms = C.c_float()
        L.check(L.lib().anc_event_elapsed_ms(self.handle, later.handle, C.byref(ms)))
        return ms.value

    def destroy(self):
        if self.handle:
            L.lib().anc_event_destroy(self.handle)
            self.handle = None
