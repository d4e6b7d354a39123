"""Device memory, streams and events over the nvq C ABI (no PyTorch involved)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib


class Stream:
    """A CUDA stream created by the library (``ptr`` is the cudaStream_t)."""

    def __init__(self, device: int = 0):
        self.device = device
        p = C.c_void_p()
        check(lib().nvq_stream_create(device, C.byref(p)))
        self.ptr = p.value

    def sync(self) -> None:
        check(lib().nvq_stream_sync(self.device, self.ptr))

    def close(self) -> None:
        if self.ptr is not None:
            lib().nvq_stream_destroy(self.device, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _sptr(stream) -> C.c_void_p:
    if stream is None:
        return C.c_void_p(None)
    if isinstance(stream, Stream):
        return C.c_void_p(stream.ptr)
    return C.c_void_p(int(stream))


class Event:
    def __init__(self, device: int = 0):
        self.device = device
        p = C.c_void_p()
        check(lib().nvq_event_create(device, C.byref(p)))
        self.ptr = p.value

    def record(self, stream=None) -> None:
        check(lib().nvq_event_record(self.device, self.ptr, _sptr(stream)))

    def sync(self) -> None:
        check(lib().nvq_event_sync(self.device, self.ptr))

    def block(self, stream) -> None:
        """Work enqueued on ``stream`` from now on waits for what this event recorded."""
        check(lib().nvq_stream_wait_event(self.device, _sptr(stream), self.ptr))

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float()
        check(lib().nvq_event_elapsed_ms(self.ptr, later.ptr, C.byref(ms)))
        return float(ms.value)

    def __del__(self):
        try:
            if self.ptr is not None:
                lib().nvq_event_destroy(self.device, self.ptr)
                self.ptr = None
        except Exception:
            pass


def device_sync(device: int = 0) -> None:
    check(lib().nvq_device_sync(device))


def device_count() -> int:
    n = C.c_int()
    check(lib().nvq_device_count(C.byref(n)))
    return n.value


def device_info(device: int = 0) -> dict:
    sm, tot, ma, mi = C.c_int(), C.c_size_t(), C.c_int(), C.c_int()
    check(lib().nvq_device_info(device, C.byref(sm), C.byref(tot), C.byref(ma), C.byref(mi)))
    return dict(sm_count=sm.value, total_bytes=tot.value, cc=(ma.value, mi.value))


class DeviceBuffer:
    """An owned allocation in the HBM of one GPU: ``nbytes`` raw bytes at ``ptr``."""

    def __init__(self, nbytes: int, device: int = 0):
        self.device = device
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(lib().nvq_malloc(device, self.nbytes, C.byref(p)))
        self.ptr = p.value or 0

    @classmethod
    def from_numpy(cls, a: np.ndarray, device: int = 0, stream=None) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes, device)
        buf.upload(a, stream)
        return buf

    def upload(self, a: np.ndarray, stream=None, offset: int = 0) -> None:
        a = np.ascontiguousarray(a)
        if offset + a.nbytes > self.nbytes:
            raise ValueError("upload larger than the buffer")
        check(lib().nvq_memcpy_h2d(C.c_void_p(self.ptr + offset), a.ctypes.data_as(C.c_void_p),
                                   a.nbytes, self.device, _sptr(stream)))
        if stream is None:
            device_sync(self.device)

    def download(self, out: np.ndarray, stream=None, offset: int = 0) -> np.ndarray:
        if not out.flags.c_contiguous:
            raise ValueError("download target must be contiguous")
        if offset + out.nbytes > self.nbytes:
            raise ValueError("download larger than the buffer")
        check(lib().nvq_memcpy_d2h(out.ctypes.data_as(C.c_void_p), C.c_void_p(self.ptr + offset),
                                   out.nbytes, self.device, _sptr(stream)))
        if stream is None:
            device_sync(self.device)
        return out

    def to_numpy(self, dtype, shape) -> np.ndarray:
        return self.download(np.empty(shape, dtype))

    def zero(self, stream=None) -> None:
        check(lib().nvq_memset(C.c_void_p(self.ptr), 0, self.nbytes, self.device, _sptr(stream)))

    def at(self, offset: int) -> C.c_void_p:
        return C.c_void_p(self.ptr + offset)

    def free(self) -> None:
        if self.ptr:
            lib().nvq_free(self.device, C.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class _Pinned:
    def __init__(self, nbytes: int):
        p = C.c_void_p()
        check(lib().nvq_host_alloc(nbytes, C.byref(p)))
        self.ptr = p.value
        self.nbytes = nbytes

    def __del__(self):
        try:
            if self.ptr:
                lib().nvq_host_free(C.c_void_p(self.ptr))
                self.ptr = None
        except Exception:
            pass


def pinned_empty(shape, dtype) -> np.ndarray:
    """A NumPy array in page-locked host memory (full-rate, asynchronous PCIe copies)."""
    dtype = np.dtype(dtype)
    n = int(np.prod(shape)) if np.ndim(shape) else int(shape)
    nbytes = max(1, n * dtype.itemsize)
    owner = _Pinned(nbytes)
    raw = (C.c_char * nbytes).from_address(owner.ptr)
    raw._owner = owner  # the array's base keeps the allocation alive
    return np.frombuffer(raw, dtype=dtype, count=n).reshape(shape)
