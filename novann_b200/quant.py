"""Casts and quantisation: the host-facing calls and their device-resident forms.

The reference converts dtypes with ``ndarray.astype`` on host arrays
(``novann/layers/linear/linear.py:81``).  ``cast`` keeps that contract (NumPy array
in, NumPy array out) and runs the conversion on the GPU; the ``*_device`` functions
work on ``DeviceBuffer``s already resident in HBM and are asynchronous on a stream.

bf16 has no NumPy dtype: bf16 data is carried as ``np.uint16`` bit patterns and
named by the string ``"bf16"``.  FP8 / FP4 codes are ``np.uint8``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, lib
from .device import DeviceBuffer, _sptr

_NP_OF = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16, "f64": np.float64}


def _dtype_name(d) -> str:
    if isinstance(d, str):
        d = d.lower()
        alias = {"float32": "f32", "float16": "f16", "bfloat16": "bf16", "fp32": "f32",
                 "fp16": "f16", "float64": "f64", "fp64": "f64"}
        d = alias.get(d, d)
        if d in _lib.DTYPE_IDS:
            return d
        raise ValueError(f"unknown dtype '{d}'")
    d = np.dtype(d)
    if d == np.float32:
        return "f32"
    if d == np.float16:
        return "f16"
    if d == np.float64:
        return "f64"
    if d.name == "bfloat16":
        return "bf16"
    raise ValueError(f"unsupported dtype {d}")


def _fmt_id(fmt: str) -> int:
    fmt = fmt.lower()
    if fmt not in ("e4m3", "e5m2"):
        raise ValueError("fmt must be 'e4m3' or 'e5m2'")
    return _lib.DTYPE_IDS[fmt]


# ------------------------------------------------------------------ device-resident
def cast_device(dst: DeviceBuffer, dst_dtype: str, src: DeviceBuffer, src_dtype: str, n: int,
                stream=None, dst_offset: int = 0, src_offset: int = 0) -> None:
    check(lib().nvq_cast(dst.at(dst_offset), _lib.DTYPE_IDS[dst_dtype], src.at(src_offset),
                         _lib.DTYPE_IDS[src_dtype], n, src.device, _sptr(stream)))


def amax_device(src: DeviceBuffer, n: int, out: DeviceBuffer, stream=None, src_offset: int = 0,
                out_offset: int = 0) -> None:
    check(lib().nvq_amax_f32(src.at(src_offset), n, out.at(out_offset), src.device, _sptr(stream)))


def quantize_fp8_device(dst: DeviceBuffer, src: DeviceBuffer, n: int, fmt: str, inv_scale: float,
                        stream=None, dst_offset: int = 0, src_offset: int = 0) -> None:
    check(lib().nvq_quantize_fp8(dst.at(dst_offset), src.at(src_offset), n, _fmt_id(fmt),
                                 C.c_float(float(inv_scale)), src.device, _sptr(stream)))


def dequantize_fp8_device(dst: DeviceBuffer, src: DeviceBuffer, n: int, fmt: str, scale: float,
                          stream=None, dst_offset: int = 0, src_offset: int = 0) -> None:
    check(lib().nvq_dequantize_fp8(dst.at(dst_offset), src.at(src_offset), n, _fmt_id(fmt),
                                   C.c_float(float(scale)), src.device, _sptr(stream)))


def quantize_fp8_tensor_device(dst: DeviceBuffer, asi: DeviceBuffer, src: DeviceBuffer, n: int,
                               fmt: str, amax_in: DeviceBuffer | None = None, stream=None) -> None:
    """amax -> scales -> codes on the device.  ``asi`` receives {amax, scale, inv_scale}."""
    check(lib().nvq_quantize_fp8_tensor(dst.at(0), asi.at(0), src.at(0), n, _fmt_id(fmt),
                                        amax_in.at(0) if amax_in is not None else None,
                                        src.device, _sptr(stream)))


def quantize_fp4_b32_device(packed: DeviceBuffer, scales: DeviceBuffer, src: DeviceBuffer,
                            rows: int, cols: int, stream=None) -> None:
    check(lib().nvq_quantize_fp4_b32(packed.at(0), scales.at(0), src.at(0), rows, cols,
                                     src.device, _sptr(stream)))


def dequantize_fp4_b32_device(dst: DeviceBuffer, packed: DeviceBuffer, scales: DeviceBuffer,
                              rows: int, cols: int, stream=None) -> None:
    check(lib().nvq_dequantize_fp4_b32(dst.at(0), packed.at(0), scales.at(0), rows, cols,
                                       dst.device, _sptr(stream)))


# ------------------------------------------------------------------ host arrays
def cast(x: np.ndarray, dtype, *, src_dtype=None, device: int = 0, out: np.ndarray | None = None
         ) -> np.ndarray:
    """GPU replacement for ``x.astype(dtype)`` between fp32 and fp16 / bf16 / fp64.

    ``x`` float32 -> ``dtype`` in {float16, "bf16", float64}; or ``x`` float16 / float64 /
    bf16-bits (``src_dtype="bf16"``, uint16 array) -> float32.  float64 -> float32 is the
    conversion the reference's layers perform on BatchNorm's float64 output
    (``novann/layers/linear/linear.py:81``).  Like ``astype(np.float32, copy=False)``, a
    request for the dtype ``x`` already has returns ``x`` itself.  Host arrays in pinned
    memory (``pinned_empty``) move at full PCIe rate.
    """
    dst = _dtype_name(dtype)
    if src_dtype is None:
        if x.dtype == np.uint16:
            raise ValueError("uint16 input: pass src_dtype='bf16'")
        src = _dtype_name(x.dtype)
    else:
        src = _dtype_name(src_dtype)
    if src == dst:
        return x
    if x.dtype != _NP_OF[src]:
        raise ValueError(f"array dtype {x.dtype} does not hold {src} data")
    x = np.ascontiguousarray(x)
    if out is None:
        out = np.empty(x.shape, _NP_OF[dst])
    elif out.dtype != _NP_OF[dst] or out.size != x.size or not out.flags.c_contiguous:
        raise ValueError("out has the wrong dtype, size or layout")
    check(lib().nvq_cast_host(out.ctypes.data_as(C.c_void_p), _lib.DTYPE_IDS[dst],
                              x.ctypes.data_as(C.c_void_p), _lib.DTYPE_IDS[src], x.size, device))
    return out


def amax(x: np.ndarray, device: int = 0) -> np.float32:
    d = DeviceBuffer.from_numpy(np.ascontiguousarray(x, np.float32), device)
    o = DeviceBuffer(4, device)
    amax_device(d, x.size, o)
    return o.to_numpy(np.float32, (1,))[0]


def fp8_scales(amax_value, fmt: str):
    """(scale, inv_scale) from an amax by the written rule: one fp32 division each,
    both 1 when amax is 0.  Host arithmetic on one scalar."""
    fmax = np.float32(448.0 if fmt.lower() == "e4m3" else 57344.0)
    a = np.float32(amax_value)
    if a == 0:
        return np.float32(1.0), np.float32(1.0)
    return np.float32(a / fmax), np.float32(fmax / a)


def quantize_fp8(x: np.ndarray, fmt: str = "e4m3", device: int = 0):
    """Per-tensor FP8 quantisation of a host fp32 array.  Returns (codes uint8 with
    x's shape, scale, inv_scale)."""
    x = np.ascontiguousarray(x, np.float32)
    d = DeviceBuffer.from_numpy(x, device)
    q = DeviceBuffer(max(1, x.size), device)
    asi = DeviceBuffer(12, device)
    quantize_fp8_tensor_device(q, asi, d, x.size, fmt)
    codes = q.to_numpy(np.uint8, x.shape) if x.size else np.empty(x.shape, np.uint8)
    a = asi.to_numpy(np.float32, (3,))
    return codes, a[1], a[2]


def dequantize_fp8(q: np.ndarray, scale, fmt: str = "e4m3", device: int = 0) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8)
    out = np.empty(q.shape, np.float32)
    if q.size == 0:
        return out
    d = DeviceBuffer.from_numpy(q, device)
    o = DeviceBuffer(q.size * 4, device)
    dequantize_fp8_device(o, d, q.size, fmt, scale)
    return o.download(out)


def quantize_fp4_b32(x_bf16_bits: np.ndarray, device: int = 0):
    """bf16 bits (rows, cols) -> (packed uint8 (rows, cols/2), scales f32 (rows, cols/32))."""
    x = np.ascontiguousarray(x_bf16_bits, np.uint16)
    rows, cols = x.shape
    packed = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 32), np.float32)
    if cols % 32:
        check(lib().nvq_quantize_fp4_b32(None, None, None, rows, cols, device, None))
    if x.size == 0:
        return packed, scales
    d = DeviceBuffer.from_numpy(x, device)
    p = DeviceBuffer(packed.nbytes, device)
    s = DeviceBuffer(scales.nbytes, device)
    quantize_fp4_b32_device(p, s, d, rows, cols)
    return p.download(packed), s.download(scales)


def dequantize_fp4_b32(packed: np.ndarray, scales: np.ndarray, device: int = 0) -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales, np.float32)
    rows, half = packed.shape
    out = np.empty((rows, half * 2), np.uint16)
    if out.size == 0:
        return out
    p = DeviceBuffer.from_numpy(packed, device)
    s = DeviceBuffer.from_numpy(scales, device)
    o = DeviceBuffer(out.nbytes, device)
    dequantize_fp4_b32_device(o, p, s, rows, half * 2)
    return o.download(out)


def quantize_weight(w: np.ndarray, fmt: str = "e4m3", device: int = 0):
    """Weight preparation for the quantised layers.

    FP8 (``"e4m3"`` / ``"e5m2"``): per-output-channel scales; returns (codes uint8 (N, K),
    scales float32 (N,)).  FP4 (``"e2m1_b32"``): the weight is rounded to bf16 and quantised
    in blocks of 32 along K; returns (packed uint8 (N, K/2), scales float32 (N, K/32))."""
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    if fmt == "e2m1_b32":
        return quantize_fp4_b32(cast(w, "bf16", device=device), device)
    d = DeviceBuffer.from_numpy(w, device)
    q = DeviceBuffer(max(1, w.size), device)
    s = DeviceBuffer(max(4, n * 4), device)
    check(lib().nvq_quantize_fp8_rows(q.at(0), s.at(0), d.at(0), n, k, _fmt_id(fmt), device, None))
    return q.to_numpy(np.uint8, (n, k)), s.to_numpy(np.float32, (n,))
