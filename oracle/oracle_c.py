"""ctypes binding of the C oracle (``oracle_c.c``): test infrastructure only.

``build()`` compiles ``liboracle_c.so`` next to the source with gcc; ``load()``
returns a thin wrapper whose methods take and return NumPy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle_c.so")
_SRC = os.path.join(_HERE, "oracle_c.c")

FMT_E4M3, FMT_E5M2 = 3, 4
_FMT = {"e4m3": FMT_E4M3, "e5m2": FMT_E5M2}


def build(force: bool = False) -> str:
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.check_call(
            ["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-shared",
             "-fPIC", "-o", _SO, _SRC])
    return _SO


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class OracleC:
    def __init__(self, path: str):
        self.lib = C.CDLL(path)
        L = self.lib
        L.orc_amax_f32.restype = C.c_float
        L.orc_amax_f32.argtypes = [C.c_void_p, C.c_size_t]
        L.orc_max_threads.restype = C.c_int
        for name in ("orc_f32_to_f16", "orc_f16_to_f32", "orc_f32_to_bf16", "orc_bf16_to_f32",
                     "orc_f64_to_f32", "orc_f32_to_f64"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
            getattr(L, name).restype = None
        L.orc_quantize_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_int]
        L.orc_quantize_fp8.restype = None
        L.orc_dequantize_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_int]
        L.orc_dequantize_fp8.restype = None
        L.orc_quantize_fp4_b32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
        L.orc_quantize_fp4_b32.restype = None
        L.orc_dequantize_fp4_b32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
        L.orc_dequantize_fp4_b32.restype = None
        L.orc_set_threads.argtypes = [C.c_int]

    def set_threads(self, n: int) -> None:
        self.lib.orc_set_threads(int(n))

    def max_threads(self) -> int:
        return int(self.lib.orc_max_threads())

    def _conv(self, fn, x, in_dt, out_dt, out=None):
        x = np.ascontiguousarray(x, in_dt)
        if out is None:
            out = np.empty(x.shape, out_dt)
        getattr(self.lib, fn)(_p(x), _p(out), x.size)
        return out

    def f32_to_f16_bits(self, x, out=None):
        return self._conv("orc_f32_to_f16", x, np.float32, np.uint16, out)

    def f16_bits_to_f32(self, h, out=None):
        return self._conv("orc_f16_to_f32", h, np.uint16, np.float32, out)

    def f32_to_bf16_bits(self, x, out=None):
        return self._conv("orc_f32_to_bf16", x, np.float32, np.uint16, out)

    def bf16_bits_to_f32(self, b, out=None):
        return self._conv("orc_bf16_to_f32", b, np.uint16, np.float32, out)

    def f64_to_f32(self, x, out=None):
        return self._conv("orc_f64_to_f32", x, np.float64, np.float32, out)

    def f32_to_f64(self, x, out=None):
        return self._conv("orc_f32_to_f64", x, np.float32, np.float64, out)

    def amax_f32(self, x) -> np.float32:
        x = np.ascontiguousarray(x, np.float32)
        return np.float32(self.lib.orc_amax_f32(_p(x), x.size))

    def quantize_fp8(self, x, inv_scale, fmt, out=None):
        x = np.ascontiguousarray(x, np.float32)
        if out is None:
            out = np.empty(x.shape, np.uint8)
        self.lib.orc_quantize_fp8(_p(x), _p(out), x.size, C.c_float(float(inv_scale)), _FMT[fmt])
        return out

    def dequantize_fp8(self, q, scale, fmt, out=None):
        q = np.ascontiguousarray(q, np.uint8)
        if out is None:
            out = np.empty(q.shape, np.float32)
        self.lib.orc_dequantize_fp8(_p(q), _p(out), q.size, C.c_float(float(scale)), _FMT[fmt])
        return out

    def quantize_fp4_b32(self, x_bf16_bits):
        x = np.ascontiguousarray(x_bf16_bits, np.uint16)
        rows, cols = x.shape
        assert cols % 32 == 0
        packed = np.empty((rows, cols // 2), np.uint8)
        scales = np.empty((rows, cols // 32), np.float32)
        self.lib.orc_quantize_fp4_b32(_p(x), _p(packed), _p(scales), rows, cols)
        return packed, scales

    def dequantize_fp4_b32(self, packed, scales):
        packed = np.ascontiguousarray(packed, np.uint8)
        scales = np.ascontiguousarray(scales, np.float32)
        rows, half = packed.shape
        out = np.empty((rows, half * 2), np.uint16)
        self.lib.orc_dequantize_fp4_b32(_p(packed), _p(scales), _p(out), rows, half * 2)
        return out


_inst = None


def load() -> OracleC:
    global _inst
    if _inst is None:
        _inst = OracleC(build())
    return _inst
