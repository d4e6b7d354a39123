"""Functional ops over the nvq C ABI, mirroring ``novann/functional.py`` for the hot path.

``linear_q*`` is ``F.linear`` (novann/functional.py:147-163) for a weight held as FP8 /
FP4 codes; the device form works on buffers resident in HBM, the host form takes and
returns NumPy arrays (bf16 as uint16 bit patterns).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check, lib
from .device import DeviceBuffer, _sptr, device_sync


def linear_workspace_bytes(n: int, k: int, fmt: str) -> int:
    out = C.c_size_t()
    check(lib().nvq_linear_workspace_bytes(n, k, _lib.DTYPE_IDS[fmt], C.byref(out)))
    return out.value


def check_device_errors(device: int = 0) -> None:
    """Raises if a tensor-core kernel recorded a bounded-wait give-up since the last call."""
    flag = C.c_int()
    check(lib().nvq_device_error_flag(device, C.byref(flag)))
    if flag.value:
        raise _lib.NvqError(_lib.ERR_TIMEOUT, f"device-side wait gave up (code {flag.value})")


def linear_q_device(y: DeviceBuffer, x: DeviceBuffer, wq: DeviceBuffer, fmt: str,
                    w_scales: DeviceBuffer, bias: DeviceBuffer | None, m: int, n: int, k: int,
                    workspace: DeviceBuffer | None, stream=None) -> None:
    """``workspace=None`` selects the in-kernel expansion of FP8 codes (M > 128, K % 16 == 0)."""
    check(lib().nvq_linear_fwd(y.at(0), x.at(0), wq.at(0), _lib.DTYPE_IDS[fmt], w_scales.at(0),
                               bias.at(0) if bias is not None else None, m, n, k,
                               workspace.at(0) if workspace is not None else None,
                               workspace.nbytes if workspace is not None else 0,
                               x.device, _sptr(stream)))


def linear_q_host(x_bf16_bits: np.ndarray, wq: np.ndarray, w_scales: np.ndarray,
                  bias: np.ndarray | None, fmt: str = "e4m3", device: int = 0,
                  use_workspace: bool = True) -> np.ndarray:
    """Host arrays in, bf16 bits (M, N) out."""
    x = np.ascontiguousarray(x_bf16_bits, np.uint16)
    m, k = x.shape
    n = wq.shape[0]
    dx = DeviceBuffer.from_numpy(x, device)
    dw = DeviceBuffer.from_numpy(np.ascontiguousarray(wq, np.uint8), device)
    ds = DeviceBuffer.from_numpy(np.ascontiguousarray(w_scales, np.float32), device)
    db = DeviceBuffer.from_numpy(np.ascontiguousarray(bias, np.float32), device) if bias is not None else None
    dy = DeviceBuffer(m * n * 2, device)
    ws = DeviceBuffer(linear_workspace_bytes(n, k, fmt), device) if use_workspace else None
    linear_q_device(dy, dx, dw, fmt, ds, db, m, n, k, ws)
    device_sync(device)
    check_device_errors(device)
    return dy.to_numpy(np.uint16, (m, n))
