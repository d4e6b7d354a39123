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


_LINEAR_PATHS = {None: _lib.LINEAR_AUTO, "auto": _lib.LINEAR_AUTO,
                 "bf16_activations": _lib.LINEAR_BF16_ACTIVATIONS,
                 "expand_in_kernel": _lib.LINEAR_EXPAND_IN_KERNEL,
                 "single_cta": _lib.LINEAR_SINGLE_CTA, "cta_pair": _lib.LINEAR_CTA_PAIR,
                 "cluster_reduce": _lib.LINEAR_CLUSTER_REDUCE}
_CONV_PATHS = {None: _lib.CONV_AUTO, "auto": _lib.CONV_AUTO, "patch_matrix": _lib.CONV_PATCH_MATRIX,
               "cta_pair": _lib.CONV_CTA_PAIR}


def linear_q_device(y: DeviceBuffer, x: DeviceBuffer, wq: DeviceBuffer, fmt: str,
                    w_scales: DeviceBuffer, bias: DeviceBuffer | None, m: int, n: int, k: int,
                    workspace: DeviceBuffer | None, stream=None, path: str | None = None,
                    codes_finite: bool = False) -> None:
    """``workspace=None`` selects the in-kernel expansion of FP8 codes (M > 128, K % 16 == 0).
    ``path`` names a kernel path of ``nvq_linear_fwd_opts``: ``"bf16_activations"`` (M <= 128:
    activations taken as bf16, no two-piece E4M3 carrier), ``"cluster_reduce"`` (M <= 32: the
    clustered stream that adds its partial sums through distributed shared memory), ``"expand_in_kernel"``,
    ``"single_cta"``, ``"cta_pair"``; ``None`` lets the library choose.  ``codes_finite``: the
    caller vouches that no weight code is NaN / inf, which the in-kernel expansion then does not test."""
    flags = _LINEAR_PATHS[path] | (_lib.LINEAR_CODES_FINITE if codes_finite else 0)
    check(lib().nvq_linear_fwd_opts(y.at(0), x.at(0), wq.at(0), _lib.DTYPE_IDS[fmt], w_scales.at(0),
                                    bias.at(0) if bias is not None else None, m, n, k,
                                    workspace.at(0) if workspace is not None else None,
                                    workspace.nbytes if workspace is not None else 0,
                                    flags, x.device, _sptr(stream)))


def linear_q_host(x_bf16_bits: np.ndarray, wq: np.ndarray, w_scales: np.ndarray,
                  bias: np.ndarray | None, fmt: str = "e4m3", device: int = 0,
                  use_workspace: bool = True, path: str | None = None) -> np.ndarray:
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
    linear_q_device(dy, dx, dw, fmt, ds, db, m, n, k, ws, path=path)
    device_sync(device)
    check_device_errors(device)
    return dy.to_numpy(np.uint16, (m, n))


# ------------------------------------------------------------------ the reference's signatures
_default_device = 0


def set_default_device(device: int) -> None:
    """GPU used by ``linear`` / ``conv2d`` below when no ``device=`` is given."""
    global _default_device
    _default_device = int(device)


def _data(p):
    """``Parameters`` (anything with ``.data``) or a bare array."""
    return p.data if hasattr(p, "data") else p


def linear(input: np.ndarray, weight, bias=None, *, device: int | None = None) -> np.ndarray:
    """``F.linear(input, weight, bias)`` with the reference's signature
    (novann/functional.py:147-163): ``weight`` / ``bias`` are ``Parameters`` (their ``.data`` is
    read; bare arrays are taken too), result ``input @ weight.data.T + bias.data`` as float32,
    computed on the GPU."""
    dev = _default_device if device is None else device
    return linear_f32_host(input, _data(weight), None if bias is None else _data(bias), dev)


def conv2d(input: np.ndarray, weight, kernel_size, stride=1, padding=0, *, bias=None,
           padding_mode: str = "zeros", extras: bool = False, device: int | None = None):
    """``F.conv2d`` with the reference's signature (novann/functional.py:275-385):
    ``kernel_size`` / ``stride`` / ``padding`` ints or pairs (``"valid"`` = 0, ``"same"``
    refused), ``padding_mode`` one of zeros / reflect / replicate / circular.  Returns ``out``
    (N, Cout, OH, OW) float32, or ``(out, col, w_col)`` with ``extras`` - ``col`` the im2col
    matrix (C*KH*KW, N*OH*OW) built on the GPU, ``w_col`` the weight viewed (Cout, C*KH*KW)."""
    from .layers import _pair
    dev = _default_device if device is None else device
    kh, kw = _pair(kernel_size)
    w = _data(weight)
    if tuple(w.shape[2:]) != (kh, kw):
        raise ValueError(f"kernel_size {(kh, kw)} does not match the weight's {tuple(w.shape[2:])}")
    res = conv2d_f32_host(input, w, None if bias is None else _data(bias), _pair(stride), _pair(padding),
                          padding_mode, dev, return_col=extras)
    if extras:
        out, col = res
        return out, col, np.asarray(w).reshape(w.shape[0], -1)
    return res


# ------------------------------------------------------------------ fp32 layers (host arrays)
def _f32(a, device: int = 0):
    """Contiguous float32 view of a host array.  float32 passes through; float64 / float16
    arrays (a reference BatchNorm hands float64 to its neighbours) are converted by the GPU
    cast, as the layers' ``astype(np.float32, copy=False)`` would on the CPU."""
    a = np.asarray(a)
    if a.dtype == np.float32:
        return np.ascontiguousarray(a)
    if a.dtype in (np.float64, np.float16) and a.size:
        from . import quant
        return quant.cast(a, np.float32, device=device)
    return np.ascontiguousarray(a, np.float32)


def linear_f32_host(x, w, b=None, device: int = 0, relu: bool = False):
    """``F.linear`` (novann/functional.py:147-163) in fp32 on the GPU.  With ``relu`` the
    fused ``F.relu`` is applied and (out, mask) is returned."""
    x, w = _f32(x, device), _f32(w, device)
    m, k = x.shape
    n = w.shape[0]
    dx, dw = DeviceBuffer.from_numpy(x, device), DeviceBuffer.from_numpy(w, device)
    db = DeviceBuffer.from_numpy(_f32(b, device).reshape(-1), device) if b is not None else None
    dy = DeviceBuffer(max(4, m * n * 4), device)
    dm = DeviceBuffer(max(4, m * n * 4), device) if relu else None
    check(lib().nvq_linear_fwd_f32(dy.at(0), dx.at(0), dw.at(0), db.at(0) if db else None, m, n, k,
                                   int(relu), dm.at(0) if dm else None, device, None))
    y = dy.to_numpy(np.float32, (m, n))
    return (y, dm.to_numpy(np.float32, (m, n))) if relu else y


def linear_bwd_f32_host(grad, x, w, with_bias: bool = True, device: int = 0, mask=None):
    """``Linear.backward`` (novann/layers/linear/linear.py:85-108): returns (dW (N,K),
    db (1,N) or None, dX (M,K)); ``mask`` (M,K) multiplies dX (``ReLU.backward``)."""
    grad, x, w = _f32(grad, device), _f32(x, device), _f32(w, device)
    m, n = grad.shape
    k = x.shape[1]
    dg, dx, dw = (DeviceBuffer.from_numpy(a, device) for a in (grad, x, w))
    o_dw, o_db, o_dx = DeviceBuffer(n * k * 4, device), DeviceBuffer(n * 4, device), DeviceBuffer(m * k * 4, device)
    dmask = DeviceBuffer.from_numpy(_f32(mask, device), device) if mask is not None else None
    check(lib().nvq_linear_bwd_f32(o_dw.at(0), o_db.at(0) if with_bias else None, o_dx.at(0), dg.at(0),
                                   dx.at(0), dw.at(0), dmask.at(0) if dmask else None, m, n, k,
                                   device, None))
    return (o_dw.to_numpy(np.float32, (n, k)),
            o_db.to_numpy(np.float32, (1, n)) if with_bias else None,
            o_dx.to_numpy(np.float32, (m, k)))


def relu_host(x, device: int = 0):
    """``F.relu(x, extras=True)`` (novann/functional.py:8-22): returns (out, mask)."""
    x = _f32(x, device)
    d = DeviceBuffer.from_numpy(x, device)
    o, mk = DeviceBuffer(max(4, x.nbytes), device), DeviceBuffer(max(4, x.nbytes), device)
    check(lib().nvq_relu_fwd_f32(o.at(0), mk.at(0), d.at(0), x.size, device, None))
    return o.to_numpy(np.float32, x.shape), mk.to_numpy(np.float32, x.shape)


def softmax_ce_host(logits, labels, device: int = 0):
    """``CrossEntropyLoss.__call__`` (novann/losses/loss_functions.py:69-75): (loss, grad)."""
    z = _f32(logits, device)
    m, c = z.shape
    lab = np.ascontiguousarray(labels, np.int32)
    dz, dl = DeviceBuffer.from_numpy(z, device), DeviceBuffer.from_numpy(lab, device)
    g, yh, ls = DeviceBuffer(z.nbytes, device), DeviceBuffer(z.nbytes, device), DeviceBuffer(4, device)
    check(lib().nvq_softmax_ce_f32(g.at(0), ls.at(0), dz.at(0), dl.at(0), yh.at(0), m, c, device, None))
    return ls.to_numpy(np.float32, (1,))[0], g.to_numpy(np.float32, (m, c))


def conv2d_out_size(h, w, kh, kw, sh, sw, ph, pw):
    oh, ow = C.c_int(), C.c_int()
    check(lib().nvq_conv2d_out_size(h, w, kh, kw, sh, sw, ph, pw, C.byref(oh), C.byref(ow)))
    return oh.value, ow.value


def _pad_mode(name: str) -> int:
    if name not in _lib.PAD_MODES:
        raise ValueError(f"padding_mode Only accept {tuple(_lib.PAD_MODES)} not '{name}'")
    return _lib.PAD_MODES[name]


def conv2d_f32_host(x, w, b=None, stride=(1, 1), padding=(0, 0), padding_mode: str = "zeros",
                    device: int = 0, return_col: bool = False):
    """``F.conv2d`` (novann/functional.py:275-385) in fp32 on the GPU: (N,Cout,OH,OW), and with
    ``return_col`` also the im2col matrix (C*KH*KW, N*OH*OW) the reference caches."""
    x, w = _f32(x, device), _f32(w, device)
    n, c, h, wd = x.shape
    cout, _, kh, kw = w.shape
    mode = _pad_mode(padding_mode)
    oh, ow = conv2d_out_size(h, wd, kh, kw, stride[0], stride[1], padding[0], padding[1])
    dx, dw = DeviceBuffer.from_numpy(x, device), DeviceBuffer.from_numpy(w, device)
    db = DeviceBuffer.from_numpy(_f32(b, device).reshape(-1), device) if b is not None else None
    col = DeviceBuffer(max(4, c * kh * kw * n * oh * ow * 4), device)
    out = DeviceBuffer(max(4, n * cout * oh * ow * 4), device)
    check(lib().nvq_conv2d_fwd_f32(out.at(0), dx.at(0), dw.at(0), db.at(0) if db else None, col.at(0),
                                   n, c, h, wd, cout, kh, kw, stride[0], stride[1], padding[0],
                                   padding[1], mode, device, None))
    y = out.to_numpy(np.float32, (n, cout, oh, ow))
    if return_col:
        return y, col.to_numpy(np.float32, (c * kh * kw, n * oh * ow))
    return y


def conv2d_q_host(x, wq, w_scales, b, kernel, stride=(1, 1), padding=(0, 0),
                  padding_mode: str = "zeros", fmt: str = "e4m3", device: int = 0,
                  path: str | None = None):
    """Quantised-weight ``F.conv2d``: ``wq`` is (Cout, kpad) FP8 codes of the zero-padded
    ``w.reshape(Cout, C*KH*KW)`` with ``w_scales`` (Cout,), or for ``fmt="e2m1_b32"`` the packed
    (Cout, kpad/2) FP4 codes with block scales (Cout, kpad/32), kpad a multiple of 32.  Returns
    fp32 (N,Cout,OH,OW)."""
    x = _f32(x, device)
    n, c, h, wd = x.shape
    kh, kw = kernel
    cout = wq.shape[0]
    mode = _pad_mode(padding_mode)
    rows, kpad = C.c_size_t(), C.c_size_t()
    check(lib().nvq_conv2d_q_sizes(n, c, h, wd, cout, kh, kw, stride[0], stride[1], padding[0], padding[1],
                                   C.byref(rows), C.byref(kpad)))
    if fmt == "e2m1_b32":
        kpad = C.c_size_t((c * kh * kw + 31) // 32 * 32)       # FP4 blocks are 32 columns
        if wq.shape[1] * 2 != kpad.value:
            raise ValueError(f"packed FP4 weight must be (Cout, {kpad.value // 2})")
    elif wq.shape[1] != kpad.value:
        raise ValueError(f"weight codes must be (Cout, {kpad.value})")
    oh, ow = conv2d_out_size(h, wd, kh, kw, stride[0], stride[1], padding[0], padding[1])
    dx = DeviceBuffer.from_numpy(x, device)
    dq = DeviceBuffer.from_numpy(np.ascontiguousarray(wq, np.uint8), device)
    ds = DeviceBuffer.from_numpy(_f32(w_scales, device), device)
    db = DeviceBuffer.from_numpy(_f32(b, device).reshape(-1), device) if b is not None else None
    col = DeviceBuffer(rows.value * kpad.value * 2, device)
    yb = DeviceBuffer(rows.value * cout * 2, device)
    ws = DeviceBuffer(linear_workspace_bytes(cout, kpad.value, fmt), device)
    out = DeviceBuffer(n * cout * oh * ow * 4, device)
    check(lib().nvq_conv2d_fwd_q_opts(out.at(0), dx.at(0), dq.at(0), _lib.DTYPE_IDS[fmt], ds.at(0),
                                      db.at(0) if db else None, col.at(0), yb.at(0), ws.at(0), ws.nbytes,
                                      n, c, h, wd, cout, kh, kw, stride[0], stride[1], padding[0],
                                      padding[1], mode, _CONV_PATHS[path], device, None))
    device_sync(device)
    check_device_errors(device)
    return out.to_numpy(np.float32, (n, cout, oh, ow))


def conv2d_q_nhwc_device(out: DeviceBuffer, x: DeviceBuffer, wq: DeviceBuffer, fmt: str,
                         w_scales: DeviceBuffer, bias: DeviceBuffer | None, workspace: DeviceBuffer,
                         n: int, c: int, h: int, w: int, cout: int, kernel, stride=(1, 1), padding=(0, 0),
                         relu: bool = False, stream=None) -> None:
    """Quantised convolution with bf16 NHWC activations in and out (``nvq_conv2d_fwd_q_nhwc``):
    the form chained quantised layers use, nothing is converted or re-laid-out per call."""
    check(lib().nvq_conv2d_fwd_q_nhwc(out.at(0), x.at(0), wq.at(0), _lib.DTYPE_IDS[fmt], w_scales.at(0),
                                      bias.at(0) if bias is not None else None, workspace.at(0),
                                      workspace.nbytes, n, c, h, w, cout, kernel[0], kernel[1], stride[0],
                                      stride[1], padding[0], padding[1], int(relu), x.device, _sptr(stream)))


def nchw_f32_to_nhwc_bf16_device(dst: DeviceBuffer, src: DeviceBuffer, n: int, c: int, s: int, stream=None) -> None:
    check(lib().nvq_nchw_f32_to_nhwc_bf16(dst.at(0), src.at(0), n, c, s, src.device, _sptr(stream)))


def nhwc_bf16_to_nchw_f32_device(dst: DeviceBuffer, src: DeviceBuffer, n: int, c: int, s: int, stream=None) -> None:
    check(lib().nvq_nhwc_bf16_to_nchw_f32(dst.at(0), src.at(0), n, c, s, src.device, _sptr(stream)))


def conv2d_bwd_f32_host(grad, col, w, x_shape, stride, padding, with_bias: bool = True, device: int = 0):
    """``Conv2d.backward`` (novann/layers/convolutional/conv2d.py:179-207): returns
    (dW (Cout,C,KH,KW), db (Cout,1) or None, dX (N,C,H,W))."""
    grad, col, w = _f32(grad, device), _f32(col, device), _f32(w, device)
    n, c, h, wd = x_shape
    cout, _, kh, kw = w.shape
    oh, ow = grad.shape[2], grad.shape[3]
    L, ckk = n * oh * ow, c * kh * kw
    dg, dc, dw_ = (DeviceBuffer.from_numpy(a, device) for a in (grad, col, w))
    o_dw, o_db, o_dx = DeviceBuffer(cout * ckk * 4, device), DeviceBuffer(cout * 4, device), DeviceBuffer(n * c * h * wd * 4, device)
    gr, dcol = DeviceBuffer(cout * L * 4, device), DeviceBuffer(ckk * L * 4, device)
    check(lib().nvq_conv2d_bwd_f32(o_dw.at(0), o_db.at(0) if with_bias else None, o_dx.at(0), dg.at(0),
                                   dc.at(0), dw_.at(0), gr.at(0), dcol.at(0), n, c, h, wd, cout, kh, kw,
                                   stride[0], stride[1], padding[0], padding[1], device, None))
    return (o_dw.to_numpy(np.float32, w.shape),
            o_db.to_numpy(np.float32, (cout, 1)) if with_bias else None,
            o_dx.to_numpy(np.float32, (n, c, h, wd)))


def im2col_f32_host(x, kernel, stride, padding, padding_mode: str = "zeros", device: int = 0):
    """``_im2col`` (novann/functional.py:346-368): (C*KH*KW, N*OH*OW) fp32."""
    x = _f32(x, device)
    n, c, h, wd = x.shape
    kh, kw = kernel
    oh, ow = conv2d_out_size(h, wd, kh, kw, stride[0], stride[1], padding[0], padding[1])
    dx = DeviceBuffer.from_numpy(x, device)
    col = DeviceBuffer(max(4, c * kh * kw * n * oh * ow * 4), device)
    check(lib().nvq_im2col_f32(col.at(0), dx.at(0), n, c, h, wd, kh, kw, stride[0], stride[1],
                               padding[0], padding[1], _pad_mode(padding_mode), device, None))
    return col.to_numpy(np.float32, (c * kh * kw, n * oh * ow))


def linear_q_bwd_host(grad, x, wq, w_scales, fmt: str = "e4m3", with_bias: bool = True, device: int = 0):
    """Backward of the quantised Linear on the tensor cores: returns (dW (N,K) fp32, db (1,N) or
    None, dX (M,K) fp32) from the output gradient, the forward input and the weight codes."""
    grad, x = _f32(grad, device), _f32(x, device)
    m, n = grad.shape
    k = x.shape[1]
    need = C.c_size_t()
    check(lib().nvq_linear_bwd_q_workspace_bytes(m, n, k, C.byref(need)))
    dg, dx_in = DeviceBuffer.from_numpy(grad, device), DeviceBuffer.from_numpy(x, device)
    dq = DeviceBuffer.from_numpy(np.ascontiguousarray(wq, np.uint8), device)
    ds = DeviceBuffer.from_numpy(_f32(w_scales, device), device)
    o_dx, o_dw, o_db = DeviceBuffer(m * k * 4, device), DeviceBuffer(n * k * 4, device), DeviceBuffer(n * 4, device)
    ws = DeviceBuffer(need.value, device)
    check(lib().nvq_linear_bwd_q(o_dx.at(0), o_dw.at(0), o_db.at(0) if with_bias else None, dg.at(0),
                                 dx_in.at(0), dq.at(0), _lib.DTYPE_IDS[fmt], ds.at(0), m, n, k,
                                 ws.at(0), ws.nbytes, device, None))
    device_sync(device)
    check_device_errors(device)
    return (o_dw.to_numpy(np.float32, (n, k)),
            o_db.to_numpy(np.float32, (1, n)) if with_bias else None,
            o_dx.to_numpy(np.float32, (m, k)))


def linear_w8a8_device(y: DeviceBuffer, x: DeviceBuffer, wq: DeviceBuffer, w_scales: DeviceBuffer,
                       bias: DeviceBuffer | None, m: int, n: int, k: int, workspace: DeviceBuffer,
                       stream=None) -> None:
    """W8A8 variant: activations quantised to E4M3 per row inside the call, FP8 x FP8 MMAs."""
    check(lib().nvq_linear_fwd_w8a8(y.at(0), x.at(0), wq.at(0), w_scales.at(0),
                                    bias.at(0) if bias is not None else None, m, n, k,
                                    workspace.at(0), workspace.nbytes, x.device, _sptr(stream)))


def linear_w8a8_workspace_bytes(m: int, k: int) -> int:
    out = C.c_size_t()
    check(lib().nvq_linear_w8a8_workspace_bytes(m, k, C.byref(out)))
    return out.value


def linear_w8a8_host(x_bf16_bits, wq, w_scales, bias, device: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x_bf16_bits, np.uint16)
    m, k = x.shape
    n = wq.shape[0]
    dx = DeviceBuffer.from_numpy(x, device)
    dw = DeviceBuffer.from_numpy(np.ascontiguousarray(wq, np.uint8), device)
    ds = DeviceBuffer.from_numpy(_f32(w_scales, device), device)
    db = DeviceBuffer.from_numpy(_f32(bias, device), device) if bias is not None else None
    dy = DeviceBuffer(m * n * 2, device)
    ws = DeviceBuffer(linear_w8a8_workspace_bytes(m, k), device)
    linear_w8a8_device(dy, dx, dw, ds, db, m, n, k, ws)
    device_sync(device)
    check_device_errors(device)
    return dy.to_numpy(np.uint16, (m, n))


def linear_expand_weight_device(wd: DeviceBuffer, wq: DeviceBuffer, fmt: str, w_scales: DeviceBuffer | None,
                                n: int, k: int, stream=None) -> None:
    check(lib().nvq_linear_expand_weight(wd.at(0), wq.at(0), _lib.DTYPE_IDS[fmt],
                                         w_scales.at(0) if w_scales is not None else None, n, k,
                                         wq.device, _sptr(stream)))


def linear_expanded_device(y: DeviceBuffer, x: DeviceBuffer, wd: DeviceBuffer,
                           chan_scales: DeviceBuffer | None, bias: DeviceBuffer | None, m: int, n: int,
                           k: int, stream=None, relu: bool = False) -> None:
    check(lib().nvq_linear_fwd_expanded(y.at(0), x.at(0), wd.at(0),
                                        chan_scales.at(0) if chan_scales is not None else None,
                                        bias.at(0) if bias is not None else None, m, n, k, int(relu),
                                        x.device, _sptr(stream)))


class LinearWeightCache:
    """Device-resident quantised weight of one Linear with its expanded bf16 copy cached
    (``nvq_linear_cache_*``).  The codes are expanded on the first forward and again only
    after ``update`` (which bumps the version the library compares); every other forward runs
    the contraction alone.  ``forward_device`` works on device buffers, ``forward_host`` on
    bf16 bit arrays; results equal ``linear_q_device``'s bit for bit."""

    def __init__(self, wq: np.ndarray, w_scales: np.ndarray, bias: np.ndarray | None = None,
                 fmt: str = "e4m3", device: int = 0) -> None:
        import ctypes as C
        self.fmt, self.device = fmt, device
        self.n = int(wq.shape[0])
        self.k = int(np.asarray(w_scales).size * 32 // self.n) if fmt == "e2m1_b32" else int(wq.shape[1])
        self.version = 0
        self.expansions = 0
        self._h = C.c_void_p()
        check(lib().nvq_linear_cache_create(C.byref(self._h), self.n, self.k, _lib.DTYPE_IDS[fmt], device))
        self.d_codes = DeviceBuffer.from_numpy(np.ascontiguousarray(wq, np.uint8), device)
        self.d_scales = DeviceBuffer.from_numpy(np.ascontiguousarray(w_scales, np.float32), device)
        self.d_bias = None if bias is None else DeviceBuffer.from_numpy(
            np.ascontiguousarray(bias, np.float32).reshape(-1), device)

    def update(self, wq: np.ndarray | None = None, w_scales: np.ndarray | None = None,
               bias: np.ndarray | None = None) -> None:
        """New codes / scales / bias written into the same device buffers; the next forward
        expands again."""
        if wq is not None:
            self.d_codes.upload(np.ascontiguousarray(wq, np.uint8))
        if w_scales is not None:
            self.d_scales.upload(np.ascontiguousarray(w_scales, np.float32))
        if bias is not None and self.d_bias is not None:
            self.d_bias.upload(np.ascontiguousarray(bias, np.float32).reshape(-1))
        self.version += 1

    def forward_device(self, y: DeviceBuffer, x: DeviceBuffer, m: int, stream=None, relu: bool = False) -> None:
        import ctypes as C
        ran = C.c_int(0)
        check(lib().nvq_linear_cache_fwd(self._h, y.at(0), x.at(0), self.d_codes.at(0), self.d_scales.at(0),
                                         self.d_bias.at(0) if self.d_bias is not None else None, m,
                                         self.version, int(relu), C.byref(ran), _sptr(stream)))
        self.expansions += ran.value

    def forward_host(self, x_bf16_bits: np.ndarray, relu: bool = False) -> np.ndarray:
        x = np.ascontiguousarray(x_bf16_bits, np.uint16)
        m = x.shape[0]
        dx = DeviceBuffer.from_numpy(x, self.device)
        dy = DeviceBuffer(m * self.n * 2, self.device)
        self.forward_device(dy, dx, m, relu=relu)
        device_sync(self.device)
        check_device_errors(self.device)
        return dy.to_numpy(np.uint16, (m, self.n))

    def close(self) -> None:
        if self._h:
            lib().nvq_linear_cache_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def mul_host(a, b, device: int = 0) -> np.ndarray:
    """Elementwise fp32 product on the GPU (``ReLU.backward``: grad * mask)."""
    a, b = _f32(a, device), _f32(b, device)
    if a.shape != b.shape:
        raise ValueError("shapes differ")
    da, db = DeviceBuffer.from_numpy(a, device), DeviceBuffer.from_numpy(b, device)
    o = DeviceBuffer(max(4, a.nbytes), device)
    check(lib().nvq_mul_f32(o.at(0), da.at(0), db.at(0), a.size, device, None))
    return o.to_numpy(np.float32, a.shape)


# ------------------------------------------------------------------ BatchNorm, pooling, Dropout
def _f64(a):
    return np.ascontiguousarray(a, np.float64)


def _ncs(shape):
    """(N, C, S) view of a BatchNorm input shape: (N,C), (N,C,L) or (N,C,H,W)."""
    if len(shape) not in (2, 3, 4):
        raise ValueError(f"BatchNorm expects 2D, 3D or 4D input, got {len(shape)}D")
    return shape[0], shape[1], int(np.prod(shape[2:], dtype=np.int64))


def batchnorm_fwd_host(x, gamma, beta, running_mean, running_var, momentum: float = 0.1,
                       eps: float = 1e-5, training: bool = True, device: int = 0):
    """``BatchNorm2d.forward`` / ``BatchNorm1d.forward`` (novann/layers/batchnorm/batchnorm2d.py:57-102,
    batchnorm1d.py:96-141).  gamma / beta / running statistics: float64, C entries.  Returns
    (y fp32, new_running_mean, new_running_var, save_stats): y is the float32 narrowing of the
    reference's float64 result; save_stats (2, C) fp32 holds the batch mean and the
    Bessel-corrected variance for ``batchnorm_bwd_host`` (None in evaluation mode)."""
    x = _f32(x, device)
    n, c, s = _ncs(x.shape)
    dx = DeviceBuffer.from_numpy(x, device)
    dg, db = DeviceBuffer.from_numpy(_f64(gamma).ravel(), device), DeviceBuffer.from_numpy(_f64(beta).ravel(), device)
    drm = DeviceBuffer.from_numpy(_f64(running_mean).ravel(), device)
    drv = DeviceBuffer.from_numpy(_f64(running_var).ravel(), device)
    dy = DeviceBuffer(max(4, x.nbytes), device)
    dst = DeviceBuffer(2 * c * 4, device)
    dsc = DeviceBuffer(lib().nvq_batchnorm_scratch_bytes(c), device)
    check(lib().nvq_batchnorm_fwd_f32(dy.at(0), dx.at(0), dg.at(0), db.at(0), drm.at(0), drv.at(0),
                                      dst.at(0), dsc.at(0), n, c, s, float(momentum), float(eps),
                                      int(bool(training)), device, None))
    y = dy.to_numpy(np.float32, x.shape) if x.size else np.empty(x.shape, np.float32)
    return (y, drm.to_numpy(np.float64, (c,)), drv.to_numpy(np.float64, (c,)),
            dst.to_numpy(np.float32, (2, c)) if training and x.size else None)


def batchnorm_bwd_host(grad, x, save_stats, gamma, eps: float = 1e-5, device: int = 0):
    """``BatchNorm2d.backward`` (batchnorm2d.py:104-146): returns (dx fp32, dgamma, dbeta float64 (C,))."""
    grad, x = _f32(grad, device), _f32(x, device)
    n, c, s = _ncs(x.shape)
    dgr, dx = DeviceBuffer.from_numpy(grad, device), DeviceBuffer.from_numpy(x, device)
    dst = DeviceBuffer.from_numpy(_f32(save_stats, device), device)
    dg = DeviceBuffer.from_numpy(_f64(gamma).ravel(), device)
    o_dx = DeviceBuffer(max(4, x.nbytes), device)
    o_dg, o_db = DeviceBuffer(c * 8, device), DeviceBuffer(c * 8, device)
    dsc = DeviceBuffer(lib().nvq_batchnorm_scratch_bytes(c), device)
    check(lib().nvq_batchnorm_bwd_f32(o_dx.at(0), o_dg.at(0), o_db.at(0), dgr.at(0), dx.at(0), dst.at(0),
                                      dg.at(0), dsc.at(0), n, c, s, float(eps), device, None))
    return (o_dx.to_numpy(np.float32, x.shape), o_dg.to_numpy(np.float64, (c,)),
            o_db.to_numpy(np.float64, (c,)))


def max_pool2d_host(x, kernel, stride, padding=(0, 0), padding_mode: str = "zeros", device: int = 0):
    """``F.max_pool2d`` (novann/functional.py:450-536): (N, C, OH, OW) fp32."""
    x = _f32(x, device)
    n, c, h, w = x.shape
    mode = _pad_mode(padding_mode)
    oh = (h + 2 * padding[0] - kernel[0]) // stride[0] + 1
    ow = (w + 2 * padding[1] - kernel[1]) // stride[1] + 1
    dx = DeviceBuffer.from_numpy(x, device)
    dy = DeviceBuffer(max(4, n * c * max(oh, 0) * max(ow, 0) * 4), device)
    check(lib().nvq_maxpool2d_fwd_f32(dy.at(0), dx.at(0), n, c, h, w, kernel[0], kernel[1], stride[0],
                                      stride[1], padding[0], padding[1], mode, device, None))
    return dy.to_numpy(np.float32, (n, c, oh, ow))


def max_pool2d_bwd_host(grad, x, kernel, stride, padding=(0, 0), padding_mode: str = "zeros",
                        device: int = 0):
    """``MaxPool2d.backward`` (novann/layers/pooling/maxpool/maxpool2d.py): dX (N, C, H, W)."""
    grad, x = _f32(grad, device), _f32(x, device)
    n, c, h, w = x.shape
    dg, dx = DeviceBuffer.from_numpy(grad, device), DeviceBuffer.from_numpy(x, device)
    o = DeviceBuffer(max(4, x.nbytes), device)
    check(lib().nvq_maxpool2d_bwd_f32(o.at(0), dg.at(0), dx.at(0), n, c, h, w, kernel[0], kernel[1],
                                      stride[0], stride[1], padding[0], padding[1],
                                      _pad_mode(padding_mode), device, None))
    return o.to_numpy(np.float32, x.shape)


def avg_pool2d_host(x, device: int = 0):
    """``F.avg_pool2d`` (novann/functional.py:550-559): (N, C, 1, 1) fp32."""
    x = _f32(x, device)
    n, c, h, w = x.shape
    dx, o = DeviceBuffer.from_numpy(x, device), DeviceBuffer(max(4, n * c * 4), device)
    check(lib().nvq_gap2d_fwd_f32(o.at(0), dx.at(0), n * c, h * w, device, None))
    return o.to_numpy(np.float32, (n, c, 1, 1))


def avg_pool2d_bwd_host(grad, x_shape, device: int = 0):
    """``GlobalAvgPool2d.backward``: (N, C, H, W) fp32."""
    grad = _f32(grad, device)
    n, c, h, w = x_shape
    dg, o = DeviceBuffer.from_numpy(grad, device), DeviceBuffer(max(4, n * c * h * w * 4), device)
    check(lib().nvq_gap2d_bwd_f32(o.at(0), dg.at(0), n * c, h * w, device, None))
    return o.to_numpy(np.float32, (n, c, h, w))


def dropout_host(x, mask, keep_prob: float, device: int = 0):
    """``(x * mask) / keep_prob`` (novann/layers/regularization/dropout.py:52-54, :66)."""
    x, mask = _f32(x, device), _f32(mask, device)
    dx, dm = DeviceBuffer.from_numpy(x, device), DeviceBuffer.from_numpy(mask, device)
    o = DeviceBuffer(max(4, x.nbytes), device)
    check(lib().nvq_dropout_f32(o.at(0), dx.at(0), dm.at(0), x.size, C.c_float(keep_prob), device, None))
    return o.to_numpy(np.float32, x.shape)
