"""CPU oracle (NumPy) for the cast / quantise / quantised-GEMM hot path.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA kernels are
compared against; only the test-suite, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it.  The
product package never does.

What it restates
----------------
NovaNN (the reference) is pure NumPy.  Its dtype-conversion primitive is
``ndarray.astype`` (call sites ``novann/layers/linear/linear.py:81,96``,
``novann/layers/convolutional/conv2d.py:159,188``) and its contraction is
``ndarray.__matmul__`` (``novann/functional.py:160,377``).  The arithmetic
therefore lives in a third-party dependency, NumPy 2.3.5 (``pyproject.toml:10``,
pinned in ``poetry.lock``), whose published behaviour for narrowing casts is IEEE-754
round-to-nearest-even with overflow to infinity.  The functions below restate that
algorithm with explicit integer arithmetic so every bit of the result is specified:

* fp32 <-> fp16: pinned against ``ndarray.astype(np.float16)`` itself.
* fp32 <-> bf16, FP8 E4M3 (finite-only "fn" flavour), FP8 E5M2, FP4 E2M1: the
  reference has no such code (PARITY UNPINNED by the reference); the rules are
  the normative spec documented per function, cross-checked in the tests against
  the ``ml_dtypes`` package where it is installed.
* fp32 Linear / Conv2d / ReLU / softmax-CE / SGD (the reference's own layers):
  restated in ``mlp_*`` / ``conv2d_*`` below and pinned by golden vectors that
  were produced by importing the reference (``tests/golden/make_golden.py``).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------
# small-float format table: (exponent bits, mantissa bits, bias, max finite code,
# code emitted for a NaN input before the sign is applied)
# ----------------------------------------------------------------------------
E4M3 = dict(name="e4m3", ebits=4, mbits=3, bias=7, max_code=0x7E, nan_code=0x7F, fmax=448.0)
E5M2 = dict(name="e5m2", ebits=5, mbits=2, bias=15, max_code=0x7B, nan_code=0x7E, fmax=57344.0)
E2M1 = dict(name="e2m1", ebits=2, mbits=1, bias=1, max_code=0x7, nan_code=None, fmax=6.0)

FP4_BLOCK = 32


def _u32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return x.view(np.uint32)


# ----------------------------------------------------------------------------
# fp32 <-> fp16   (reference primitive: ndarray.astype, novann/layers/linear/linear.py:81)
# ----------------------------------------------------------------------------
def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> fp16 bit patterns (uint16), identical to ``x.astype(np.float16)``.

    RNE, subnormals honoured, |x| >= 65520 -> inf.  NaN: sign kept, the top ten
    mantissa bits kept (not quieted); if those ten bits are zero the result is
    ``sign | 0x7c01`` (NumPy's behaviour, observed black-box).
    """
    u = _u32(x)
    sign = ((u >> 16) & 0x8000).astype(np.uint32)
    a = u & np.uint32(0x7FFFFFFF)
    e = (a >> 23).astype(np.int64)
    # normal range of the target (a >= 2^-14): rebias and round 13 bits away
    v = (a.astype(np.int64) - 0x38000000)
    h = v >> 13
    r = v & 0x1FFF
    h = h + ((r > 0x1000) | ((r == 0x1000) & ((h & 1) == 1)))
    h = np.minimum(h, 0x7C00)  # rounds/overflows to inf
    # subnormal range of the target: value = m * 2^(e-150); unit 2^-24
    m = ((a & 0x7FFFFF) | 0x800000).astype(np.int64)
    sh = np.clip(126 - e, 0, 40)
    hs = m >> sh
    rs = m & ((np.int64(1) << sh) - 1)
    half = np.int64(1) << np.maximum(sh - 1, 0)
    hs = hs + ((rs > half) | ((rs == half) & ((hs & 1) == 1)))
    out = np.where(a >= 0x38800000, h, hs)
    out = np.where(a >= 0x47800000, 0x7C00, out)  # >= 65536 (and inf)
    # NaN
    pay = (a >> 13) & 0x3FF
    nan = 0x7C00 | np.where(pay == 0, 1, pay)
    out = np.where(a > 0x7F800000, nan, out)
    return (out.astype(np.uint32) | sign).astype(np.uint16)


def f16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    """fp16 bit patterns -> fp32, exact; NaN payload shifted left 13, not quieted
    (identical to ``h.view(np.float16).astype(np.float32)``)."""
    h = np.ascontiguousarray(h, dtype=np.uint16).astype(np.uint32)
    sign = (h & 0x8000) << 16
    e = (h >> 10) & 0x1F
    m = h & 0x3FF
    # normal
    out = ((e + 112) << 23) | (m << 13)
    # inf / NaN
    out = np.where(e == 0x1F, np.uint32(0x7F800000) | (m << 13), out)
    # subnormal: m * 2^-24, exact in fp32
    sub = (m.astype(np.float32) * np.float32(2.0 ** -24)).view(np.uint32)
    out = np.where(e == 0, sub, out)
    return (out | sign).astype(np.uint32).view(np.float32)


# ----------------------------------------------------------------------------
# fp64 <-> fp32   (reference primitive: ndarray.astype(np.float32) on BatchNorm's float64
# output, novann/layers/linear/linear.py:81 fed by novann/layers/batchnorm/batchnorm2d.py:40-41,87)
# ----------------------------------------------------------------------------
def f64_to_f32_bits(x: np.ndarray) -> np.ndarray:
    """fp64 -> fp32 bit patterns (uint32), identical to ``x.astype(np.float32)``.

    RNE on the 29 dropped mantissa bits, subnormal results honoured, |x| >= 2^128 (after
    rounding) -> inf.  NaN: sign kept, top 22 payload bits kept, quiet bit set
    (``sign | 0x7fc00000 | payload >> 29``; NumPy's behaviour, observed black-box).
    """
    u = np.ascontiguousarray(x, dtype=np.float64).view(np.uint64)
    sign = ((u >> np.uint64(32)) & np.uint64(0x80000000)).astype(np.uint64)
    a = u & np.uint64(0x7FFFFFFFFFFFFFFF)
    e = (a >> np.uint64(52)).astype(np.int64)
    m = a & np.uint64((1 << 52) - 1)
    # normal range of the target (|x| >= 2^-126, biased fp64 exponent >= 897): rebias, drop 29 bits
    v = a.astype(np.int64) - (np.int64(896) << 52)
    h = v >> 29
    r = v & ((1 << 29) - 1)
    h = h + ((r > (1 << 28)) | ((r == (1 << 28)) & ((h & 1) == 1)))
    h = np.minimum(h, 0x7F800000)
    # subnormal range: value = (m | 2^52) * 2^(e - 1075); the target's unit is 2^-149
    mm = (m | np.uint64(1 << 52)).astype(np.int64)
    sh = np.clip(926 - e, 0, 62)
    hs = mm >> sh
    rs = mm & ((np.int64(1) << sh) - 1)
    half = np.int64(1) << np.maximum(sh - 1, 0)
    hs = hs + ((rs > half) | ((rs == half) & ((hs & 1) == 1)))
    hs = np.where(e == 0, 0, hs)            # fp64 zeros and subnormals are far below 2^-150
    out = np.where(e >= 897, h, hs)
    out = np.where(a >= np.uint64(0x47F0000000000000), 0x7F800000, out)
    nan = np.int64(0x7FC00000) | (m >> np.uint64(29)).astype(np.int64)
    out = np.where(a > np.uint64(0x7FF0000000000000), nan, out)
    return (out.astype(np.uint64) | sign).astype(np.uint32)


def f32_bits_to_f64_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> fp64 bit patterns (uint64), identical to ``x.astype(np.float64)``: exact;
    a NaN comes out quiet with its payload shifted left 29."""
    u = _u32(x).astype(np.uint64)
    sign = (u & np.uint64(0x80000000)) << np.uint64(32)
    e = (u >> np.uint64(23)) & np.uint64(0xFF)
    m = u & np.uint64(0x7FFFFF)
    out = ((e + np.uint64(896)) << np.uint64(52)) | (m << np.uint64(29))
    out = np.where(e == 0xFF, np.uint64(0x7FF0000000000000) | (m << np.uint64(29)) |
                   np.where(m != 0, np.uint64(0x0008000000000000), np.uint64(0)), out)
    # fp32 subnormal m * 2^-149: normalise (the leading one of m moves to the hidden bit)
    mi = m.astype(np.int64)
    lead = np.zeros(m.shape, np.int64)
    for b in range(23):
        lead = np.where((mi >> b) > 0, b, lead)
    sub = ((np.uint64(1023 - 149) + lead.astype(np.uint64)) << np.uint64(52)) | \
          ((m << (np.uint64(52) - lead.astype(np.uint64))) & np.uint64((1 << 52) - 1))
    out = np.where((e == 0) & (m != 0), sub, out)
    out = np.where((e == 0) & (m == 0), np.uint64(0), out)
    return (out | sign).astype(np.uint64)


# ----------------------------------------------------------------------------
# fp32 <-> bf16   (no reference code; spec: RNE, NaN -> sign|0x7fc0)
# ----------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16): RNE on the low 16 bits including
    overflow to inf (0x7f7fffff -> 0x7f80); any NaN -> ``sign | 0x7fc0``."""
    u = _u32(x).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    nan = ((u >> 16) & 0x8000) | 0x7FC0
    out = np.where((u & 0x7FFFFFFF) > 0x7F800000, nan, r)
    return out.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """bf16 bit patterns -> fp32: ``bits << 16``; payloads preserved."""
    b = np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32)
    return (b << 16).view(np.float32)


# ----------------------------------------------------------------------------
# generic saturating RNE fp32 -> tiny float (E4M3 / E5M2 / E2M1)
# ----------------------------------------------------------------------------
def _f32_to_small_sat(x: np.ndarray, fmt: dict) -> np.ndarray:
    """Saturating ("satfinite") RNE conversion of fp32 to a <=8-bit float code.

    |y| is clamped to the format's largest finite value (so +-inf saturate), then
    rounded to nearest, ties to even, subnormals honoured.  The sign goes to the
    top bit of the code (bit 7 for FP8, bit 3 for FP4); -0 keeps its sign.
    """
    ebits, mbits, bias = fmt["ebits"], fmt["mbits"], fmt["bias"]
    u = _u32(x)
    sbit = (u >> 31).astype(np.uint32)
    a = (u & np.uint32(0x7FFFFFFF)).astype(np.int64)
    e = a >> 23
    shift = 23 - mbits
    # normal range
    v = a - (np.int64(127 - bias) << 23)
    h = v >> shift
    r = v & ((np.int64(1) << shift) - 1)
    half = np.int64(1) << (shift - 1)
    h = h + ((r > half) | ((r == half) & ((h & 1) == 1)))
    # subnormal range: unit = 2^(1-bias-mbits); value = m * 2^(e-150)
    m = (a & 0x7FFFFF) | 0x800000
    sh = np.clip((150 + (1 - bias - mbits)) - e, 0, 40)
    hs = m >> sh
    rs = m & ((np.int64(1) << sh) - 1)
    halfs = np.int64(1) << np.maximum(sh - 1, 0)
    hs = hs + ((rs > halfs) | ((rs == halfs) & ((hs & 1) == 1)))
    min_normal = np.int64(127 + 1 - bias) << 23
    out = np.where(a >= min_normal, h, hs)
    fmax_bits = np.array([fmt["fmax"]], np.float32).view(np.uint32)[0]
    out = np.where(a >= int(fmax_bits), fmt["max_code"], out)
    signpos = ebits + mbits
    out = out.astype(np.uint32) | (sbit << signpos)
    isnan = a > 0x7F800000
    if fmt["nan_code"] is not None:
        out = np.where(isnan, np.uint32(fmt["nan_code"]) | (sbit << signpos), out)
    else:
        # E2M1 has no NaN: +NaN -> 0x8, -NaN -> 0x0 (the behaviour of the
        # ml_dtypes float4_e2m1fn cast, observed black-box)
        out = np.where(isnan, (np.uint32(1) - sbit) << signpos, out)
    return out.astype(np.uint8)


def f32_to_e4m3_bits(x):
    """fp32 -> FP8 E4M3 "fn" (bias 7, no inf, NaN 0x7f/0xff, max 448), saturating
    RNE.  Equals ``np.clip(x,-448,448).astype(ml_dtypes.float8_e4m3fn)``; NaN ->
    ``sign|0x7f``."""
    return _f32_to_small_sat(x, E4M3)


def f32_to_e5m2_bits(x):
    """fp32 -> FP8 E5M2 (bias 15, max finite 57344), saturating RNE (inf clamps
    to +-57344); NaN -> ``sign|0x7e``."""
    return _f32_to_small_sat(x, E5M2)


def f32_to_e2m1_codes(x):
    """fp32 -> FP4 E2M1 code (0..15, sign in bit 3), saturating RNE over the code
    points {0,.5,1,1.5,2,3,4,6}."""
    return _f32_to_small_sat(x, E2M1)


def _small_table(fmt: dict) -> np.ndarray:
    """Exact fp32 value of every code of a tiny float format.  NaN codes decode to
    the canonical quiet NaN carrying the code's sign (``sign|0x7fc00000``)."""
    ebits, mbits, bias = fmt["ebits"], fmt["mbits"], fmt["bias"]
    n = 1 << (1 + ebits + mbits)
    t = np.zeros(n, np.float32)
    for c in range(n):
        s = -1.0 if (c >> (ebits + mbits)) & 1 else 1.0
        e = (c >> mbits) & ((1 << ebits) - 1)
        m = c & ((1 << mbits) - 1)
        if e == 0:
            val = m * 2.0 ** (1 - bias - mbits)
        else:
            val = (1 + m / (1 << mbits)) * 2.0 ** (e - bias)
        t[c] = s * val
    tu = t.view(np.uint32)
    if fmt["name"] == "e4m3":
        tu[0x7F] = 0x7FC00000
        tu[0xFF] = 0xFFC00000
    if fmt["name"] == "e5m2":
        tu[0x7C] = 0x7F800000
        tu[0xFC] = 0xFF800000
        for c in (0x7D, 0x7E, 0x7F):
            tu[c] = 0x7FC00000
            tu[c | 0x80] = 0xFFC00000
    return t


E4M3_TABLE = _small_table(E4M3)
E5M2_TABLE = _small_table(E5M2)
E2M1_TABLE = _small_table(E2M1)


def _fmt(fmt):
    if isinstance(fmt, dict):
        return fmt
    return {"e4m3": E4M3, "e5m2": E5M2, "e2m1": E2M1}[fmt]


def _table(fmt):
    return {"e4m3": E4M3_TABLE, "e5m2": E5M2_TABLE, "e2m1": E2M1_TABLE}[_fmt(fmt)["name"]]


# ----------------------------------------------------------------------------
# per-tensor FP8 quantise / dequantise
# ----------------------------------------------------------------------------
def amax_f32(x: np.ndarray) -> np.float32:
    """max |x| over the tensor, NaNs ignored (exact; order independent)."""
    a = _u32(x).ravel() & np.uint32(0x7FFFFFFF)
    if a.size == 0:
        return np.float32(0.0)
    a = np.where(a > 0x7F800000, np.uint32(0), a)
    return a.max().reshape(1).view(np.float32)[0]


def fp8_scales(amax, fmt) -> tuple[np.float32, np.float32]:
    """(scale, inv_scale) from a tensor's amax: ``scale = amax/FMAX`` and
    ``inv_scale = FMAX/amax``, each ONE fp32 round-to-nearest division; both 1.0
    when amax == 0."""
    fmax = np.float32(_fmt(fmt)["fmax"])
    amax = np.float32(amax)
    if amax == 0:
        return np.float32(1.0), np.float32(1.0)
    with np.errstate(over="ignore", divide="ignore"):
        return np.float32(amax / fmax), np.float32(fmax / amax)


def quantize_fp8(x: np.ndarray, inv_scale, fmt) -> np.ndarray:
    """``q_i = cvt_sat_rne(x_i * inv_scale)`` with a single fp32 multiply."""
    with np.errstate(over="ignore", invalid="ignore"):
        y = np.ascontiguousarray(x, np.float32) * np.float32(inv_scale)
    return _f32_to_small_sat(y, _fmt(fmt)).reshape(np.shape(x))


def dequantize_fp8(q: np.ndarray, scale, fmt) -> np.ndarray:
    """``x'_i = float(q_i) * scale`` (one fp32 multiply).  NaN codes give the
    canonical quiet NaN with the code's sign regardless of the scale."""
    q = np.ascontiguousarray(q, np.uint8)
    t = _table(fmt)[q]
    with np.errstate(over="ignore", invalid="ignore"):
        y = t * np.float32(scale)
    nan = np.isnan(t)
    if nan.any():
        yu = y.view(np.uint32)
        yu[nan] = t.view(np.uint32)[nan]
    return y


def quantize_fp8_tensor(x: np.ndarray, fmt):
    """amax -> scales -> codes.  Returns (codes u8, scale f32, inv_scale f32)."""
    scale, inv = fp8_scales(amax_f32(x), fmt)
    return quantize_fp8(x, inv, fmt), scale, inv


# ----------------------------------------------------------------------------
# FP4 E2M1, one fp32 scale per 32 consecutive elements of the last dimension
# ----------------------------------------------------------------------------
def quantize_fp4_b32(x_bf16_bits: np.ndarray):
    """bf16 (rows, cols) -> (packed u8 (rows, cols/2), scales f32 (rows, cols/32)).

    Per block of 32: ``amax_b`` exact; ``scale_b = amax_b / 6`` (fp32 RN);
    ``inv_b = 6 / amax_b`` if amax_b > 0 else 0; ``code = cvt_sat_rne_e2m1(
    float(x) * inv_b)``; byte j = code[2j] | code[2j+1] << 4 (low nibble first).
    NaN elements are ignored by the amax.
    """
    b = np.ascontiguousarray(x_bf16_bits, np.uint16)
    rows, cols = b.shape
    assert cols % FP4_BLOCK == 0
    x = bf16_bits_to_f32(b).reshape(rows, cols // FP4_BLOCK, FP4_BLOCK)
    a = x.view(np.uint32) & np.uint32(0x7FFFFFFF)
    a = np.where(a > 0x7F800000, np.uint32(0), a)
    amax = a.max(axis=2).view(np.float32)
    with np.errstate(over="ignore", divide="ignore", invalid="ignore"):
        scale = (amax / np.float32(6.0)).astype(np.float32)
        inv = np.where(amax > 0, np.float32(6.0) / amax, np.float32(0.0)).astype(np.float32)
        y = x * inv[:, :, None]
    codes = _f32_to_small_sat(y, E2M1).reshape(rows, cols)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return packed, scale


def dequantize_fp4_b32(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """(packed u8 (rows, cols/2), scales (rows, cols/32)) -> bf16 bits (rows, cols):
    ``bf16_rne(e2m1_value(code) * scale_b)``."""
    p = np.ascontiguousarray(packed, np.uint8)
    rows, half = p.shape
    cols = half * 2
    codes = np.empty((rows, cols), np.uint8)
    codes[:, 0::2] = p & 0xF
    codes[:, 1::2] = p >> 4
    v = E2M1_TABLE[codes].reshape(rows, cols // FP4_BLOCK, FP4_BLOCK)
    with np.errstate(over="ignore", invalid="ignore"):
        y = v * np.ascontiguousarray(scales, np.float32)[:, :, None]
    return f32_to_bf16_bits(y.reshape(rows, cols)).reshape(rows, cols)


# ----------------------------------------------------------------------------
# quantised-weight Linear forward
# ----------------------------------------------------------------------------
def quantize_weight_per_channel(w: np.ndarray, fmt="e4m3"):
    """Per-output-channel weight quantisation: ``s_n = max_k|W[n,k]| / FMAX``;
    ``Wq[n,k] = cvt_sat(W[n,k] * (FMAX / amax_n))``.  Returns (codes (N,K) u8,
    scales (N,) f32)."""
    w = np.ascontiguousarray(w, np.float32)
    f = _fmt(fmt)
    fmax = np.float32(f["fmax"])
    amax = np.abs(w).max(axis=1).astype(np.float32)
    safe = np.where(amax > 0, amax, np.float32(1.0))
    scale = np.where(amax > 0, safe / fmax, np.float32(1.0)).astype(np.float32)
    inv = np.where(amax > 0, fmax / safe, np.float32(1.0)).astype(np.float32)
    codes = _f32_to_small_sat(w * inv[:, None], f).reshape(w.shape)
    return codes, scale


def linear_fwd_qweight(x_bf16_bits, wq, w_scales, bias, fmt="e4m3", acc=np.float64):
    """``Y[m,n] = bf16_rne(s_n * sum_k float(X[m,k]) * float(Wq[n,k]) + b_n)``.

    Mirrors ``F.linear`` (novann/functional.py:147-163: ``input @ weight.T`` then
    ``+= bias``) on the dequantised operands.  ``acc`` chooses the accumulation
    type of the CPU contraction (float64 separates the kernel's own error from
    sgemm's; float32 is what the reference's NumPy ``@`` does).  Returns
    (bf16 bits (M,N), fp32 pre-rounding values (M,N)).
    """
    x = bf16_bits_to_f32(x_bf16_bits).astype(acc)
    w = _table(fmt)[np.ascontiguousarray(wq, np.uint8)].astype(acc)
    y = (x @ w.T).astype(np.float32)
    y = y * np.ascontiguousarray(w_scales, np.float32)[None, :]
    if bias is not None:
        y = y + np.ascontiguousarray(bias, np.float32).reshape(1, -1)
    y = y.astype(np.float32)
    return f32_to_bf16_bits(y).reshape(y.shape), y


def dequantize_fp4_weight(packed, scales) -> np.ndarray:
    """Packed E2M1 block-32 weight (N, K/2) + scales (N, K/32) -> fp32 (N,K) exact
    product ``e2m1_value * scale`` (fp32)."""
    p = np.ascontiguousarray(packed, np.uint8)
    n, half = p.shape
    k = half * 2
    codes = np.empty((n, k), np.uint8)
    codes[:, 0::2] = p & 0xF
    codes[:, 1::2] = p >> 4
    v = E2M1_TABLE[codes].reshape(n, k // FP4_BLOCK, FP4_BLOCK)
    return (v * np.ascontiguousarray(scales, np.float32)[:, :, None]).reshape(n, k)


def max_abs_rel(y, y_ref) -> float:
    """The GEMM parity metric: ``max|y - y_ref| / max|y_ref|``."""
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    return float(np.max(np.abs(y - y_ref)) / np.max(np.abs(y_ref)))


# ----------------------------------------------------------------------------
# fp32 layers of the reference (config: MLP train step) and Conv2d forward
# ----------------------------------------------------------------------------
def linear_fwd_f32(x, w, b):
    """``F.linear`` (novann/functional.py:147-163): ``x @ w.T`` then ``+= b``."""
    out = np.asarray(x, np.float32) @ np.asarray(w, np.float32).T
    if b is not None:
        out += np.asarray(b, np.float32).reshape(1, -1)
    return out


def linear_bwd_f32(x, w, grad):
    """``Linear.backward`` (novann/layers/linear/linear.py:85-108).  Returns
    (dW (N,K), db (1,N), dx (M,K))."""
    grad = np.asarray(grad, np.float32)
    return grad.T @ x, np.sum(grad, axis=0, keepdims=True), grad @ w


def relu_fwd(x):
    """``F.relu`` (novann/functional.py:8-22): ``mask=(x>0)``; ``x*mask``."""
    mask = (x > 0).astype(x.dtype)
    return x * mask, mask


def softmax_ce(logits, labels):
    """``CrossEntropyLoss`` (novann/losses/loss_functions.py:29-75).

    Returns (loss, grad).  ``grad = (softmax(logits,1) - onehot)/N`` in fp32 after
    a float64 subtraction (the int32 one-hot promotes it).  The loss VALUE follows
    the reference literally: softmax is applied a second time, along the batch axis,
    inside ``F.cross_entropy`` (novann/functional.py:108-128) with eps 1e-8.
    """
    logits = np.asarray(logits, np.float32)
    n, c = logits.shape
    z = logits - logits.max(axis=1, keepdims=True)
    ez = np.exp(z)
    y_hat = (ez / ez.sum(axis=1, keepdims=True)).astype(np.float32)
    onehot = np.eye(c, dtype=np.int32)[np.asarray(labels)]
    grad = ((y_hat - onehot) / n).astype(np.float32)
    z2 = y_hat - y_hat.max(axis=0, keepdims=True)
    e2 = np.exp(z2)
    p2 = (e2 / e2.sum(axis=0, keepdims=True)).astype(np.float32)
    loss = np.float32(-np.sum(onehot * np.log(p2 + 1e-8)) / n)
    return loss, grad


def mlp_train_step(params, x, labels, lr):
    """One step of ``Sequential(Linear, ReLU, Linear, ReLU, ..., Linear)`` +
    ``CrossEntropyLoss`` + vanilla ``SGD`` (novann/optim/sgd.py:58-82), i.e. the
    body of the reference's train loop (novann/utils/train/train.py:60-75).

    ``params`` = [W0, b0, W1, b1, ...] with W (out,in), b (1,out).  Returns a dict
    with logits, loss, grads (same order as params) and the updated params.
    """
    nl = len(params) // 2
    acts, masks = [np.asarray(x, np.float32)], []
    h = acts[0]
    for i in range(nl):
        h = linear_fwd_f32(h, params[2 * i], params[2 * i + 1])
        if i < nl - 1:
            h, m = relu_fwd(h)
            masks.append(m)
            acts.append(h)
    logits = h
    loss, g = softmax_ce(logits, labels)
    grads = [None] * len(params)
    for i in reversed(range(nl)):
        dw, db, dx = linear_bwd_f32(acts[i], params[2 * i], g)
        grads[2 * i], grads[2 * i + 1] = dw, db
        if i > 0:
            g = dx * masks[i - 1]
    new = [(p - np.float32(lr) * gr).astype(np.float32) for p, gr in zip(params, grads)]
    return dict(logits=logits, loss=loss, grads=grads, params=new)


def conv2d_out_size(h, w, kh, kw, sh, sw, ph, pw):
    """``_calc_out_size`` (novann/functional.py:319-323)."""
    return (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1


_PAD_MODES = {"zeros": "constant", "reflect": "reflect", "replicate": "edge", "circular": "wrap"}


def im2col(x, kh, kw, sh, sw, ph, pw, padding_mode="zeros"):
    """``_im2col`` (novann/functional.py:346-368): rows ordered (c, kh, kw),
    columns ordered (n, oh, ow).  Written as explicit gathers, not as_strided."""
    if padding_mode not in _PAD_MODES:
        raise ValueError(f"padding_mode Only accept {tuple(_PAD_MODES)} not '{padding_mode}'")
    x = np.asarray(x, np.float32)
    n, c, h, w = x.shape
    xp = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)), mode=_PAD_MODES[padding_mode])
    oh, ow = conv2d_out_size(h, w, kh, kw, sh, sw, ph, pw)
    col = np.empty((c, kh, kw, n, oh, ow), np.float32)
    for i in range(kh):
        for j in range(kw):
            win = xp[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw]  # (n,c,oh,ow)
            col[:, i, j] = win.transpose(1, 0, 2, 3)
    return col.reshape(c * kh * kw, n * oh * ow), oh, ow


def conv2d_fwd_f32(x, w, b, stride=(1, 1), padding=(0, 0), padding_mode="zeros"):
    """``F.conv2d`` (novann/functional.py:275-385): ``w_col @ col (+ b)`` reshaped
    to (N, Cout, OH, OW)."""
    w = np.asarray(w, np.float32)
    cout, cin, kh, kw = w.shape
    n = x.shape[0]
    col, oh, ow = im2col(x, kh, kw, stride[0], stride[1], padding[0], padding[1], padding_mode)
    out = w.reshape(cout, -1) @ col
    if b is not None:
        out += np.asarray(b, np.float32).reshape(cout, 1)
    return np.ascontiguousarray(out.reshape(cout, n, oh, ow).transpose(1, 0, 2, 3))


def conv2d_bwd_f32(grad, col, w, x_shape, stride=(1, 1), padding=(0, 0)):
    """``Conv2d.backward`` with ``_col2im`` (novann/layers/convolutional/conv2d.py:117-148,
    179-207).  Returns (dW, db (Cout,1), dX).  col2im is written as strided slice adds in
    (kh, kw) order, the order in which np.add.at applies the contributions; gradient that
    lands on padding is cropped away, as the reference does for every padding mode."""
    grad = np.asarray(grad, np.float32)
    w = np.asarray(w, np.float32)
    n, c, h, wd = x_shape
    cout, _, kh, kw = w.shape
    sh, sw = stride
    ph, pw = padding
    oh, ow = grad.shape[2], grad.shape[3]
    g_r = grad.transpose(1, 0, 2, 3).reshape(cout, -1)
    dw = (g_r @ np.asarray(col, np.float32).T).reshape(w.shape)
    db = np.sum(g_r, axis=1).reshape(-1, 1)
    dcol = (w.reshape(cout, -1).T @ g_r).reshape(c, kh, kw, n, oh, ow)
    dxp = np.zeros((n, c, h + 2 * ph, wd + 2 * pw), np.float32)
    for i in range(kh):
        for j in range(kw):
            dxp[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw] += dcol[:, i, j].transpose(1, 0, 2, 3)
    return dw, db, np.ascontiguousarray(dxp[:, :, ph:ph + h, pw:pw + wd])


def adamw_step(p, g, m, v, t, lr, b1=0.9, b2=0.999, eps=1e-8, wd=0.0, decay=True):
    """One ``AdamW.step`` on one tensor (novann/optim/adamw.py:41-65), NumPy fp32 arithmetic
    with Python-float scalars exactly as the reference writes it.  Returns (p, m, v)."""
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * (g ** 2)
    m_hat = m / (1 - b1 ** t)
    v_hat = v / (1 - b2 ** t)
    p = p - lr * m_hat / (np.sqrt(v_hat) + eps)
    if wd > 0 and decay:
        p = p - lr * wd * p
    return p.astype(np.float32), m.astype(np.float32), v.astype(np.float32)


# ----------------------------------------------------------------------------
# BatchNorm, pooling, Dropout and the CNN step of the reference's main.py
# ----------------------------------------------------------------------------
def _bn_axes(x):
    if x.ndim == 4:
        return (0, 2, 3), (1, -1, 1, 1)
    if x.ndim == 3:
        return (0, 2), (1, -1, 1)
    if x.ndim == 2:
        return (0,), (1, -1)
    raise ValueError(f"BatchNorm expects 2D, 3D or 4D input, got {x.ndim}D")


def batchnorm_fwd(x, gamma, beta, running_mean, running_var, momentum=0.1, eps=1e-5, training=True):
    """``BatchNorm2d.forward`` (novann/layers/batchnorm/batchnorm2d.py:57-102) and
    ``BatchNorm1d.forward`` (batchnorm1d.py:96-141).  gamma / beta / running statistics are
    float64 vectors of length C (the reference creates them with np.ones / np.zeros), x is
    fp32.  Returns (out float64, new_running_mean, new_running_var, cache); the cache holds
    what backward needs.  The float64 output is what the reference returns; its consumers
    narrow it with astype(float32)."""
    x = np.asarray(x, np.float32)
    axes, shp = _bn_axes(x)
    ga, be = np.asarray(gamma, np.float64).reshape(shp), np.asarray(beta, np.float64).reshape(shp)
    rm, rv = np.asarray(running_mean, np.float64).reshape(shp), np.asarray(running_var, np.float64).reshape(shp)
    m = x.size // x.shape[1]
    if not training:
        x_hat = (x - rm) / np.sqrt(rv + eps)
        return ga * x_hat + be, rm.ravel(), rv.ravel(), None
    mu = np.mean(x, axis=axes, keepdims=True)
    var = np.var(x, axis=axes, keepdims=True)
    if m > 1:
        var = var * (m / (m - 1))
    x_mu = x - mu
    x_hat = x_mu / np.sqrt(var + eps)
    out = ga * x_hat + be
    new_rm = (1 - momentum) * rm + momentum * mu
    new_rv = (1 - momentum) * rv + momentum * var
    cache = dict(x_hat=x_hat, x_mu=x_mu, var=var, mu=mu, m=m, axes=axes, gamma=ga, eps=eps)
    return out, new_rm.ravel(), new_rv.ravel(), cache


def batchnorm_bwd(grad, cache):
    """``BatchNorm2d.backward`` (batchnorm2d.py:104-146).  Returns (dx, dgamma, dbeta), the
    parameter gradients as flat length-C vectors."""
    x_hat, x_mu, var, m, axes, ga, eps = (cache[k] for k in ("x_hat", "x_mu", "var", "m", "axes", "gamma", "eps"))
    dgamma = np.sum(grad * x_hat, axis=axes, keepdims=True)
    dbeta = np.sum(grad, axis=axes, keepdims=True)
    dx_hat = grad * ga
    inv_std = (var + eps) ** (-0.5)
    inv_std3 = (var + eps) ** (-1.5)
    dvar = np.sum(dx_hat * x_mu * (-0.5) * inv_std3, axis=axes, keepdims=True)
    dmu = np.sum(dx_hat * (-inv_std), axis=axes, keepdims=True) + \
        dvar * np.sum(-2.0 * x_mu, axis=axes, keepdims=True) / m
    dx = dx_hat * inv_std + dvar * (2.0 * x_mu) / m + dmu / m
    return dx, dgamma.ravel(), dbeta.ravel()


def _pool_windows(x, kh, kw, sh, sw, ph, pw, padding_mode):
    """(N, C, OH, OW, KH, KW) windows of the padded input, gathered explicitly."""
    if padding_mode not in _PAD_MODES:
        raise ValueError(f"padding_mode Only accept {tuple(_PAD_MODES)} not '{padding_mode}'")
    n, c, h, w = x.shape
    xp = np.pad(x, ((0, 0), (0, 0), (ph, ph), (pw, pw)), mode=_PAD_MODES[padding_mode])
    oh, ow = conv2d_out_size(h, w, kh, kw, sh, sw, ph, pw)
    win = np.empty((n, c, oh, ow, kh, kw), x.dtype)
    for i in range(kh):
        for j in range(kw):
            win[..., i, j] = xp[:, :, i:i + sh * oh:sh, j:j + sw * ow:sw]
    return win, xp.shape


def maxpool2d_fwd(x, kernel, stride=None, padding=(0, 0), padding_mode="zeros"):
    """``F.max_pool2d`` (novann/functional.py:450-536).  Returns (out, windows, padded_shape)."""
    x = np.asarray(x, np.float32)
    stride = kernel if stride is None else stride
    win, pshape = _pool_windows(x, kernel[0], kernel[1], stride[0], stride[1], padding[0], padding[1],
                                padding_mode)
    return win.max(axis=(4, 5)), win, pshape


def maxpool2d_bwd(grad, windows, padded_shape, x_shape, kernel, stride, padding):
    """``MaxPool2d.backward`` (novann/layers/pooling/maxpool/maxpool2d.py): ties share the
    gradient evenly; windows are added back in (oh, ow) order; padding is cropped."""
    grad = np.asarray(grad, np.float32)
    kh, kw = kernel
    sh, sw = stride
    ph, pw = padding
    mx = windows.max(axis=(4, 5), keepdims=True)
    mask = (windows == mx).astype(np.float32)
    counts = mask.sum(axis=(4, 5), keepdims=True)
    counts[counts == 0] = 1.0
    gw = mask * (grad[..., None, None] / counts)
    dxp = np.zeros(padded_shape, np.float32)
    for i in range(grad.shape[2]):
        for j in range(grad.shape[3]):
            dxp[:, :, i * sh:i * sh + kh, j * sw:j * sw + kw] += gw[:, :, i, j]
    h, w = x_shape[2], x_shape[3]
    return np.ascontiguousarray(dxp[:, :, ph:ph + h, pw:pw + w])


def gap2d_fwd(x):
    """``F.avg_pool2d`` (novann/functional.py:550-559) on fp32 input."""
    return np.mean(np.asarray(x, np.float32), axis=(2, 3), keepdims=True)


def gap2d_bwd(grad, x_shape):
    """``GlobalAvgPool2d.backward``: ones * (grad * (1 / (H*W)))."""
    grad = np.asarray(grad, np.float32)
    factor = 1.0 / (x_shape[2] * x_shape[3])
    return np.ones(x_shape, np.float32) * (grad * factor)


def dropout(x, mask, p):
    """``Dropout.forward`` / ``backward`` (novann/layers/regularization/dropout.py:40-70) with
    the mask given: (x * mask) / (1 - p)."""
    return (x * mask) / (1.0 - p)


def cnn_main_spec():
    """The layer list of the reference's main.py (main.py:24-46) as (kind, args) tuples."""
    return [
        ("conv", dict(cin=1, cout=16, k=3, s=1, p=1)), ("bn2d", dict(c=16)), ("relu", {}),
        ("conv", dict(cin=16, cout=32, k=3, s=2, p=1)), ("bn2d", dict(c=32)), ("relu", {}),
        ("maxpool", dict(k=2, s=2)),
        ("conv", dict(cin=32, cout=64, k=3, s=1, p=1)), ("bn2d", dict(c=64)), ("relu", {}),
        ("gap", {}), ("flatten", {}),
        ("linear", dict(fin=64, fout=32, bias=False)), ("bn1d", dict(c=32)), ("relu", {}),
        ("dropout", dict(p=0.5)),
        ("linear", dict(fin=32, fout=10, bias=True)),
    ]


def cnn_train_step(spec, params, state, x, labels, drop_masks, opt, t):
    """One training step of a Sequential CNN given as ``spec`` (see ``cnn_main_spec``):
    zero_grad -> forward -> CrossEntropyLoss -> backward -> AdamW.step, written layer by layer
    with the functions above (novann/model/nn.py:185-223 drives the same loop).

    params: list in ``Sequential.parameters()`` order (conv weight; bn gamma, beta (float64);
    linear weight [, bias (1, N)]).  state: {"running": [(mean, var) per BatchNorm], "m": [...],
    "v": [...]} AdamW moments per parameter.  drop_masks: one 0/1 array per Dropout layer.
    opt: dict(lr, b1, b2, eps, wd).  Returns dict(logits, loss, grads, params, state)."""
    pi = bi = di = 0
    tape = []
    h = np.asarray(x, np.float32)
    for kind, a in spec:
        if kind == "conv":
            w = params[pi]
            h32 = h.astype(np.float32, copy=False)
            col, _, _ = im2col(h32, a["k"], a["k"], a["s"], a["s"], a["p"], a["p"])
            out = conv2d_fwd_f32(h32, w, None, (a["s"], a["s"]), (a["p"], a["p"]))
            tape.append((kind, a, pi, dict(col=col, x_shape=h32.shape)))
            pi += 1
            h = out
        elif kind in ("bn2d", "bn1d"):
            ga, be = params[pi], params[pi + 1]
            rm, rv = state["running"][bi]
            out, nrm, nrv, cache = batchnorm_fwd(h.astype(np.float32, copy=False), ga.ravel(), be.ravel(),
                                                 rm, rv, training=True)
            state["running"][bi] = (nrm, nrv)
            tape.append((kind, a, pi, cache))
            pi += 2
            bi += 1
            h = out
        elif kind == "relu":
            mask = (h > 0).astype(h.dtype)
            tape.append((kind, a, None, mask))
            h = h * mask
        elif kind == "maxpool":
            h32 = h.astype(np.float32, copy=False)
            out, win, pshape = maxpool2d_fwd(h32, (a["k"], a["k"]), (a["s"], a["s"]))
            tape.append((kind, a, None, dict(win=win, pshape=pshape, x_shape=h32.shape)))
            h = out
        elif kind == "gap":
            h32 = h.astype(np.float32, copy=False)
            tape.append((kind, a, None, h32.shape))
            h = gap2d_fwd(h32)
        elif kind == "flatten":
            tape.append((kind, a, None, h.shape))
            h = h.reshape(h.shape[0], -1)
        elif kind == "linear":
            w = params[pi]
            b = params[pi + 1] if a["bias"] else None
            h32 = h.astype(np.float32, copy=False)
            tape.append((kind, a, pi, h32))
            h = h32 @ w.T
            if b is not None:
                h = h + b
            pi += 2 if a["bias"] else 1
        elif kind == "dropout":
            mask = drop_masks[di].astype(h.dtype)
            di += 1
            tape.append((kind, a, None, mask))
            h = dropout(h, mask, a["p"])
        else:
            raise ValueError(kind)
    logits = h
    loss, g = softmax_ce(logits, labels)
    grads = [None] * len(params)
    for kind, a, p0, c in reversed(tape):
        if kind == "conv":
            dw, _, dx = conv2d_bwd_f32(g.astype(np.float32, copy=False), c["col"], params[p0], c["x_shape"],
                                       (a["s"], a["s"]), (a["p"], a["p"]))
            grads[p0] = dw
            g = dx
        elif kind in ("bn2d", "bn1d"):
            dx, dga, dbe = batchnorm_bwd(g, c)
            grads[p0], grads[p0 + 1] = dga.reshape(params[p0].shape), dbe.reshape(params[p0 + 1].shape)
            g = dx
        elif kind == "relu":
            g = g * c
        elif kind == "maxpool":
            g = maxpool2d_bwd(g.astype(np.float32, copy=False), c["win"], c["pshape"], c["x_shape"],
                              (a["k"], a["k"]), (a["s"], a["s"]), (0, 0))
        elif kind == "gap":
            g = gap2d_bwd(g, c)
        elif kind == "flatten":
            g = g.reshape(c)
        elif kind == "linear":
            g32 = g.astype(np.float32, copy=False)
            grads[p0] = g32.T @ c
            if a["bias"]:
                grads[p0 + 1] = np.sum(g32, axis=0, keepdims=True)
            g = g32 @ params[p0]
        elif kind == "dropout":
            g = dropout(g, c, a["p"])
    new = []
    for i, (p, gr) in enumerate(zip(params, grads)):
        is_bn = p.dtype == np.float64
        m = opt["b1"] * state["m"][i] + (1 - opt["b1"]) * gr
        v = opt["b2"] * state["v"][i] + (1 - opt["b2"]) * (gr ** 2)
        m_hat = m / (1 - opt["b1"] ** t)
        v_hat = v / (1 - opt["b2"] ** t)
        q = p - opt["lr"] * m_hat / (np.sqrt(v_hat) + opt["eps"])
        if opt["wd"] > 0 and not is_bn:
            q = q - opt["lr"] * opt["wd"] * q
        state["m"][i], state["v"][i] = m.astype(p.dtype), v.astype(p.dtype)
        new.append(q.astype(p.dtype))
    return dict(logits=logits, loss=loss, grads=grads, params=new, state=state)
