"""The CUDA casts and quantisers against the ``ml_dtypes`` package directly.

NovaNN holds no bf16 / FP8 / FP4 code, so nothing of the reference can pin these formats; the
written rules are pinned to an independent third-party implementation instead.  The CPU suite
compares the oracle with ``ml_dtypes``; here the device output itself is compared, so the chain
kernel == oracle == ml_dtypes is closed on the kernel's side too.  Saturation is the written
rule's (clamp to the largest finite value first), which ``ml_dtypes`` does not do by itself.
"""
import numpy as np
import pytest

from novann_b200 import quant, workloads
from novann_b200.device import DeviceBuffer

pytestmark = pytest.mark.gpu
ml_dtypes = pytest.importorskip("ml_dtypes")


def _values(n=1 << 24, seed=0):
    """2^24 seeded values: the cast-sweep distribution, magnitudes spread over fp32's range, raw
    bit patterns, and the 4096-element edge block (NaN payloads, infinities, ties, subnormals)."""
    rng = np.random.default_rng(seed)
    q = n // 4
    a = workloads.cast_input(q, seed=seed, edge=False)
    b = (rng.standard_normal(q) * 10.0 ** rng.integers(-12, 6, q)).astype(np.float32)
    c = rng.integers(0, 1 << 32, q, dtype=np.uint64).astype(np.uint32).view(np.float32)
    d = (rng.standard_normal(n - 3 * q) * 3).astype(np.float32)
    x = np.concatenate([a, b, c, d])
    x[-4096:] = workloads.edge_block_f32()
    return x


def test_bf16_cast_equals_ml_dtypes(gpu):
    x = _values()
    got = quant.cast(x, "bf16", device=gpu)
    with np.errstate(all="ignore"):
        want = x.astype(ml_dtypes.bfloat16).view(np.uint16)
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, (hex(int(x.view(np.uint32)[bad[0]])), hex(int(got[bad[0]])), hex(int(want[bad[0]])))
    back = quant.cast(got, "f32", src_dtype="bf16", device=gpu)
    assert np.array_equal(back.view(np.uint32), got.view(ml_dtypes.bfloat16).astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("fmt,mlt,fmax", [("e4m3", "float8_e4m3fn", 448.0), ("e5m2", "float8_e5m2", 57344.0)])
def test_fp8_quantize_equals_ml_dtypes(gpu, fmt, mlt, fmax):
    """nvq_quantize_fp8 at inverse scale 1 and at a non-trivial scale: codes = ml_dtypes' cast of
    the clamped product; nvq_dequantize_fp8: every code x scale."""
    mt = getattr(ml_dtypes, mlt)
    x = _values(seed=1)
    d = DeviceBuffer.from_numpy(x, gpu)
    q = DeviceBuffer(x.size, gpu)
    for inv in (1.0, 0.3712):
        quant.quantize_fp8_device(q, d, x.size, fmt, inv)
        got = q.to_numpy(np.uint8, x.shape)
        with np.errstate(all="ignore"):
            y = x * np.float32(inv)
            want = np.clip(y, -fmax, fmax).astype(mt).view(np.uint8)
        nan = np.isnan(y)
        assert np.array_equal(got[~nan], want[~nan]), (fmt, inv)
        # NaN lanes: the sign bit of the input and the format's NaN code
        assert np.array_equal(got[nan] & 0x7F, np.full(nan.sum(), 0x7F if fmt == "e4m3" else 0x7E, np.uint8))
    codes = np.tile(np.arange(256, dtype=np.uint8), 64)
    out = quant.dequantize_fp8(codes, 0.5, fmt, gpu)
    want = codes.view(mt).astype(np.float32) * np.float32(0.5)
    fin = ~np.isnan(want)
    assert np.array_equal(out[fin].view(np.uint32), want[fin].view(np.uint32))
    assert np.all(np.isnan(out[~fin]))


def test_fp8_per_tensor_equals_ml_dtypes(gpu):
    """The whole per-tensor call (amax, scales, codes) on the FP8 config's distribution."""
    x = workloads.fp8_input(1024, 4096, seed=2)
    for fmt, mt, fmax in (("e4m3", ml_dtypes.float8_e4m3fn, 448.0), ("e5m2", ml_dtypes.float8_e5m2, 57344.0)):
        codes, scale, inv = quant.quantize_fp8(x, fmt, gpu)
        amax = np.max(np.abs(x))
        assert scale == np.float32(amax / np.float32(fmax)) and inv == np.float32(np.float32(fmax) / amax)
        want = np.clip(x * inv, -fmax, fmax).astype(mt).view(np.uint8)
        assert np.array_equal(codes, want)


def test_fp4_block32_equals_ml_dtypes(gpu):
    """nvq_quantize_fp4_b32: block scales amax / 6, codes = ml_dtypes' float4_e2m1fn cast of the
    clamped scaled values, low nibble first; the dequantiser against ml_dtypes' decode."""
    rng = np.random.default_rng(3)
    rows, cols = 2048, 4096
    xb = workloads.fp4_input_bits(rows, cols, seed=3)
    xb[5, 64:96] = 0                                        # an all-zero block
    xb[6, 0:32] = xb[6, 0] & 0x7FFF                         # a constant block
    xb[7, :] = (rng.integers(0, 0x7F80, cols, dtype=np.uint64)).astype(np.uint16)   # any finite bf16
    packed, scales = quant.quantize_fp4_b32(xb, gpu)
    x = (xb.astype(np.uint32) << 16).view(np.float32).reshape(rows, cols // 32, 32)
    amax = np.max(np.abs(x), axis=2)
    assert np.array_equal(scales.view(np.uint32), (amax / np.float32(6)).astype(np.float32).view(np.uint32))
    with np.errstate(all="ignore"):
        inv = np.where(amax > 0, np.float32(6) / amax, np.float32(0)).astype(np.float32)
        y = (x * inv[:, :, None]).astype(np.float32)
    codes = np.clip(y, -6, 6).astype(ml_dtypes.float4_e2m1fn).view(np.uint8).reshape(rows, cols) & 0xF
    want = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(packed, want)
    back = quant.dequantize_fp4_b32(packed, scales, gpu)
    vals = codes.astype(np.uint8).view(ml_dtypes.float4_e2m1fn).astype(np.float32).reshape(rows, cols // 32, 32)
    wantb = (vals * scales[:, :, None]).astype(np.float32).astype(ml_dtypes.bfloat16).view(np.uint16)
    assert np.array_equal(back, wantb.reshape(rows, cols))
