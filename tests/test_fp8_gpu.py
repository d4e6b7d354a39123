"""Bit-exact parity of the FP8 per-tensor quantise / dequantise kernels with the oracle."""
import ctypes as C

import numpy as np
import pytest

from novann_b200 import _lib, quant, workloads
from novann_b200.device import DeviceBuffer
from oracle import oracle_np as o

pytestmark = pytest.mark.gpu
FMTS = ["e4m3", "e5m2"]


@pytest.mark.parametrize("n", [0, 1, 5, 15, 16, 17, 1000, (1 << 20) + 3])
def test_amax_sizes_and_nan_ignored(gpu, oracle_c, n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 7).astype(np.float32)
    if n > 4:
        x[n // 2] = np.nan
        x[1] = -123.5
    d = DeviceBuffer.from_numpy(x, gpu) if n else DeviceBuffer(4, gpu)
    out = DeviceBuffer.from_numpy(np.array([777.0], np.float32), gpu)  # must be overwritten
    quant.amax_device(d, n, out)
    got = out.to_numpy(np.float32, (1,))[0]
    assert got.view(np.uint32) == oracle_c.amax_f32(x).view(np.uint32)
    assert got.view(np.uint32) == o.amax_f32(x).view(np.uint32)


@pytest.mark.parametrize("fmt", FMTS)
def test_quantize_config_like_tensor(gpu, oracle_c, fmt):
    """N(0,1)*U[0.1,10] rows (the FP8 config's distribution) with the edge block
    appended: codes, scales and dequantised words all bit-exact; idempotence."""
    x = workloads.fp8_input(2048, 2048, seed=1)
    x.ravel()[-4096:] = workloads.edge_block_f32()
    fin = np.where(np.isfinite(x), x, 0)
    x[~np.isfinite(x) & ~np.isnan(x)] = 0  # keep NaNs, drop infs: amax stays finite
    codes, scale, inv = quant.quantize_fp8(x, fmt, gpu)
    s_ref, i_ref = o.fp8_scales(oracle_c.amax_f32(x), fmt)
    assert scale.view(np.uint32) == s_ref.view(np.uint32)
    assert inv.view(np.uint32) == i_ref.view(np.uint32)
    want = oracle_c.quantize_fp8(x, i_ref, fmt)
    bad = np.flatnonzero(codes.ravel() != want.ravel())
    assert bad.size == 0, (x.ravel()[bad[:4]], codes.ravel()[bad[:4]], want.ravel()[bad[:4]])
    back = quant.dequantize_fp8(codes, scale, fmt, gpu)
    assert np.array_equal(back.view(np.uint32), oracle_c.dequantize_fp8(want, s_ref, fmt).view(np.uint32))
    # quant(dequant(q)) == q wherever q is not a NaN code
    d = DeviceBuffer.from_numpy(back, gpu)
    q2 = DeviceBuffer(back.size, gpu)
    quant.quantize_fp8_device(q2, d, back.size, fmt, inv)
    again = q2.to_numpy(np.uint8, codes.shape)
    ok = ~np.isnan(back)
    assert np.array_equal(again[ok], codes[ok])


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("inv", [1.0, 0.37, 123.4, 3.0e-3])
def test_quantize_special_values_with_infs(gpu, oracle_c, fmt, inv):
    x = np.concatenate([workloads.edge_block_f32(), workloads.cast_input(10007, seed=2, edge=False)])
    d = DeviceBuffer.from_numpy(x, gpu)
    q = DeviceBuffer(x.size, gpu)
    quant.quantize_fp8_device(q, d, x.size, fmt, inv)
    got = q.to_numpy(np.uint8, x.shape)
    want = oracle_c.quantize_fp8(x, inv, fmt)
    bad = np.flatnonzero(got != want)
    assert bad.size == 0, (x.view(np.uint32)[bad[:4]], got[bad[:4]], want[bad[:4]])
    with np.errstate(all="ignore"):
        assert np.array_equal(got, o.quantize_fp8(x, inv, fmt))


@pytest.mark.parametrize("fmt", FMTS)
def test_exhaustive_all_fp32_patterns_scale_one(gpu, oracle_c, fmt):
    chunk = 1 << 28
    d_in = DeviceBuffer(chunk * 4, gpu)
    d_out = DeviceBuffer(chunk, gpu)
    got = np.empty(chunk, np.uint8)
    want = np.empty(chunk, np.uint8)
    for c in range(16):
        u = np.arange(c * chunk, (c + 1) * chunk, dtype=np.uint32)
        d_in.upload(u)
        quant.quantize_fp8_device(d_out, d_in, chunk, fmt, 1.0)
        d_out.download(got)
        oracle_c.quantize_fp8(u.view(np.float32), 1.0, fmt, out=want)
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, (hex(int(u[bad[0]])), hex(int(got[bad[0]])), hex(int(want[bad[0]])))


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("n", [1, 15, 16, 33, 256, 4099])
def test_dequantize_all_codes_sizes_scales(gpu, oracle_c, fmt, n):
    q = np.resize(np.arange(256, dtype=np.uint8), n)
    for scale in (1.0, 0.0123, 7.5e-4, 3.0e30, 1e-38):
        got = quant.dequantize_fp8(q, scale, fmt, gpu)
        want = oracle_c.dequantize_fp8(q, scale, fmt)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), scale


def test_scale_validation(gpu):
    d = DeviceBuffer(256, gpu)
    L = _lib.lib()
    for bad in (0.0, -1.0, float("inf"), float("nan")):
        assert L.nvq_quantize_fp8(d.at(0), d.at(0), 16, _lib.E4M3, C.c_float(bad), gpu, None) == _lib.ERR_INVALID
        assert L.nvq_dequantize_fp8(d.at(0), d.at(0), 16, _lib.E5M2, C.c_float(bad), gpu, None) == _lib.ERR_INVALID
    assert L.nvq_quantize_fp8(d.at(0), d.at(0), 16, _lib.F16, C.c_float(1.0), gpu, None) == _lib.ERR_INVALID


def test_zero_tensor_and_empty_tensor(gpu):
    codes, scale, inv = quant.quantize_fp8(np.zeros((4, 8), np.float32), "e4m3", gpu)
    assert not codes.any() and scale == 1 and inv == 1
    codes, scale, inv = quant.quantize_fp8(np.zeros((0, 8), np.float32), "e5m2", gpu)
    assert codes.shape == (0, 8) and scale == 1 and inv == 1


@pytest.mark.parametrize("fmt", FMTS)
def test_row_sharded_equals_whole_tensor(gpu, oracle_c, fmt):
    """Shards of rows quantised with the host-combined amax give the bytes of the
    one-GPU result (what 2/4/8-GPU runs do; here the shards run on one device)."""
    x = workloads.fp8_input(512, 1024, seed=7)
    whole, scale, inv = quant.quantize_fp8(x, fmt, gpu)
    for g in (2, 4, 8):
        rows = 512 // g
        partial = [quant.amax(x[r * rows:(r + 1) * rows], gpu) for r in range(g)]
        amax = max(partial)
        s2, i2 = quant.fp8_scales(amax, fmt)
        assert s2 == scale and i2 == inv
        a_in = DeviceBuffer.from_numpy(np.array([amax], np.float32), gpu)
        for r in range(g):
            shard = np.ascontiguousarray(x[r * rows:(r + 1) * rows])
            d = DeviceBuffer.from_numpy(shard, gpu)
            q = DeviceBuffer(shard.size, gpu)
            asi = DeviceBuffer(12, gpu)
            quant.quantize_fp8_tensor_device(q, asi, d, shard.size, fmt, amax_in=a_in)
            assert np.array_equal(q.to_numpy(np.uint8, shard.shape), whole[r * rows:(r + 1) * rows])
            assert asi.to_numpy(np.float32, (3,))[2] == inv


def test_full_size_roundtrip_idempotence(gpu):
    """fp32 [16384,16384] (the FP8 config size), generated on the host in pieces;
    quant -> dequant -> quant reproduces the codes, and a checksum of a sample of
    rows matches the oracle."""
    rows, cols = 16384, 16384
    n = rows * cols
    d = DeviceBuffer(n * 4, gpu)
    piece = 1024
    keep = {}
    for r in range(0, rows, piece):
        blk = workloads.fp8_input(piece, cols, seed=100 + r)
        d.upload(blk, offset=r * cols * 4)
        if r in (0, 8192, rows - piece):
            keep[r] = blk
    host_amax = np.float32(0)
    q = DeviceBuffer(n, gpu)
    asi = DeviceBuffer(12, gpu)
    quant.quantize_fp8_tensor_device(q, asi, d, n, "e4m3")
    amax, scale, inv = asi.to_numpy(np.float32, (3,))
    assert scale == np.float32(amax / np.float32(448)) and inv == np.float32(np.float32(448) / amax)
    for r, blk in keep.items():
        got = q.download(np.empty((piece, cols), np.uint8), offset=r * cols)
        assert np.array_equal(got, o.quantize_fp8(blk, inv, "e4m3"))
    quant.dequantize_fp8_device(d, q, n, "e4m3", scale)
    q2 = DeviceBuffer(n, gpu)
    quant.quantize_fp8_device(q2, d, n, "e4m3", inv)
    for off in (0, n // 2, n - (1 << 24)):
        a = q.download(np.empty(1 << 24, np.uint8), offset=off)
        b = q2.download(np.empty(1 << 24, np.uint8), offset=off)
        assert np.array_equal(a, b)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("inv", [0.37, 37.5])
def test_every_pattern_of_two_chunks_with_scaling(gpu, oracle_c, fmt, inv):
    """All fp32 patterns in [0x38000000, 0x48000000) (2^-15 .. 2^17, where the products land on
    both formats' subnormal, normal and saturating ranges) times a non-trivial scale, positive
    and negative."""
    chunk = 1 << 28
    d_in = DeviceBuffer(chunk * 4, gpu)
    d_out = DeviceBuffer(chunk, gpu)
    got = np.empty(chunk, np.uint8)
    want = np.empty(chunk, np.uint8)
    for start in (0x38000000, 0xB8000000):
        u = np.arange(start, start + chunk, dtype=np.uint32)
        d_in.upload(u)
        quant.quantize_fp8_device(d_out, d_in, chunk, fmt, inv)
        d_out.download(got)
        oracle_c.quantize_fp8(u.view(np.float32), inv, fmt, out=want)
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, (hex(int(u[bad[0]])), hex(int(got[bad[0]])), hex(int(want[bad[0]])))
