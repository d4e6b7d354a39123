"""Bit-exact parity of the CUDA casts (through the C ABI) with the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

from novann_b200 import _lib, quant, workloads
from novann_b200.device import DeviceBuffer, Stream, pinned_empty
from oracle import oracle_np as o

pytestmark = pytest.mark.gpu

PAIRS = [("f32", "bf16"), ("f32", "f16"), ("bf16", "f32"), ("f16", "f32")]
NP = {"f32": np.float32, "f16": np.uint16, "bf16": np.uint16}  # 16-bit data compared as bits


def _oracle(oc, x, src, dst):
    with np.errstate(all="ignore"):
        if (src, dst) == ("f32", "bf16"):
            return oc.f32_to_bf16_bits(x)
        if (src, dst) == ("f32", "f16"):
            return oc.f32_to_f16_bits(x)
        if (src, dst) == ("bf16", "f32"):
            return oc.bf16_bits_to_f32(x)
        return oc.f16_bits_to_f32(x)


def _device_cast(x, src, dst, gpu, src_off=0, dst_off=0):
    n = x.size
    dsize = 4 if dst == "f32" else 2
    d_in = DeviceBuffer(x.nbytes + 64, gpu)
    d_out = DeviceBuffer(n * dsize + 128, gpu)
    d_out.zero()
    d_in.upload(x, offset=src_off)
    quant.cast_device(d_out, dst, d_in, src, n, dst_offset=dst_off, src_offset=src_off)
    out = d_out.download(np.empty(n, NP[dst]), offset=dst_off)
    # nothing may be written past the end
    guard = d_out.download(np.empty(32, np.uint8), offset=dst_off + n * dsize)
    assert not guard.any()
    return out


def _source(src, n, seed=0):
    if src == "f32":
        x = workloads.cast_input(max(n, 4096), seed)[-n:] if n else np.empty(0, np.float32)
        return np.ascontiguousarray(x)
    rng = np.random.default_rng(seed)
    return rng.integers(0, 1 << 16, n, dtype=np.uint64).astype(np.uint16)


@pytest.mark.parametrize("src,dst", PAIRS)
@pytest.mark.parametrize("n", [0, 1, 3, 7, 8, 9, 31, 33, 255, 1000, 4096, (1 << 20) + 7])
def test_cast_sizes(gpu, oracle_c, src, dst, n):
    x = _source(src, n, seed=n)
    got = _device_cast(x, src, dst, gpu)
    want = _oracle(oracle_c, x, src, dst)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("src,dst", PAIRS)
@pytest.mark.parametrize("src_off,dst_off", [(4, 0), (0, 4), (8, 2 * 2), (16, 16)])
def test_cast_misaligned_buffers(gpu, oracle_c, src, dst, src_off, dst_off):
    x = _source(src, 5000, seed=3)
    got = _device_cast(x, src, dst, gpu, src_off=src_off, dst_off=dst_off)
    want = _oracle(oracle_c, x, src, dst)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("src", ["f16", "bf16"])
def test_widen_all_65536_codes(gpu, oracle_c, src):
    h = np.arange(1 << 16, dtype=np.uint16)
    got = _device_cast(h, src, "f32", gpu)
    assert np.array_equal(got.view(np.uint32), _oracle(oracle_c, h, src, "f32").view(np.uint32))
    ref = h.view(np.float16).astype(np.float32) if src == "f16" else None
    if ref is not None:  # NumPy's own widening, the reference primitive
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("n", [1 << 20, 1 << 26])
def test_cast_config_tensors_and_numpy_astype(gpu, oracle_c, n):
    """The cast-sweep tensors (1 Mi and 64 Mi elements): all four directions, and for
    fp16 also against NumPy's astype, which is the reference's own code path."""
    x = workloads.cast_input(n, seed=0)
    for dst in ("bf16", "f16"):
        got = _device_cast(x, "f32", dst, gpu)
        assert np.array_equal(got, _oracle(oracle_c, x, "f32", dst))
        if dst == "f16":
            with np.errstate(all="ignore"):
                assert np.array_equal(got, x.astype(np.float16).view(np.uint16))
        back = _device_cast(got, dst, "f32", gpu)
        assert np.array_equal(back.view(np.uint32), _oracle(oracle_c, got, dst, "f32").view(np.uint32))


@pytest.mark.parametrize("dst", ["bf16", "f16"])
def test_exhaustive_all_fp32_patterns(gpu, oracle_c, dst):
    """Every one of the 2^32 fp32 bit patterns, in 16 chunks of 256 Mi."""
    chunk = 1 << 28
    d_in = DeviceBuffer(chunk * 4, gpu)
    d_out = DeviceBuffer(chunk * 2, gpu)
    got = np.empty(chunk, np.uint16)
    want = np.empty(chunk, np.uint16)
    for c in range(16):
        u = np.arange(c * chunk, (c + 1) * chunk, dtype=np.uint32)
        d_in.upload(u)
        quant.cast_device(d_out, dst, d_in, "f32", chunk)
        d_out.download(got)
        x = u.view(np.float32)
        if dst == "bf16":
            oracle_c.f32_to_bf16_bits(x, out=want)
        else:
            oracle_c.f32_to_f16_bits(x, out=want)
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, (hex(int(u[bad[0]])), hex(int(got[bad[0]])), hex(int(want[bad[0]])))


def test_cast_host_api_multi_chunk(gpu, oracle_c):
    """The host-array call (NumPy in, NumPy out) across several staging chunks, from
    pinned and from pageable memory, plus the float32 -> float32 identity."""
    n = (40 << 20) + 13
    x = pinned_empty(n, np.float32)
    workloads.cast_input(n, seed=4, out=x)
    out = pinned_empty(n, np.uint16)
    got = quant.cast(x, "bf16", out=out)
    assert got is out
    assert np.array_equal(got, oracle_c.f32_to_bf16_bits(x))
    y = np.array(x[: (17 << 20) + 5])  # pageable copy
    h = quant.cast(y, np.float16)
    with np.errstate(all="ignore"):
        assert np.array_equal(h.view(np.uint16), y.astype(np.float16).view(np.uint16))
    back = quant.cast(h, np.float32)
    assert back.dtype == np.float32
    assert np.array_equal(back.view(np.uint32), h.astype(np.float32).view(np.uint32))
    assert quant.cast(y, np.float32) is y
    b32 = quant.cast(got[:1000].copy(), "f32", src_dtype="bf16")
    assert np.array_equal(b32.view(np.uint32), got[:1000].astype(np.uint32) << 16)


def test_cast_rejects_bad_pairs(gpu):
    d = DeviceBuffer(64, gpu)
    st = _lib.lib().nvq_cast(d.at(0), _lib.F16, d.at(0), _lib.BF16, 4, gpu, None)
    assert st == _lib.ERR_INVALID
    st = _lib.lib().nvq_cast(None, _lib.F16, d.at(0), _lib.F32, 4, gpu, None)
    assert st == _lib.ERR_INVALID


def test_full_size_roundtrip_properties(gpu):
    """1 Gi elements (the largest config): properties that need no CPU pass.
    widen(narrow(x)) is idempotent under a second narrow, and narrowing a widened
    16-bit tensor gives the tensor back (every non-NaN 16-bit value is exactly
    representable)."""
    n = 1 << 30
    st = Stream(gpu)
    d16 = DeviceBuffer(n * 2, gpu)
    d32 = DeviceBuffer(n * 4, gpu)
    d16b = DeviceBuffer(n * 2, gpu)
    # fill the 16-bit tensor with all 65536 patterns repeated; NaNs excluded from the check
    pat = np.tile(np.arange(1 << 16, dtype=np.uint16), 1 << 8)  # 16 Mi
    for i in range(0, n, pat.size):
        d16.upload(pat, stream=st, offset=i * 2)
    st.sync()
    for name in ("bf16", "f16"):
        quant.cast_device(d32, "f32", d16, name, n, stream=st)
        quant.cast_device(d16b, name, d32, "f32", n, stream=st)
        st.sync()
        for off in (0, n - pat.size, (n // 2) + 4096):
            a = d16b.download(np.empty(pat.size, np.uint16), offset=off * 2)
            b = d16.download(np.empty(pat.size, np.uint16), offset=off * 2)
            exp = (b >> 7) & 0xFF if name == "bf16" else (b >> 10) & 0x1F
            man = b & (0x7F if name == "bf16" else 0x3FF)
            notnan = ~((exp == (0xFF if name == "bf16" else 0x1F)) & (man != 0))
            assert np.array_equal(a[notnan], b[notnan])


# ---------------------------------------------------------------- float64 <-> float32
# The narrowing NovaNN really performs: its BatchNorm layers emit float64 and the next layer's
# astype(np.float32) narrows it (novann/layers/linear/linear.py:81).  Pinned against
# ndarray.astype itself, the reference's primitive, and against the integer oracle.
def _f64_edge_block() -> np.ndarray:
    bits = [
        0x0000000000000000, 0x0000000000000001, 0x000FFFFFFFFFFFFF, 0x0010000000000000,   # zero, fp64 denormals
        0x3690000000000000, 0x3690000000000001, 0x368FFFFFFFFFFFFF, 0x36A0000000000000,   # half of fp32's least subnormal
        0x36A8000000000000, 0x36B0000000000000, 0x36B8000000000000, 0x380FFFFFFFFFFFFF,   # subnormal ties, below min normal
        0x380FFFFFF0000000, 0x3810000000000000, 0x380FFFFFE0000000,                       # rounds up into the normals
        0x3FF0000010000000, 0x3FF0000030000000, 0x3FF000000FFFFFFF, 0x3FF0000010000001,   # ties at 1 + half ulp
        0x3FF0000020000000, 0x3FF00000EFFFFFFF, 0x3FF00000F0000000,
        0x47EFFFFFE0000000, 0x47EFFFFFEFFFFFFF, 0x47EFFFFFF0000000, 0x47F0000000000000,   # fp32 max / overflow tie
        0x7FEFFFFFFFFFFFFF, 0x7FF0000000000000,                                           # fp64 max, inf
        0x7FF0000000000001, 0x7FF8000000000000, 0x7FF0000020000000, 0x7FF4000000000000,   # NaNs: payload kept >> 29, quieted
        0x7FF0000010000000, 0x7FF7FFFFFFFFFFFF, 0x7FF00000E0000000, 0x7FFFFFFFFFFFFFFF,
    ]
    base = np.array(bits, dtype=np.uint64)
    return np.concatenate([base, base | np.uint64(1 << 63)]).view(np.float64)


def _f64_source(n, seed):
    """Doubles that land all over fp32's range, ties at fp32's half ulp, and the edge block."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n) * 10.0 ** rng.integers(-46, 39, n)
    k = n // 4
    if k:
        f = rng.integers(0, 0x7F800000, k, dtype=np.uint64).astype(np.uint32).view(np.float32).astype(np.float64)
        t = f.view(np.uint64) | np.uint64(1 << 28)                 # exactly half way between two fp32 values
        t += rng.integers(-1, 2, k).astype(np.int64).view(np.uint64)  # ... or one fp64 ulp either side
        x[:k] = t.view(np.float64) * rng.choice([-1.0, 1.0], k)
    e = _f64_edge_block()
    if n >= e.size:
        x[n - e.size:] = e
    return x


def _device_cast_f64(x, src, dst, gpu, src_off=0, dst_off=0):
    n = x.size
    dsize = 8 if dst == "f64" else 4
    d_in = DeviceBuffer(x.nbytes + 64, gpu)
    d_out = DeviceBuffer(n * dsize + 128, gpu)
    d_out.zero()
    d_in.upload(x, offset=src_off)
    quant.cast_device(d_out, dst, d_in, src, n, dst_offset=dst_off, src_offset=src_off)
    out = d_out.download(np.empty(n, np.float64 if dst == "f64" else np.float32), offset=dst_off)
    guard = d_out.download(np.empty(32, np.uint8), offset=dst_off + n * dsize)
    assert not guard.any()
    return out


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 31, 33, 1000, 4099, (1 << 20) + 3])
@pytest.mark.parametrize("offs", [(0, 0), (8, 4), (16, 0), (0, 8), (24, 12)])
def test_f64_to_f32_sizes_and_alignment(gpu, oracle_c, n, offs):
    x = _f64_source(n, seed=n + offs[0])
    got = _device_cast_f64(x, "f64", "f32", gpu, *offs)
    with np.errstate(all="ignore"):
        assert np.array_equal(got.view(np.uint32), x.astype(np.float32).view(np.uint32))
    assert np.array_equal(got.view(np.uint32), o.f64_to_f32_bits(x))
    assert np.array_equal(got.view(np.uint32), oracle_c.f64_to_f32(x).view(np.uint32))


def test_f64_to_f32_2pow26_doubles_against_numpy(gpu, oracle_c):
    """2^26 doubles (512 MiB in): random magnitudes, fp32 half-ulp ties and the edge block,
    bit-compared with ndarray.astype(np.float32)."""
    x = _f64_source(1 << 26, seed=7)
    got = _device_cast_f64(x, "f64", "f32", gpu)
    with np.errstate(all="ignore"):
        want = x.astype(np.float32)
    bad = np.flatnonzero(got.view(np.uint32) != want.view(np.uint32))
    assert bad.size == 0, (hex(int(x.view(np.uint64)[bad[0]])), hex(int(got.view(np.uint32)[bad[0]])))
    assert np.array_equal(oracle_c.f64_to_f32(x).view(np.uint32), want.view(np.uint32))


def test_f64_every_fp32_neighbourhood(gpu):
    """Every fp32 exponent (subnormals included) x the 5 doubles around each of 64 mantissa
    ties per exponent: the rounding decision at every scale."""
    e = np.arange(0, 255, dtype=np.uint32)[:, None] << 23
    m = np.random.default_rng(3).integers(0, 1 << 23, (1, 64), dtype=np.uint64).astype(np.uint32)
    f = (e | m).reshape(-1).view(np.float32).astype(np.float64)
    half = np.spacing(f.astype(np.float32)).astype(np.float64) / 2
    x = np.concatenate([f + half * k for k in (0.0, 0.5, 1.0, 1.5)] +
                       [np.nextafter(f + half, np.inf), np.nextafter(f + half, -np.inf)])
    x = np.concatenate([x, -x])
    got = _device_cast_f64(x, "f64", "f32", gpu)
    with np.errstate(all="ignore"):
        assert np.array_equal(got.view(np.uint32), x.astype(np.float32).view(np.uint32))


@pytest.mark.parametrize("n", [0, 1, 5, 1000, (1 << 20) + 1])
def test_f32_to_f64_exact(gpu, oracle_c, n):
    x = _source("f32", n, seed=n)
    got = _device_cast_f64(x, "f32", "f64", gpu)
    assert np.array_equal(got.view(np.uint64), x.astype(np.float64).view(np.uint64))
    assert np.array_equal(got.view(np.uint64), o.f32_bits_to_f64_bits(x))
    got2 = _device_cast_f64(x, "f32", "f64", gpu, 4, 8)
    assert np.array_equal(got2.view(np.uint64), got.view(np.uint64))


def test_f32_to_f64_all_exponents_and_nans(gpu):
    """Every exponent with 2^15 mantissas, both signs, subnormals and NaN payloads included,
    against ndarray.astype(np.float64)."""
    u = (np.arange(256, dtype=np.uint32)[:, None] << 23) | \
        (np.arange(1 << 15, dtype=np.uint32)[None, :] * np.uint32(257) & np.uint32(0x7FFFFF))
    u = np.concatenate([u.reshape(-1), u.reshape(-1) | np.uint32(0x80000000)])
    got = _device_cast_f64(u.view(np.float32), "f32", "f64", gpu)
    assert np.array_equal(got.view(np.uint64), u.view(np.float32).astype(np.float64).view(np.uint64))


def test_f64_host_api(gpu):
    """quant.cast on host float64 arrays (several staging chunks), and the layer-entry helper."""
    from novann_b200.layers import _as_f32
    x = _f64_source((20 << 20) + 5, seed=11)
    got = quant.cast(x, np.float32)
    with np.errstate(all="ignore"):
        want = x.astype(np.float32)
    assert got.dtype == np.float32 and np.array_equal(got.view(np.uint32), want.view(np.uint32))
    back = quant.cast(got, np.float64)
    assert back.dtype == np.float64
    assert np.array_equal(back.view(np.uint64), got.astype(np.float64).view(np.uint64))
    x2 = x[:1000].reshape(10, 100)
    y = _as_f32(x2, gpu)
    with np.errstate(all="ignore"):
        assert y.shape == (10, 100) and np.array_equal(y.view(np.uint32), x2.astype(np.float32).view(np.uint32))
    f = np.ones((3, 4), np.float32)
    assert _as_f32(f, gpu) is f or np.shares_memory(_as_f32(f, gpu), f)
    with pytest.raises(TypeError):
        _as_f32(np.ones(4, np.int32), gpu)


@pytest.mark.parametrize("src_pinned,dst_pinned", [(False, False), (True, False), (False, True)])
def test_cast_host_api_pageable_arrays_are_staged(gpu, oracle_c, src_pinned, dst_pinned):
    """Plain (pageable) NumPy arrays - what ndarray.astype is handed - go through the library's
    page-locked staging buffers, filled and drained by host threads: several chunks, a ragged
    last chunk, either side pageable; same bits as the page-locked path and as the oracle."""
    n = (16 << 20) * 3 + 12345                       # three full staging chunks and a tail (fp32 side)
    x = pinned_empty(n, np.float32) if src_pinned else np.empty(n, np.float32)
    workloads.cast_input(n, seed=8, out=x)
    out = pinned_empty(n, np.uint16) if dst_pinned else np.empty(n, np.uint16)
    out[:] = 0xFFFF
    got = quant.cast(x, "bf16", out=out, device=gpu)
    assert got is out
    assert np.array_equal(got, oracle_c.f32_to_bf16_bits(x))
    back = quant.cast(got, "f32", src_dtype="bf16", device=gpu)          # pageable result array
    assert np.array_equal(back.view(np.uint32), got.astype(np.uint32) << 16)


def test_cast_host_api_from_two_threads(gpu, oracle_c):
    """Two host threads cast different arrays on one device at once: the calls are serialised
    per device and both results are right."""
    import threading
    xs = [workloads.cast_input((9 << 20) + i, seed=20 + i) for i in range(2)]
    outs = [None, None]

    def work(i):
        outs[i] = quant.cast(xs[i], np.float16, device=gpu)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for x, h in zip(xs, outs):
        with np.errstate(all="ignore"):
            assert np.array_equal(h.view(np.uint16), x.astype(np.float16).view(np.uint16))
