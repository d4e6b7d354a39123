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
