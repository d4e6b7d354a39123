"""Bit-exact parity of the FP4 E2M1 block-32 kernels with the oracle."""
import numpy as np
import pytest

from novann_b200 import _lib, quant, workloads
from novann_b200.device import DeviceBuffer
from oracle import oracle_np as o

pytestmark = pytest.mark.gpu


def _check(gpu, oracle_c, xb):
    p, s = quant.quantize_fp4_b32(xb, gpu)
    with np.errstate(all="ignore"):
        pw, sw = oracle_c.quantize_fp4_b32(xb)
    bad = np.argwhere(s.view(np.uint32) != sw.view(np.uint32))
    assert bad.size == 0, (bad[:4], s[tuple(bad[0])], sw[tuple(bad[0])])
    bad = np.argwhere(p != pw)
    assert bad.size == 0, (bad[:4], p[tuple(bad[0])], pw[tuple(bad[0])])
    back = quant.dequantize_fp4_b32(p, s, gpu)
    with np.errstate(all="ignore"):
        want = oracle_c.dequantize_fp4_b32(pw, sw)
    bad = np.argwhere(back != want)
    assert bad.size == 0, (bad[:4], back[tuple(bad[0])], want[tuple(bad[0])])
    return p, s, back


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 64), (7, 96), (128, 1024), (1000, 4096)])
def test_shapes(gpu, oracle_c, rows, cols):
    _check(gpu, oracle_c, workloads.fp4_input_bits(rows, cols, seed=rows))


def test_special_blocks(gpu, oracle_c):
    xb = workloads.fp4_input_bits(64, 512, seed=5)
    rng = np.random.default_rng(9)
    xb[0, :32] = 0
    xb[1, :] = rng.integers(0, 1 << 16, 512)
    xb[2, :64] = rng.integers(0, 0x0080, 64)
    xb[3, :32] = 0x7F80
    xb[4, :32] = 0x7FC0
    xb[5, 5] = 0xFF80
    xb[6, 40] = 0xFFC1
    xb[7, :32] = 0x8000
    _check(gpu, oracle_c, xb)


def test_every_bf16_pattern_in_every_lane_position(gpu, oracle_c):
    """All 65536 bf16 patterns, arranged so each block mixes magnitudes, in four
    different shuffles (so patterns meet different block maxima)."""
    base = np.arange(1 << 16, dtype=np.uint16)
    for seed in range(4):
        rng = np.random.default_rng(seed)
        xb = rng.permutation(base).reshape(256, 256)
        _check(gpu, oracle_c, xb)
    # and sorted order: blocks of near-equal values, incl. all-NaN / all-subnormal blocks
    _check(gpu, oracle_c, base.reshape(256, 256))


def test_all_codes_times_assorted_scales(gpu, oracle_c):
    """Dequantise every byte value against scales including 0, subnormal, huge, inf, NaN."""
    scales = np.array([0.0, 1.0, 0.33, 1e-40, 3e38, np.inf, -2.5, np.nan, 2 ** -126, 1.7e-3],
                      np.float32)
    packed = np.tile(np.arange(256, dtype=np.uint8).reshape(16, 16), (scales.size, 1))
    packed = packed.reshape(scales.size, 256)       # each row: 16 blocks of 16 bytes
    sc = np.repeat(scales[:, None], 16, axis=1)
    got = quant.dequantize_fp4_b32(packed, sc, gpu)
    with np.errstate(all="ignore"):
        want = oracle_c.dequantize_fp4_b32(packed, sc)
        assert np.array_equal(want, o.dequantize_fp4_b32(packed, sc))
    assert np.array_equal(got, want)


def test_config_tensor_full_size(gpu, oracle_c):
    """bf16 [8192, 8192] N(0,1), the FP4 config: packed (8192,4096) + scales (8192,256)."""
    xb = workloads.fp4_input_bits(8192, 8192, seed=0)
    p, s, back = _check(gpu, oracle_c, xb)
    assert p.shape == (8192, 4096) and s.shape == (8192, 256)
    # requantising the dequantised tensor keeps every code whose value is representable:
    # the block maximum maps to +-6 again, so scales are reproduced exactly
    p2, s2 = quant.quantize_fp4_b32(back, gpu)
    with np.errstate(all="ignore"):
        pw, sw = oracle_c.quantize_fp4_b32(back)
    assert np.array_equal(p2, pw) and np.array_equal(s2.view(np.uint32), sw.view(np.uint32))


def test_rejects_bad_shape(gpu):
    with pytest.raises(_lib.NvqError):
        quant.quantize_fp4_b32(np.zeros((4, 40), np.uint16), gpu)
