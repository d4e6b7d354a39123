"""Pins the CPU oracle: the NumPy restatement and the C restatement agree with each
other, with NumPy's own ``astype`` (the reference's cast primitive) for fp16, and,
where the package is installed, with ml_dtypes for bf16 / FP8 / FP4."""
import numpy as np
import pytest

from novann_b200 import workloads
from oracle import oracle_np as o


def _patterns():
    """Every value of the upper 19 bits crossed with rounding-critical low bits, the
    edge block and 4 Mi random words."""
    hi = np.arange(1 << 19, dtype=np.uint32) << 13
    lows = np.array([0, 1, 0xFFF, 0x1000, 0x1001, 0x1FFF], dtype=np.uint32)
    rng = np.random.default_rng(7)
    rnd = rng.integers(0, 1 << 32, 1 << 22, dtype=np.uint64).astype(np.uint32)
    return np.concatenate([(hi[:, None] | lows[None, :]).ravel(), rnd,
                           workloads.edge_block_f32().view(np.uint32)]).view(np.float32)


X = _patterns()


def test_f32_to_f16_equals_numpy_astype(oracle_c):
    with np.errstate(all="ignore"):
        want = X.astype(np.float16).view(np.uint16)
    assert np.array_equal(o.f32_to_f16_bits(X), want)
    assert np.array_equal(oracle_c.f32_to_f16_bits(X), want)


def test_f16_to_f32_all_codes_equals_numpy(oracle_c):
    h = np.arange(1 << 16, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32).view(np.uint32)
    assert np.array_equal(o.f16_bits_to_f32(h).view(np.uint32), want)
    assert np.array_equal(oracle_c.f16_bits_to_f32(h).view(np.uint32), want)


def test_known_answers_f16_nan_and_ties():
    # observed NumPy behaviour: payload kept, not quieted, zero payload -> ...01
    cases = {0x7F800001: 0x7C01, 0x7FA00000: 0x7D00, 0xFFC12345: 0xFE09, 0x7F801FFF: 0x7C01,
             0x477FF000: 0x7C00, 0x477FEFFF: 0x7BFF, 0x33000000: 0x0000, 0x33000001: 0x0001}
    u = np.array(list(cases), dtype=np.uint32)
    got = o.f32_to_f16_bits(u.view(np.float32))
    assert [int(g) for g in got] == list(cases.values())
    assert o.f16_bits_to_f32(np.array([0x7C01], np.uint16)).view(np.uint32)[0] == 0x7F802000


def test_bf16_rules(oracle_c):
    got = o.f32_to_bf16_bits(X)
    assert np.array_equal(got, oracle_c.f32_to_bf16_bits(X))
    u = np.array([0x7F7FFFFF, 0x7F800001, 0xFFC12345, 0x3F808000, 0x3F818000], np.uint32)
    assert [int(v) for v in o.f32_to_bf16_bits(u.view(np.float32))] == \
        [0x7F80, 0x7FC0, 0xFFC0, 0x3F80, 0x3F82]
    h = np.arange(1 << 16, dtype=np.uint16)
    assert np.array_equal(o.bf16_bits_to_f32(h).view(np.uint32), h.astype(np.uint32) << 16)
    assert np.array_equal(oracle_c.bf16_bits_to_f32(h).view(np.uint32), h.astype(np.uint32) << 16)


def test_against_ml_dtypes():
    m = pytest.importorskip("ml_dtypes")
    with np.errstate(all="ignore"):
        assert np.array_equal(o.f32_to_bf16_bits(X), X.astype(m.bfloat16).view(np.uint16))
        assert np.array_equal(o.f32_to_e4m3_bits(X),
                              np.clip(X, -448, 448).astype(m.float8_e4m3fn).view(np.uint8))
        assert np.array_equal(o.f32_to_e5m2_bits(X),
                              np.clip(X, -57344, 57344).astype(m.float8_e5m2).view(np.uint8))
        assert np.array_equal(o.f32_to_e2m1_codes(X),
                              np.clip(X, -6, 6).astype(m.float4_e2m1fn).view(np.uint8))
    c = np.arange(256, dtype=np.uint8)
    assert np.array_equal(o.E4M3_TABLE.view(np.uint32),
                          c.view(m.float8_e4m3fn).astype(np.float32).view(np.uint32))
    assert np.array_equal(o.E5M2_TABLE.view(np.uint32),
                          c.view(m.float8_e5m2).astype(np.float32).view(np.uint32))
    assert np.array_equal(o.E2M1_TABLE, np.arange(16, dtype=np.uint8).view(m.float4_e2m1fn)
                          .astype(np.float32))


def test_fp8_known_answers():
    x = np.array([448, 464, 1e9, np.inf, -np.inf, 440, 2 ** -9, 2 ** -10, 2 ** -10 * 1.0001, -0.0],
                 np.float32)
    assert [int(v) for v in o.f32_to_e4m3_bits(x)] == \
        [0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0x7E, 0x01, 0x00, 0x01, 0x80]
    x = np.array([57344, 61440, np.inf, 2 ** -16, 2 ** -17, -(2 ** -17) * 1.01], np.float32)
    assert [int(v) for v in o.f32_to_e5m2_bits(x)] == [0x7B, 0x7B, 0x7B, 0x01, 0x00, 0x81]
    nan = np.array([0x7FC00000, 0xFFC00000], np.uint32).view(np.float32)
    assert [int(v) for v in o.f32_to_e4m3_bits(nan)] == [0x7F, 0xFF]
    assert [int(v) for v in o.f32_to_e5m2_bits(nan)] == [0x7E, 0xFE]


def test_e2m1_ties():
    x = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 100.0, -0.0, -0.25, 0.2500001],
                 np.float32)
    assert [int(v) for v in o.f32_to_e2m1_codes(x)] == [0, 2, 2, 4, 4, 6, 6, 7, 7, 8, 8, 1]


@pytest.mark.parametrize("fmt", ["e4m3", "e5m2"])
def test_fp8_quant_dequant_c_equals_numpy(oracle_c, fmt):
    x = workloads.fp8_input(64, 1024, seed=3)
    x.ravel()[-4096:] = workloads.edge_block_f32()
    amax = o.amax_f32(x)
    assert amax == oracle_c.amax_f32(x)
    fin = x[np.isfinite(x)]
    scale, inv = o.fp8_scales(np.abs(fin).max(), fmt)
    with np.errstate(all="ignore"):
        q = o.quantize_fp8(x, inv, fmt)
    assert np.array_equal(q, oracle_c.quantize_fp8(x, inv, fmt))
    allq = np.arange(256, dtype=np.uint8)
    for s in (scale, np.float32(1.0), np.float32(3e-5), np.float32(1e30)):
        assert np.array_equal(o.dequantize_fp8(allq, s, fmt).view(np.uint32),
                              oracle_c.dequantize_fp8(allq, s, fmt).view(np.uint32))
    # idempotence: quant(dequant(q)) == q for every finite code
    finite = allq[np.isfinite(o._table(fmt)[allq])]
    assert np.array_equal(o.quantize_fp8(o.dequantize_fp8(finite, scale, fmt), inv, fmt), finite)


def test_fp8_scale_rule():
    s, i = o.fp8_scales(np.float32(0.0), "e4m3")
    assert s == 1 and i == 1
    s, i = o.fp8_scales(np.float32(3.5), "e4m3")
    assert s == np.float32(np.float32(3.5) / np.float32(448)) and i == np.float32(448) / np.float32(3.5)


def test_fp4_c_equals_numpy_including_specials(oracle_c):
    xb = workloads.fp4_input_bits(64, 512, seed=5)
    rng = np.random.default_rng(9)
    xb[0, :32] = 0                                   # all-zero block: scale 0, inv 0
    xb[1, :] = rng.integers(0, 1 << 16, 512)         # arbitrary bit patterns: NaN, inf, subnormal
    xb[2, :64] = rng.integers(0, 0x0080, 64)         # bf16 subnormals: reciprocal overflows
    xb[3, :32] = 0x7F80                              # all inf
    xb[4, :32] = 0x7FC0                              # all NaN
    xb[5, 5] = 0xFF80
    with np.errstate(all="ignore"):
        p1, s1 = o.quantize_fp4_b32(xb)
        p2, s2 = oracle_c.quantize_fp4_b32(xb)
        assert np.array_equal(p1, p2)
        assert np.array_equal(s1.view(np.uint32), s2.view(np.uint32))
        assert np.array_equal(o.dequantize_fp4_b32(p1, s1), oracle_c.dequantize_fp4_b32(p1, s1))
    # packing: low nibble first
    one = np.zeros((1, 32), np.uint16)
    one[0, 0] = 0x40C0  # 6.0 -> code 7 at element 0; everything else 0
    p, s = o.quantize_fp4_b32(one)
    assert p[0, 0] == 0x07 and s[0, 0] == np.float32(1.0)
    one[0, 0], one[0, 1] = 0, 0xC0C0  # -6.0 at element 1 -> high nibble 0xF
    p, _ = o.quantize_fp4_b32(one)
    assert p[0, 0] == 0xF0


def test_fp4_roundtrip_error_bound():
    xb = workloads.fp4_input_bits(32, 256, seed=1)
    p, s = o.quantize_fp4_b32(xb)
    back = o.bf16_bits_to_f32(o.dequantize_fp4_b32(p, s))
    x = o.bf16_bits_to_f32(xb)
    amax = np.abs(x.reshape(32, 8, 32)).max(axis=2, keepdims=True)
    # E2M1 spacing is at most 2 (between 4 and 6) in units of amax/6 -> half of it, + bf16 rounding
    assert np.all(np.abs(back.reshape(32, 8, 32) - x.reshape(32, 8, 32)) <= amax * (1 / 6 + 1 / 128))


def test_weight_quant_and_linear_oracle():
    xb, w, b = workloads.linear_inputs(16, 24, 64, seed=2)
    wq, s = o.quantize_weight_per_channel(w, "e4m3")
    assert wq.shape == (24, 64) and s.shape == (24,)
    assert np.all((wq & 0x7F).max(axis=1) == 0x7E)  # every channel uses the full range
    yb, y = o.linear_fwd_qweight(xb, wq, s, b)
    ref = o.bf16_bits_to_f32(xb).astype(np.float64) @ w.T.astype(np.float64) + b
    assert o.max_abs_rel(o.bf16_bits_to_f32(yb), ref) < 5e-2  # FP8 weight error only


def test_two_piece_e4m3_split_of_bf16_activations():
    """The few-rows FP8 kernel carries a bf16 activation v (already divided by its row's power of
    two, so v < 256) as p1 = e4m3(v), p2 = e4m3(16 (v - p1)).  v = p1 + p2 / 16 must hold exactly
    for every bf16 value in [2^-6, 256), and within 2^-14 below that."""
    ml_dtypes = pytest.importorskip("ml_dtypes")
    bits = np.arange(0, 0x8000, dtype=np.uint16)
    v = (bits.astype(np.uint32) << 16).view(np.float32)
    for sign in (1.0, -1.0):
        exact = v[(v >= 2.0 ** -6) & (v < 256)] * np.float32(sign)
        p1 = exact.astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
        p2 = ((exact - p1) * 16).astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
        assert exact.size == 1792 and np.array_equal(p1 + p2 / 16, exact)
        small = v[(v > 0) & (v < 2.0 ** -6)] * np.float32(sign)
        p1 = small.astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
        p2 = ((small - p1) * 16).astype(ml_dtypes.float8_e4m3fn).astype(np.float32)
        assert np.max(np.abs(p1 + p2 / 16 - small)) <= 2.0 ** -14


def _f64_patterns():
    """Doubles across fp32's whole range, ties at fp32's half ulp (and one fp64 ulp either side),
    every fp32 exponent, fp64 specials."""
    rng = np.random.default_rng(5)
    raw = rng.integers(0, 1 << 64, 1 << 21, dtype=np.uint64).view(np.float64)
    spread = rng.standard_normal(1 << 21) * 10.0 ** rng.integers(-46, 39, 1 << 21)
    f = rng.integers(0, 0x7F800000, 1 << 21, dtype=np.uint64).astype(np.uint32).view(np.float32)
    t = f.astype(np.float64).view(np.uint64) | np.uint64(1 << 28)
    ties = np.concatenate([t, t + np.uint64(1), t - np.uint64(1)]).view(np.float64)
    spec = np.array([0, 1, 0x3690000000000000, 0x3690000000000001, 0x36A0000000000000, 0x380FFFFFF0000000,
                     0x47EFFFFFEFFFFFFF, 0x47EFFFFFF0000000, 0x7FF0000000000000, 0x7FF0000000000001,
                     0x7FF8000000000000, 0x7FF0000020000000, 0x7FF7FFFFFFFFFFFF, 0x7FF00000E0000000],
                    np.uint64)
    spec = np.concatenate([spec, spec | np.uint64(1 << 63)]).view(np.float64)
    return np.concatenate([raw, spread, ties, -ties, spec])


def test_f64_to_f32_equals_numpy_astype(oracle_c):
    """float64 -> float32 is the narrowing the reference's layers apply to BatchNorm's float64
    output (novann/layers/linear/linear.py:81): pinned against ndarray.astype itself."""
    d = _f64_patterns()
    with np.errstate(all="ignore"):
        want = d.astype(np.float32).view(np.uint32)
    assert np.array_equal(o.f64_to_f32_bits(d), want)
    assert np.array_equal(oracle_c.f64_to_f32(d).view(np.uint32), want)
    known = {0x7FF0000000000001: 0x7FC00000, 0xFFF0000020000000: 0xFFC00001, 0x7FF4000000000000: 0x7FE00000,
             0x47EFFFFFEFFFFFFF: 0x7F7FFFFF, 0x47EFFFFFF0000000: 0x7F800000, 0x3690000000000000: 0x0,
             0x3690000000000001: 0x1, 0x36A8000000000000: 0x2, 0x380FFFFFFFFFFFFF: 0x00800000}
    got = o.f64_to_f32_bits(np.array(list(known), np.uint64).view(np.float64))
    assert [int(g) for g in got] == list(known.values())


def test_f32_to_f64_equals_numpy_astype(oracle_c):
    want = X.astype(np.float64).view(np.uint64)
    assert np.array_equal(o.f32_bits_to_f64_bits(X), want)
    assert np.array_equal(oracle_c.f32_to_f64(X).view(np.uint64), want)
    sub = np.arange(0, 1 << 23, 97, dtype=np.uint32).view(np.float32)      # fp32 subnormals normalise
    assert np.array_equal(o.f32_bits_to_f64_bits(sub), sub.astype(np.float64).view(np.uint64))
    assert np.array_equal(oracle_c.f32_to_f64(sub).view(np.uint64), sub.astype(np.float64).view(np.uint64))
