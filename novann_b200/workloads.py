"""Seeded synthetic inputs of the benchmark configurations (no dataset involved).

All generators use ``numpy.random.Generator(PCG64(seed))`` so that the CPU oracle and
the device see identical bits.
"""
from __future__ import annotations

import numpy as np


def edge_block_f32() -> np.ndarray:
    """4096 fp32 values that hit every special path of the narrowing casts: signed
    zeros, fp32 / fp16 / bf16 subnormals, round-to-even ties, the fp16 overflow
    threshold (65504 / 65520), FP8 / FP4 saturation points, fp32 max, infinities and
    NaNs with assorted payloads."""
    bits = [
        0x00000000, 0x80000000, 0x00000001, 0x80000001, 0x007FFFFF, 0x00800000,  # zeros, denormals
        0x33000000, 0x33000001, 0x32FFFFFF, 0x33800000, 0x33C00000, 0x337FFFFF,  # fp16 underflow ties
        0x387FC000, 0x387FE000, 0x38800000, 0x387FFFFF, 0x38000000,              # fp16 subnormal edge
        0x477FE000, 0x477FEFFF, 0x477FF000, 0x477FFFFF, 0x47800000,              # 65504 / 65520 / 65536
        0x7F7FFFFF, 0xFF7FFFFF, 0x7F7F8000, 0x7F7F7FFF,                          # fp32 max, bf16 overflow
        0x7F800000, 0xFF800000,                                                  # inf
        0x7F800001, 0x7FA00000, 0xFFC12345, 0x7F801FFF, 0x7FC00000, 0xFFC00000,  # NaNs
        0x7FFFFFFF, 0xFFFFFFFF, 0x7F802000, 0xFF800001,
        0x43E00000, 0x43E80000, 0x43DFFFFF, 0x43F00000, 0x43D80000, 0x43D00000,  # 448 region (E4M3)
        0x47600000, 0x47700000, 0x475FFFFF, 0x47500000,                          # 57344 region (E5M2)
        0x3B000000, 0x3A800000, 0x3AFFFFFF, 0x3B000001, 0x3C800000,              # E4M3 subnormals
        0x37800000, 0x37000000, 0x37000001, 0x36FFFFFF,                          # E5M2 subnormals
        0x3E800000, 0x3F400000, 0x3FA00000, 0x3FE00000, 0x40200000, 0x40600000,  # E2M1 ties
        0x40A00000, 0x40C00000, 0x40E00000, 0x3E7FFFFF, 0x3E800001,
        0x3F800000, 0x3F801000, 0x3F803000, 0x3F802FFF, 0x3F803001,              # fp16 mantissa ties
        0x3F808000, 0x3F818000, 0x3F807FFF, 0x3F808001,                          # bf16 mantissa ties
    ]
    base = np.array(bits, dtype=np.uint32)
    neg = base ^ np.uint32(0x80000000)
    rng = np.random.default_rng(12345)
    rest = rng.integers(0, 1 << 32, 4096 - 2 * base.size, dtype=np.uint64).astype(np.uint32)
    return np.concatenate([base, neg, rest]).view(np.float32)


def cast_input(n: int, seed: int = 0, edge: bool = True, out: np.ndarray | None = None) -> np.ndarray:
    """Cast-sweep tensor: N(0,1) with 1 % of the entries replaced by draws from
    N(0, sigma=100) (variance 1e4), generated in 16 Mi-element pieces, with the
    4096-element edge block overwriting the tail when ``edge`` is set."""
    x = np.empty(n, np.float32) if out is None else out
    rng = np.random.default_rng(seed)
    step = 1 << 24
    for i in range(0, n, step):
        m = min(step, n - i)
        v = rng.standard_normal(m, dtype=np.float32)
        mask = rng.random(m, dtype=np.float32) < 0.01
        k = int(mask.sum())
        v[mask] = rng.standard_normal(k, dtype=np.float32) * np.float32(100.0)
        x[i:i + m] = v
    if edge and n >= 4096:
        x[n - 4096:] = edge_block_f32()
    return x


def fp8_input(rows: int, cols: int, seed: int = 0) -> np.ndarray:
    """FP8 config tensor: N(0,1)[rows, cols] * U[0.1, 10][rows, 1], fp32."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    x *= rng.uniform(0.1, 10.0, (rows, 1)).astype(np.float32)
    return x


def fp4_input_bits(rows: int, cols: int, seed: int = 0) -> np.ndarray:
    """FP4 config tensor: bf16_rne(N(0,1)) as uint16 bit patterns (no NaN occurs, so
    plain integer RNE is the full rule here)."""
    rng = np.random.default_rng(seed)
    u = rng.standard_normal((rows, cols), dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def linear_inputs(m: int, n: int, k: int, seed: int = 0):
    """FP8-weight Linear config: X bf16 bits (m,k) from N(0,1); W fp32 (n,k) from
    N(0, sigma=0.02); bias fp32 (n,) from N(0, sigma=0.01)."""
    rng = np.random.default_rng(seed)
    u = rng.standard_normal((m, k), dtype=np.float32).view(np.uint32)
    x_bits = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    b = rng.standard_normal(n, dtype=np.float32) * np.float32(0.01)
    return x_bits, w, b


def mlp_inputs(batch: int = 128, dims=(784, 256, 128, 10), seed: int = 0):
    """MLP train-step config: X ~ U[0,1) fp32 (batch, dims[0]); labels uniform in
    [0, dims[-1]); weights N(0, 2/fan_in) (the Kaiming-normal-ReLU law the reference's
    Sequential applies, novann/model/nn.py:85-143), biases zero (1, out)."""
    rng = np.random.default_rng(seed)
    x = rng.random((batch, dims[0]), dtype=np.float32)
    y = rng.integers(0, dims[-1], batch).astype(np.int32)
    params = []
    for fi, fo in zip(dims[:-1], dims[1:]):
        params.append((rng.standard_normal((fo, fi), dtype=np.float32)
                       * np.float32(np.sqrt(2.0 / fi))).astype(np.float32))
        params.append(np.zeros((1, fo), np.float32))
    return x, y, params


def cnn_inputs(batch: int = 128, steps: int = 1, seed: int = 0):
    """Seeded stand-in for the reference's MNIST CNN job (main.py:14-46): ``steps`` batches of
    normalised-pixel-like images U[0,1] fp32 (batch, 1, 28, 28) with labels in [0, 10), and the
    parameter list of that CNN in ``Sequential.parameters()`` order -- conv weights N(0, 2/fan_in)
    fp32, BatchNorm gamma ~ 1 and beta ~ 0 as float64 (the reference's dtype for them) with the
    reference's shapes, Linear weights fp32, final bias (1, 10)."""
    rng = np.random.default_rng(seed)
    x = rng.random((steps, batch, 1, 28, 28), dtype=np.float32)
    y = rng.integers(0, 10, (steps, batch)).astype(np.int64)

    def w(*shape):
        fan_in = int(np.prod(shape[1:]))
        return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)

    def bn(c, nd):
        shp = (1, c, 1, 1) if nd == 4 else (1, c)
        return [1.0 + 0.1 * rng.standard_normal(shp), 0.1 * rng.standard_normal(shp)]

    params = [w(16, 1, 3, 3), *bn(16, 4), w(32, 16, 3, 3), *bn(32, 4), w(64, 32, 3, 3), *bn(64, 4),
              w(32, 64), *bn(32, 2), w(10, 32), (0.01 * rng.standard_normal((1, 10))).astype(np.float32)]
    return x, y, params
