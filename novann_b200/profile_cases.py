"""Small, self-ending cases of each kernel for profiler captures.

    python -m novann_b200.profile_cases cast   [log2_elems=26]
    python -m novann_b200.profile_cases fp8    [rows=8192]
    python -m novann_b200.profile_cases fp4    [rows=8192]
    python -m novann_b200.profile_cases linear [M=4096 N=4096 K=4096]
    python -m novann_b200.profile_cases w8a8   [M=4096 N=4096 K=4096]
    python -m novann_b200.profile_cases cnn    [batch=128 steps=3]
    python -m novann_b200.profile_cases mlp    [batch=128 steps=3]
    python -m novann_b200.profile_cases conv   [N=128 C=64 HW=56 Cout=128 reps=2]
    python -m novann_b200.profile_cases fewrows [M=16 N=8192 K=8192 reps=3]

Each case uploads seeded inputs, launches the kernels a few times and exits; sizes are
larger than the 126 MB L2 (so DRAM counters mean something) but hold at most a few GB.
"""
from __future__ import annotations

import sys

import numpy as np

from . import functional as F, quant, workloads
from .device import DeviceBuffer, Stream, device_sync


def case_cast(log2n: int = 26, reps: int = 3) -> None:
    n = 1 << log2n
    st = Stream(0)
    x = workloads.cast_input(n, seed=0)
    d32 = DeviceBuffer.from_numpy(x, 0)
    d16 = DeviceBuffer(n * 2, 0)
    for _ in range(reps):
        quant.cast_device(d16, "bf16", d32, "f32", n, stream=st)
        quant.cast_device(d32, "f32", d16, "bf16", n, stream=st)
        quant.cast_device(d16, "f16", d32, "f32", n, stream=st)
        quant.cast_device(d32, "f32", d16, "f16", n, stream=st)
    st.sync()


def case_fp8(rows: int = 8192, reps: int = 3) -> None:
    cols = 8192
    n = rows * cols
    st = Stream(0)
    x = workloads.fp8_input(rows, cols, seed=0)
    d = DeviceBuffer.from_numpy(x, 0)
    q = DeviceBuffer(n, 0)
    asi = DeviceBuffer(12, 0)
    for _ in range(reps):
        quant.quantize_fp8_tensor_device(q, asi, d, n, "e4m3", stream=st)
        quant.dequantize_fp8_device(d, q, n, "e4m3", 0.01, stream=st)
    st.sync()


def case_fp4(rows: int = 8192, reps: int = 3) -> None:
    cols = 8192
    st = Stream(0)
    xb = workloads.fp4_input_bits(rows, cols, seed=0)
    d = DeviceBuffer.from_numpy(xb, 0)
    p = DeviceBuffer(rows * cols // 2, 0)
    s = DeviceBuffer(rows * cols // 32 * 4, 0)
    for _ in range(reps):
        quant.quantize_fp4_b32_device(p, s, d, rows, cols, stream=st)
        quant.dequantize_fp4_b32_device(d, p, s, rows, cols, stream=st)
    st.sync()


def case_linear(m: int = 4096, n: int = 4096, k: int = 4096, reps: int = 3) -> None:
    st = Stream(0)
    xb, w, b = workloads.linear_inputs(m, n, k, seed=0)
    # weight codes straight from a seeded generator (no oracle in the product path)
    rng = np.random.default_rng(1)
    wq = rng.integers(0, 0x7F, (n, k), dtype=np.uint64).astype(np.uint8)
    wq |= (rng.integers(0, 2, (n, k), dtype=np.uint64).astype(np.uint8) << 7)
    sc = np.full(n, 1e-3, np.float32)
    dx = DeviceBuffer.from_numpy(xb, 0)
    dw = DeviceBuffer.from_numpy(wq, 0)
    ds = DeviceBuffer.from_numpy(sc, 0)
    db = DeviceBuffer.from_numpy(b, 0)
    dy = DeviceBuffer(m * n * 2, 0)
    ws = DeviceBuffer(F.linear_workspace_bytes(n, k, "e4m3"), 0)
    for _ in range(reps):
        F.linear_q_device(dy, dx, dw, "e4m3", ds, db, m, n, k, ws, stream=st)
    st.sync()
    F.check_device_errors(0)


def case_w8a8(m: int = 4096, n: int = 4096, k: int = 4096, reps: int = 3) -> None:
    st = Stream(0)
    xb, _, b = workloads.linear_inputs(m, 8, k, seed=0)
    rng = np.random.default_rng(1)
    wq = rng.integers(0, 0x7F, (n, k), dtype=np.uint64).astype(np.uint8)
    dx, dw = DeviceBuffer.from_numpy(xb, 0), DeviceBuffer.from_numpy(wq, 0)
    ds = DeviceBuffer.from_numpy(np.full(n, 1e-3, np.float32), 0)
    dy = DeviceBuffer(m * n * 2, 0)
    ws = DeviceBuffer(F.linear_w8a8_workspace_bytes(m, k), 0)
    for _ in range(reps):
        F.linear_w8a8_device(dy, dx, dw, ds, None, m, n, k, ws, stream=st)
    st.sync()
    F.check_device_errors(0)


def case_cnn(batch: int = 128, steps: int = 3) -> None:
    """Training steps of the reference's main.py CNN, eager launches (one kernel per line in a
    profiler's launch list)."""
    from .train_cnn import CNNTrainStep, main_cnn_spec
    xs, ys, params = workloads.cnn_inputs(batch, steps=1, seed=0)
    step = CNNTrainStep(main_cnn_spec(), params, batch, (1, 28, 28))
    for _ in range(steps):
        step.step(xs[0], ys[0])


def case_mlp(batch: int = 128, steps: int = 3) -> None:
    """Training steps of the 784-256-128-10 MLP, eager launches."""
    from .train import MLPTrainStep
    x, y, params = workloads.mlp_inputs(batch, seed=0)
    step = MLPTrainStep(params, batch, lr=0.01)
    for _ in range(steps):
        step.step(x, y)


def case_conv(n: int = 128, c: int = 64, hw: int = 56, cout: int = 128, reps: int = 2) -> None:
    """FP8-weight 3x3 convolution (stride 1, pad 1) through nvq_conv2d_fwd_q, device resident."""
    from . import _lib
    from ._lib import check, lib
    from .device import _sptr
    st = Stream(0)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, c, hw, hw), dtype=np.float32)
    wq = rng.integers(0, 0x7F, (cout, c * 9), dtype=np.uint64).astype(np.uint8)
    dx, dq = DeviceBuffer.from_numpy(x, 0), DeviceBuffer.from_numpy(wq, 0)
    ds = DeviceBuffer.from_numpy(np.full(cout, 1e-3, np.float32), 0)
    rows, kpad = n * hw * hw, c * 9
    col, yb = DeviceBuffer(rows * kpad * 2, 0), DeviceBuffer(rows * cout * 2, 0)
    ws = DeviceBuffer(F.linear_workspace_bytes(cout, kpad, "e4m3"), 0)
    out = DeviceBuffer(rows * cout * 4, 0)
    for _ in range(reps):
        check(lib().nvq_conv2d_fwd_q(out.at(0), dx.at(0), dq.at(0), _lib.DTYPE_IDS["e4m3"], ds.at(0), None,
                                     col.at(0), yb.at(0), ws.at(0), ws.nbytes, n, c, hw, hw, cout, 3, 3,
                                     1, 1, 1, 1, 0, 0, _sptr(st)))
    st.sync()
    F.check_device_errors(0)


def case_fewrows(m: int = 16, n: int = 8192, k: int = 8192, reps: int = 3) -> None:
    """FP8-weight Linear with few rows (the weight-streaming kernel), rotating over four weight
    copies so that every call reads its codes from DRAM."""
    st = Stream(0)
    rng = np.random.default_rng(1)
    xb, _, b = workloads.linear_inputs(m, 8, k, seed=0)
    sets = []
    for i in range(4):
        wq = rng.integers(0, 0x7F, (n, k), dtype=np.uint64).astype(np.uint8)
        sets.append((DeviceBuffer.from_numpy(wq, 0), DeviceBuffer(F.linear_workspace_bytes(n, k, "e4m3"), 0)))
    dx = DeviceBuffer.from_numpy(xb, 0)
    ds = DeviceBuffer.from_numpy(np.full(n, 1e-3, np.float32), 0)
    dy = DeviceBuffer(m * n * 2, 0)
    for r in range(reps * 4):
        dw, ws = sets[r % 4]
        F.linear_q_device(dy, dx, dw, "e4m3", ds, None, m, n, k, ws, stream=st)
    st.sync()
    F.check_device_errors(0)


def main(argv) -> None:
    what = argv[1] if len(argv) > 1 else "cast"
    args = [int(a) for a in argv[2:]]
    if what == "cast":
        case_cast(*args)
    elif what == "fp8":
        case_fp8(*args)
    elif what == "fp4":
        case_fp4(*args)
    elif what == "linear":
        case_linear(*args)
    elif what == "w8a8":
        case_w8a8(*args)
    elif what == "cnn":
        case_cnn(*args)
    elif what == "mlp":
        case_mlp(*args)
    elif what == "conv":
        case_conv(*args)
    elif what == "fewrows":
        case_fewrows(*args)
    else:
        raise SystemExit(f"unknown case {what}")
    device_sync(0)


if __name__ == "__main__":
    main(sys.argv)
