"""The allocation-free Linear entry point (``nvq_linear_fwd_static``).

Hosts that cannot allocate device memory where they need a Linear (fixed memory budgets,
latency-critical steps in which cudaMalloc would stall the device) call this form: its
scratch is an array built into the library.  The test drives it through the C ABI and
requires the same output as ``nvq_linear_fwd`` with a caller workspace, on two calls in a
row; the second call uses a smaller weight so that it runs over the first call's leftovers
in the shared scratch.  The file name sorts last on purpose: a run that stops at the first
failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from novann_b200 import _lib, functional as F, workloads
from novann_b200.device import DeviceBuffer, device_sync
from oracle import oracle_np as o

pytestmark = pytest.mark.gpu

STATIC_BYTES = 8 << 20


def _codes(n, k, seed):
    rng = np.random.default_rng(seed)
    wq = rng.integers(0, 0x7F, (n, k), dtype=np.uint64).astype(np.uint8)      # finite E4M3 codes
    wq |= rng.integers(0, 2, (n, k), dtype=np.uint64).astype(np.uint8) << 7   # random signs
    sc = rng.uniform(1e-4, 1e-3, n).astype(np.float32)
    return wq, sc


def _both_ways(gpu, m, n, k, seed):
    xb, _, b = workloads.linear_inputs(m, n, k, seed=seed)
    wq, sc = _codes(n, k, seed)
    L = _lib.lib()
    dx, dw = DeviceBuffer.from_numpy(xb, gpu), DeviceBuffer.from_numpy(wq, gpu)
    ds, db = DeviceBuffer.from_numpy(sc, gpu), DeviceBuffer.from_numpy(b, gpu)
    y_ref, y_new = DeviceBuffer(m * n * 2, gpu), DeviceBuffer(m * n * 2, gpu)
    status = DeviceBuffer.from_numpy(np.zeros(1, np.int32), gpu)
    # the caller-workspace form gets exactly the bytes the built-in array has, so both calls
    # take the same kernel path (few rows: the partial sums must fit the same 8 MiB)
    ws = DeviceBuffer(max(STATIC_BYTES, F.linear_workspace_bytes(n, k, "e4m3")), gpu)
    ws_bytes = C.c_size_t(STATIC_BYTES)
    _lib.check(L.nvq_linear_fwd(y_ref.at(0), dx.at(0), dw.at(0), _lib.E4M3, ds.at(0), db.at(0), m, n, k,
                                ws.at(0), ws_bytes, gpu, None))
    _lib.check(L.nvq_linear_fwd_static(y_new.at(0), dx.at(0), dw.at(0), _lib.E4M3, ds.at(0), db.at(0),
                                       m, n, k, status.at(0), gpu, None))
    device_sync(gpu)
    F.check_device_errors(gpu)
    assert status.to_numpy(np.int32, (1,))[0] == 0
    a = y_ref.to_numpy(np.uint16, (m, n))
    c = y_new.to_numpy(np.uint16, (m, n))
    # and against the CPU oracle (float64 accumulation), within the FP8 bound of the other tests
    rows = np.unique(np.concatenate([np.arange(0, m, max(1, m // 16)), [m - 1]]))
    want, _ = o.linear_fwd_qweight(xb[rows], wq, sc, b, "e4m3")
    err = o.max_abs_rel(o.bf16_bits_to_f32(c[rows]), o.bf16_bits_to_f32(want))
    assert err <= 2.0 ** -7, err
    return a, c


def test_static_scratch_matches_workspace_form_twice_in_a_row(gpu):
    # first call fills the whole built-in scratch (2048 x 2048 weights = 8 MiB expanded);
    # 128 rows keep it on the kernel that reads the expanded weight from scratch
    a, c = _both_ways(gpu, 128, 2048, 2048, seed=1)
    assert np.array_equal(a, c)
    # second call: smaller weight, run over the first call's leftovers (K = 328 is not a
    # multiple of 16, which also keeps this shape on the scratch path)
    a, c = _both_ways(gpu, 200, 264, 328, seed=2)
    assert np.array_equal(a, c)
    # third call: few rows.  The same array now holds the few-rows kernels' fp32 partial sums,
    # activation codes and row scales instead of an expanded weight, over the leftovers of the
    # two calls before; bit for bit the caller-workspace form, and twice the same bits.
    a, c = _both_ways(gpu, 16, 1024, 1024, seed=3)
    assert np.array_equal(a, c)
    a2, c2 = _both_ways(gpu, 16, 1024, 1024, seed=3)
    assert np.array_equal(c, c2) and np.array_equal(a, a2)


def test_static_scratch_rejects_oversized_weight(gpu):
    L = _lib.lib()
    d = DeviceBuffer(64, gpu)
    n, k = 2048, 2056                      # N * K * 2 just above the 8 MiB limit
    assert n * k * 2 > STATIC_BYTES
    st = L.nvq_linear_fwd_static(d.at(0), d.at(0), d.at(0), _lib.E4M3, d.at(0), None, 16, n, k,
                                 None, gpu, None)
    assert st == _lib.ERR_INVALID
    msg = L.nvq_last_error().decode()
    assert "built-in" in msg and str(STATIC_BYTES) in msg
