#!/usr/bin/env python
"""Benchmark of the cast / quantised-Linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case NAME [ints ...]          one small case of one kernel (profiler captures)

One "step" is one pass of the cast sweep over one 1 Gi-element tensor resident in HBM:
fp32->bf16, bf16->fp32, fp32->fp16, fp16->fp32 (6 algorithmic bytes per element each,
24 per element per step).  The headline metric is achieved HBM GB/s summed over all
ranks (weak scaling: every rank owns its own 1 Gi-element shard, no collective).

`e2e` repeats the same sweep through the host-array call that replaces
``ndarray.astype`` (NumPy array in pinned memory in, NumPy array out), so every byte
crosses PCIe inside the timed region; next to it the same bytes are moved by plain copies
with no kernel (the ceiling of that path) and the sweep is repeated on pageable arrays.

The FP8-weight Linear (the other half of the headline metric), the smaller cast sizes, the
float64 cast, the quantisers, the convolution and the training steps are measured in the
same run and reported as flat keys; with more than one rank the data-parallel MLP step runs
with its NCCL all-reduce over all ranks.

`--impl reference` times the reference's CPU path for the same sweep on the host, at the
same size: ``ndarray.astype`` for fp16 (NovaNN's own primitive, single-threaded by nature)
and the CPU oracle's C restatement on all cores for bf16 (the reference has no bf16).
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ELEMS = 1 << 30          # per rank
TILE = 1 << 26             # seeded block the big tensor is tiled from
BYTES_PER_ELEM_STEP = 24   # 4 directions x 6 B
DIRECTIONS = [("f32", "bf16"), ("bf16", "f32"), ("f32", "f16"), ("f16", "f32")]
MLP_PARAMS = 235146        # floats in the 784-256-128-10 gradient bucket


def workload_config(n: int = N_ELEMS) -> dict:
    """The workload both arms run; identical in the GPU line and the reference line."""
    return {"workload": "cast sweep fp32->bf16->fp32->fp16->fp32, 1 Gi elements per GPU "
                        "(BASELINE configs[1], largest size)",
            "elements_per_gpu": n, "bytes_per_element_step": BYTES_PER_ELEM_STEP,
            "l2": "inputs (4 GiB + 2 GiB) far exceed the 126 MB L2; no flush needed",
            "input": "N(0,1) with 1% N(0,sigma=100) + 4096-element edge block; "
                     "2^26-element seeded tile repeated 16x"}


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms on a thread."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for nm, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


_T0 = time.time()


def phase(name: str, limit_s: int = 240) -> None:
    """Marks the start of a phase on stderr and re-arms a watchdog: a phase that takes longer than
    ``limit_s`` dumps every thread's stack and ends the process (a hung rank then costs minutes,
    not the launcher's whole time limit, and the dump says where it stood)."""
    rank = os.environ.get("RANK", "0")
    sys.stderr.write(f"[bench rank {rank} +{time.time() - _T0:6.1f}s] {name}\n")
    sys.stderr.flush()
    faulthandler.cancel_dump_traceback_later()
    faulthandler.dump_traceback_later(limit_s, exit=True)


def _host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# ------------------------------------------------------------------ CPU arm
class CpuSweep:
    """The CPU path of the sweep on n elements: fp16 legs = ``ndarray.astype`` (the reference's
    own primitive, one thread), bf16 legs = the C oracle with OpenMP on every host thread this
    process may use (set explicitly: a launcher that exports OMP_NUM_THREADS=1 does not shrink it)."""

    def __init__(self, n: int):
        from novann_b200 import workloads
        from oracle import oracle_c
        self.oc = oracle_c.load()
        self.threads = _host_threads()
        self.oc.set_threads(self.threads)
        self.n = n
        self.x = np.empty(n, np.float32)
        tile = workloads.cast_input(min(n, TILE), seed=0)
        for off in range(0, n, tile.size):
            self.x[off:off + tile.size] = tile[:n - off]
        self.b16 = np.empty(n, np.uint16)
        self.f32 = np.empty(n, np.float32)

    def run(self):
        """One sweep; returns (seconds, GB/s per direction)."""
        n, oc, x = self.n, self.oc, self.x
        t0 = time.perf_counter()
        oc.f32_to_bf16_bits(x, out=self.b16)
        t1 = time.perf_counter()
        oc.bf16_bits_to_f32(self.b16, out=self.f32)
        t2 = time.perf_counter()
        with np.errstate(all="ignore"):
            h = x.astype(np.float16)       # the reference's own primitive
        t3 = time.perf_counter()
        h.astype(np.float32)
        t4 = time.perf_counter()
        g = 6 * n / 1e9
        return t4 - t0, {"f32->bf16_c_omp": g / (t1 - t0), "bf16->f32_c_omp": g / (t2 - t1),
                         "f32->f16_numpy_astype": g / (t3 - t2), "f16->f32_numpy_astype": g / (t4 - t3)}


def run_reference(args):
    """The reference arm: the full 1 Gi-element sweep per step on the host.  A step takes about
    ten seconds, so the number of steps is cut to what fits ~200 s; `steps` reports what ran."""
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    n = N_ELEMS
    cpu = CpuSweep(n)
    budget_s = 200.0
    t_begin = time.perf_counter()
    warm = min(args.warmup, 1)
    for _ in range(warm):
        cpu.run()
    times, detail = [], None
    for i in range(max(1, args.steps)):
        s, detail = cpu.run()
        times.append(s)
        elapsed = time.perf_counter() - t_begin
        if elapsed + s > budget_s:
            break
    tot = sum(times)
    value = BYTES_PER_ELEM_STEP * n * len(times) / tot / 1e9
    sample = (f"full size: {n} elements per step, {len(times)} timed steps (+{warm} warm-up); fp16 legs "
              f"ndarray.astype (1 thread), bf16 legs C oracle OpenMP ({cpu.threads} threads)")
    line = {
        "impl": "reference", "metric": "cast_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": warm, "steps_requested": args.steps,
        "ms_per_step": tot / len(times) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32<->bf16/f16", "data": "synthetic",
        "config": workload_config(n),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cpu.threads, "kind": "reference",
                         "sample": sample,
                         **{"gbs_" + k.replace("->", "_to_"): v for k, v in detail.items()}},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ GPU arm: helpers
class Timing:
    """CUDA-event timing on the library's stream.  Where a call's working set is below the 126 MB
    L2, launches rotate over enough operand sets that every launch finds its inputs in DRAM (a
    flushing write between launches would leave dirty lines whose write-back lands inside the
    next timed kernel)."""

    def __init__(self, dev, st):
        self.dev, self.st = dev, st

    def events(self):
        from novann_b200.device import Event
        return Event(self.dev), Event(self.dev)

    def rotating(self, fn, sets, rounds=4):
        k = len(sets)
        for i in range(k):
            fn(*sets[i])
        self.st.sync()
        e0, e1 = self.events()
        e0.record(self.st)
        for i in range(rounds * k):
            fn(*sets[i % k])
        e1.record(self.st)
        e1.sync()
        return e0.elapsed_ms(e1) / (rounds * k)

    def graph(self, fn, sets, rounds=4):
        """The same rotation recorded once into a CUDA graph (one call per buffer set) and
        replayed: the device time of a call without the host's launch cost."""
        import ctypes as C
        from novann_b200._lib import check, lib
        from novann_b200.device import _sptr
        dev, st = self.dev, self.st
        for a in sets:
            fn(*a)
        st.sync()
        check(lib().nvq_graph_begin_capture(dev, _sptr(st)))
        try:
            for a in sets:
                fn(*a)
        finally:
            h = C.c_void_p()
            check(lib().nvq_graph_end_capture(dev, _sptr(st), C.byref(h)))
        graph = C.c_void_p(h.value)
        check(lib().nvq_graph_launch(dev, graph, _sptr(st)))
        st.sync()
        e0, e1 = self.events()
        e0.record(st)
        for _ in range(rounds):
            check(lib().nvq_graph_launch(dev, graph, _sptr(st)))
        e1.record(st)
        e1.sync()
        check(lib().nvq_graph_destroy(dev, graph))
        return e0.elapsed_ms(e1) / (rounds * len(sets))

    @staticmethod
    def n_sets_for(set_bytes):
        return max(2, int(np.ceil((512 << 20) / set_bytes)) + 1)


def _free(sets):
    for bufs in sets:
        for b in bufs:
            if b is not None:
                b.free()


def _random_codes(rng, n, k):
    wq = rng.integers(0, 0x7F, (n, k), dtype=np.uint64).astype(np.uint8)      # finite E4M3 codes
    wq |= rng.integers(0, 2, (n, k), dtype=np.uint64).astype(np.uint8) << 7
    return wq


# ------------------------------------------------------------------ GPU arm: the other kernels
def measure_cast_sizes(T, rank):
    """The other sizes of the cast-sweep config (1 Mi and 64 Mi elements) and the float64 pair:
    the four-direction sweep over rotating buffer pairs; GB/s over 24 B (12 B for float64) per
    element."""
    from novann_b200 import quant, workloads
    from novann_b200.device import DeviceBuffer
    out = {}
    for name, n in (("cast_1Mi_gbs", 1 << 20), ("cast_64Mi_gbs", 1 << 26)):
        x = workloads.cast_input(n, seed=rank)
        sets = [(DeviceBuffer.from_numpy(x, T.dev), DeviceBuffer(n * 2, T.dev))
                for _ in range(Timing.n_sets_for(6 * n))]

        def sweep(d32, d16):
            for src, dst in DIRECTIONS:
                a, b = (d32, d16) if src == "f32" else (d16, d32)
                quant.cast_device(b, dst, a, src, n, stream=T.st)
        t = T.rotating(sweep, sets, rounds=4 if n > (1 << 22) else 8)
        out[name] = BYTES_PER_ELEM_STEP * n / t / 1e6
        if n == 1 << 20:
            out["cast_1Mi_us_per_sweep"] = t * 1e3
            out["cast_1Mi_us_per_sweep_graph"] = T.graph(sweep, sets, rounds=8) * 1e3
        _free(sets)
    # float64 -> float32 (what the reference's layers do to BatchNorm's output) and back: 2^28
    # elements (2 GiB of float64), 12 algorithmic bytes per element and direction
    n = 1 << 28
    rng = np.random.default_rng(rank)
    tile = rng.standard_normal(1 << 24)
    d64, d32 = DeviceBuffer(n * 8, T.dev), DeviceBuffer(n * 4, T.dev)
    for off in range(0, n, tile.size):
        d64.upload(tile, offset=off * 8)
    sets = [(d64, d32)]
    t = T.rotating(lambda a, b: quant.cast_device(b, "f32", a, "f64", n, stream=T.st), sets, rounds=10)
    out["cast_f64_to_f32_gbs"] = 12 * n / t / 1e6
    t = T.rotating(lambda a, b: quant.cast_device(a, "f64", b, "f32", n, stream=T.st), sets, rounds=10)
    out["cast_f32_to_f64_gbs"] = 12 * n / t / 1e6
    _free(sets)
    return out


def measure_quantisers(T, rank, world):
    from novann_b200 import quant, workloads
    from novann_b200.device import DeviceBuffer
    out = {}
    # FP8 per tensor: fp32 [16384, 16384 / world] row shard (1 GiB per GPU at world = 1)
    rows = 16384 // world
    n = rows * 16384
    x = workloads.fp8_input(min(rows, 1024), 16384, seed=rank)
    asi = DeviceBuffer(12, T.dev)
    sets = []
    for _ in range(Timing.n_sets_for(5 * n)):
        d32 = DeviceBuffer(n * 4, T.dev)
        for off in range(0, n, x.size):
            d32.upload(x, offset=off * 4)
        sets.append((d32, DeviceBuffer(n, T.dev)))
    t = T.rotating(lambda d32, d8: quant.quantize_fp8_tensor_device(d8, asi, d32, n, "e4m3", stream=T.st), sets)
    out["fp8_e4m3_amax_quantize_gbs"] = 9 * n / t / 1e6
    t = T.rotating(lambda d32, d8: quant.dequantize_fp8_device(d32, d8, n, "e4m3", 0.02, stream=T.st), sets)
    out["fp8_e4m3_dequantize_gbs"] = 5 * n / t / 1e6
    _free(sets)
    # FP4 block 32: bf16 [8192 / world, 8192]
    r4 = 8192 // world
    xb = workloads.fp4_input_bits(r4, 8192, seed=rank)
    set_bytes = r4 * 8192 * 2.625
    sets = [(DeviceBuffer.from_numpy(xb, T.dev), DeviceBuffer(r4 * 4096, T.dev),
             DeviceBuffer(r4 * 256 * 4, T.dev)) for _ in range(Timing.n_sets_for(set_bytes))]
    t = T.rotating(lambda dx, dp, dsc: quant.quantize_fp4_b32_device(dp, dsc, dx, r4, 8192, stream=T.st), sets)
    out["fp4_quantize_gbs"] = set_bytes / t / 1e6
    t = T.rotating(lambda dx, dp, dsc: quant.dequantize_fp4_b32_device(dx, dp, dsc, r4, 8192, stream=T.st), sets)
    out["fp4_dequantize_gbs"] = set_bytes / t / 1e6
    _free(sets)
    return out


def measure_linear(T, rank, world):
    """FP8-weight Linear forward: M = 4096 (one GPU) or 8192 / world rows per GPU; N = K = 4096.
    Rotating operand sets (x, codes, workspace, y): a set comes round again only after the other
    sets' >= 512 MB went through L2, so every call finds its operands in DRAM."""
    from novann_b200 import functional as F, workloads
    from novann_b200.device import DeviceBuffer
    dev, st = T.dev, T.st
    _, peak_bf16, _ = _peaks()
    m = 4096 if world == 1 else 8192 // world
    nn = kk = 4096
    rng = np.random.default_rng(rank)
    xb, _, _ = workloads.linear_inputs(m, 8, kk, seed=rank)
    wq = _random_codes(rng, nn, kk)
    dss = DeviceBuffer.from_numpy(np.full(nn, 1e-3, np.float32), dev)
    dbb = DeviceBuffer.from_numpy(np.zeros(nn, np.float32), dev)
    per_set = m * kk * 2 + nn * kk + nn * kk * 2 + m * nn * 2
    lsets = [(DeviceBuffer.from_numpy(xb, dev), DeviceBuffer.from_numpy(wq, dev),
              DeviceBuffer(F.linear_workspace_bytes(nn, kk, "e4m3"), dev), DeviceBuffer(m * nn * 2, dev))
             for _ in range(Timing.n_sets_for(per_set))]
    flops = 2.0 * m * nn * kk
    out = {"linear_fp8_M_per_gpu": m}

    def call(path=None, use_ws=True):
        return lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, m, nn, kk,
                                                         ws if use_ws else None, stream=st, path=path)
    t = T.rotating(call(), lsets)
    F.check_device_errors(dev)
    out["linear_fp8_ms"] = t
    out["linear_fp8_tflops_per_gpu"] = flops / t / 1e9
    out["linear_fp8_frac_bf16_peak"] = flops / t / 1e9 / peak_bf16
    out["linear_fp8_frac_nominal_fp8_4500"] = flops / t / 1e9 / 4500.0
    t = T.rotating(call(use_ws=False), lsets)
    F.check_device_errors(dev)
    out["linear_fp8_in_kernel_expansion_tflops_per_gpu"] = flops / t / 1e9
    # fixed weights (inference): the library's weight cache expands the codes on the first forward
    # and runs the contraction alone afterwards; one cache per rotating set
    caches = [F.LinearWeightCache(wq, np.full(nn, 1e-3, np.float32), np.zeros(nn, np.float32), "e4m3", dev)
              for _ in lsets]
    csets = [(dxx, c, dy) for (dxx, _, _, dy), c in zip(lsets, caches)]
    t = T.rotating(lambda dxx, c, dy: c.forward_device(dy, dxx, m, stream=st), csets)
    F.check_device_errors(dev)
    assert all(c.expansions == 1 for c in caches)
    out["linear_fp8_weight_expanded_once_tflops_per_gpu"] = flops / t / 1e9
    for c in caches:
        c.close()
    del caches, csets
    ws8 = DeviceBuffer(F.linear_w8a8_workspace_bytes(m, kk), dev)
    t = T.rotating(lambda dxx, dw, ws, dy: F.linear_w8a8_device(dy, dxx, dw, dss, dbb, m, nn, kk, ws8, stream=st), lsets)
    F.check_device_errors(dev)
    out["linear_w8a8_variant_tflops_per_gpu"] = flops / t / 1e9     # NOT the parity path (2.4-3.2e-2 off)
    # few rows (serving shape): the weight-streaming kernel; same rotating sets, so the 16 MB of
    # codes come from DRAM on every call
    ms_ = 16

    def few(dxx, dw, ws, dy):
        F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, ms_, nn, kk, ws, stream=st)
    t = T.rotating(few, lsets)
    tg = T.graph(few, lsets)
    F.check_device_errors(dev)
    hbm, _, _ = _peaks()
    out["linear_fp8_few_rows_us"] = t * 1e3
    out["linear_fp8_few_rows_us_graph"] = tg * 1e3
    out["linear_fp8_few_rows_frac_hbm_graph"] = nn * kk / tg / 1e6 / hbm
    _free(lsets)
    ws8.free()
    # the same kernel on a weight far larger than L2 (an 8192 x 28672 projection, 235 MB of codes)
    nl, kl = 28672, 8192
    wl = np.tile(rng.integers(0, 0x7F, (nl // 8, kl), dtype=np.uint8), (8, 1))
    xl, _, _ = workloads.linear_inputs(ms_, 8, kl, seed=rank)
    dsl = DeviceBuffer.from_numpy(np.full(nl, 1e-3, np.float32), dev)
    big = [(DeviceBuffer.from_numpy(xl, dev), DeviceBuffer.from_numpy(wl, dev),
            DeviceBuffer(64 << 20, dev), DeviceBuffer(ms_ * nl * 2, dev)) for _ in range(2)]
    t = T.rotating(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dsl, None, ms_, nl, kl, ws,
                                                             stream=st), big, rounds=5)
    F.check_device_errors(dev)
    out["linear_fp8_few_rows_large_us"] = t * 1e3
    out["linear_fp8_few_rows_large_frac_hbm"] = nl * kl / t / 1e6 / hbm
    _free(big)
    for b in (dsl, dss, dbb):
        b.free()
    return out


def measure_conv(T, rank, world):
    """FP8-weight Conv2d forward as an implicit GEMM: x fp32 [128 / world, 64, 56, 56], 3x3, pad 1,
    128 output channels; NCHW fp32 in and out, all kernels of the call in the time."""
    from novann_b200 import _lib, functional as F
    from novann_b200._lib import check, lib
    from novann_b200.device import DeviceBuffer, _sptr
    dev, st = T.dev, T.st
    rng = np.random.default_rng(rank)
    cn, cc, chw, cco = max(1, 128 // world), 64, 56, 128
    xcv = rng.standard_normal((cn, cc, chw, chw), dtype=np.float32)
    wcv = rng.integers(0, 0x7F, (cco, cc * 9), dtype=np.uint64).astype(np.uint8)
    d_xc, d_wc = DeviceBuffer.from_numpy(xcv, dev), DeviceBuffer.from_numpy(wcv, dev)
    d_sc = DeviceBuffer.from_numpy(np.full(cco, 1e-3, np.float32), dev)
    crows, ckp = cn * chw * chw, cc * 9
    d_col, d_yb = DeviceBuffer(crows * ckp * 2, dev), DeviceBuffer(crows * cco * 2, dev)
    d_wsc = DeviceBuffer(F.linear_workspace_bytes(cco, ckp, "e4m3"), dev)
    d_oc = DeviceBuffer(crows * cco * 4, dev)

    def conv_call(*_):
        check(lib().nvq_conv2d_fwd_q(d_oc.at(0), d_xc.at(0), d_wc.at(0), _lib.DTYPE_IDS["e4m3"], d_sc.at(0),
                                     None, d_col.at(0), d_yb.at(0), d_wsc.at(0), d_wsc.nbytes, cn, cc,
                                     chw, chw, cco, 3, 3, 1, 1, 1, 1, 0, dev, _sptr(st)))
    t = T.rotating(conv_call, [()], rounds=10)
    F.check_device_errors(dev)
    # the same convolution between chained quantised layers: bf16 NHWC in and out, no layout pass
    d_xh, d_yh = DeviceBuffer(cn * cc * chw * chw * 2, dev), DeviceBuffer(crows * cco * 2, dev)
    F.nchw_f32_to_nhwc_bf16_device(d_xh, d_xc, cn, cc, chw * chw, stream=st)

    def nhwc_call(*_):
        F.conv2d_q_nhwc_device(d_yh, d_xh, d_wc, "e4m3", d_sc, None, d_wsc, cn, cc, chw, chw, cco, (3, 3),
                               (1, 1), (1, 1), relu=True, stream=st)
    t2 = T.rotating(nhwc_call, [()], rounds=10)
    F.check_device_errors(dev)
    for b in (d_xc, d_wc, d_col, d_yb, d_wsc, d_oc, d_sc, d_xh, d_yh):
        b.free()
    flops = 2.0 * crows * cco * ckp
    return {"conv2d_fp8_ms": t, "conv2d_fp8_tflops_per_gpu": flops / t / 1e9, "conv2d_fp8_N_per_gpu": cn,
            "conv2d_fp8_nhwc_ms": t2, "conv2d_fp8_nhwc_tflops_per_gpu": flops / t2 / 1e9}


def measure_train_steps(T, rank, world):
    """The fp32 MLP step (784-256-128-10) and the CNN of the reference's main.py, batch 128 / world
    per GPU, replayed as CUDA graphs; no collective in these two figures."""
    from novann_b200 import workloads
    from novann_b200.train import MLPTrainStep
    from novann_b200.train_cnn import CNNTrainStep, main_cnn_spec
    dev = T.dev
    out = {}
    bsz = max(1, 128 // world)
    xm, ym, params = workloads.mlp_inputs(128, (784, 256, 128, 10), seed=0)
    step = MLPTrainStep(params, bsz, 0.01, dev)
    step.step(xm[:bsz], ym[:bsz])
    step.capture()
    for _ in range(5):
        step.replay()
    step.stream.sync()
    T2 = Timing(dev, step.stream)
    e0, e1 = T2.events()
    e0.record(step.stream)
    for _ in range(50):
        step.replay()
    e1.record(step.stream)
    e1.sync()
    out["mlp_step_us"] = e0.elapsed_ms(e1) / 50 * 1e3
    xc, yc, cparams = workloads.cnn_inputs(bsz, steps=1, seed=0)
    cnn = CNNTrainStep(main_cnn_spec(), cparams, bsz, (1, 28, 28), device=dev)
    cnn.step(xc[0], yc[0])
    cnn.capture()
    for _ in range(3):
        cnn.step(xc[0], yc[0])
    T3 = Timing(dev, cnn.stream)
    e0, e1 = T3.events()
    e0.record(cnn.stream)
    for _ in range(20):
        cnn.replay()
    e1.record(cnn.stream)
    e1.sync()
    out["cnn_step_us"] = e0.elapsed_ms(e1) / 20 * 1e3
    return out


def measure_dp_step(dev, rank, world, dist, local):
    """The one collective of the project: the data-parallel MLP step, batch 128 split over the
    ranks, its flat 235 146-float gradient bucket summed by nvq_allreduce_sum_f32 (NCCL over
    NVLink), 1 / world folded into the SGD kernel.  Times are the max over ranks.
    dp_step_us: device time per step, 50 steps enqueued back to back, each step = a CUDA graph of
    the library's nine forward / loss / backward kernels, then the all-reduce and the SGD kernel
    launched eagerly (the NCCL collective is never captured); dp_step_eager_us: all eleven launches
    eager; allreduce_us: the all-reduce alone."""
    import torch
    from novann_b200 import workloads
    from novann_b200.device import DeviceBuffer
    from novann_b200.train import Communicator, MLPTrainStep, shard_rows

    def max_over_ranks(v):
        t = torch.tensor([v], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    uid = torch.zeros(128, dtype=torch.uint8, device=f"cuda:{local}")
    if rank == 0:
        uid = torch.tensor(list(Communicator.make_unique_id()), dtype=torch.uint8, device=f"cuda:{local}")
    dist.broadcast(uid, src=0)
    comm = Communicator(bytes(uid.cpu().tolist()), rank, world, device=dev)
    out = {}
    x, y, params = workloads.mlp_inputs(128, (784, 256, 128, 10), seed=0)
    lo, hi = shard_rows(128, rank, world)
    step = MLPTrainStep(params, hi - lo, 0.01, dev, comm=comm)
    T = Timing(dev, step.stream)
    for _ in range(3):
        step.step(x[lo:hi], y[lo:hi])
    dist.barrier()
    e0, e1 = T.events()
    e0.record(step.stream)
    for _ in range(50):
        step.launch()
    e1.record(step.stream)
    step.sync()
    out["dp_step_eager_us"] = max_over_ranks(e0.elapsed_ms(e1) / 50 * 1e3)
    step.capture()
    for _ in range(3):
        step.replay()
    step.sync()
    dist.barrier()
    e0, e1 = T.events()
    e0.record(step.stream)
    for _ in range(50):
        step.replay()
    e1.record(step.stream)
    step.sync()
    out["dp_step_us"] = max_over_ranks(e0.elapsed_ms(e1) / 50 * 1e3)
    # the same step with the all-reduce and the SGD update fused into one kernel over NVLink peer
    # memory (no NCCL on the data path): graph of the nine compute kernels + that kernel
    from novann_b200.train import PeerGroup

    def gather(payload):
        t = torch.zeros(64, dtype=torch.uint8, device=f"cuda:{local}")
        t[:len(payload)] = torch.tensor(list(payload), dtype=torch.uint8)
        outs = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(outs, t)
        return [bytes(o.cpu().tolist())[:len(payload)] for o in outs]

    def all_ranks_ok(flag):
        t = torch.tensor([1.0 if flag else 0.0], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return t.item() > 0

    # Every stage ends with an agreement over all ranks, so that a rank on which CUDA IPC or a
    # step failed never leaves the others inside a collective: the figure is then reported as null.
    peer, why = None, None
    try:
        peer = PeerGroup(rank, world, MLP_PARAMS, dev, allgather=gather, timeout_ms=20000)
    except Exception as e:      # noqa: BLE001 - reported in the line
        why = f"peer group: {e}"
    if not all_ranks_ok(peer is not None):
        out["dp_step_peer_us"] = None
        out["dp_step_peer_skipped"] = (why or "another rank could not map peer memory")[:120]
    else:
        t_step = None
        try:
            pstep = MLPTrainStep(params, hi - lo, 0.01, dev, peer=peer)
            Tp = Timing(dev, pstep.stream)
            for _ in range(2):
                pstep.step(x[lo:hi], y[lo:hi])
            pstep.capture()
            for _ in range(4):
                pstep.replay()
            pstep.sync()
            e0, e1 = Tp.events()
            e0.record(pstep.stream)
            for _ in range(50):
                pstep.replay()
            e1.record(pstep.stream)
            pstep.sync()
            t_step = e0.elapsed_ms(e1) / 50 * 1e3
        except Exception as e:      # noqa: BLE001
            why = f"peer step: {e}"
        if all_ranks_ok(t_step is not None):
            out["dp_step_peer_us"] = max_over_ranks(t_step)
        else:
            out["dp_step_peer_us"] = None
            out["dp_step_peer_skipped"] = (why or "the step failed on another rank")[:120]
    dist.barrier()
    if peer is not None:
        peer._allgather = None       # the barrier above was the rendezvous
        peer.close()
    # the all-reduce alone, on the gradient bucket
    buf = DeviceBuffer(MLP_PARAMS * 4, dev)
    buf.zero(stream=step.stream)
    for _ in range(5):
        comm.allreduce_sum(buf, MLP_PARAMS, stream=step.stream)
    step.sync()
    dist.barrier()
    e0, e1 = T.events()
    e0.record(step.stream)
    for _ in range(50):
        comm.allreduce_sum(buf, MLP_PARAMS, stream=step.stream)
    e1.record(step.stream)
    step.sync()
    out["allreduce_us"] = max_over_ranks(e0.elapsed_ms(e1) / 50 * 1e3)
    out["allreduce_floats"] = MLP_PARAMS
    dist.barrier()
    buf.free()
    comm.close()
    return out


def measure_e2e(dev, tile, n, steps, barrier, max_over_ranks):
    """The sweep through the host-array call on pinned arrays (the headline e2e figure), the same
    bytes moved by plain pinned copies with no kernel (H2D and D2H of each cast issued together,
    one synchronisation per cast: what a synchronous astype replacement can reach at best), and
    the sweep on pageable arrays at a quarter of the size."""
    from novann_b200 import quant
    from novann_b200._lib import check, lib
    from novann_b200.device import DeviceBuffer, Stream, _sptr, device_sync, pinned_empty
    import ctypes as C
    h32 = pinned_empty(n, np.float32)
    h16 = pinned_empty(n, np.uint16)
    for off in range(0, n, tile.size):
        h32[off:off + tile.size] = tile
    h16f = h16.view(np.float16)

    def sweep_host(a32, a16, a16f):
        quant.cast(a32, "bf16", out=a16, device=dev)
        quant.cast(a16, "f32", src_dtype="bf16", out=a32, device=dev)
        quant.cast(a32, np.float16, out=a16f, device=dev)
        quant.cast(a16f, np.float32, out=a32, device=dev)

    sweep_host(h32, h16, h16f)
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        sweep_host(h32, h16, h16f)
    device_sync(dev)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    out = {"e2e_s": e2e_s}
    # ---- ceiling: the same bytes, copies only
    d_in, d_out = DeviceBuffer(n * 4, dev), DeviceBuffer(n * 4, dev)
    s_in, s_out = Stream(dev), Stream(dev)
    vp = C.c_void_p

    def copies_only():
        for src_b, dst_b, hs, hd in ((4, 2, h32, h16), (2, 4, h16, h32), (4, 2, h32, h16), (2, 4, h16, h32)):
            check(lib().nvq_memcpy_h2d(d_in.at(0), vp(hs.ctypes.data), n * src_b, dev, _sptr(s_in)))
            check(lib().nvq_memcpy_d2h(vp(hd.ctypes.data), d_out.at(0), n * dst_b, dev, _sptr(s_out)))
            s_in.sync()
            s_out.sync()
    d_out.zero()
    copies_only()
    barrier()
    t0 = time.perf_counter()
    copies_only()
    out["copy_s"] = max_over_ranks(time.perf_counter() - t0)
    d_in.free()
    d_out.free()
    # ---- pageable arrays (what a plain ndarray is): a quarter of the size
    npg = n // 4
    p32 = np.empty(npg, np.float32)
    p16 = np.empty(npg, np.uint16)
    p32[:] = h32[:npg]
    sweep_host(p32, p16, p16.view(np.float16))
    barrier()
    t0 = time.perf_counter()
    sweep_host(p32, p16, p16.view(np.float16))
    device_sync(dev)
    out["pageable_s"] = max_over_ranks(time.perf_counter() - t0)
    out["pageable_elems"] = npg
    return out


# ------------------------------------------------------------------ GPU arm
def run_ours(args):
    rank, world, local = _dist_env()
    from novann_b200 import _lib, quant, workloads
    from novann_b200.device import DeviceBuffer, Event, Stream, device_sync

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = local
    L = _lib.lib()
    st = Stream(dev)
    n = N_ELEMS

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- inputs resident in HBM before the timed region
    phase("cast sweep: inputs")
    tile = workloads.cast_input(TILE, seed=rank)
    d32 = DeviceBuffer(n * 4, dev)
    d16 = DeviceBuffer(n * 2, dev)
    for off in range(0, n, TILE):
        d32.upload(tile, offset=off * 4)

    def barrier():
        device_sync(dev)
        if dist is not None:
            dist.barrier()
        device_sync(dev)

    def sweep(events=None):
        for i, (src, dst) in enumerate(DIRECTIONS):
            a, b = (d32, d16) if src == "f32" else (d16, d32)
            quant.cast_device(b, dst, a, src, n, stream=st)
            if events is not None:
                events[i + 1].record(st)

    phase("cast sweep: warm-up and timed steps")
    warm = max(3, args.warmup)
    for _ in range(warm):
        sweep()
    barrier()
    sampler = ClockSampler(dev)
    sampler.start()
    ev = [[Event(dev) for _ in range(5)] for _ in range(args.steps)]
    launches0 = L.nvq_launch_count()
    t_start, t_stop = Event(dev), Event(dev)
    t_start.record(st)
    for k in range(args.steps):
        ev[k][0].record(st)
        sweep(ev[k])
    t_stop.record(st)
    barrier()
    launches = L.nvq_launch_count() - launches0
    ms_total = max_over_ranks(t_start.elapsed_ms(t_stop))
    per_kernel = {}
    for i, (src, dst) in enumerate(DIRECTIONS):
        per_kernel[f"{src}->{dst}"] = statistics.mean(ev[k][i].elapsed_ms(ev[k][i + 1])
                                                      for k in range(args.steps))
    value = BYTES_PER_ELEM_STEP * n * args.steps * world / (ms_total * 1e-3) / 1e9
    d32.free()
    d16.free()

    T = Timing(dev, st)
    flat = {}
    for name, fn in (("other cast sizes", measure_cast_sizes), ("quantisers", measure_quantisers),
                     ("linear", measure_linear), ("conv", measure_conv), ("train steps", measure_train_steps)):
        phase(name)
        flat.update(fn(T, rank) if fn is measure_cast_sizes else fn(T, rank, world))
    clocks = sampler.stop()   # sampled over the timed region and the other kernels
    if dist is not None:
        phase("data-parallel step")
        barrier()
        flat.update(measure_dp_step(dev, rank, world, dist, local))
        barrier()
        # aggregate Linear throughput of the job: every rank multiplies its own row shard
        import torch
        t = torch.tensor([flat["linear_fp8_tflops_per_gpu"]], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        flat["linear_fp8_tflops"] = float(t.item())
        t = torch.tensor([flat["linear_fp8_tflops_per_gpu"]], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        flat["linear_fp8_tflops_per_gpu"] = float(t.item())      # the slowest rank's
    else:
        flat["linear_fp8_tflops"] = flat["linear_fp8_tflops_per_gpu"]

    # ---- e2e: host arrays through the astype-replacement call
    phase("e2e through host arrays", 400)
    e2e_steps = max(1, min(args.steps, 5))
    e = measure_e2e(dev, tile, n, e2e_steps, barrier, max_over_ranks)
    e2e_value = BYTES_PER_ELEM_STEP * n * e2e_steps * world / e["e2e_s"] / 1e9
    copy_ceiling = BYTES_PER_ELEM_STEP * n * world / e["copy_s"] / 1e9
    pageable = BYTES_PER_ELEM_STEP * e["pageable_elems"] * world / e["pageable_s"] / 1e9

    phase("cpu baseline and report")
    if rank == 0:
        peak, peak_bf16, which = _peaks()
        dom = max(per_kernel, key=per_kernel.get)
        achieved = 6 * n / (per_kernel[dom] * 1e-3) / 1e9
        cpu = None
        if world == 1:
            cpu_n = 1 << 27
            sweep_cpu = CpuSweep(cpu_n)
            best, detail = None, None
            for _ in range(3):
                s, dt = sweep_cpu.run()
                if best is None or s < best:
                    best, detail = s, dt
            cpu = {"value": BYTES_PER_ELEM_STEP * cpu_n / best / 1e9, "unit": "GB/s", "cores": sweep_cpu.threads,
                   "kind": "port",
                   "sample": f"{cpu_n} of {n} elements, best of 3; bf16 legs C oracle OpenMP "
                             f"{sweep_cpu.threads} threads, fp16 legs ndarray.astype (1 thread)",
                   **{"gbs_" + k.replace("->", "_to_"): v for k, v in detail.items()}}
        # DRAM bytes of the dominant kernel per launch: one ncu capture at 64 Mi elements
        # (profiles/cast_kernels_64Mi_elements.md) counted dram reads equal to the algorithmic
        # reads (no re-reads) and writes short of the algorithmic writes by what was still in L2
        # when the single profiled launch ended; scaled by elements (x16) to this size.
        narrow = dom.startswith("f32")
        ncu_64mi = (268.4e6 + 88.8e6) if narrow else (134.2e6 + 210.7e6)
        line = {
            "metric": "cast_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32<->bf16/f16", "data": "synthetic",
            "config": workload_config(n),
            "roofline": {"bound": "hbm", "kernel": f"cast {dom}", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": which,
                         "traffic": ncu_64mi * 16,
                         "traffic_source": "ncu dram read+write at 64 Mi elements x16 (reads = algorithmic; "
                                           "writes short by the L2-resident tail of the one profiled launch)",
                         "algorithmic_bytes": 6.0 * n, "frac_uses": "algorithmic_bytes",
                         "frac_of_nominal_8tbs": achieved / 8000.0,
                         **{"ms_" + k.replace("->", "_to_"): v for k, v in per_kernel.items()},
                         "cast_64Mi_gbs": flat["cast_64Mi_gbs"], "cast_1Mi_gbs": flat["cast_1Mi_gbs"],
                         "cast_f64_to_f32_gbs": flat["cast_f64_to_f32_gbs"],
                         "linear_fp8_tflops_per_gpu": flat["linear_fp8_tflops_per_gpu"],
                         "linear_fp8_frac_bf16_peak": flat["linear_fp8_frac_bf16_peak"],
                         "linear_fp8_M_per_gpu": flat["linear_fp8_M_per_gpu"],
                         "dp_step_us": flat.get("dp_step_us"), "allreduce_us": flat.get("allreduce_us"),
                         "dp_step_peer_us": flat.get("dp_step_peer_us")},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 12 * n,
                    "d2h_bytes_per_step": 12 * n, "steps": e2e_steps,
                    "api": "novann_b200.quant.cast(host array) -> nvq_cast_host, pinned arrays",
                    "copy_ceiling_gbs": copy_ceiling, "frac_of_copy_ceiling": e2e_value / copy_ceiling,
                    "pageable_gbs": pageable, "pageable_elements": e["pageable_elems"]},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        line.update(flat)       # flat scalar keys: the Linear, the other cast sizes, the DP step ...
        print(json.dumps(line), flush=True)
    faulthandler.cancel_dump_traceback_later()
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------ single small cases
def run_case(name: str, a: list[int]) -> None:
    """One small, self-ending case of one kernel on device 0, for profiler captures: seeded
    inputs, a few launches, exit.  Sizes are larger than the 126 MB L2 (so DRAM counters mean
    something) but hold at most a few GB.

        cast [log2_elems=26 reps=3]      cast64 [log2_elems=26 reps=3]    fp8 [rows=8192 reps=3]
        fp4 [rows=8192 reps=3]           linear [M=4096 N=4096 K=4096 reps=3 in_kernel=0]
        w8a8 [M N K reps]                fewrows [M=16 N=8192 K=8192 reps=3]
        conv [N=128 C=64 HW=56 Cout=128 reps=2]     convnhwc [N=128 C=64 HW=56 Cout=128 reps=3]
        mlp [batch=128 steps=3]          cnn [batch=128 steps=3]
    """
    from novann_b200 import _lib, functional as F, quant, workloads
    from novann_b200._lib import check, lib
    from novann_b200.device import DeviceBuffer, Stream, _sptr, device_sync

    def arg(i, default):
        return a[i] if len(a) > i else default
    st = Stream(0)
    rng = np.random.default_rng(1)
    if name == "cast":
        n, reps = 1 << arg(0, 26), arg(1, 3)
        d32 = DeviceBuffer.from_numpy(workloads.cast_input(n, seed=0), 0)
        d16 = DeviceBuffer(n * 2, 0)
        for _ in range(reps):
            for src, dst in DIRECTIONS:
                s_, d_ = (d32, d16) if src == "f32" else (d16, d32)
                quant.cast_device(d_, dst, s_, src, n, stream=st)
    elif name == "cast64":
        n, reps = 1 << arg(0, 26), arg(1, 3)
        d64 = DeviceBuffer.from_numpy(np.random.default_rng(0).standard_normal(n), 0)
        d32 = DeviceBuffer(n * 4, 0)
        for _ in range(reps):
            quant.cast_device(d32, "f32", d64, "f64", n, stream=st)
            quant.cast_device(d64, "f64", d32, "f32", n, stream=st)
    elif name == "fp8":
        rows, reps, cols = arg(0, 8192), arg(1, 3), 8192
        n = rows * cols
        d = DeviceBuffer.from_numpy(workloads.fp8_input(rows, cols, seed=0), 0)
        q, asi = DeviceBuffer(n, 0), DeviceBuffer(12, 0)
        for _ in range(reps):
            quant.quantize_fp8_tensor_device(q, asi, d, n, "e4m3", stream=st)
            quant.dequantize_fp8_device(d, q, n, "e4m3", 0.01, stream=st)
    elif name == "fp4":
        rows, reps, cols = arg(0, 8192), arg(1, 3), 8192
        d = DeviceBuffer.from_numpy(workloads.fp4_input_bits(rows, cols, seed=0), 0)
        p, s = DeviceBuffer(rows * cols // 2, 0), DeviceBuffer(rows * cols // 32 * 4, 0)
        for _ in range(reps):
            quant.quantize_fp4_b32_device(p, s, d, rows, cols, stream=st)
            quant.dequantize_fp4_b32_device(d, p, s, rows, cols, stream=st)
    elif name in ("linear", "w8a8"):
        m, n, k, reps, in_kernel = arg(0, 4096), arg(1, 4096), arg(2, 4096), arg(3, 3), arg(4, 0)
        xb, _, b = workloads.linear_inputs(m, 8, k, seed=0)
        dx, dw = DeviceBuffer.from_numpy(xb, 0), DeviceBuffer.from_numpy(_random_codes(rng, n, k), 0)
        ds = DeviceBuffer.from_numpy(np.full(n, 1e-3, np.float32), 0)
        dy = DeviceBuffer(m * n * 2, 0)
        if name == "w8a8":
            ws = DeviceBuffer(F.linear_w8a8_workspace_bytes(m, k), 0)
            for _ in range(reps):
                F.linear_w8a8_device(dy, dx, dw, ds, None, m, n, k, ws, stream=st)
        else:
            ws = None if in_kernel else DeviceBuffer(F.linear_workspace_bytes(n, k, "e4m3"), 0)
            for _ in range(reps):
                F.linear_q_device(dy, dx, dw, "e4m3", ds, None, m, n, k, ws, stream=st)
    elif name == "fewrows":
        m, n, k, reps = arg(0, 16), arg(1, 8192), arg(2, 8192), arg(3, 3)
        xb, _, _ = workloads.linear_inputs(m, 8, k, seed=0)
        sets = [(DeviceBuffer.from_numpy(rng.integers(0, 0x7F, (n, k), dtype=np.uint64).astype(np.uint8), 0),
                 DeviceBuffer(F.linear_workspace_bytes(n, k, "e4m3"), 0)) for _ in range(4)]
        dx = DeviceBuffer.from_numpy(xb, 0)
        ds = DeviceBuffer.from_numpy(np.full(n, 1e-3, np.float32), 0)
        dy = DeviceBuffer(m * n * 2, 0)
        for r in range(reps * 4):       # four weight copies in rotation: every call reads DRAM
            dw, ws = sets[r % 4]
            F.linear_q_device(dy, dx, dw, "e4m3", ds, None, m, n, k, ws, stream=st)
    elif name == "conv":
        n, c, hw, cout, reps = arg(0, 128), arg(1, 64), arg(2, 56), arg(3, 128), arg(4, 2)
        x = np.random.default_rng(0).standard_normal((n, c, hw, hw), dtype=np.float32)
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
    elif name == "convnhwc":
        n, c, hw, cout, reps = arg(0, 128), arg(1, 64), arg(2, 56), arg(3, 128), arg(4, 3)
        x = np.random.default_rng(0).standard_normal((n, c, hw, hw), dtype=np.float32)
        wq = rng.integers(0, 0x7F, (cout, c * 9), dtype=np.uint64).astype(np.uint8)
        dx32, dq = DeviceBuffer.from_numpy(x, 0), DeviceBuffer.from_numpy(wq, 0)
        ds = DeviceBuffer.from_numpy(np.full(cout, 1e-3, np.float32), 0)
        dxh, dyh = DeviceBuffer(x.size * 2, 0), DeviceBuffer(n * hw * hw * cout * 2, 0)
        ws = DeviceBuffer(cout * c * 9 * 2, 0)
        F.nchw_f32_to_nhwc_bf16_device(dxh, dx32, n, c, hw * hw, stream=st)
        for _ in range(reps):
            F.conv2d_q_nhwc_device(dyh, dxh, dq, "e4m3", ds, None, ws, n, c, hw, hw, cout, (3, 3), (1, 1), (1, 1),
                                   relu=True, stream=st)
    elif name == "mlp":
        from novann_b200.train import MLPTrainStep
        batch, steps = arg(0, 128), arg(1, 3)
        x, y, params = workloads.mlp_inputs(batch, seed=0)
        step = MLPTrainStep(params, batch, lr=0.01)
        for _ in range(steps):
            step.step(x, y)
    elif name == "cnn":
        from novann_b200.train_cnn import CNNTrainStep, main_cnn_spec
        batch, steps = arg(0, 128), arg(1, 3)
        xs, ys, params = workloads.cnn_inputs(batch, steps=1, seed=0)
        step = CNNTrainStep(main_cnn_spec(), params, batch, (1, 28, 28))
        for _ in range(steps):
            step.step(xs[0], ys[0])
    else:
        raise SystemExit(f"unknown case {name}")
    st.sync()
    device_sync(0)
    F.check_device_errors(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="run one small case of one kernel and exit")
    ap.add_argument("case_args", nargs="*", type=int)
    args = ap.parse_args()
    if args.case:
        run_case(args.case, args.case_args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
