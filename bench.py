#!/usr/bin/env python
"""Benchmark of the cast hot path (and, as extra fields, the FP8-weight Linear).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the cast sweep over one 1 Gi-element tensor resident in HBM:
fp32->bf16, bf16->fp32, fp32->fp16, fp16->fp32 (6 algorithmic bytes per element each,
24 per element per step).  The headline metric is achieved HBM GB/s summed over all
ranks (weak scaling: every rank owns its own 1 Gi-element shard, no collective).

`e2e` repeats the same sweep through the host-array call that replaces
``ndarray.astype`` (NumPy array in pinned memory in, NumPy array out), so every byte
crosses PCIe inside the timed region.

`--impl reference` times the reference's CPU path for the same sweep on the host:
``ndarray.astype`` for fp16 (NovaNN's own primitive, single-threaded by nature) and
the CPU oracle's C restatement on all cores for bf16 (the reference has no bf16).
"""
from __future__ import annotations

import argparse
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


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def cpu_cast_sweep(n: int, reps: int = 1):
    """The CPU path for the sweep on n elements; returns (seconds per sweep, detail)."""
    from novann_b200 import workloads
    from oracle import oracle_c
    oc = oracle_c.load()
    x = workloads.cast_input(n, seed=0)
    b16 = np.empty(n, np.uint16)
    f32 = np.empty(n, np.float32)
    t = {}
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        oc.f32_to_bf16_bits(x, out=b16)
        t1 = time.perf_counter()
        oc.bf16_bits_to_f32(b16, out=f32)
        t2 = time.perf_counter()
        with np.errstate(all="ignore"):
            h = x.astype(np.float16)       # the reference's own primitive
        t3 = time.perf_counter()
        h.astype(np.float32)
        t4 = time.perf_counter()
        tot = t4 - t0
        if best is None or tot < best:
            best = tot
            t = {"f32->bf16_c_omp": 6 * n / (t1 - t0) / 1e9, "bf16->f32_c_omp": 6 * n / (t2 - t1) / 1e9,
                 "f32->f16_numpy_astype": 6 * n / (t3 - t2) / 1e9,
                 "f16->f32_numpy_astype": 6 * n / (t4 - t3) / 1e9}
    return best, t, oc.max_threads()


def run_reference(args):
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    n = 1 << 27  # bounded sample of the 1 Gi-element sweep
    sec, detail, threads = None, None, None
    times = []
    for i in range(args.warmup + args.steps):
        s, detail, threads = cpu_cast_sweep(n)
        if i >= args.warmup:
            times.append(s)
    tot = sum(times)
    value = BYTES_PER_ELEM_STEP * n * len(times) / tot / 1e9
    sample = (f"{n} of {N_ELEMS} elements per step, 4 directions: fp16 legs = ndarray.astype "
              f"(1 thread), bf16 legs = C oracle with OpenMP ({threads} threads)")
    line = {
        "impl": "reference", "metric": "cast_hbm_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": tot / len(times) * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32<->bf16/f16", "data": "synthetic",
        "config": {"workload": "cast sweep fp32<->bf16, fp32<->fp16 (CPU sample)", "elements": n},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "reference",
                         "sample": sample, "per_direction_gbs": detail},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def measure_extras(dev, st, rank, world, dist, local):
    """The other kernels of the path, timed with CUDA events on the library's stream.  Where a
    call's working set is below the 126 MB L2, launches rotate over enough operand sets that
    every launch finds its inputs in DRAM (a flushing write between launches would leave dirty
    lines whose write-back lands inside the next timed kernel).  Reported under "extra"; the
    headline metric above is the cast sweep."""
    from novann_b200 import functional as F, quant, workloads
    from novann_b200.device import DeviceBuffer, Event
    from novann_b200.train import MLPTrainStep

    flush = DeviceBuffer(256 << 20, dev)

    def timed(fn, iters=10, warm=3, do_flush=False):
        for _ in range(warm):
            fn()
        tot = 0.0
        for _ in range(iters):
            if do_flush:
                flush.zero(stream=st)
            e0, e1 = Event(dev), Event(dev)
            e0.record(st)
            fn()
            e1.record(st)
            e1.sync()
            tot += e0.elapsed_ms(e1)
        return tot / iters

    out = {}
    peak_bf16 = None
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak_bf16 = float(json.load(open(pk))["bf16_tflops"])
    def timed_rotating(fn, sets, rounds=4):
        """Back-to-back launches that rotate over buffer sets, so that a set is touched again
        only after >= 512 MB of other traffic: every launch reads DRAM, and no flush write-back
        lands inside the timed region."""
        k = len(sets)
        for i in range(k):
            fn(*sets[i])
        st.sync()
        e0, e1 = Event(dev), Event(dev)
        e0.record(st)
        for i in range(rounds * k):
            fn(*sets[i % k])
        e1.record(st)
        e1.sync()
        return e0.elapsed_ms(e1) / (rounds * k)

    def timed_graph(fn, sets, rounds=4):
        """The same rotation recorded once into a CUDA graph (one call per buffer set) and replayed:
        the device time of a call without the host's launch cost, as a serving loop would issue it."""
        import ctypes as C
        from novann_b200._lib import check, lib
        from novann_b200.device import _sptr
        for args_ in sets:
            fn(*args_)
        st.sync()
        check(lib().nvq_graph_begin_capture(dev, _sptr(st)))
        try:
            for args_ in sets:
                fn(*args_)
        finally:
            h = C.c_void_p()
            check(lib().nvq_graph_end_capture(dev, _sptr(st), C.byref(h)))
        graph = C.c_void_p(h.value)
        check(lib().nvq_graph_launch(dev, graph, _sptr(st)))
        st.sync()
        e0, e1 = Event(dev), Event(dev)
        e0.record(st)
        for _ in range(rounds):
            check(lib().nvq_graph_launch(dev, graph, _sptr(st)))
        e1.record(st)
        e1.sync()
        check(lib().nvq_graph_destroy(dev, graph))
        return e0.elapsed_ms(e1) / (rounds * len(sets))

    def n_sets_for(set_bytes):
        return max(2, int(np.ceil((512 << 20) / set_bytes)) + 1)

    # ---- FP8 per tensor: fp32 [16384, 16384 / world] row shard (1 GiB per GPU at world = 1)
    rows = 16384 // world
    n = rows * 16384
    x = workloads.fp8_input(min(rows, 1024), 16384, seed=rank)
    asi = DeviceBuffer(12, dev)
    sets = []
    for _ in range(n_sets_for(5 * n)):
        d32 = DeviceBuffer(n * 4, dev)
        for off in range(0, n, x.size):
            d32.upload(x, offset=off * 4)
        sets.append((d32, DeviceBuffer(n, dev)))
    t = timed_rotating(lambda d32, d8: quant.quantize_fp8_tensor_device(d8, asi, d32, n, "e4m3", stream=st), sets)
    out["fp8_e4m3_amax_quantize_gbs"] = 9 * n / t / 1e6
    t = timed_rotating(lambda d32, d8: quant.dequantize_fp8_device(d32, d8, n, "e4m3", 0.02, stream=st), sets)
    out["fp8_e4m3_dequantize_gbs"] = 5 * n / t / 1e6
    out["fp8_note"] = "%d rotating buffer sets of %.0f MB" % (len(sets), 5 * n / 1e6)
    for bufs in sets:
        for b_ in bufs:
            b_.free()
    # ---- FP4 block 32: bf16 [8192, 8192] (128 MiB in, about the L2 size), rotating sets as above
    r4 = 8192 // world
    xb = workloads.fp4_input_bits(r4, 8192, seed=rank)
    set_bytes = r4 * 8192 * 2.625
    sets = [(DeviceBuffer.from_numpy(xb, dev), DeviceBuffer(r4 * 4096, dev),
             DeviceBuffer(r4 * 256 * 4, dev)) for _ in range(n_sets_for(set_bytes))]
    n_sets = len(sets)
    t = timed_rotating(lambda dx, dp, dsc: quant.quantize_fp4_b32_device(dp, dsc, dx, r4, 8192, stream=st), sets)
    out["fp4_quantize_gbs"] = 2.625 * r4 * 8192 / t / 1e6
    t = timed_rotating(lambda dx, dp, dsc: quant.dequantize_fp4_b32_device(dx, dp, dsc, r4, 8192, stream=st), sets)
    out["fp4_dequantize_gbs"] = 2.625 * r4 * 8192 / t / 1e6
    out["fp4_note"] = "%d rotating buffer sets of %.0f MB, %d launches back to back" % (
        n_sets, set_bytes / 1e6, 4 * n_sets)
    for bufs in sets:
        for b_ in bufs:
            b_.free()
    # ---- FP8-weight Linear forward: M = 4096 (world 1) or 8192 / world rows per GPU; N = K = 4096
    m = 4096 if world == 1 else 8192 // world
    nn = kk = 4096
    rng = np.random.default_rng(rank)
    xb, _, b = workloads.linear_inputs(m, 8, kk, seed=rank)
    wq = rng.integers(0, 0x7F, (nn, kk), dtype=np.uint64).astype(np.uint8)
    wq |= rng.integers(0, 2, (nn, kk), dtype=np.uint64).astype(np.uint8) << 7
    dss = DeviceBuffer.from_numpy(np.full(nn, 1e-3, np.float32), dev)
    dbb = DeviceBuffer.from_numpy(np.zeros(nn, np.float32), dev)
    # rotating operand sets (x, codes, workspace, y): a set comes round again only after the other
    # sets' >= 512 MB went through L2, so every call finds its operands in DRAM
    per_set = m * kk * 2 + nn * kk + nn * kk * 2 + m * nn * 2
    lsets = [(DeviceBuffer.from_numpy(xb, dev), DeviceBuffer.from_numpy(wq, dev),
              DeviceBuffer(F.linear_workspace_bytes(nn, kk, "e4m3"), dev), DeviceBuffer(m * nn * 2, dev))
             for _ in range(n_sets_for(per_set))]
    t = timed_rotating(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, m, nn, kk, ws,
                                                                 stream=st), lsets)
    F.check_device_errors(dev)
    tf = 2.0 * m * nn * kk / t / 1e9
    t_warm = timed_rotating(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, m, nn, kk,
                                                                      ws, stream=st), lsets[:1], rounds=20)
    out["linear_fp8"] = {"M_per_gpu": m, "N": nn, "K": kk, "ms": t, "tflops_per_gpu": tf,
                         "tflops_per_gpu_l2_warm": 2.0 * m * nn * kk / t_warm / 1e9,
                         "frac_of_measured_bf16_peak": tf / peak_bf16 if peak_bf16 else None,
                         "frac_of_nominal_fp8_peak_4500": tf / 4500.0,
                         "note": "bf16 activations x FP8 weight codes; weight expansion pass "
                                 "included; tcgen05 kind::f16 (a bf16-activation GEMM cannot "
                                 "exceed half of FP8 peak); tflops_per_gpu: %d rotating operand sets, every call reads "
                                 "its 112 MB of operands from DRAM; _l2_warm: the same buffers back to back "
                                 "(operands stay in the 126 MB L2)" % len(lsets)}
    for dxx, dw, ws, dy in lsets:
        F.linear_expand_weight_device(ws, dw, "e4m3", None, nn, kk, stream=st)
    t = timed_rotating(lambda dxx, dw, ws, dy: F.linear_expanded_device(dy, dxx, ws, dss, dbb, m, nn, kk,
                                                                        stream=st), lsets)
    F.check_device_errors(dev)
    tfe = 2.0 * m * nn * kk / t / 1e9
    t_warm = timed_rotating(lambda dxx, dw, ws, dy: F.linear_expanded_device(dy, dxx, ws, dss, dbb, m, nn, kk,
                                                                             stream=st), lsets[:1], rounds=20)
    out["linear_fp8_weight_expanded_once"] = {
        "ms": t, "tflops_per_gpu": tfe, "tflops_per_gpu_l2_warm": 2.0 * m * nn * kk / t_warm / 1e9,
        "frac_of_measured_bf16_peak": tfe / peak_bf16 if peak_bf16 else None,
        "note": "contraction alone: the codes were expanded to bf16 once, outside the call "
                "(nvq_linear_expand_weight + nvq_linear_fwd_expanded; 2 bytes per weight kept)"}
    ws8 = DeviceBuffer(F.linear_w8a8_workspace_bytes(m, kk), dev)
    t = timed_rotating(lambda dxx, dw, ws, dy: F.linear_w8a8_device(dy, dxx, dw, dss, dbb, m, nn, kk, ws8,
                                                                    stream=st), lsets)
    F.check_device_errors(dev)
    tf8 = 2.0 * m * nn * kk / t / 1e9
    out["linear_w8a8_variant"] = {"M_per_gpu": m, "N": nn, "K": kk, "ms": t, "tflops_per_gpu": tf8,
                                  "frac_of_nominal_fp8_peak_4500": tf8 / 4500.0,
                                  "note": "NOT the parity path: activations quantised to E4M3 per row "
                                          "inside the call (included in the time), FP8 x FP8 MMAs "
                                          "(kind::f8f6f4); max-abs-rel vs the bf16-activation result "
                                          "is 2.4-3.2e-2, outside the 1e-2 bound"}
    # few rows (serving shape): the weight-streaming kernel; same rotating sets, so the 16 MB of
    # codes come from DRAM on every call
    ms_ = 16
    t = timed_rotating(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, ms_, nn, kk, ws,
                                                                 stream=st), lsets)
    t_warm = timed_rotating(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, ms_, nn, kk,
                                                                      ws, stream=st), lsets[:1], rounds=20)
    t_graph = timed_graph(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dss, dbb, ms_, nn, kk, ws,
                                                                    stream=st), lsets)
    F.check_device_errors(dev)
    out["linear_fp8_few_rows"] = {"M": ms_, "N": nn, "K": kk, "us": t * 1e3, "us_l2_warm": t_warm * 1e3,
                                  "us_cuda_graph": t_graph * 1e3,
                                  "weight_gbs": nn * kk / t / 1e6,
                                  "note": "M <= 128: codes read once (1 byte per weight) and fed to "
                                          "kind::f8f6f4 MMAs as they are, activations carried as two rows "
                                          "of E4M3 codes, operands swapped, split along K with a "
                                          "deterministic reduction kernel; weight_gbs = code bytes / time; us = eager "
                                          "calls from Python (three launches, host-bound), us_cuda_graph = the "
                                          "same rotation replayed from one CUDA graph"}
    for bufs in lsets:
        for b_ in bufs:
            b_.free()
    ws8.free()
    # the same kernel on a weight far larger than L2 (an 8192 x 28672 projection, 235 MB of codes):
    # the streaming rate without the fixed cost of a 16 MB call; two rotating weights
    nl, kl = 28672, 8192
    wl = np.tile(rng.integers(0, 0x7F, (nl // 8, kl), dtype=np.uint8), (8, 1))   # values do not matter here
    xl, _, _ = workloads.linear_inputs(ms_, 8, kl, seed=rank)
    dsl = DeviceBuffer.from_numpy(np.full(nl, 1e-3, np.float32), dev)
    big = [(DeviceBuffer.from_numpy(xl, dev), DeviceBuffer.from_numpy(wl, dev),
            DeviceBuffer(64 << 20, dev), DeviceBuffer(ms_ * nl * 2, dev))   # partial sums need < 8 MB
           for _ in range(2)]
    t = timed_rotating(lambda dxx, dw, ws, dy: F.linear_q_device(dy, dxx, dw, "e4m3", dsl, None, ms_, nl, kl, ws,
                                                                 stream=st), big, rounds=5)
    F.check_device_errors(dev)
    peak_hbm, _ = _peaks()
    out["linear_fp8_few_rows_large"] = {"M": ms_, "N": nl, "K": kl, "us": t * 1e3,
                                        "weight_gbs": nl * kl / t / 1e6,
                                        "frac_of_measured_hbm_peak": nl * kl / t / 1e6 / peak_hbm,
                                        "note": "three kernels per call (activation split, stream, reduction) "
                                                "in the time; 235 MB of codes per call from DRAM"}
    for bufs in big:
        for b_ in bufs:
            b_.free()
    dsl.free()
    # ---- FP8-weight Conv2d forward as an implicit GEMM: x fp32 [128 / world, 64, 56, 56], 3x3, pad 1,
    # 128 output channels (a ResNet-style block); NCHW fp32 in and out, everything on the device
    from novann_b200 import _lib as _l
    cn, cc, chw, cco = max(1, 128 // world), 64, 56, 128
    xcv = rng.standard_normal((cn, cc, chw, chw), dtype=np.float32)
    wcv = rng.integers(0, 0x7F, (cco, cc * 9), dtype=np.uint64).astype(np.uint8)
    d_xc, d_wc = DeviceBuffer.from_numpy(xcv, dev), DeviceBuffer.from_numpy(wcv, dev)
    d_sc = DeviceBuffer.from_numpy(np.full(cco, 1e-3, np.float32), dev)
    crows, ckp = cn * chw * chw, cc * 9
    d_col, d_yb = DeviceBuffer(crows * ckp * 2, dev), DeviceBuffer(crows * cco * 2, dev)
    d_wsc = DeviceBuffer(F.linear_workspace_bytes(cco, ckp, "e4m3"), dev)
    d_oc = DeviceBuffer(crows * cco * 4, dev)
    from novann_b200._lib import check as _check, lib as _lib_fn
    from novann_b200.device import _sptr

    def conv_call():
        _check(_lib_fn().nvq_conv2d_fwd_q(d_oc.at(0), d_xc.at(0), d_wc.at(0), _l.DTYPE_IDS["e4m3"], d_sc.at(0),
                                          None, d_col.at(0), d_yb.at(0), d_wsc.at(0), d_wsc.nbytes, cn, cc,
                                          chw, chw, cco, 3, 3, 1, 1, 1, 1, 0, dev, _sptr(st)))
    t = timed(conv_call, iters=10)
    F.check_device_errors(dev)
    out["conv2d_fp8"] = {"N_per_gpu": cn, "C": cc, "HW": chw, "Cout": cco, "kernel": 3, "ms": t,
                         "tflops_per_gpu": 2.0 * crows * cco * ckp / t / 1e9,
                         "note": "nvq_conv2d_fwd_q: fp32 NCHW -> bf16 NHWC pass, weight expansion, tcgen05 "
                                 "implicit GEMM with 4-D TMA boxes (no patch matrix; output channels on the "
                                 "MMA's M side), fp32 NCHW written by TMA stores from the epilogue; all "
                                 "three kernels in the time"}
    for b_ in (d_xc, d_wc, d_col, d_yb, d_wsc, d_oc):
        b_.free()
    # ---- fp32 MLP train step, batch 128 / world rows per GPU, CUDA-graph replay
    bsz = 128 // world
    xm, ym, params = workloads.mlp_inputs(128, (784, 256, 128, 10), seed=0)
    step = MLPTrainStep(params, bsz, 0.01, dev)
    step.step(xm[:bsz], ym[:bsz])
    step.capture()
    e0, e1 = Event(dev), Event(dev)
    for _ in range(5):
        step.replay()
    step.stream.sync()
    e0.record(step.stream)
    for _ in range(50):
        step.replay()
    e1.record(step.stream)
    e1.sync()
    out["mlp_step_us"] = e0.elapsed_ms(e1) / 50 * 1e3
    # ---- the CNN of the reference's main.py, batch 128 / world per GPU: forward + CE + backward
    # replayed as one CUDA graph, then the two AdamW launches
    from novann_b200.train_cnn import CNNTrainStep, main_cnn_spec
    cb = 128 // world
    xc, yc, cparams = workloads.cnn_inputs(cb, steps=1, seed=0)
    cnn = CNNTrainStep(main_cnn_spec(), cparams, cb, (1, 28, 28), device=dev)
    cnn.step(xc[0], yc[0])
    cnn.capture()
    for _ in range(3):
        cnn.step(xc[0], yc[0])
    e0, e1 = Event(dev), Event(dev)
    e0.record(cnn.stream)
    for _ in range(20):
        cnn.replay()
    e1.record(cnn.stream)
    e1.sync()
    out["cnn_step_us"] = e0.elapsed_ms(e1) / 20 * 1e3
    out["cnn_step_note"] = ("main.py CNN (3 conv + 4 BatchNorm + pool + 2 Linear + Dropout), batch %d per GPU, "
                            "forward + CE + backward + AdamW, %d kernels per step, inputs resident" %
                            (cb, cnn.launches_per_step))
    out["mlp_step_note"] = ("fp32 784-256-128-10, batch %d per GPU, forward + CE + backward + SGD, "
                            "%d kernels replayed as one CUDA graph, no all-reduce in this figure" % (bsz, step.kernels_per_step()))
    return out


def run_ours(args):
    rank, world, local = _dist_env()
    from novann_b200 import _lib, quant, workloads
    from novann_b200.device import DeviceBuffer, Event, Stream, device_sync, pinned_empty

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

    # ---- inputs resident in HBM before the timed region
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

    for _ in range(max(3, args.warmup)):
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
    ms_total = t_start.elapsed_ms(t_stop)
    per_kernel = {}
    for i, (src, dst) in enumerate(DIRECTIONS):
        per_kernel[f"{src}->{dst}"] = statistics.mean(ev[k][i].elapsed_ms(ev[k][i + 1])
                                                      for k in range(args.steps))
    if dist is not None:
        import torch
        t = torch.tensor([ms_total], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    value = BYTES_PER_ELEM_STEP * n * args.steps * world / (ms_total * 1e-3) / 1e9

    d32.free()
    d16.free()
    extra = measure_extras(dev, st, rank, world, dist, local)
    clocks = sampler.stop()   # sampled over the timed region and the extra kernels

    # ---- e2e: host arrays through the astype-replacement call
    h32 = pinned_empty(n, np.float32)
    h16 = pinned_empty(n, np.uint16)
    for off in range(0, n, TILE):
        h32[off:off + TILE] = tile
    h16f = h16.view(np.float16)

    def sweep_host():
        quant.cast(h32, "bf16", out=h16, device=dev)
        quant.cast(h16, "f32", src_dtype="bf16", out=h32, device=dev)
        quant.cast(h32, np.float16, out=h16f, device=dev)
        quant.cast(h16f, np.float32, out=h32, device=dev)

    e2e_steps = max(1, min(args.steps, 5))
    sweep_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        sweep_host()
    device_sync(dev)
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        import torch
        t = torch.tensor([e2e_s], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = BYTES_PER_ELEM_STEP * n * e2e_steps * world / e2e_s / 1e9

    if rank == 0:
        peak, which = _peaks()
        dom = max(per_kernel, key=per_kernel.get)
        achieved = 6 * n / (per_kernel[dom] * 1e-3) / 1e9
        cpu = None
        if world == 1:
            cpu_n = 1 << 27
            sec, detail, threads = cpu_cast_sweep(cpu_n, reps=3)
            cpu = {"value": BYTES_PER_ELEM_STEP * cpu_n / sec / 1e9, "unit": "GB/s", "cores": threads,
                   "kind": "port",
                   "sample": f"{cpu_n} of {n} elements, best of 3 sweeps; bf16 legs: C oracle "
                             f"OpenMP {threads} threads; fp16 legs: ndarray.astype (1 thread)",
                   "per_direction_gbs": detail}
        line = {
            "metric": "cast_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32<->bf16/f16", "data": "synthetic",
            "config": {"workload": "cast sweep fp32->bf16->fp32->fp16->fp32, 1 Gi elements per GPU "
                                   "(BASELINE configs[1], largest size)",
                       "elements_per_gpu": n, "bytes_per_element_step": BYTES_PER_ELEM_STEP,
                       "l2": "inputs (4 GiB + 2 GiB) far exceed the 126 MB L2; no flush needed",
                       "input": "N(0,1) with 1% N(0,sigma=100) + 4096-element edge block; "
                                "2^26-element seeded tile repeated 16x"},
            "roofline": {"bound": "hbm", "kernel": f"cast {dom}", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": which,
                         # dram read + write of the dominant kernel per launch: the ncu capture at
                         # 64 Mi elements (profiles/cast_kernels_64Mi_elements.md) shows reads equal
                         # to the algorithmic reads and no re-reads; scaled by elements to this size
                         "traffic": 6.0 * n, "traffic_source": "ncu at 64 Mi elements, scaled x16",
                         "per_kernel_ms": per_kernel,
                         "frac_of_nominal_8tbs": achieved / 8000.0},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 12 * n,
                    "d2h_bytes_per_step": 12 * n, "steps": e2e_steps,
                    "api": "novann_b200.quant.cast(host array) -> nvq_cast_host"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
