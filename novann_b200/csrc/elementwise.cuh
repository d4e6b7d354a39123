// Grid-stride driver for the HBM-bound elementwise conversions.
//
// An "op" converts packets of Op::VEC consecutive elements held in registers:
//   Op::In  load(const void* src, size_t packet)        256/128-bit streaming loads
//   void    store(void* dst, size_t packet, const In&)   convert + 128/256-bit stores
//   void    scalar(const void* src, void* dst, size_t i) one element by the written rules
//   void    init()                                        once per thread, before the loop
//   Op::RESIDENT                                          cap on resident blocks per SM (0 = none)
// Every thread keeps Op::UNROLL packets in flight; consecutive threads own
// consecutive packets so each warp-wide access covers whole 32-byte sectors once.
#pragma once

#include <stdlib.h>

#include "nvq_common.cuh"

constexpr int kEwThreads = 256;

template <class Op>
__global__ void __launch_bounds__(kEwThreads)
ew_vector_kernel(Op op, const void* __restrict__ src, void* __restrict__ dst, size_t n_packets,
                 size_t n) {
    const size_t tid = (size_t)blockIdx.x * kEwThreads + threadIdx.x;
    op.init();
    // grid-stride over packets: at any moment the whole grid works on one contiguous window
    // of the tensor (a per-block contiguous slice measured the same at 1 Gi elements and 5 %
    // slower at 64 Mi)
    const size_t stride = (size_t)gridDim.x * kEwThreads;
    for (size_t base = tid; base < n_packets; base += stride * Op::UNROLL) {
        typename Op::In in[Op::UNROLL];
#pragma unroll
        for (int u = 0; u < Op::UNROLL; u++) {
            size_t p = base + (size_t)u * stride;
            if (p < n_packets) in[u] = op.load(src, p);
        }
#pragma unroll
        for (int u = 0; u < Op::UNROLL; u++) {
            size_t p = base + (size_t)u * stride;
            if (p < n_packets) op.store(dst, p, in[u]);
        }
    }

    // ragged tail: fewer than VEC elements, one per thread
    size_t tail0 = n_packets * Op::VEC;
    if (tail0 + tid < n) op.scalar(src, dst, tail0 + tid);
}

template <class Op>
__global__ void __launch_bounds__(kEwThreads)
ew_scalar_kernel(Op op, const void* __restrict__ src, void* __restrict__ dst, size_t n) {
    const size_t stride = (size_t)gridDim.x * kEwThreads;
    op.init();
    for (size_t i = (size_t)blockIdx.x * kEwThreads + threadIdx.x; i < n; i += stride)
        op.scalar(src, dst, i);
}

// Launch heuristic: a grid that fills every SM to the occupancy the kernel reaches
// (resident blocks x SM count) and no more, so each thread walks a long grid-stride
// loop; small inputs get just enough blocks to cover their packets.
template <class Op>
nvq_status ew_launch(Op op, const void* src, void* dst, size_t n, int device, cudaStream_t st,
                     size_t src_align, size_t dst_align) {
    if (n == 0) return NVQ_OK;
    int sms = nvq_sm_count(device);
    if (nvq_aligned(src, src_align) && nvq_aligned(dst, dst_align)) {
        static std::atomic<int> per_sm_of[64];   // resident blocks per SM, per device (0 = not asked yet)
        int per_sm = per_sm_of[device].load(std::memory_order_relaxed);
        if (per_sm == 0) {
            int b = 0;
            NVQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, ew_vector_kernel<Op>,
                                                                   kEwThreads, 0));
            per_sm = b > 0 ? b : 1;
            // Mixed read/write streams lose DRAM efficiency when too much traffic is in flight
            // (measured on B200: ~80-100 KB of loads + stores per SM is the sweet spot; full
            // occupancy costs the write-heavy kernels 5-7 %), so an op may cap its resident blocks.
            if (Op::RESIDENT > 0 && Op::RESIDENT < per_sm) per_sm = Op::RESIDENT;
            per_sm_of[device].store(per_sm, std::memory_order_relaxed);
        }
        size_t n_packets = n / Op::VEC;
        size_t want = (n_packets + (size_t)kEwThreads * Op::UNROLL - 1) /
                      ((size_t)kEwThreads * Op::UNROLL);
        size_t cap = (size_t)sms * per_sm;
        unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
        ew_vector_kernel<Op><<<grid, kEwThreads, 0, st>>>(op, src, dst, n_packets, n);
    } else {
        size_t want = (n + kEwThreads - 1) / kEwThreads;
        size_t cap = (size_t)sms * 8;
        unsigned grid = (unsigned)(want < cap ? want : cap);
        ew_scalar_kernel<Op><<<grid, kEwThreads, 0, st>>>(op, src, dst, n);
    }
    NVQ_LAUNCHED();
    return NVQ_OK;
}

// ---- packet level helpers -------------------------------------------------------

// true when any of the 8 fp32 words is inf or NaN (x*0 is NaN exactly then)
__device__ __forceinline__ bool any_nonfinite8(const u32x8& a) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) acc = fmaf(__uint_as_float(a.v[i]), 0.f, acc);
    return acc != acc;
}
