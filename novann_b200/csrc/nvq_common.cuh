// Shared host/device helpers of the nvq library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/nvq.h"

// ---------------------------------------------------------------- host side
void nvq_set_error(const char* fmt, ...);
extern std::atomic<uint64_t> g_nvq_launches;

#define NVQ_FAIL(code, ...)          \
    do {                             \
        nvq_set_error(__VA_ARGS__);  \
        return (code);               \
    } while (0)

#define NVQ_CUDA(expr)                                                                  \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess)                                                          \
            NVQ_FAIL(NVQ_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                     __FILE__, __LINE__);                                               \
    } while (0)

#define NVQ_REQUIRE(cond, ...)                          \
    do {                                                \
        if (!(cond)) NVQ_FAIL(NVQ_ERR_INVALID, __VA_ARGS__); \
    } while (0)

// Counts a kernel launch and converts a launch error into a status.
#define NVQ_LAUNCHED()                                                                   \
    do {                                                                                 \
        g_nvq_launches.fetch_add(1, std::memory_order_relaxed);                          \
        cudaError_t _e = cudaGetLastError();                                             \
        if (_e != cudaSuccess)                                                           \
            NVQ_FAIL(NVQ_ERR_CUDA, "kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), \
                     __FILE__, __LINE__);                                                \
    } while (0)

// Programmatic dependent launch for kernels that follow one another in a stream: a kernel launched
// with nvq_launch_chained may be scheduled while the previous kernel of the stream is still
// running; its first statement, nvq_chain_sync(), lets the NEXT kernel be scheduled in the same
// way and then waits until the previous one has completed and its writes are visible.  Every
// thread executes it before anything else (a block that returned without waiting would let the
// grid complete, and its successor start, before the predecessor's writes have landed).  Launched
// without the attribute, or after something that is not such a kernel, the two instructions do
// nothing.  Used by the latency-bound fp32 step kernels (2-4 % per training step).  The
// bandwidth-bound elementwise kernels do NOT use it: measured on B200, blocks of the next kernel
// that were placed while the previous one still ran end up unevenly spread over the SMs (64 Mi
// cast 6030 -> 4964 GB/s, FP4 quantise 5664 -> 5241 GB/s).
#ifdef __CUDACC__
__device__ __forceinline__ void nvq_chain_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
static inline void nvq_launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);   // the error, if any, is read by NVQ_LAUNCHED
}
#endif

// Makes `device` current for the calling thread; fails when it is not an sm_100 part.
nvq_status nvq_use_device(int device);
int nvq_sm_count(int device);

static inline bool nvq_aligned(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

// ---------------------------------------------------------------- device side
#ifdef __CUDACC__

// ---- the written conversion rules, scalar, integer only ("spec" path) ----------
// Used for tails, misaligned buffers and every packet that holds a non-finite value,
// so that NaN / inf lanes never depend on what the hardware converters do.

__device__ __forceinline__ uint32_t rne_shift_u32(uint32_t v, int sh) {
    if (sh <= 0) return v;
    if (sh > 31) return 0u;
    uint32_t h = v >> sh;
    uint32_t r = v & ((1u << sh) - 1u);
    uint32_t half = 1u << (sh - 1);
    return h + ((r > half) || (r == half && (h & 1u)));
}

// Saturating RNE of an fp32 magnitude (not NaN) to a tiny float: mbits mantissa bits,
// exponent bias `bias`; fmax_bits = fp32 pattern of the largest finite value.
__device__ __forceinline__ uint32_t small_from_abs(uint32_t a, int mbits, int bias,
                                                   uint32_t fmax_bits, uint32_t max_code) {
    if (a >= fmax_bits) return max_code;
    uint32_t min_normal = (uint32_t)(127 + 1 - bias) << 23;
    if (a >= min_normal) return rne_shift_u32(a - ((uint32_t)(127 - bias) << 23), 23 - mbits);
    int e = (int)(a >> 23);
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    return rne_shift_u32(m, (150 + (1 - bias - mbits)) - e);
}

__device__ __forceinline__ uint32_t spec_f32_to_f16(uint32_t u) {
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) {
        uint32_t pay = (a >> 13) & 0x3FFu;
        return sign | 0x7C00u | (pay ? pay : 1u);
    }
    if (a >= 0x47800000u) return sign | 0x7C00u;
    uint32_t h;
    if (a >= 0x38800000u) {
        h = rne_shift_u32(a - 0x38000000u, 13);
        h = h > 0x7C00u ? 0x7C00u : h;
    } else {
        h = rne_shift_u32((a & 0x7FFFFFu) | 0x800000u, 126 - (int)(a >> 23));
    }
    return sign | h;
}

__device__ __forceinline__ uint32_t spec_f16_to_f32(uint32_t h) {
    uint32_t sign = (h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0x1Fu) return sign | 0x7F800000u | (m << 13);
    if (e == 0u) {
        if (m == 0u) return sign;
        int s = __clz(m) - 21;  // shifts needed to bring the leading one to bit 10
        m <<= s;
        return sign | ((uint32_t)(113 - s) << 23) | ((m & 0x3FFu) << 13);
    }
    return sign | ((e + 112u) << 23) | (m << 13);
}

__device__ __forceinline__ uint32_t spec_f32_to_bf16(uint32_t u) {
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return ((u >> 16) & 0x8000u) | 0x7FC0u;
    return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}

template <int FMT>
__device__ __forceinline__ uint32_t spec_f32_to_fp8(uint32_t u) {
    uint32_t s = (u >> 24) & 0x80u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (FMT == NVQ_E4M3) {
        if (a > 0x7F800000u) return s | 0x7Fu;
        return s | small_from_abs(a, 3, 7, 0x43E00000u, 0x7Eu);
    }
    if (a > 0x7F800000u) return s | 0x7Eu;
    return s | small_from_abs(a, 2, 15, 0x47600000u, 0x7Bu);
}

__device__ __forceinline__ uint32_t spec_f32_to_e2m1(uint32_t u) {
    uint32_t s = (u >> 28) & 0x8u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return s ^ 0x8u;
    return s | small_from_abs(a, 1, 1, 0x40C00000u, 0x7u);
}

template <int FMT>
__device__ __forceinline__ uint32_t spec_fp8_to_f32(uint32_t c) {
    uint32_t sign = (c & 0x80u) << 24;
    uint32_t a = c & 0x7Fu;
    const int mbits = FMT == NVQ_E4M3 ? 3 : 2, bias = FMT == NVQ_E4M3 ? 7 : 15;
    if (FMT == NVQ_E4M3 && a == 0x7Fu) return sign | 0x7FC00000u;
    if (FMT == NVQ_E5M2 && a == 0x7Cu) return sign | 0x7F800000u;
    if (FMT == NVQ_E5M2 && a > 0x7Cu) return sign | 0x7FC00000u;
    uint32_t e = a >> mbits, m = a & ((1u << mbits) - 1u);
    if (e == 0u) {
        if (m == 0u) return sign;
        int s = __clz(m) - (31 - mbits);
        m <<= s;
        return sign | ((uint32_t)(127 + 1 - bias - s) << 23) |
               ((m & ((1u << mbits) - 1u)) << (23 - mbits));
    }
    return sign | ((e + 127u - bias) << 23) | (m << (23 - mbits));
}

// fp32 product x*y with the NaN results a host (SSE) multiply gives, which is what
// the CPU statement of the rules computes: a NaN operand propagates quieted with its
// own sign (x first); 0*inf gives the default NaN 0xffc00000.  Finite results are the
// ordinary round-to-nearest product.
__device__ __forceinline__ uint32_t spec_mul_bits(uint32_t xu, uint32_t yu) {
    if ((xu & 0x7FFFFFFFu) > 0x7F800000u) return xu | 0x00400000u;
    if ((yu & 0x7FFFFFFFu) > 0x7F800000u) return yu | 0x00400000u;
    float p = __fmul_rn(__uint_as_float(xu), __uint_as_float(yu));
    if (p != p) return 0xFFC00000u;
    return __float_as_uint(p);
}

// ---- memory access helpers: streaming 128/256-bit global loads and stores -------
struct __align__(32) u32x8 { uint32_t v[8]; };

// instruction spellings, overridable for measurements
#ifndef NVQ_ST256
#define NVQ_ST256 "st.global.L1::no_allocate.v8.b32"
#endif
#ifndef NVQ_LD128
#define NVQ_LD128 "ld.global.nc.L1::no_allocate.v4.b32"
#endif

__device__ __forceinline__ u32x8 ldg_stream_256(const void* p) {
    u32x8 r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]),
                   "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint4 ldg_stream_128(const void* p) {
    uint4 r;
    asm volatile(NVQ_LD128 " {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_stream_64(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ void stg_stream_256(void* p, const u32x8& r) {
    asm volatile(NVQ_ST256 " [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p),
                 "r"(r.v[0]), "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]),
                 "r"(r.v[6]), "r"(r.v[7])
                 : "memory");
}
__device__ __forceinline__ void stg_stream_128(void* p, const uint4& r) {
    asm volatile("st.global.L1::no_allocate.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x),
                 "r"(r.y), "r"(r.z), "r"(r.w)
                 : "memory");
}
__device__ __forceinline__ void stg_stream_64(void* p, const uint2& r) {
    asm volatile("st.global.L1::no_allocate.v2.b32 [%0], {%1,%2};" ::"l"(p), "r"(r.x), "r"(r.y)
                 : "memory");
}

#endif  // __CUDACC__
