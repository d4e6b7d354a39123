// Per-tensor FP8 (E4M3 "fn" saturating, E5M2 saturating) quantise / dequantise and
// the amax reduction that feeds them.  NovaNN has no quantisation; the rules are:
//   amax = max|x| (NaN ignored);  scale = amax/FMAX, inv = FMAX/amax (1 when amax==0)
//   q = cvt_sat_rne(x * inv)  -- one fp32 multiply, then the conversion
//   x' = float(q) * scale     -- one fp32 multiply
// HBM-bound: amax 4 B/elem, quantise 5 B/elem, dequantise 5 B/elem.
#include <math.h>

#include "elementwise.cuh"

namespace {

template <int FMT>
__device__ __forceinline__ float fmt_max() { return FMT == NVQ_E4M3 ? 448.0f : 57344.0f; }

// two fp32 -> two FP8 codes in a b16 (lo in the low byte)
template <int FMT>
__device__ __forceinline__ uint32_t cvt_fp8x2(float lo, float hi) {
    uint16_t r;
    if (FMT == NVQ_E4M3)
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- amax ---------------------------------------------------------------------
// fmaxf(m, |x|) returns the non-NaN operand, so NaNs drop out; the running maximum of
// non-negative floats is then combined as an unsigned integer (same ordering), which
// makes the result independent of the reduction order.
__global__ void __launch_bounds__(256)
amax_kernel(const float* __restrict__ src, size_t n, unsigned int* __restrict__ out, int vec_ok) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    float m = 0.f;
    size_t n_packets = vec_ok ? n / 8 : 0;
    constexpr int U = 4;
    for (size_t base = tid; base < n_packets; base += stride * U) {
        u32x8 in[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            size_t p = base + (size_t)u * stride;
            if (p < n_packets) in[u] = ldg_stream_256(src + p * 8);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            size_t p = base + (size_t)u * stride;
            if (p < n_packets) {
#pragma unroll
                for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(__uint_as_float(in[u].v[i])));
            }
        }
    }
    for (size_t i = n_packets * 8 + tid; i < n; i += stride) m = fmaxf(m, fabsf(src[i]));
    // warp-shuffle reduction, then one value per warp through shared memory
    unsigned int b = __float_as_uint(m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
    __shared__ unsigned int warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x < 32) {
        b = threadIdx.x < (blockDim.x >> 5) ? warp_max[threadIdx.x] : 0u;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
        if (threadIdx.x == 0 && b) atomicMax(out, b);
    }
}

// ---- quantise: 16 elements per packet (2 x 256-bit loads, one 128-bit store) ----
struct In16 { u32x8 a, b; };

template <int FMT, bool DEVICE_SCALE>
#ifndef NVQ_FP8_UNROLL
#define NVQ_FP8_UNROLL 2
#endif
struct QuantOp {
    static constexpr int VEC = 16;
    static constexpr int UNROLL = NVQ_FP8_UNROLL;
    static constexpr int RESIDENT = 2;
    using In = In16;
    float inv;                 // host-provided (DEVICE_SCALE == false)
    const float* d_amax;       // device amax (DEVICE_SCALE == true)
    float* d_asi;              // {amax, scale, inv} written by thread 0 of block 0

    __device__ __forceinline__ void init() {
        if (DEVICE_SCALE) {
            float amax = *d_amax;
            float scale = 1.f;
            inv = 1.f;
            if (amax != 0.f) {
                scale = __fdiv_rn(amax, fmt_max<FMT>());
                inv = __fdiv_rn(fmt_max<FMT>(), amax);
            }
            if (blockIdx.x == 0 && threadIdx.x == 0) {
                d_asi[0] = amax;
                d_asi[1] = scale;
                d_asi[2] = inv;
            }
        }
    }
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        In r;
        r.a = ldg_stream_256((const char*)src + p * 64);
        r.b = ldg_stream_256((const char*)src + p * 64 + 32);
        return r;
    }
    __device__ __forceinline__ uint32_t one(uint32_t xu) const {
        return spec_f32_to_fp8<FMT>(spec_mul_bits(xu, __float_as_uint(inv)));
    }
    __device__ __forceinline__ void half(const u32x8& a, uint32_t& w0, uint32_t& w1) const {
        if (!any_nonfinite8(a)) {
            float y[8];
#pragma unroll
            for (int i = 0; i < 8; i++) y[i] = __fmul_rn(__uint_as_float(a.v[i]), inv);
            w0 = cvt_fp8x2<FMT>(y[0], y[1]) | (cvt_fp8x2<FMT>(y[2], y[3]) << 16);
            w1 = cvt_fp8x2<FMT>(y[4], y[5]) | (cvt_fp8x2<FMT>(y[6], y[7]) << 16);
        } else {
            w0 = one(a.v[0]) | (one(a.v[1]) << 8) | (one(a.v[2]) << 16) | (one(a.v[3]) << 24);
            w1 = one(a.v[4]) | (one(a.v[5]) << 8) | (one(a.v[6]) << 16) | (one(a.v[7]) << 24);
        }
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& in) const {
        uint4 o;
        half(in.a, o.x, o.y);
        half(in.b, o.z, o.w);
        stg_stream_128((char*)dst + p * 16, o);
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        ((uint8_t*)dst)[i] = (uint8_t)one(((const uint32_t*)src)[i]);
    }
};

// ---- dequantise: 16 codes per packet (128-bit load, 2 x 256-bit stores) ----------
template <int FMT>
struct DequantOp {
    static constexpr int VEC = 16;
    static constexpr int UNROLL = NVQ_FP8_UNROLL;
    static constexpr int RESIDENT = 2;
    using In = uint4;
    float scale;
    __device__ __forceinline__ void init() {}
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        return ldg_stream_128((const char*)src + p * 16);
    }
    __device__ __forceinline__ uint32_t one(uint32_t c) const {
        uint32_t t = spec_fp8_to_f32<FMT>(c);
        if ((t & 0x7FFFFFFFu) > 0x7F800000u) return t;  // NaN code: canonical, signed
        return spec_mul_bits(t, __float_as_uint(scale));
    }
    // four codes of one 32-bit word -> four fp32 words
    __device__ __forceinline__ void word(uint32_t w, uint32_t* o) const {
        // inf / NaN codes take the integer path
        uint32_t special = FMT == NVQ_E4M3 ? ((w & 0x7F7F7F7Fu) + 0x01010101u)
                                           : ((w & 0x7F7F7F7Fu) + 0x04040404u);
        if (!(special & 0x80808080u)) {
            uint32_t h01, h23;
            if (FMT == NVQ_E4M3) {
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)(w & 0xFFFFu)));
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(w >> 16)));
            } else {
                h01 = __byte_perm(w, 0u, 0x1404);  // E5M2 code = top byte of an fp16
                h23 = __byte_perm(w, 0u, 0x3424);
            }
            float f0, f1, f2, f3;
            asm("cvt.f32.f16 %0, %1;" : "=f"(f0) : "h"((uint16_t)(h01 & 0xFFFFu)));
            asm("cvt.f32.f16 %0, %1;" : "=f"(f1) : "h"((uint16_t)(h01 >> 16)));
            asm("cvt.f32.f16 %0, %1;" : "=f"(f2) : "h"((uint16_t)(h23 & 0xFFFFu)));
            asm("cvt.f32.f16 %0, %1;" : "=f"(f3) : "h"((uint16_t)(h23 >> 16)));
            o[0] = __float_as_uint(__fmul_rn(f0, scale));
            o[1] = __float_as_uint(__fmul_rn(f1, scale));
            o[2] = __float_as_uint(__fmul_rn(f2, scale));
            o[3] = __float_as_uint(__fmul_rn(f3, scale));
        } else {
            o[0] = one(w & 0xFFu);
            o[1] = one((w >> 8) & 0xFFu);
            o[2] = one((w >> 16) & 0xFFu);
            o[3] = one(w >> 24);
        }
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& in) const {
        u32x8 lo, hi;
        word(in.x, lo.v);
        word(in.y, lo.v + 4);
        word(in.z, hi.v);
        word(in.w, hi.v + 4);
        stg_stream_256((char*)dst + p * 64, lo);
        stg_stream_256((char*)dst + p * 64 + 32, hi);
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        ((uint32_t*)dst)[i] = one(((const uint8_t*)src)[i]);
    }
};

// ---- per-row (per output channel) quantisation of a weight matrix ----------------------
//   s_r = amax_r / FMAX (1 when the row is all zero);  q = cvt_sat_rne(w * (FMAX / amax_r))
// One block per row: block-wide amax, then the row is read again (from L1/L2) and converted.
__device__ __forceinline__ float load_as_f32(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float load_as_f32(const uint16_t* p, size_t i) {   // bf16 bits
    return __uint_as_float((uint32_t)p[i] << 16);
}

template <int FMT, class T>
__global__ void __launch_bounds__(256)
quantize_rows_kernel(uint8_t* __restrict__ dst, float* __restrict__ scales,
                     const T* __restrict__ src, size_t cols) {
    const T* row = src + (size_t)blockIdx.x * cols;
    uint8_t* out = dst + (size_t)blockIdx.x * cols;
    float m = 0.f;
    for (size_t i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, fabsf(load_as_f32(row, i)));
    unsigned int b = __float_as_uint(m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
    __shared__ unsigned int warp_max[8];
    __shared__ float s_inv;
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) b = max(b, warp_max[w]);
        float amax = __uint_as_float(b), scale = 1.f, inv = 1.f;
        if (amax != 0.f) {
            scale = __fdiv_rn(amax, fmt_max<FMT>());
            inv = __fdiv_rn(fmt_max<FMT>(), amax);
        }
        scales[blockIdx.x] = scale;
        s_inv = inv;
    }
    __syncthreads();
    const uint32_t invu = __float_as_uint(s_inv);
    for (size_t i = threadIdx.x; i < cols; i += blockDim.x)
        out[i] = (uint8_t)spec_f32_to_fp8<FMT>(spec_mul_bits(__float_as_uint(load_as_f32(row, i)), invu));
}

// Fast per-row E4M3 quantisation of bf16 rows (the activations of the W8A8 Linear): one block
// per row, 8 values per 16-byte load, hardware converters.  The row maximum is taken on the bit
// patterns; a row that holds inf / NaN (pattern >= 0x7f80), or whose reciprocal scale overflows,
// is redone lane by lane with the written rules (NaN ignored by the maximum, integer conversion).
__global__ void __launch_bounds__(256)
quantize_rows_bf16_fast_kernel(uint8_t* __restrict__ dst, float* __restrict__ scales,
                               const uint16_t* __restrict__ src, size_t cols) {
    // the GEMM that consumes these codes may start its set-up now; it waits for this grid to
    // finish before its first load
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint16_t* row = src + (size_t)blockIdx.x * cols;
    uint8_t* out = dst + (size_t)blockIdx.x * cols;
    const size_t chunks = cols / 8;
    __shared__ unsigned int warp_max[8];
    __shared__ float s_inv;
    __shared__ int s_slow;
    // rows of up to 8192 values stay in registers between the two passes (4 chunks a thread)
    constexpr int KEEP = 4;
    const bool in_regs = chunks <= (size_t)KEEP * 256;
    uint4 keep[KEEP];
    uint32_t m2 = 0u;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            size_t c = threadIdx.x + (size_t)j * 256;
            keep[j] = c < chunks ? ldg_stream_128(row + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < KEEP; j++) {
            m2 = __vmaxu2(m2, keep[j].x & 0x7FFF7FFFu);
            m2 = __vmaxu2(m2, keep[j].y & 0x7FFF7FFFu);
            m2 = __vmaxu2(m2, keep[j].z & 0x7FFF7FFFu);
            m2 = __vmaxu2(m2, keep[j].w & 0x7FFF7FFFu);
        }
    } else {
        for (size_t c = threadIdx.x; c < chunks; c += blockDim.x) {
            uint4 v = *(const uint4*)(row + c * 8);
            m2 = __vmaxu2(m2, v.x & 0x7FFF7FFFu);
            m2 = __vmaxu2(m2, v.y & 0x7FFF7FFFu);
            m2 = __vmaxu2(m2, v.z & 0x7FFF7FFFu);
            m2 = __vmaxu2(m2, v.w & 0x7FFF7FFFu);
        }
    }
    unsigned int b = max(m2 & 0xFFFFu, m2 >> 16);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) b = max(b, warp_max[w]);
        float amax = __uint_as_float(b << 16), scale = 1.f, inv = 1.f;
        if (amax != 0.f) {
            scale = __fdiv_rn(amax, 448.0f);
            inv = __fdiv_rn(448.0f, amax);
        }
        s_slow = (b >= 0x7F80u) || (__float_as_uint(inv) >= 0x7F800000u);
        scales[blockIdx.x] = scale;
        s_inv = inv;
    }
    __syncthreads();
    if (!s_slow) {
        const float inv = s_inv;
        if (in_regs) {
#pragma unroll
            for (int j = 0; j < KEEP; j++) {
                size_t c = threadIdx.x + (size_t)j * 256;
                if (c >= chunks) continue;
                const uint32_t w[4] = {keep[j].x, keep[j].y, keep[j].z, keep[j].w};
                uint32_t q[4];
#pragma unroll
                for (int i = 0; i < 4; i++)
                    q[i] = cvt_fp8x2<NVQ_E4M3>(__fmul_rn(__uint_as_float(w[i] << 16), inv),
                                               __fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), inv));
                *(uint2*)(out + c * 8) = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
            }
            return;
        }
        for (size_t c = threadIdx.x; c < chunks; c += blockDim.x) {
            uint4 v = *(const uint4*)(row + c * 8);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t q[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                q[i] = cvt_fp8x2<NVQ_E4M3>(__fmul_rn(__uint_as_float(w[i] << 16), inv),
                                           __fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), inv));
            *(uint2*)(out + c * 8) = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
        }
        return;
    }
    // slow path: the written rules
    float m = 0.f;
    for (size_t i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, fabsf(load_as_f32(row, i)));
    b = __float_as_uint(m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) b = max(b, __shfl_xor_sync(0xFFFFFFFFu, b, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) b = max(b, warp_max[w]);
        float amax = __uint_as_float(b), scale = 1.f, inv = 1.f;
        if (amax != 0.f) {
            scale = __fdiv_rn(amax, 448.0f);
            inv = __fdiv_rn(448.0f, amax);
        }
        scales[blockIdx.x] = scale;
        s_inv = inv;
    }
    __syncthreads();
    const uint32_t invu = __float_as_uint(s_inv);
    for (size_t i = threadIdx.x; i < cols; i += blockDim.x)
        out[i] = (uint8_t)spec_f32_to_fp8<NVQ_E4M3>(spec_mul_bits(__float_as_uint(load_as_f32(row, i)), invu));
}

nvq_status launch_amax(const float* d_src, size_t n, float* d_amax, int device, cudaStream_t st) {
    NVQ_CUDA(cudaMemsetAsync(d_amax, 0, sizeof(float), st));
    if (n == 0) return NVQ_OK;
    static std::atomic<int> per_sm_of[64];   // per device
    int per_sm = per_sm_of[device].load(std::memory_order_relaxed);
    if (per_sm == 0) {
        int b = 0;
        NVQ_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, amax_kernel, 256, 0));
        per_sm = b > 0 ? b : 1;
        per_sm_of[device].store(per_sm, std::memory_order_relaxed);
    }
    size_t want = (n / 8 + 256 * 4 - 1) / (256 * 4);
    size_t cap = (size_t)nvq_sm_count(device) * per_sm;
    unsigned grid = (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
    amax_kernel<<<grid, 256, 0, st>>>(d_src, n, (unsigned int*)d_amax, nvq_aligned(d_src, 32));
    NVQ_LAUNCHED();
    return NVQ_OK;
}

bool scale_ok(float s) { return isfinite(s) && s > 0.f; }

}  // namespace

extern "C" nvq_status nvq_amax_f32(const float* d_src, size_t n, float* d_amax, int device,
                                   void* stream) {
    NVQ_REQUIRE(d_amax && (n == 0 || d_src), "nvq_amax_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    return launch_amax(d_src, n, d_amax, device, (cudaStream_t)stream);
}

extern "C" nvq_status nvq_quantize_fp8(uint8_t* d_dst, const float* d_src, size_t n, nvq_dtype fmt,
                                       float inv_scale, int device, void* stream) {
    NVQ_REQUIRE(n == 0 || (d_dst && d_src), "nvq_quantize_fp8: null buffer");
    NVQ_REQUIRE(fmt == NVQ_E4M3 || fmt == NVQ_E5M2, "nvq_quantize_fp8: fmt must be E4M3 or E5M2");
    NVQ_REQUIRE(scale_ok(inv_scale), "nvq_quantize_fp8: inv_scale must be finite and > 0");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (fmt == NVQ_E4M3)
        return ew_launch(QuantOp<NVQ_E4M3, false>{inv_scale, nullptr, nullptr}, d_src, d_dst, n,
                         device, st, 32, 16);
    return ew_launch(QuantOp<NVQ_E5M2, false>{inv_scale, nullptr, nullptr}, d_src, d_dst, n, device,
                     st, 32, 16);
}

extern "C" nvq_status nvq_dequantize_fp8(float* d_dst, const uint8_t* d_src, size_t n,
                                         nvq_dtype fmt, float scale, int device, void* stream) {
    NVQ_REQUIRE(n == 0 || (d_dst && d_src), "nvq_dequantize_fp8: null buffer");
    NVQ_REQUIRE(fmt == NVQ_E4M3 || fmt == NVQ_E5M2, "nvq_dequantize_fp8: fmt must be E4M3 or E5M2");
    NVQ_REQUIRE(scale_ok(scale), "nvq_dequantize_fp8: scale must be finite and > 0");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (fmt == NVQ_E4M3)
        return ew_launch(DequantOp<NVQ_E4M3>{scale}, d_src, d_dst, n, device, st, 16, 32);
    return ew_launch(DequantOp<NVQ_E5M2>{scale}, d_src, d_dst, n, device, st, 16, 32);
}

extern "C" nvq_status nvq_quantize_fp8_tensor(uint8_t* d_dst, float* d_amax_scale_inv,
                                              const float* d_src, size_t n, nvq_dtype fmt,
                                              const float* d_amax_in, int device, void* stream) {
    NVQ_REQUIRE(d_amax_scale_inv && (n == 0 || (d_dst && d_src)),
                "nvq_quantize_fp8_tensor: null buffer");
    NVQ_REQUIRE(fmt == NVQ_E4M3 || fmt == NVQ_E5M2,
                "nvq_quantize_fp8_tensor: fmt must be E4M3 or E5M2");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const float* amax = d_amax_in;
    if (!amax) {
        s = launch_amax(d_src, n, d_amax_scale_inv, device, st);
        if (s != NVQ_OK) return s;
        amax = d_amax_scale_inv;
    }
    // n == 0 still publishes the scales: run one block over zero packets
    size_t n_eff = n;
    if (fmt == NVQ_E4M3) {
        QuantOp<NVQ_E4M3, true> op{1.f, amax, d_amax_scale_inv};
        if (n_eff == 0) {
            ew_vector_kernel<<<1, kEwThreads, 0, st>>>(op, (const void*)d_src, (void*)d_dst, 0, 0);
            NVQ_LAUNCHED();
            return NVQ_OK;
        }
        return ew_launch(op, d_src, d_dst, n, device, st, 32, 16);
    }
    QuantOp<NVQ_E5M2, true> op{1.f, amax, d_amax_scale_inv};
    if (n_eff == 0) {
        ew_vector_kernel<<<1, kEwThreads, 0, st>>>(op, (const void*)d_src, (void*)d_dst, 0, 0);
        NVQ_LAUNCHED();
        return NVQ_OK;
    }
    return ew_launch(op, d_src, d_dst, n, device, st, 32, 16);
}

extern "C" nvq_status nvq_quantize_fp8_rows(uint8_t* d_dst, float* d_scales, const float* d_src,
                                            size_t rows, size_t cols, nvq_dtype fmt, int device,
                                            void* stream) {
    NVQ_REQUIRE(fmt == NVQ_E4M3 || fmt == NVQ_E5M2, "nvq_quantize_fp8_rows: fmt must be E4M3 or E5M2");
    if (rows == 0 || cols == 0) return NVQ_OK;
    NVQ_REQUIRE(d_dst && d_scales && d_src, "nvq_quantize_fp8_rows: null buffer");
    NVQ_REQUIRE(rows < (1u << 31), "nvq_quantize_fp8_rows: too many rows");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (fmt == NVQ_E4M3)
        quantize_rows_kernel<NVQ_E4M3, float><<<(unsigned)rows, 256, 0, st>>>(d_dst, d_scales, d_src, cols);
    else
        quantize_rows_kernel<NVQ_E5M2, float><<<(unsigned)rows, 256, 0, st>>>(d_dst, d_scales, d_src, cols);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

// the same rule for bf16 input rows (activations of the quantised Linear)
nvq_status nvq_quantize_e4m3_rows_bf16(uint8_t* d_dst, float* d_scales, const uint16_t* d_src,
                                       size_t rows, size_t cols, cudaStream_t st) {
    if (cols % 8 == 0 && nvq_aligned(d_src, 16) && nvq_aligned(d_dst, 8))
        quantize_rows_bf16_fast_kernel<<<(unsigned)rows, 256, 0, st>>>(d_dst, d_scales, d_src, cols);
    else
        quantize_rows_kernel<NVQ_E4M3, uint16_t><<<(unsigned)rows, 256, 0, st>>>(d_dst, d_scales, d_src, cols);
    NVQ_LAUNCHED();
    return NVQ_OK;
}
