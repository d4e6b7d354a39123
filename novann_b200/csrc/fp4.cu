// FP4 E2M1 quantisation with one fp32 scale per 32 consecutive elements of a row,
// two codes per byte (low nibble first), and the inverse.  NovaNN has no
// quantisation; the rules are:
//   amax_b = max|x| over the block (NaN ignored);  scale_b = amax_b / 6
//   inv_b  = amax_b > 0 ? 6 / amax_b : 0
//   code   = cvt_sat_rne_e2m1(float(x) * inv_b);   byte j = code[2j] | code[2j+1] << 4
//   x'     = bf16_rne(e2m1_value(code) * scale_b)
// One thread owns one block: 64 bytes of bf16 in, 16 bytes of codes + one scale out
// (2.625 bytes per element either way), no shuffles, every access full-sector.
#include <math.h>
#include <stdlib.h>

#include "nvq_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 2;

struct Block32 { u32x8 a, b; };  // 32 bf16 values

// two fp32 -> one byte holding two E2M1 codes (lo in the low nibble)
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; mov.b16 %0, {t, 0}; }"
        : "=h"(r)
        : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t quant_word_fast(uint32_t w0, uint32_t w1, uint32_t w2,
                                                    uint32_t w3, float inv) {
    // 8 bf16 values (four words) -> 8 codes (one word): four converter results (one byte each)
    // gathered with three byte permutes
    const uint32_t w[4] = {w0, w1, w2, w3};
    uint32_t q[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float lo = __fmul_rn(__uint_as_float(w[i] << 16), inv);
        float hi = __fmul_rn(__uint_as_float(w[i] & 0xFFFF0000u), inv);
        q[i] = cvt_e2m1x2(lo, hi);
    }
    return __byte_perm(__byte_perm(q[0], q[1], 0x0040), __byte_perm(q[2], q[3], 0x0040), 0x5410);
}

__device__ __forceinline__ uint32_t quant_one_spec(uint32_t xu, uint32_t invu) {
    return spec_f32_to_e2m1(spec_mul_bits(xu, invu));
}

__device__ __forceinline__ uint32_t quant_word_spec(uint32_t w0, uint32_t w1, uint32_t w2,
                                                    uint32_t w3, uint32_t invu) {
    const uint32_t w[4] = {w0, w1, w2, w3};
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t lo = quant_one_spec(w[i] << 16, invu);
        uint32_t hi = quant_one_spec(w[i] & 0xFFFF0000u, invu);
        out |= (lo | (hi << 4)) << (8 * i);
    }
    return out;
}

__device__ __forceinline__ void quant_block(const Block32& in, uint4& codes, float& scale) {
    // block maximum on the bit patterns: |x| of a bf16 orders like its low 15 bits, two values
    // per word; inf / NaN patterns (>= 0x7f80) come out on top and send the block down the
    // integer path, which recomputes the maximum with NaNs ignored
    uint32_t m2 = 0u;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        m2 = __vmaxu2(m2, in.a.v[i] & 0x7FFF7FFFu);
        m2 = __vmaxu2(m2, in.b.v[i] & 0x7FFF7FFFu);
    }
    const uint32_t m16 = max(m2 & 0xFFFFu, m2 >> 16);
    bool slow = m16 >= 0x7F80u;
    float amax = __uint_as_float(m16 << 16);
    if (slow) {
        amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(in.a.v[i] << 16)),
                                     fabsf(__uint_as_float(in.a.v[i] & 0xFFFF0000u))));
            amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(in.b.v[i] << 16)),
                                     fabsf(__uint_as_float(in.b.v[i] & 0xFFFF0000u))));
        }
    }
    scale = __fdiv_rn(amax, 6.0f);
    float inv = amax > 0.f ? __fdiv_rn(6.0f, amax) : 0.f;
    // a reciprocal that overflowed (subnormal block maximum) also takes the integer path
    slow = slow || (__float_as_uint(inv) >= 0x7F800000u);
    if (!slow) {
        codes.x = quant_word_fast(in.a.v[0], in.a.v[1], in.a.v[2], in.a.v[3], inv);
        codes.y = quant_word_fast(in.a.v[4], in.a.v[5], in.a.v[6], in.a.v[7], inv);
        codes.z = quant_word_fast(in.b.v[0], in.b.v[1], in.b.v[2], in.b.v[3], inv);
        codes.w = quant_word_fast(in.b.v[4], in.b.v[5], in.b.v[6], in.b.v[7], inv);
    } else {
        uint32_t iu = __float_as_uint(inv);
        codes.x = quant_word_spec(in.a.v[0], in.a.v[1], in.a.v[2], in.a.v[3], iu);
        codes.y = quant_word_spec(in.a.v[4], in.a.v[5], in.a.v[6], in.a.v[7], iu);
        codes.z = quant_word_spec(in.b.v[0], in.b.v[1], in.b.v[2], in.b.v[3], iu);
        codes.w = quant_word_spec(in.b.v[4], in.b.v[5], in.b.v[6], in.b.v[7], iu);
    }
}

__global__ void __launch_bounds__(kThreads)
fp4_quant_kernel(const uint16_t* __restrict__ src, uint8_t* __restrict__ packed,
                 float* __restrict__ scales, size_t n_blocks) {
    const size_t stride = (size_t)gridDim.x * kThreads;
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (size_t base = tid; base < n_blocks; base += stride * kUnroll) {
        Block32 in[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            size_t b = base + (size_t)u * stride;
            if (b < n_blocks) {
                in[u].a = ldg_stream_256((const char*)src + b * 64);
                in[u].b = ldg_stream_256((const char*)src + b * 64 + 32);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            size_t b = base + (size_t)u * stride;
            if (b < n_blocks) {
                uint4 codes;
                float scale;
                quant_block(in[u], codes, scale);
                stg_stream_128(packed + b * 16, codes);
                __stcs(scales + b, scale);
            }
        }
    }
}

// ---- dequantise -------------------------------------------------------------------
__device__ __forceinline__ float e2m1_value(uint32_t c) {
    // {0,.5,1,1.5,2,3,4,6}: magnitudes as fp32 patterns from a 3-bit code
    uint32_t m = c & 7u;
    uint32_t bits = m == 0 ? 0u : m == 1 ? 0x3F000000u : (((m >> 1) + 126u) << 23) | ((m & 1u) << 22);
    return __uint_as_float(bits | ((c & 8u) << 28));
}

__device__ __forceinline__ uint32_t dequant_one_spec(uint32_t c, uint32_t su) {
    return spec_f32_to_bf16(spec_mul_bits(__float_as_uint(e2m1_value(c)), su));
}

// one byte (two codes, low nibble first) -> f16x2 holding their exact values
__device__ __forceinline__ uint32_t cvt_f16x2_e2m1x2(uint32_t byte) {
    uint32_t r;
    asm("{ .reg .b8 t, z; mov.b16 {t, z}, %1; cvt.rn.f16x2.e2m1x2 %0, t; }"
        : "=r"(r)
        : "h"((uint16_t)byte));
    return r;
}

// 8 codes (one word) -> 8 bf16 (four words)
__device__ __forceinline__ void dequant_word_fast(uint32_t w, float s, uint32_t* o) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t f01 = cvt_f16x2_e2m1x2((w >> (8 * i)) & 0xFFu);
        float v0, v1;
        asm("cvt.f32.f16 %0, %1;" : "=f"(v0) : "h"((uint16_t)(f01 & 0xFFFFu)));
        asm("cvt.f32.f16 %0, %1;" : "=f"(v1) : "h"((uint16_t)(f01 >> 16)));
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;"
            : "=r"(o[i])
            : "f"(__fmul_rn(v1, s)), "f"(__fmul_rn(v0, s)));
    }
}

__device__ __forceinline__ void dequant_word_spec(uint32_t w, uint32_t su, uint32_t* o) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t lo = dequant_one_spec((w >> (8 * i)) & 0xFu, su);
        uint32_t hi = dequant_one_spec((w >> (8 * i + 4)) & 0xFu, su);
        o[i] = lo | (hi << 16);
    }
}

__global__ void __launch_bounds__(kThreads)
fp4_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                   uint16_t* __restrict__ dst, size_t n_blocks) {
    const size_t stride = (size_t)gridDim.x * kThreads;
    const size_t tid = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (size_t base = tid; base < n_blocks; base += stride * kUnroll) {
        uint4 in[kUnroll];
        float sc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            size_t b = base + (size_t)u * stride;
            if (b < n_blocks) {
                in[u] = ldg_stream_128(packed + b * 16);
                sc[u] = __ldcs(scales + b);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            size_t b = base + (size_t)u * stride;
            if (b < n_blocks) {
                u32x8 lo, hi;
                uint32_t su = __float_as_uint(sc[u]);
                if ((su & 0x7F800000u) != 0x7F800000u) {
                    dequant_word_fast(in[u].x, sc[u], lo.v);
                    dequant_word_fast(in[u].y, sc[u], lo.v + 4);
                    dequant_word_fast(in[u].z, sc[u], hi.v);
                    dequant_word_fast(in[u].w, sc[u], hi.v + 4);
                } else {
                    dequant_word_spec(in[u].x, su, lo.v);
                    dequant_word_spec(in[u].y, su, lo.v + 4);
                    dequant_word_spec(in[u].z, su, hi.v);
                    dequant_word_spec(in[u].w, su, hi.v + 4);
                }
                stg_stream_256((char*)dst + b * 64, lo);
                stg_stream_256((char*)dst + b * 64 + 32, hi);
            }
        }
    }
}

template <class K>
unsigned pick_grid(K kernel, size_t n_blocks, int device, std::atomic<int>* per_sm_of, int resident_cap) {
    int per_sm = per_sm_of[device].load(std::memory_order_relaxed);
    if (per_sm == 0) {
        int b = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kernel, kThreads, 0);
        per_sm = b > 0 ? b : 1;
        // fewer resident blocks = less mixed traffic in flight = better DRAM efficiency
        if (resident_cap > 0 && resident_cap < per_sm) per_sm = resident_cap;
        per_sm_of[device].store(per_sm, std::memory_order_relaxed);
    }
    size_t want = (n_blocks + (size_t)kThreads * kUnroll - 1) / ((size_t)kThreads * kUnroll);
    size_t cap = (size_t)nvq_sm_count(device) * per_sm;
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace

extern "C" nvq_status nvq_quantize_fp4_b32(uint8_t* d_packed, float* d_scales,
                                           const uint16_t* d_src_bf16, size_t rows, size_t cols,
                                           int device, void* stream) {
    NVQ_REQUIRE(cols % 32 == 0, "nvq_quantize_fp4_b32: cols (%zu) must be a multiple of 32", cols);
    size_t n_blocks = rows * (cols / 32);
    if (n_blocks == 0) return NVQ_OK;
    NVQ_REQUIRE(d_packed && d_scales && d_src_bf16, "nvq_quantize_fp4_b32: null buffer");
    NVQ_REQUIRE(nvq_aligned(d_src_bf16, 32) && nvq_aligned(d_packed, 16) && nvq_aligned(d_scales, 4),
                "nvq_quantize_fp4_b32: src must be 32-byte, packed 16-byte, scales 4-byte aligned");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    static std::atomic<int> per_sm_of[64];
    unsigned grid = pick_grid(fp4_quant_kernel, n_blocks, device, per_sm_of, 3);
    fp4_quant_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(d_src_bf16, d_packed, d_scales,
                                                                  n_blocks);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_dequantize_fp4_b32(uint16_t* d_dst_bf16, const uint8_t* d_packed,
                                             const float* d_scales, size_t rows, size_t cols,
                                             int device, void* stream) {
    NVQ_REQUIRE(cols % 32 == 0, "nvq_dequantize_fp4_b32: cols (%zu) must be a multiple of 32", cols);
    size_t n_blocks = rows * (cols / 32);
    if (n_blocks == 0) return NVQ_OK;
    NVQ_REQUIRE(d_packed && d_scales && d_dst_bf16, "nvq_dequantize_fp4_b32: null buffer");
    NVQ_REQUIRE(nvq_aligned(d_dst_bf16, 32) && nvq_aligned(d_packed, 16) && nvq_aligned(d_scales, 4),
                "nvq_dequantize_fp4_b32: dst must be 32-byte, packed 16-byte, scales 4-byte aligned");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    static std::atomic<int> per_sm_of[64];
    unsigned grid = pick_grid(fp4_dequant_kernel, n_blocks, device, per_sm_of, 2);
    fp4_dequant_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(d_packed, d_scales, d_dst_bf16,
                                                                    n_blocks);
    NVQ_LAUNCHED();
    return NVQ_OK;
}
