// Pieces shared by the single-CTA and the CTA-pair Linear kernels.
#pragma once

#include "tc_common.cuh"

struct LinearParams {
    uint16_t* y;           // M x N output: bf16, or fp32 when out_f32 is set
    int out_f32;           // bit 0: fp32 output; bit 1: fused ReLU (v * (v > 0), the reference's formula)
    const uint8_t* wq;     // fused kernels: the weight codes (N x K bytes); else unused
    const float* scales;   // N per-output-channel factors or nullptr (= 1)
    const float* row_scales;  // M per-row factors (quantised activations) or nullptr
    const float* bias;     // N or nullptr (= 0)
    int M, N, K;
    int m_blocks, n_blocks;   // in units of the kernel's own tile
    int num_big;              // work items [0, num_big) are full tiles
    int num_items;            // items [num_big, num_items) are half-width tiles
    int group_m;              // rasterisation: m-blocks per group
    int* status;              // mapped host word: first non-zero give-up code
    // implicit-GEMM convolution (stride 1, zero padding): a CTA's 128-row operand tile is a box
    // of conv_bw x conv_bh output positions of one image; M tiles are numbered image-major
    int conv_bw, conv_bh;     // box (conv_bw = OW)
    int conv_th;              // boxes per image = ceil(OH / conv_bh)
    int conv_images, conv_OH, conv_OW;
    int conv_KW, conv_ph, conv_pw;
    int conv_cpb;             // 64-channel blocks per filter tap = C / 64
};

nvq_status nvq_status_word(int device, int** dev_ptr);

// Y = scale_n * X @ Wd^T + bias_n with Wd (N x K) already 16-bit; Y bf16 or fp32 (out_f32)
nvq_status nvq_linear_bf16_launch(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w_bf16,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int out_f32, int device, cudaStream_t st);

// launchers (gemm.cu: one CTA per 128 x 256 tile; gemm_pair.cu: CTA pair per 256 x 256 tile)
nvq_status nvq_linear_launch_single(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w,
                                    const float* d_scales, const float* d_bias, size_t M, size_t N,
                                    size_t K, int out_f32, int device, cudaStream_t st);
nvq_status nvq_linear_launch_pair(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int out_f32, int device, cudaStream_t st);

nvq_status nvq_linear_launch_pair_fused(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                        nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                        size_t M, size_t N, size_t K, int out_f32, int device, cudaStream_t st);

nvq_status nvq_linear_launch_pair_w8a8(uint16_t* d_y, const uint8_t* d_xq, const float* d_x_scales,
                                       const uint8_t* d_wq, const float* d_w_scales,
                                       const float* d_bias, size_t M, size_t N, size_t K, int device,
                                       cudaStream_t st);

// Convolution as an implicit GEMM on the CTA-pair kernel: x bf16 NHWC, weight bf16 (Cout x
// KH*KW*C, columns ordered (kh, kw, c)), out fp32 NCHW holding bf16-rounded values.
nvq_status nvq_conv_launch_pair_implicit(float* d_out, const uint16_t* d_x_nhwc, const uint16_t* d_w,
                                         const float* d_scales, const float* d_bias, int N, int C,
                                         int H, int W, int Cout, int KH, int KW, int ph, int pw,
                                         int device, cudaStream_t st);

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// AND-reduction + barrier over the THREADS epilogue threads (named barrier 1)
template <int THREADS = 128>
__device__ __forceinline__ bool epilogue_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)ok), "n"(THREADS)
        : "memory");
    return r != 0;
}

// Work item -> tile origin.  Full tiles are walked in groups of `group_m` row blocks (all
// column blocks of a group before the next group) so that the tiles in flight at any time
// form a roughly square patch and share their A and B panels through L2.  The tiles that
// would form a partial last wave are cut into two half-width tiles so that the wave
// spreads over (almost) every CTA.
struct TileRef { int m_blk, n_blk, half, is_half; };
__device__ __forceinline__ TileRef tile_ref(const LinearParams& p, int item) {
    TileRef t;
    int big = item;
    t.half = 0;
    t.is_half = 0;
    if (item >= p.num_big) {
        big = p.num_big + ((item - p.num_big) >> 1);
        t.half = (item - p.num_big) & 1;
        t.is_half = 1;
    }
    const int per_group = p.group_m * p.n_blocks;
    const int g = big / per_group, r = big % per_group;
    const int first = g * p.group_m;
    const int gsize = min(p.group_m, p.m_blocks - first);
    t.m_blk = first + r % gsize;
    t.n_blk = r / gsize;
    // a last column block with at most 128 valid columns runs as a half-width tile
    if (!t.is_half && p.N - t.n_blk * 256 <= 128) t.is_half = 1;
    return t;
}

// fp32 flavour of store_chunk: 32 accumulators -> scale, bias -> 128 bytes of the row
__device__ __forceinline__ void store_chunk_f32(const uint32_t* r, const float* scale, const float* bias,
                                                float* yrow, int n_base, int N, bool vec32, bool relu) {
#pragma unroll
    for (int g = 0; g < 4; g++) {
        u32x8 o;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int cc = g * 8 + j;
            float v = fmaf(__uint_as_float(r[cc]), scale[cc], bias[cc]);
            if (relu) v = __fmul_rn(v, v > 0.f ? 1.f : 0.f);
            o.v[j] = __float_as_uint(v);
        }
        const int n = n_base + g * 8;
        if (n + 8 <= N) {
            if (vec32) {
                stg_stream_256(yrow + g * 8, o);
            } else {
                stg_stream_128(yrow + g * 8, make_uint4(o.v[0], o.v[1], o.v[2], o.v[3]));
                stg_stream_128(yrow + g * 8 + 4, make_uint4(o.v[4], o.v[5], o.v[6], o.v[7]));
            }
        }
    }
}

// Epilogue of one 32-column chunk: 32 fp32 accumulators of this thread's row -> scale,
// bias, bf16, global stores.  `vec32` = rows start on 32-byte boundaries.
__device__ __forceinline__ void store_chunk(const uint32_t* r, const float* scale, const float* bias,
                                            uint16_t* yrow, int n_base, int N, bool vec32, bool relu) {
#pragma unroll
    for (int g = 0; g < 2; g++) {
        u32x8 o;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int cc = g * 16 + 2 * j;
            float v0 = fmaf(__uint_as_float(r[cc]), scale[cc], bias[cc]);
            float v1 = fmaf(__uint_as_float(r[cc + 1]), scale[cc + 1], bias[cc + 1]);
            if (relu) {
                v0 = __fmul_rn(v0, v0 > 0.f ? 1.f : 0.f);
                v1 = __fmul_rn(v1, v1 > 0.f ? 1.f : 0.f);
            }
            o.v[j] = pack_bf16(v0, v1);
        }
        const int n = n_base + g * 16;
        if (vec32 && n + 16 <= N) {
            stg_stream_256(yrow + g * 16, o);
        } else {
            if (n + 8 <= N) stg_stream_128(yrow + g * 16, make_uint4(o.v[0], o.v[1], o.v[2], o.v[3]));
            if (n + 16 <= N) stg_stream_128(yrow + g * 16 + 8, make_uint4(o.v[4], o.v[5], o.v[6], o.v[7]));
        }
    }
}
// one 32-column chunk of output row `row`, columns [n, n + 32), in the output's own type
__device__ __forceinline__ void store_row_chunk(const LinearParams& p, const uint32_t* r,
                                                const float* scale, const float* bias, int row, int n,
                                                bool vec32) {
    const bool relu = (p.out_f32 & 2) != 0;
    if (p.out_f32 & 1)
        store_chunk_f32(r, scale, bias, (float*)p.y + (size_t)row * p.N + n, n, p.N, (p.N % 8) == 0, relu);
    else
        store_chunk(r, scale, bias, p.y + (size_t)row * p.N + n, n, p.N, vec32, relu);
}
#endif
