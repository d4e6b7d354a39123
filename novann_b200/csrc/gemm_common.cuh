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
    int codes_finite;         // fused kernels: the caller vouches that no weight code is NaN / inf
    // implicit-GEMM convolution (stride 1, zero padding): a CTA's 128-row operand tile is a box
    // of conv_bw x conv_bh output positions of one image; M tiles are numbered image-major
    int conv_bw, conv_bh;     // box (conv_bw = OW)
    int conv_th;              // boxes per image = ceil(OH / conv_bh)
    int conv_images, conv_OH, conv_OW;
    int conv_KW, conv_ph, conv_pw, conv_sh;
    int conv_cpb;             // 64-channel blocks per filter tap = C / 64
};

nvq_status nvq_status_word(int device, int** dev_ptr);

// Y = scale_n * X @ Wd^T + bias_n with Wd (N x K) already 16-bit; Y bf16 or fp32 (out_f32).
// kernel: 0 = chosen by M, 1 = one CTA per 128 x 256 tile, 2 = CTA pair per 256 x 256 tile.
nvq_status nvq_linear_bf16_launch(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w_bf16,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int out_f32, int device, cudaStream_t st, int kernel = 0);

// launchers (gemm.cu: one CTA per 128 x 256 tile; gemm_pair.cu: CTA pair per 256 x 256 tile)
nvq_status nvq_linear_launch_single(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w,
                                    const float* d_scales, const float* d_bias, size_t M, size_t N,
                                    size_t K, int out_f32, int device, cudaStream_t st);
nvq_status nvq_linear_launch_pair(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int out_f32, int device, cudaStream_t st);

nvq_status nvq_linear_launch_pair_fused(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                        nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                        size_t M, size_t N, size_t K, int out_f32, int device, cudaStream_t st,
                                        int codes_finite = 0);

nvq_status nvq_linear_launch_pair_w8a8(uint16_t* d_y, const uint8_t* d_xq, const float* d_x_scales,
                                       const uint8_t* d_wq, const float* d_w_scales,
                                       const float* d_bias, size_t M, size_t N, size_t K, int device,
                                       cudaStream_t st);

// Few rows (M <= 128), FP8 codes: weight-streaming kernel with the dequantisation fused (the codes
// are read once, nothing expanded is written); d_partial holds nvq_linear_small_m_workspace bytes.
size_t nvq_linear_small_m_workspace(size_t M, size_t N, size_t K, int device);
// FP8 codes only: the weight codes are the MMA operand as they are (kind::f8f6f4) and each
// activation row is split into two rows of E4M3 codes; workspace = partial sums + those codes.
size_t nvq_linear_small_m_direct_workspace(size_t M, size_t N, size_t K, int device);
// use_cluster: at most 32 rows and a weight that one wave of thread-block clusters covers run
// as two kernels (split, then a clustered stream whose CTAs add their partial sums through
// distributed shared memory) instead of three; other shapes ignore the request.
nvq_status nvq_linear_launch_small_m_direct(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                            nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                            size_t M, size_t N, size_t K, void* d_workspace, int device,
                                            cudaStream_t st, bool use_cluster = false);
nvq_status nvq_linear_launch_small_m(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                     nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                     size_t M, size_t N, size_t K, float* d_partial, int device,
                                     cudaStream_t st);

// Convolution as an implicit GEMM on the CTA-pair kernel: x bf16 NHWC, weight bf16 (Cout x
// KH*KW*C, columns ordered (kh, kw, c)), out fp32 NCHW holding bf16-rounded values.
nvq_status nvq_conv_launch_pair_implicit(float* d_out, const uint16_t* d_x_nhwc, const uint16_t* d_w,
                                         const float* d_scales, const float* d_bias, int N, int C,
                                         int H, int W, int Cout, int KH, int KW, int ph, int pw, int sh, int sw,
                                         int device, cudaStream_t st);

// The same convolution with the operands swapped (output channels on the MMA's M side, up to 256
// output positions on its N side): the form for few output channels.
// With d_out_nhwc set the result goes there as bf16 (N*OH*OW) x Cout (NHWC) instead, ReLU optional.
nvq_status nvq_conv_launch_swapped(float* d_out, const uint16_t* d_x_nhwc, const uint16_t* d_w,
                                   const float* d_scales, const float* d_bias, int N, int C, int H, int W,
                                   int Cout, int KH, int KW, int ph, int pw, int sh, int sw, int device,
                                   cudaStream_t st, uint16_t* d_out_nhwc = nullptr, int relu = 0);

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---- exact FP8 -> bf16 expansion in registers (the converter warps of the fused kernels) ----
// Two FP8 codes (bytes 2*PAIR and 2*PAIR+1 of w) -> two bf16 values.  The code's exponent and
// mantissa bits are dropped into the low end of the bf16 exponent and the top of its mantissa,
// the sign into bit 15; one bf16 multiply by 2^(127 - bias) then fixes the exponent bias and,
// because bf16 arithmetic keeps subnormals, also normalises the codes whose exponent field is
// zero.  Exact for every finite code; the non-finite codes are patched by expand16.
// With b = s << 7 | mag the placed pattern s << 15 | mag << SH equals b << SH + (b & 0x80) *
// (2^8 - 2^SH), per 16-bit lane and without carries between lanes.  It is written as two
// integer multiply-adds on purpose: they issue on the FMA pipe, and the converter warps are
// bound by the half-rate integer / logic pipe that shifts and logic operations use.
template <int FMT, int PAIR>
__device__ __forceinline__ uint32_t expand2(uint32_t w) {
    const uint32_t L = __byte_perm(w, 0u, PAIR == 0 ? 0x4140 : 0x4342);   // codes -> low byte of each lane
    constexpr uint32_t up = FMT == NVQ_E4M3 ? 16u : 32u;                    // 2^SH: mantissa top at bit 6
    constexpr uint32_t lift = 256u - up;
    constexpr uint32_t rebias = FMT == NVQ_E4M3 ? 0x7B807B80u               // 2^120 as bf16, twice
                                                : 0x77807780u;              // 2^112
    uint32_t t, r;
    asm("{\n\t.reg .b32 s, u;\n\t"
        "and.b32 s, %1, 0x00800080;\n\t"
        "mul.lo.u32 u, s, %2;\n\t"
        "mad.lo.u32 %0, %1, %3, u;\n\t}"
        : "=r"(t)
        : "r"(L), "r"(lift), "r"(up));
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(t), "r"(rebias));
    return r;
}

// Lanes of an expand2 result whose code is non-finite (E4M3: 0x7f / 0xff = NaN; E5M2: 0x7c = inf,
// 0x7d.. = NaN) get all exponent bits (and for E4M3 the top mantissa bit) set on top of what the
// bit placement produced: 0x7f -> NaN; 0x7c -> inf exactly (its mantissa is zero), 0x7d.. -> NaN.
// `flags` has bit 7 of a byte set where that code is non-finite.
template <int FMT>
__device__ __forceinline__ uint32_t patch_non_finite(uint32_t r, uint32_t flags, uint32_t sel) {
    const uint32_t f = __byte_perm(flags, 0u, sel);              // flag -> bit 15 / 31 of its lane
    return r | (f - (f >> (FMT == NVQ_E4M3 ? 9 : 8)));           // 0x7fc0 / 0x7f80 per flagged lane
}

// 16 FP8 codes (four words) -> 16 bf16 values (eight words), so that the fused kernels give what
// the expansion pass gives for every code.  The test for non-finite codes is two operations per
// word; the patch itself runs only for chunks that hold one.
template <int FMT>
__device__ __forceinline__ uint32_t non_finite_flags(uint32_t w) {
    const uint32_t x = w | 0x80808080u;      // sign out of the way: 0xff / >= 0xfc marks a non-finite code
    return FMT == NVQ_E4M3 ? __vcmpeq4(x, 0xFFFFFFFFu) : __vcmpgeu4(x, 0xFCFCFCFCu);
}

// CHECK = false: the caller vouches for finite codes and the test (two operations per word, a
// quarter of the converter warps' time) is left out; a NaN / inf code then expands to the finite
// value its bits spell.
template <int FMT, bool CHECK = true>
__device__ __forceinline__ void expand16(const uint4& in, uint4& lo, uint4& hi) {
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        o[2 * i] = expand2<FMT, 0>(w[i]);       // bytes 0, 1
        o[2 * i + 1] = expand2<FMT, 1>(w[i]);   // bytes 2, 3
    }
    const uint32_t any = !CHECK ? 0u : (non_finite_flags<FMT>(w[0]) | non_finite_flags<FMT>(w[1]) |
                                        non_finite_flags<FMT>(w[2]) | non_finite_flags<FMT>(w[3]));
    if (CHECK && __builtin_expect(any != 0, 0)) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t fl = non_finite_flags<FMT>(w[i]) & 0x80808080u;
            o[2 * i] = patch_non_finite<FMT>(o[2 * i], fl, 0x1404);
            o[2 * i + 1] = patch_non_finite<FMT>(o[2 * i + 1], fl, 0x3424);
        }
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
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
    if (p.n_blocks == 1) {
        // one column block: tiles are the row blocks in order (and the single-thread roles that
        // call this once per tile are spared four integer divisions)
        t.m_blk = big;
        t.n_blk = 0;
    } else {
        const int per_group = p.group_m * p.n_blocks;
        const int g = big / per_group, r = big % per_group;
        const int first = g * p.group_m;
        const int gsize = min(p.group_m, p.m_blocks - first);
        t.m_blk = first + r % gsize;
        t.n_blk = r / gsize;
    }
    // a last column block with at most 128 valid columns runs as a half-width tile
    if (!t.is_half && p.N - t.n_blk * 256 <= 128) t.is_half = 1;
    return t;
}

// eight consecutive floats of a 16-byte aligned (shared-memory) array as two 128-bit loads: the
// epilogue's scale / bias reads are broadcasts, and four times fewer of them leave the
// shared-memory pipe to the MMAs' operand reads
__device__ __forceinline__ void load8_f32(float* dst, const float* src) {
    const float4 a = *reinterpret_cast<const float4*>(src);
    const float4 b = *reinterpret_cast<const float4*>(src + 4);
    dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
    dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
}

// fp32 flavour of store_chunk: 32 accumulators -> scale, bias -> 128 bytes of the row
__device__ __forceinline__ void store_chunk_f32(const uint32_t* r, const float* scale, const float* bias,
                                                float* yrow, int n_base, int N, bool vec32, bool relu) {
#pragma unroll
    for (int g = 0; g < 4; g++) {
        u32x8 o;
        float sc[8], bi[8];
        load8_f32(sc, scale + g * 8);
        load8_f32(bi, bias + g * 8);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float v = fmaf(__uint_as_float(r[g * 8 + j]), sc[j], bi[j]);
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
        float sc[16], bi[16];
        load8_f32(sc, scale + g * 16);
        load8_f32(sc + 8, scale + g * 16 + 8);
        load8_f32(bi, bias + g * 16);
        load8_f32(bi + 8, bias + g * 16 + 8);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int cc = g * 16 + 2 * j;
            float v0 = fmaf(__uint_as_float(r[cc]), sc[2 * j], bi[2 * j]);
            float v1 = fmaf(__uint_as_float(r[cc + 1]), sc[2 * j + 1], bi[2 * j + 1]);
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
