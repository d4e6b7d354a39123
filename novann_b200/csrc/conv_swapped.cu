// Quantised Conv2d forward as an implicit GEMM with the operands swapped, for few output
// channels (Cout <= 128 per tile):
//
//   Out^T[co, pos] = sum_{kh, kw, c} W[co, (kh, kw, c)] * X[img, oh*sh + kh - ph, ow*sw + kw - pw, c]
//
// MMA M = 128 output channels (the expanded, tap-ordered weight; rows past Cout read as zeros),
// MMA N = up to 256 output positions of one image (whole output rows), K = 64 channels of one
// filter tap per k-block.  Against the CTA-pair kernel, whose tiles are 256 positions x 128
// channels, one wait / issue / commit round of the MMA warp covers twice the work (the round,
// not the tensor pipe, limits tiles of nine k-blocks), and the epilogue thread owns a channel
// whose positions are consecutive in the NCHW plane: 128-bit stores, scale and bias in registers.
//
//   warp 0     TMA producer: 128 x 64 weight tile (2-D box) + one 4-D box of the bf16 NHWC input
//              (64 channels x OW x bh pixels, traversal strides = the convolution's strides;
//              pixels outside the image read as zeros) per k-block, ring of four 48 KB slots
//   warp 1     TMEM allocation; one lane issues tcgen05.mma kind::f16 (128 x NP x 16) and commits
//   warps 2-5  epilogue: TMEM -> scale, bias, bf16 rounding -> swizzled staging buffer -> TMA store
//              of 32-channel x 32-position boxes into the fp32 NCHW output (register stores for
//              ragged tails and unaligned shapes).  NHWC form (activations that stay bf16 NHWC
//              between chained quantised layers): the box is staged position-major and stored
//              into the bf16 (N*OH*OW) x Cout output, optional ReLU before the rounding
// One CTA per SM, cta_group::1, persistent over (image, row block, channel block) tiles.
// Every wait is bounded.
#include "gemm_common.cuh"

namespace {

constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int CH_ROWS = 128;                // output channels per tile = MMA M
constexpr int MAX_POS = 256;                // output positions per tile = MMA N (at most)
constexpr int A_BYTES = CH_ROWS * BK * 2;   // 16 KB weight tile
constexpr int B_BYTES = MAX_POS * BK * 2;   // 32 KB input tile
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4;
constexpr int THREADS = 192;
constexpr int ACC_COLS = 256;
constexpr int TMEM_COLS = 2 * ACC_COLS;
constexpr int STG_BYTES = 32 * 128;          // one 32-channel x 32-position fp32 box of the output
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 1024 + 4 * 2 * STG_BYTES;

enum { ERR_PRODUCER = 41, ERR_MMA_FULL = 42, ERR_MMA_TMEM = 43, ERR_EPILOGUE = 44 };

struct ConvParams {
    float* out;            // N x Cout x OH x OW fp32 (NCHW form)
    uint16_t* out16;       // (N*OH*OW) x Cout bf16 (NHWC form)
    int relu;              // NHWC form: v * (v > 0) before the bf16 rounding
    const float* scales;   // Cout per-channel factors or nullptr (= 1)
    const float* bias;     // Cout or nullptr
    int images, Cout, OH, OW;
    int bh, th;            // output rows per tile, tiles per image
    int c_blocks;          // ceil(Cout / 128)
    int cpb, KW, num_kb;   // channel blocks per tap, filter width, k-blocks per tile
    int ph, pw, sh;
    int num_tiles;
    int tma_out;           // the epilogue stores whole 32 x 32 boxes by TMA (alignment permitting)
    int* status;
};

struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct Tile { int img, oh0, cb; };
// channel block fastest: the tiles that share an input window run back to back
__device__ __forceinline__ Tile tile_of(const ConvParams& p, int t) {
    Tile r;
    r.cb = t % p.c_blocks;
    const int rest = t / p.c_blocks;
    r.img = rest / p.th;
    r.oh0 = (rest - r.img * p.th) * p.bh;
    return r;
}

template <bool NHWC>
__global__ void __launch_bounds__(THREADS, 1)
conv_swapped_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_out, const ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    Shared* sh = (Shared*)(smem_raw + (tiles - raw) + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;
    const int npos = p.bh * p.OW;                          // positions a full tile holds
    const uint32_t NP = (uint32_t)((npos + 15) / 16 * 16); // MMA N

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            tc::mbar_init(tc::smem_u32(&sh->full[s]), 1);
            tc::mbar_init(tc::smem_u32(&sh->empty[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            tc::mbar_init(tc::smem_u32(&sh->tmem_full[a]), 1);
            tc::mbar_init(tc::smem_u32(&sh->tmem_empty[a]), 4);
        }
        sh->abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&map_w);
        tc::tma_prefetch_desc(&map_x);
        if (p.tma_out) tc::tma_prefetch_desc(&map_out);
    }
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(&sh->tmem_base), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    // the layout pass and the weight expansion run just before this kernel
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
                const Tile tl = tile_of(p, t);
                int kh = 0, kw = 0, cb = 0;
                for (int kb = 0; kb < p.num_kb; kb++) {
                    ok = tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_PRODUCER);
                    if (!ok) break;
                    const uint32_t dst = tiles + stage * STAGE_BYTES;
                    const uint32_t fbar = tc::smem_u32(&sh->full[stage]);
                    tc::mbar_arrive_expect_tx(fbar, A_BYTES + npos * BK * 2);
                    tc::tma_load_2d(dst, &map_w, fbar, kb * BK, tl.cb * CH_ROWS);
                    tc::tma_load_4d(dst + A_BYTES, &map_x, fbar, cb * BK, kw - p.pw,
                                    tl.oh0 * p.sh + kh - p.ph, tl.img);
                    if (++cb == p.cpb) { cb = 0; if (++kw == p.KW) { kw = 0; kh++; } }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int it = 0;
            const uint32_t idesc = tc::idesc_f16(CH_ROWS, NP, 1, 1);   // bf16 x bf16
            for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x, it++) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_empty[acc]), acc_phase ^ 1, abort_flag, ERR_MMA_TMEM);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                for (int kb = 0; kb < p.num_kb; kb++) {
                    ok = tc::mbar_wait(tc::smem_u32(&sh->full[stage]), phase, abort_flag, ERR_MMA_FULL);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        tc::tc_mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    tc::tc_commit(tc::smem_u32(&sh->empty[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc::tc_commit(tc::smem_u32(&sh->tmem_full[acc]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2-5)
        const int quarter = warp & 3;
        const int S = p.OH * p.OW;
        bool ok = true;
        int it = 0;
        uint32_t chunk_no = 0;
        const uint32_t stg_base = tiles + STAGES * STAGE_BYTES + 1024 + (uint32_t)(warp - 2) * 2 * STG_BYTES;
        for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x, it++) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            const Tile tl = tile_of(p, t);
            // thread = output channel; its scale and bias stay in registers for the whole tile
            const int ch = tl.cb * CH_ROWS + quarter * 32 + lane;
            const bool ch_ok = ch < p.Cout;
            const float sc = (p.scales && ch_ok) ? p.scales[ch] : 1.f;
            const float bi = (p.bias && ch_ok) ? p.bias[ch] : 0.f;
            ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_full[acc]), acc_phase, abort_flag, ERR_EPILOGUE);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc::tc_fence_after();
            const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            // column j of the accumulator is position oh0 * OW + j of the image's plane; rows of
            // the box below the image's last output row are not stored
            const int valid = min(p.bh, p.OH - tl.oh0) * p.OW;
            if (NHWC) {
                // row of the (N*OH*OW) x Cout output that holds position 0 of this tile
                const size_t row0 = (size_t)tl.img * S + (size_t)tl.oh0 * p.OW;
#pragma unroll 1
                for (int c = 0; c < valid; c += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(taddr + c, r);
                    tc::tmem_ld_wait();
                    uint32_t h[16];            // bf16 results of positions c + 2j (low half), c + 2j + 1 (high half)
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        float a = fmaf(__uint_as_float(r[2 * j]), sc, bi), b = fmaf(__uint_as_float(r[2 * j + 1]), sc, bi);
                        if (p.relu) { a = a * (a > 0.f ? 1.f : 0.f); b = b * (b > 0.f ? 1.f : 0.f); }
                        h[j] = pack_bf16(a, b);
                    }
                    if (p.tma_out && c + 32 <= valid) {
                        // staged position-major: row = position (64 bytes: this warp's 32 channels),
                        // so for one position the warp's 32 two-byte stores are one contiguous row
                        const uint32_t stg = stg_base + (uint32_t)(chunk_no & 1) * STG_BYTES;
                        chunk_no++;
                        if (lane == 0) tc::bulk_wait_read<1>();
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            asm volatile("st.shared.b16 [%0], %1;" ::"r"(stg + (uint32_t)(2 * j) * 64u + (uint32_t)lane * 2u),
                                         "h"((uint16_t)(h[j] & 0xFFFFu)) : "memory");
                            asm volatile("st.shared.b16 [%0], %1;" ::"r"(stg + (uint32_t)(2 * j + 1) * 64u + (uint32_t)lane * 2u),
                                         "h"((uint16_t)(h[j] >> 16)) : "memory");
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            tc::tma_store_2d(&map_out, stg, tl.cb * CH_ROWS + quarter * 32, (int)(row0 + c));
                            tc::bulk_commit();
                        }
                    } else if (ch_ok) {
                        uint16_t* o = p.out16 + (row0 + c) * (size_t)p.Cout + ch;
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            if (c + 2 * j < valid) o[(size_t)(2 * j) * p.Cout] = (uint16_t)(h[j] & 0xFFFFu);
                            if (c + 2 * j + 1 < valid) o[(size_t)(2 * j + 1) * p.Cout] = (uint16_t)(h[j] >> 16);
                        }
                    }
                }
                tc::tc_fence_before();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(tc::smem_u32(&sh->tmem_empty[acc]));
                continue;
            }
            float* plane = p.out + ((size_t)tl.img * p.Cout + (ch_ok ? ch : 0)) * S + (size_t)tl.oh0 * p.OW;
            const bool vec = ((reinterpret_cast<uintptr_t>(plane) & 15) == 0);
#pragma unroll 1
            for (int c = 0; c < valid; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c, r);
                tc::tmem_ld_wait();
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const uint32_t pk = pack_bf16(fmaf(__uint_as_float(r[j]), sc, bi),
                                                  fmaf(__uint_as_float(r[j + 1]), sc, bi));
                    v[j] = __uint_as_float(pk << 16);                   // the bf16 result, widened again
                    v[j + 1] = __uint_as_float(pk & 0xFFFF0000u);
                }
                if (p.tma_out && c + 32 <= valid) {
                    // A thread's 32 positions are one 128-byte row of a 32-channel box.  Stored from
                    // registers, every warp instruction would touch 32 different lines; the box goes
                    // through a swizzled staging buffer and one TMA store instead (two buffers per
                    // warp: the store of chunk i reads while chunk i + 1 is written).
                    const uint32_t stg = stg_base + (uint32_t)(chunk_no & 1) * STG_BYTES;
                    chunk_no++;
                    if (lane == 0) tc::bulk_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int j8 = 0; j8 < 8; j8++)
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                                         stg + (uint32_t)lane * 128u + (uint32_t)((j8 ^ (lane & 7)) << 4)),
                                     "f"(v[4 * j8]), "f"(v[4 * j8 + 1]), "f"(v[4 * j8 + 2]), "f"(v[4 * j8 + 3])
                                     : "memory");
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tc::tma_store_3d(&map_out, stg, tl.oh0 * p.OW + c, tl.cb * CH_ROWS + quarter * 32, tl.img);
                        tc::bulk_commit();
                    }
                } else if (ch_ok) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        if (vec && c + j + 4 <= valid) {
                            *reinterpret_cast<float4*>(plane + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
#pragma unroll
                            for (int q = 0; q < 4; q++)
                                if (c + j + q < valid) plane[c + j + q] = v[j + q];
                        }
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&sh->tmem_empty[acc]));
        }
        if (lane == 0) tc::bulk_wait_all();     // the staging buffers are read, the boxes written
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(20000);   // let copies in flight land
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    if (warp == 1) tc::tmem_dealloc(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, 0, *abort_flag);
}

}  // namespace

nvq_status nvq_conv_launch_swapped(float* d_out, const uint16_t* d_x_nhwc, const uint16_t* d_w,
                                   const float* d_scales, const float* d_bias, int N, int C, int H, int W,
                                   int Cout, int KH, int KW, int ph, int pw, int sh, int sw, int device,
                                   cudaStream_t st, uint16_t* d_out_nhwc, int relu) {
    const bool nhwc = d_out_nhwc != nullptr;
    const int OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
    NVQ_REQUIRE(OH > 0 && OW > 0 && OW * sw <= 256 && C % 64 == 0 && Cout >= 1,
                "swapped implicit convolution: needs OW * stride <= 256 and C %% 64 == 0");
    // box height: whole output rows, at most 256 positions (and 256 pixels walked down), fewest
    // tiles per image
    int bh = 1;
    long best = -1;
    for (int h = 1; h <= OH && h * OW <= MAX_POS && h * sh <= 256; h++) {
        long tiles = (OH + h - 1) / h;
        if (best < 0 || tiles < best) { best = tiles; bh = h; }
    }
    const size_t K = (size_t)KH * KW * C;
    CUtensorMap map_w, map_x, map_out;
    nvq_status s = nvq_make_tmap_2d(&map_w, d_w, Cout, K, CH_ROWS, BK, 2, 1);
    if (s != NVQ_OK) return s;
    s = nvq_make_tmap_nhwc(&map_x, d_x_nhwc, N, H, W, C, OW, bh, sw, sh);
    if (s != NVQ_OK) return s;
    // TMA stores need every box to start on a 16-byte boundary: planes and tiles of a multiple of
    // four positions; otherwise the epilogue stores from registers
    const size_t S = (size_t)OH * OW;
    // NHWC form: boxes of 32 channels x 32 rows of the (N*OH*OW) x Cout bf16 matrix; a box may start
    // at any row, its channel offset is a multiple of 32 (64 bytes)
    const bool tma_out = nhwc ? (Cout % 8 == 0 && nvq_aligned(d_out_nhwc, 16) && (size_t)N * S < (1u << 31))
                              : (S % 4 == 0 && (bh * OW) % 4 == 0 && nvq_aligned(d_out, 16));
    if (tma_out && nhwc) {
        s = nvq_make_tmap_2d(&map_out, d_out_nhwc, (uint64_t)N * S, (uint64_t)Cout, 32, 32, 2, 0);
        if (s != NVQ_OK) return s;
    } else if (tma_out) {
        s = nvq_make_tmap_nchw_out(&map_out, d_out, N, Cout, S);
        if (s != NVQ_OK) return s;
    } else {
        map_out = map_w;   // never used
    }
    static std::atomic<bool> attr_set[64];   // per device; setting the attribute twice is harmless
    if (!attr_set[device]) {
        NVQ_CUDA(cudaFuncSetAttribute(conv_swapped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        NVQ_CUDA(cudaFuncSetAttribute(conv_swapped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set[device] = true;
    }
    ConvParams p = {};
    p.out = d_out;
    p.out16 = d_out_nhwc;
    p.relu = relu;
    p.scales = d_scales;
    p.bias = d_bias;
    p.images = N; p.Cout = Cout; p.OH = OH; p.OW = OW;
    p.bh = bh; p.th = (OH + bh - 1) / bh;
    p.c_blocks = (Cout + CH_ROWS - 1) / CH_ROWS;
    p.cpb = C / 64; p.KW = KW; p.num_kb = KH * KW * (C / 64);
    p.ph = ph; p.pw = pw; p.sh = sh;
    p.num_tiles = N * p.th * p.c_blocks;
    p.tma_out = tma_out ? 1 : 0;
    s = nvq_status_word(device, &p.status);
    if (s != NVQ_OK) return s;
    int grid = nvq_sm_count(device);
    if (grid > p.num_tiles) grid = p.num_tiles;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // set up under the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (nhwc) NVQ_CUDA(cudaLaunchKernelEx(&cfg, conv_swapped_kernel<true>, map_w, map_x, map_out, p));
    else NVQ_CUDA(cudaLaunchKernelEx(&cfg, conv_swapped_kernel<false>, map_w, map_x, map_out, p));
    NVQ_LAUNCHED();
    return NVQ_OK;
}
