// Quantised-weight Linear forward for few rows (M <= 128): the weight-streaming regime, where
// the time is the time to read the weight once.  The FP8 codes are read from HBM exactly once
// (1 byte per weight; no expanded copy is ever written) and the roles of the operands are
// swapped so that every SM streams a slice of the weight:
//
//   Y^T[n, m] = sum_k W[n, k] * X[m, k]     MMA M = 128 weight rows, MMA N = MP = M rounded up to 16
//
// Work is the list of (128-row weight block, k-block) units, cut into equal contiguous runs,
// one per CTA (so every SM reads the same number of weight bytes whatever N and K are).  A run
// may end in the middle of a weight block: each CTA writes the fp32 partial sums of every
// block it touched to its own slot, and a second kernel adds a block's slots in CTA order
// (deterministic), applies scale and bias and rounds to bf16.
//
// Kernel (one CTA per SM, cta_group::1, warp specialised):
//   warp 0      TMA producer: 128 x 64 weight codes (8 KB, linear) + MP x 64 activations (bf16,
//               128-byte swizzle) per k-block into a ring of five (MP = 128) to eight (MP = 16) slots
//   warp 1      TMEM allocation; one lane issues tcgen05.mma kind::f16 (128 x MP x 16)
//   warps 2-5   epilogue: TMEM -> fp32 partial slot in global memory
//   warps 6-13  converters: expand the codes to bf16 (exact) into the swizzled A-operand slot;
//               groups of warps take alternate k-blocks, so several are expanded concurrently
// Every wait is bounded.
#include "gemm_common.cuh"

namespace {

constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int WROWS = 128;                  // weight rows per block = MMA M
constexpr int A_BYTES = WROWS * BK * 2;     // expanded weight tile
constexpr int RAW_BYTES = WROWS * BK;       // the same weight tile as codes
constexpr int MAX_STAGES = 8;
constexpr int RING_BYTES = 212992;          // 208 KB of operand ring
// A ring slot holds the expanded tile, MP activation rows and the codes; with few rows the
// slots are small and the ring deeper (more weight bytes in flight per SM):
// MP = 16: 26 KB x 8 slots, MP = 128: 40 KB x 5 slots.
__host__ __device__ constexpr int stage_bytes(int MP) { return A_BYTES + MP * BK * 2 + RAW_BYTES; }
__host__ __device__ constexpr int num_stages(int MP) {
    return RING_BYTES / stage_bytes(MP) < MAX_STAGES ? RING_BYTES / stage_bytes(MP) : MAX_STAGES;
}
constexpr int THREADS = 448;                // 2 + 4 epilogue + 8 converter warps
#ifndef NVQ_SMALL_CONV_GROUPS
#define NVQ_SMALL_CONV_GROUPS 2
#endif
constexpr int CONV_GROUPS = NVQ_SMALL_CONV_GROUPS;   // k-blocks being expanded concurrently
static_assert(CONV_GROUPS == 1 || CONV_GROUPS == 2, "more groups than the shallowest ring (5 slots) can feed");
constexpr int ACC_COLS = 128;               // TMEM columns per accumulator
constexpr int TMEM_COLS = 2 * ACC_COLS;
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 1024;

enum { ERR_PRODUCER = 21, ERR_MMA_FULL = 22, ERR_MMA_TMEM = 23, ERR_EPILOGUE = 24, ERR_CONVERT = 25 };

struct SmallParams {
    float* partial;       // [n_blocks][pieces][MP][128] fp32
    int M, MP, N, K;
    int n_blocks, num_kb;
    int total;            // n_blocks * num_kb units
    int quota;            // units per CTA
    int pieces;           // partial slots per weight block
    const float* wscales; // FP4 only: block scales, N x K/32 (folded into the expanded weight)
    int* status;
};

struct Shared {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t raw_full[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// first CTA whose run reaches into weight block nb
__host__ __device__ inline int first_cta_of(int nb, int num_kb, int quota) { return (nb * num_kb) / quota; }

// 16 FP4 E2M1 codes (eight bytes, low nibble first) times their block scale -> 16 bf16 values:
// bf16_rne(fp32(value) * scale), the rule of the FP4 dequantiser.
__device__ __forceinline__ void expand16_fp4(uint32_t w0, uint32_t w1, float scale, uint4& lo, uint4& hi) {
    const uint32_t w[2] = {w0, w1};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t byte = (w[i >> 2] >> (8 * (i & 3))) & 0xFFu;
        uint32_t f01;
        asm("{ .reg .b8 t, z; mov.b16 {t, z}, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(f01) : "h"((uint16_t)byte));
        float v0, v1;
        asm("cvt.f32.f16 %0, %1;" : "=f"(v0) : "h"((uint16_t)(f01 & 0xFFFFu)));
        asm("cvt.f32.f16 %0, %1;" : "=f"(v1) : "h"((uint16_t)(f01 >> 16)));
        o[i] = pack_bf16(__fmul_rn(v0, scale), __fmul_rn(v1, scale));
    }
    lo = make_uint4(o[0], o[1], o[2], o[3]);
    hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// Calls f(nb, kb0, kb1, piece) for every weight block this CTA's run touches, in order.
template <class F>
__device__ __forceinline__ bool for_each_segment(const SmallParams& p, F f) {
    const int u_begin = blockIdx.x * p.quota;
    const int u_end = min(p.total, u_begin + p.quota);
    for (int u = u_begin; u < u_end;) {
        const int nb = u / p.num_kb, kb0 = u - nb * p.num_kb;
        const int kb1 = min(p.num_kb, kb0 + (u_end - u));
        if (!f(nb, kb0, kb1, (int)blockIdx.x - first_cta_of(nb, p.num_kb, p.quota))) return false;
        u += kb1 - kb0;
    }
    return true;
}

template <int FMT>
__global__ void __launch_bounds__(THREADS, 1)
linear_small_m_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const SmallParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    Shared* sh = (Shared*)(smem_raw + (tiles - raw) + RING_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t STAGES = (uint32_t)num_stages(p.MP), STAGE_BYTES = (uint32_t)stage_bytes(p.MP);
    const uint32_t X_OFF = A_BYTES, RAW_OFF = A_BYTES + (uint32_t)p.MP * BK * 2;
    constexpr bool FP4 = FMT == NVQ_E2M1_B32;
    constexpr int CODE_ROW_BYTES = FP4 ? BK / 2 : BK;     // bytes of codes per weight row and k-block
    // the finalising kernel may be scheduled now; it waits for this grid before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; s++) {
            tc::mbar_init(tc::smem_u32(&sh->full[s]), 1 + 8 / CONV_GROUPS);   // producer + a group's warps
            tc::mbar_init(tc::smem_u32(&sh->empty[s]), 1);
            tc::mbar_init(tc::smem_u32(&sh->raw_full[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            tc::mbar_init(tc::smem_u32(&sh->tmem_full[a]), 1);
            tc::mbar_init(tc::smem_u32(&sh->tmem_empty[a]), 4);
        }
        sh->abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&map_w);
        tc::tma_prefetch_desc(&map_x);
    }
    if (warp == 1) {
        tc::tmem_alloc(tc::smem_u32(&sh->tmem_base), TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for_each_segment(p, [&](int nb, int kb0, int kb1, int) {
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_PRODUCER))
                        return false;
                    const uint32_t dst = tiles + stage * STAGE_BYTES;
                    const uint32_t fbar = tc::smem_u32(&sh->full[stage]);
                    tc::mbar_arrive_expect_tx(fbar, p.MP * BK * 2);
                    tc::tma_load_2d(dst + X_OFF, &map_x, fbar, kb * BK, 0);
                    const uint32_t rbar = tc::smem_u32(&sh->raw_full[stage]);
                    tc::mbar_arrive_expect_tx(rbar, WROWS * CODE_ROW_BYTES);
                    tc::tma_load_2d(dst + RAW_OFF, &map_w, rbar, kb * CODE_ROW_BYTES, nb * WROWS);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                return true;
            });
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            int it = 0;
            const uint32_t idesc = tc::idesc_f16(WROWS, p.MP, 1, 1);
            for_each_segment(p, [&](int, int kb0, int kb1, int) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                it++;
                if (!tc::mbar_wait(tc::smem_u32(&sh->tmem_empty[acc]), acc_phase ^ 1, abort_flag, ERR_MMA_TMEM))
                    return false;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!tc::mbar_wait(tc::smem_u32(&sh->full[stage]), phase, abort_flag, ERR_MMA_FULL))
                        return false;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + X_OFF);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        tc::tc_mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc::tc_commit(tc::smem_u32(&sh->empty[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                tc::tc_commit(tc::smem_u32(&sh->tmem_full[acc]));
                return true;
            });
        }
    } else if (warp >= 6) {
        // ------------------------------------------------------------ converters
        // The eight warps form CONV_GROUPS groups; group g expands the units g, g + CONV_GROUPS, ...
        // of this CTA's run, so CONV_GROUPS k-blocks are being expanded at any time.  A group reads
        // the codes of its next unit before it expands the current one, so CONV_GROUPS must stay
        // below the ring depth minus one (the producer refills a slot only after the MMAs of
        // the unit CONV_GROUPS - ring depth back have completed).
        constexpr int GT = 256 / CONV_GROUPS;                 // threads per group
        constexpr int CH = 512 / GT;                          // 16-code chunks per thread and unit
        const int grp = (threadIdx.x - 192) / GT, ct = (threadIdx.x - 192) % GT;
        const int my_units = min(p.total, ((int)blockIdx.x + 1) * p.quota) - (int)blockIdx.x * p.quota;
        // chunk i = 16 codes: row i / 4, quarter i % 4 of the code row (16 bytes of FP8 codes,
        // 8 bytes of packed FP4 codes); FP4 also fetches the chunk's block scale
        uint4 nxt[CH];
        float nsc[CH];
        auto load_codes = [&](uint32_t st, int unit) {
            const uint32_t codes = tiles + st * STAGE_BYTES + RAW_OFF;
#pragma unroll
            for (int j = 0; j < CH; j++) {
                if constexpr (FP4) {
                    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];"
                                 : "=r"(nxt[j].x), "=r"(nxt[j].y)
                                 : "r"(codes + (ct + GT * j) * 8));
                } else {
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(nxt[j].x), "=r"(nxt[j].y), "=r"(nxt[j].z), "=r"(nxt[j].w)
                                 : "r"(codes + (ct + GT * j) * 16));
                }
            }
            if constexpr (FP4) {
                const int ug = (int)blockIdx.x * p.quota + unit;
                const int nb = ug / p.num_kb, kb = ug - nb * p.num_kb;
                const int kblocks = p.K / 32;
#pragma unroll
                for (int j = 0; j < CH; j++) {
                    const int i = ct + GT * j;
                    const int row = nb * WROWS + (i >> 2), blk = kb * 2 + ((i & 3) >> 1);
                    nsc[j] = (row < p.N && blk < kblocks) ? __ldg(p.wscales + (size_t)row * kblocks + blk) : 0.f;
                }
            }
        };
        // ring position of this group's current unit and of its next one, advanced by
        // CONV_GROUPS slots per step (no divisions in the loop)
        uint32_t stage = (uint32_t)grp % STAGES, phase = ((uint32_t)grp / STAGES) & 1u;
        auto advance = [&](uint32_t& st, uint32_t& ph) {
            st += CONV_GROUPS;
            if (st >= STAGES) { st -= STAGES; ph ^= 1u; }
        };
        uint32_t nstage = stage, nphase = phase;
        advance(nstage, nphase);
        bool ok = grp < my_units;
        if (ok) {   // the codes of a unit are read into registers one unit of this group ahead
            ok = tc::mbar_wait(tc::smem_u32(&sh->raw_full[stage]), phase, abort_flag, ERR_CONVERT);
            if (ok) load_codes(stage, grp);
        }
        for (int u = grp; u < my_units && ok; u += CONV_GROUPS) {
            uint4 in[CH];
            float sc[CH];
#pragma unroll
            for (int j = 0; j < CH; j++) { in[j] = nxt[j]; sc[j] = FP4 ? nsc[j] : 0.f; }
            if (u + CONV_GROUPS < my_units) {
                ok = tc::mbar_wait(tc::smem_u32(&sh->raw_full[nstage]), nphase, abort_flag, ERR_CONVERT);
                if (ok) load_codes(nstage, u + CONV_GROUPS);
            }
            // the operand slot is free once the MMAs of its previous use have completed
            ok = ok && tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_CONVERT);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            const uint32_t a_dst = tiles + stage * STAGE_BYTES;
            // 16 codes -> 16-byte chunks 2q, 2q+1 of the 128-byte operand row, placed by the
            // 128-byte swizzle (chunk index XOR row mod 8)
#pragma unroll
            for (int j = 0; j < CH; j++) {
                const int i = ct + GT * j;
                const int r = i >> 2, q = i & 3;
                uint4 lo, hi;
                if constexpr (FP4) expand16_fp4(in[j].x, in[j].y, sc[j], lo, hi);
                else expand16<FMT>(in[j], lo, hi);
                const uint32_t row_base = a_dst + (r >> 3) * 1024 + (r & 7) * 128;
                const uint32_t c0 = (uint32_t)((2 * q) ^ (r & 7)), c1 = (uint32_t)((2 * q + 1) ^ (r & 7));
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(row_base + c0 * 16),
                             "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(row_base + c1 * 16),
                             "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
            }
            // generic-proxy writes -> visible to the tensor core's (async proxy) reads
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&sh->full[stage]));
            stage = nstage;
            phase = nphase;
            advance(nstage, nphase);
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2-5)
        const int quarter = warp & 3;
        int it = 0;
        for_each_segment(p, [&](int nb, int, int, int piece) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            it++;
            bool ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_full[acc]), acc_phase, abort_flag, ERR_EPILOGUE);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) return false;
            tc::tc_fence_after();
            const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            // thread = weight row quarter*32 + lane of the block; column m of the accumulator is
            // activation row m: for a fixed m a warp writes 32 consecutive floats
            float* out = p.partial + ((size_t)(nb * p.pieces + piece) * p.MP) * WROWS + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < p.MP; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (c + j < p.M) out[(size_t)(c + j) * WROWS] = __uint_as_float(r[j]);
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&sh->tmem_empty[acc]));
            return true;
        });
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

// y[m, n] = bf16(scale_n * sum over the slots of n's weight block + bias_n)
__global__ void small_m_finalize_kernel(uint16_t* __restrict__ y, const float* __restrict__ partial,
                                        const float* __restrict__ scales, const float* __restrict__ bias,
                                        SmallParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the partial sums are complete
    const int total = p.M * p.N;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int m = e / p.N, n = e - m * p.N;
        const int nb = n / WROWS, nl = n - nb * WROWS;
        const int first = first_cta_of(nb, p.num_kb, p.quota);
        const int last = ((nb + 1) * p.num_kb - 1) / p.quota;
        const float* src = partial + ((size_t)(nb * p.pieces) * p.MP + m) * WROWS + nl;
        float s = src[0];
        for (int pc = 1; pc <= last - first; pc++) s = __fadd_rn(s, src[(size_t)pc * p.MP * WROWS]);
        const float v = fmaf(s, scales ? scales[n] : 1.f, bias ? bias[n] : 0.f);
        y[e] = (uint16_t)(pack_bf16(v, 0.f) & 0xFFFFu);
    }
}

}  // namespace

size_t nvq_linear_small_m_workspace(size_t M, size_t N, size_t K, int device) {
    const int MP = (int)((M + 15) / 16 * 16);
    const int n_blocks = (int)((N + WROWS - 1) / WROWS), num_kb = (int)((K + BK - 1) / BK);
    const int total = n_blocks * num_kb;
    int grid = nvq_sm_count(device);
    if (grid > total) grid = total;
    const int quota = (total + grid - 1) / grid;
    const int pieces = (num_kb + quota - 1) / quota + 1;
    return (size_t)n_blocks * pieces * MP * WROWS * sizeof(float);
}

nvq_status nvq_linear_launch_small_m(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                     nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                     size_t M, size_t N, size_t K, float* d_partial, int device,
                                     cudaStream_t st) {
    NVQ_REQUIRE(M >= 1 && M <= 128 && K % 16 == 0, "small-M Linear: needs 1 <= M <= 128 and K %% 16 == 0");
    NVQ_REQUIRE(fmt == NVQ_E4M3 || fmt == NVQ_E5M2 || (fmt == NVQ_E2M1_B32 && K % 32 == 0),
                "small-M Linear: FP8 codes, or FP4 block-32 codes with K %% 32 == 0");
    const bool fp4 = fmt == NVQ_E2M1_B32;
    NVQ_REQUIRE(M * N < (1u << 31) && N < (1u << 24) && K < (1u << 24) && N * K < (1ull << 40),
                "small-M Linear: dimension too large");
    SmallParams p;
    p.partial = d_partial;
    p.M = (int)M;
    p.MP = (int)((M + 15) / 16 * 16);
    p.N = (int)N;
    p.K = (int)K;
    p.n_blocks = (int)((N + WROWS - 1) / WROWS);
    p.num_kb = (int)((K + BK - 1) / BK);
    p.total = p.n_blocks * p.num_kb;
    int grid = nvq_sm_count(device);
    if (grid > p.total) grid = p.total;
    p.quota = (p.total + grid - 1) / grid;
    grid = (p.total + p.quota - 1) / p.quota;
    p.pieces = (p.num_kb + p.quota - 1) / p.quota + 1;
    p.wscales = fp4 ? d_scales : nullptr;
    nvq_status s = nvq_status_word(device, &p.status);
    if (s != NVQ_OK) return s;
    CUtensorMap map_w, map_x;
    // codes: linear rows of 64 bytes (FP8) or 32 bytes (64 packed FP4 codes) per k-block
    s = fp4 ? nvq_make_tmap_2d(&map_w, d_wq, N, K / 2, WROWS, BK / 2, 1, 0)
            : nvq_make_tmap_2d(&map_w, d_wq, N, K, WROWS, BK, 1, 0);
    if (s != NVQ_OK) return s;
    s = nvq_make_tmap_2d(&map_x, d_x, M, K, (uint32_t)p.MP, BK, 2, 1);  // bf16, 128-byte swizzle
    if (s != NVQ_OK) return s;
    static std::atomic<bool> attr_set[64][3];   // per device and format; setting twice is harmless
    const int fi = fmt == NVQ_E4M3 ? 0 : (fmt == NVQ_E5M2 ? 1 : 2);
    if (!attr_set[device][fi]) {
        if (fi == 0)
            NVQ_CUDA(cudaFuncSetAttribute(linear_small_m_kernel<NVQ_E4M3>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        else if (fi == 1)
            NVQ_CUDA(cudaFuncSetAttribute(linear_small_m_kernel<NVQ_E5M2>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        else
            NVQ_CUDA(cudaFuncSetAttribute(linear_small_m_kernel<NVQ_E2M1_B32>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set[device][fi] = true;
    }
    if (fi == 0) linear_small_m_kernel<NVQ_E4M3><<<grid, THREADS, SMEM_BYTES, st>>>(map_w, map_x, p);
    else if (fi == 1) linear_small_m_kernel<NVQ_E5M2><<<grid, THREADS, SMEM_BYTES, st>>>(map_w, map_x, p);
    else linear_small_m_kernel<NVQ_E2M1_B32><<<grid, THREADS, SMEM_BYTES, st>>>(map_w, map_x, p);
    NVQ_LAUNCHED();
    if (fp4) d_scales = nullptr;          // block scales are already in the expanded weight
    const int total = p.M * p.N;
    int fgrid = (total + 255) / 256;
    const int cap = nvq_sm_count(device) * 8;
    if (fgrid > cap) fgrid = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(fgrid);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // launch under the main kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NVQ_CUDA(cudaLaunchKernelEx(&cfg, small_m_finalize_kernel, d_y, (const float*)d_partial, d_scales, d_bias, p));
    NVQ_LAUNCHED();
    return NVQ_OK;
}
