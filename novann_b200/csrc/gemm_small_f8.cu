// FP8-weight Linear forward for few rows (M <= 128), direct form: the weight codes go from HBM
// into the tensor cores' operand slots by TMA and are never touched by a thread.
//
// tcgen05.mma.kind::f8f6f4 multiplies 8-bit float codes by 8-bit float codes.  The activations are
// bf16 (8 significant bits), so each row of X is first written as TWO rows of E4M3 codes:
//
//   a_m  = 2^(floor(log2 max_k |x[m,k]|) - 7)              a power of two: x / a_m is exact, < 256
//   p1   = e4m3_rn(x / a_m)                                 the leading 4 significant bits
//   p2   = e4m3_rn(16 * (x / a_m - p1))                     the remaining 4 bits (exact: the
//                                                           residual of an 8-bit value has <= 4)
//   x    = a_m * (p1 + p2 / 16)                             exactly, for |x| >= a_m / 64; smaller
//                                                           elements (below 2^-13 of the row's
//                                                           maximum) keep an absolute error
//                                                           <= a_m * 2^-14 (E4M3 subnormal spacing)
//
//   Y[m, n] = bf16( a_m * s_n * (sum_k w[n,k] p1[m,k] + sum_k w[n,k] p2[m,k] / 16) + b_n )
//
// Operands are swapped as in the converter kernel of gemm_small.cu: MMA M = 128 weight rows,
// MMA N = 2 * MP (MP = M rounded up to 16; columns [0, MP) hold the p1 sums, [MP, 2 MP) the p2
// sums), K = 32 codes per instruction.  A unit is (128-row weight block, one or two 128-code k-blocks); each
// CTA takes a contiguous run of units, writes fp32 partial sums per weight block it touched, and
// a second kernel adds them in CTA order, applies a_m, s_n, b_n and rounds to bf16.
//
//   warp 0      TMA producer: 128 x 128 weight codes (16 KB) + 2 MP x 128 activation codes per
//               k-block, both with the 128-byte swizzle; a ring slot holds one k-block, or two
//               when MP <= 32 (ring of 4 to 7 slots)
//   warp 1      TMEM allocation; one lane issues the MMAs (128 x 2MP x 32) and commits
//   warps 2-5   epilogue: TMEM -> p1 sum + p2 sum / 16 -> fp32 partial slot
// Every wait is bounded.  A non-finite activation makes its whole output row NaN.
#include "gemm_common.cuh"

namespace {

constexpr int BKC = 128;                    // codes per k-block = one 128-byte operand row
constexpr int WROWS = 128;                  // weight rows per block = MMA M
constexpr int A_BYTES = WROWS * BKC;        // 16 KB
constexpr int MAX_STAGES = 10;
constexpr int RING_BYTES = 212992;          // 208 KB of operand ring
// A ring slot holds `ukb` k-blocks (weight tiles first, then the activation tiles): with few
// activation rows a k-block is only 16-20 KB and four tiny MMAs, less than the MMA warp's wait /
// issue / commit round, so two k-blocks share a round.
__host__ __device__ constexpr int stage_bytes(int MP, int ukb) { return ukb * (A_BYTES + 2 * MP * BKC); }
__host__ __device__ constexpr int num_stages(int MP, int ukb) {
    return RING_BYTES / stage_bytes(MP, ukb) < MAX_STAGES ? RING_BYTES / stage_bytes(MP, ukb) : MAX_STAGES;
}
__host__ __device__ constexpr int unit_kblocks(int MP) { return MP <= 32 ? 2 : 1; }
constexpr int THREADS = 192;                // producer, MMA, four epilogue warps
constexpr int ACC_COLS = 256;               // TMEM columns per accumulator (2 MP <= 256)
constexpr int TMEM_COLS = 2 * ACC_COLS;
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 1024;

enum { ERR_PRODUCER = 31, ERR_MMA_FULL = 32, ERR_MMA_TMEM = 33, ERR_EPILOGUE = 34 };

struct DirectParams {
    float* partial;       // [n_blocks][pieces][MP][128] fp32
    const float* xscale;  // a_m, MP floats
    int M, MP, N, K;
    int n_blocks, num_kb; // num_kb: units along K (each `ukb` k-blocks of 128 codes)
    int ukb, k_blocks;    // k-blocks per unit; k-blocks in all (the last unit may hold fewer)
    int total;            // n_blocks * num_kb units
    int quota;            // units per CTA
    int pieces;           // partial slots per weight block
    int* status;
};

struct Shared {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__host__ __device__ inline int first_cta_of(int nb, int num_kb, int quota) { return (nb * num_kb) / quota; }

__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void e4m3x2_to_f32(uint32_t codes, float& lo, float& hi) {
    uint32_t h;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((uint16_t)codes));
    asm("cvt.f32.f16 %0, %1;" : "=f"(lo) : "h"((uint16_t)(h & 0xFFFFu)));
    asm("cvt.f32.f16 %0, %1;" : "=f"(hi) : "h"((uint16_t)(h >> 16)));
}

// One block per activation row (rows M .. MP-1 are written as zeros): row maximum, then the two
// code rows.  x8 is [2 MP][K] bytes: row m = p1 of activation row m, row MP + m = p2.  A row of
// up to 16384 values is read once (eight 128-bit loads per thread, all issued before the first
// use) and kept in registers between the two passes; longer rows are read again.
constexpr int SPLIT_KEEP = 8;
__device__ __forceinline__ void split8(const uint4& w, float inv, bool non_finite, uint2& c1, uint2& c2) {
    const uint32_t in[4] = {w.x, w.y, w.z, w.w};
    uint32_t o1[4], o2[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float v0 = __uint_as_float(in[i] << 16) * inv, v1 = __uint_as_float(in[i] & 0xFFFF0000u) * inv;
        o1[i] = e4m3x2(v0, v1);
        float f0, f1;
        e4m3x2_to_f32(o1[i], f0, f1);
        o2[i] = e4m3x2((v0 - f0) * 16.f, (v1 - f1) * 16.f);
    }
    c1 = non_finite ? make_uint2(0u, 0u) : make_uint2(o1[0] | (o1[1] << 16), o1[2] | (o1[3] << 16));
    c2 = non_finite ? make_uint2(0u, 0u) : make_uint2(o2[0] | (o2[1] << 16), o2[2] | (o2[3] << 16));
}
__global__ void __launch_bounds__(256)
split_activations_kernel(uint8_t* __restrict__ x8, float* __restrict__ xscale,
                         const uint16_t* __restrict__ x, int M, int MP, int K) {
    __shared__ float red[8];
    __shared__ int bad_s;
    // the streaming kernel may be scheduled now: it sets itself up and starts fetching weight
    // codes on the SMs this kernel leaves free, and waits for this grid before it reads x8
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int m = blockIdx.x;
    const int nvec = K / 8;                        // K % 16 == 0
    uint2* row1 = (uint2*)(x8 + (size_t)m * K);
    uint2* row2 = (uint2*)(x8 + (size_t)(MP + m) * K);
    if (m >= M) {
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) { row1[i] = make_uint2(0u, 0u); row2[i] = make_uint2(0u, 0u); }
        if (threadIdx.x == 0) xscale[m] = 0.f;
        return;
    }
    const uint4* xr = (const uint4*)(x + (size_t)m * K);
    // The row is taken in batches of SPLIT_KEEP x 256 vectors whose loads are all in flight
    // together; the first batch stays in registers between the two passes (rows up to 16384
    // elements are read once), later batches are read again (from L2) by the second pass.
    constexpr int BATCH = SPLIT_KEEP * 256;
    const int n_batches = (nvec + BATCH - 1) / BATCH;
    uint4 keep[SPLIT_KEEP];
    float amax = 0.f;
    int bad = 0;
    auto look = [&](const uint4& w) {
        const uint32_t in[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float a = fabsf(__uint_as_float(in[i] << 16)), b = fabsf(__uint_as_float(in[i] & 0xFFFF0000u));
            bad |= !(a <= 3.4e38f) | !(b <= 3.4e38f);   // inf or NaN
            amax = fmaxf(amax, fmaxf(a, b));
        }
    };
#pragma unroll
    for (int j = 0; j < SPLIT_KEEP; j++) {
        const int i = threadIdx.x + 256 * j;
        keep[j] = i < nvec ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < SPLIT_KEEP; j++) look(keep[j]);
    for (int b = 1; b < n_batches; b++) {
        uint4 t[SPLIT_KEEP];
#pragma unroll
        for (int j = 0; j < SPLIT_KEEP; j++) {
            const int i = b * BATCH + threadIdx.x + 256 * j;
            t[j] = i < nvec ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < SPLIT_KEEP; j++) look(t[j]);
    }
    if (threadIdx.x == 0) bad_s = 0;
    __syncthreads();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    if (bad) bad_s = 1;
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
    const bool non_finite = bad_s != 0;
    // a = 2^(e - 7) with e the exponent of the row maximum; an all-zero row keeps a = 1.
    // Exponents are clamped so that a and 1 / a stay normal fp32 numbers.
    int e = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xFF) - 127 : 7;
    e = max(-119, min(127, e));
    const float a = __uint_as_float((uint32_t)(e - 7 + 127) << 23);
    const float inv = __uint_as_float((uint32_t)(7 - e + 127) << 23);
    if (threadIdx.x == 0) xscale[m] = non_finite ? __uint_as_float(0x7FC00000u) : a;
#pragma unroll
    for (int j = 0; j < SPLIT_KEEP; j++) {
        const int i = threadIdx.x + 256 * j;
        if (i < nvec) split8(keep[j], inv, non_finite, row1[i], row2[i]);
    }
    for (int b = 1; b < n_batches; b++) {
        uint4 t[SPLIT_KEEP];
#pragma unroll
        for (int j = 0; j < SPLIT_KEEP; j++) {
            const int i = b * BATCH + threadIdx.x + 256 * j;
            t[j] = i < nvec ? xr[i] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int j = 0; j < SPLIT_KEEP; j++) {
            const int i = b * BATCH + threadIdx.x + 256 * j;
            if (i < nvec) split8(t[j], inv, non_finite, row1[i], row2[i]);
        }
    }
}

// Calls f(nb, kb0, kb1, piece) for every weight block this CTA's run touches, in order.
template <class F>
__device__ __forceinline__ bool for_each_segment(const DirectParams& p, F f) {
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
linear_small_m_direct_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                             const DirectParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    Shared* sh = (Shared*)(smem_raw + (tiles - raw) + RING_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t STAGES = (uint32_t)num_stages(p.MP, p.ukb), STAGE_BYTES = (uint32_t)stage_bytes(p.MP, p.ukb);
    const uint32_t NP = 2u * (uint32_t)p.MP;           // MMA N: p1 columns, then p2 columns
    const uint32_t X_OFF = (uint32_t)p.ukb * A_BYTES, X_BYTES = NP * BKC;
    // the finalising kernel may be scheduled now; it waits for this grid before it reads
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; s++) {
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
            // The weight does not depend on the kernel that splits the activations, which may
            // still be running: the first ring of weight tiles is requested before the wait for
            // that kernel, the activation tiles of those slots after it.
            uint32_t early = 0;
            for_each_segment(p, [&](int nb, int kb0, int kb1, int) {
                for (int kb = kb0; kb < kb1; kb++) {
                    if (early == STAGES) return false;
                    const uint32_t dst = tiles + early * STAGE_BYTES;
                    const uint32_t fbar = tc::smem_u32(&sh->full[early]);
                    const int k0 = kb * p.ukb, nk = min(p.ukb, p.k_blocks - k0);
                    tc::mbar_arrive_expect_tx(fbar, nk * (A_BYTES + X_BYTES));
                    for (int j = 0; j < nk; j++)
                        tc::tma_load_2d(dst + j * A_BYTES, &map_w, fbar, (k0 + j) * BKC, nb * WROWS);
                    early++;
                }
                return true;
            });
            asm volatile("griddepcontrol.wait;" ::: "memory");   // x8 is complete and visible
            uint32_t stage = 0, phase = 0, unit = 0;
            for_each_segment(p, [&](int nb, int kb0, int kb1, int) {
                for (int kb = kb0; kb < kb1; kb++, unit++) {
                    const uint32_t dst = tiles + stage * STAGE_BYTES;
                    const uint32_t fbar = tc::smem_u32(&sh->full[stage]);
                    const int k0 = kb * p.ukb, nk = min(p.ukb, p.k_blocks - k0);
                    if (unit >= early) {
                        if (!tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_PRODUCER))
                            return false;
                        tc::mbar_arrive_expect_tx(fbar, nk * (A_BYTES + X_BYTES));
                        for (int j = 0; j < nk; j++)
                            tc::tma_load_2d(dst + j * A_BYTES, &map_w, fbar, (k0 + j) * BKC, nb * WROWS);
                    }
                    for (int j = 0; j < nk; j++)
                        tc::tma_load_2d(dst + X_OFF + j * X_BYTES, &map_x, fbar, (k0 + j) * BKC, 0);
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
            // A = weight codes (E4M3 = 0, E5M2 = 1), B = activation codes (E4M3)
            const uint32_t idesc = tc::idesc_f16(WROWS, NP, FMT == NVQ_E5M2 ? 1u : 0u, 0u);
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
                    const int nk = min(p.ukb, p.k_blocks - kb * p.ukb);
                    for (int j = 0; j < nk; j++) {
                        const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr + j * A_BYTES);
                        const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + X_OFF + j * X_BYTES);
#pragma unroll
                        for (int k = 0; k < 4; k++)      // four 32-byte k-steps of 32 codes
                            tc::tc_mma_f8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                          (kb > kb0 || j > 0 || k > 0) ? 1u : 0u);
                    }
                    tc::tc_commit(tc::smem_u32(&sh->empty[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                tc::tc_commit(tc::smem_u32(&sh->tmem_full[acc]));
                return true;
            });
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
            // thread = weight row quarter*32 + lane of the block; column m is activation row m:
            // for a fixed m a warp writes 32 consecutive floats
            float* out = p.partial + ((size_t)(nb * p.pieces + piece) * p.MP) * WROWS + quarter * 32 + lane;
#pragma unroll 1
            for (int c = 0; c < p.MP; c += 16) {
                uint32_t r1[16], r2[16];
                tc::tmem_ld_32x16(taddr + c, r1);
                tc::tmem_ld_32x16(taddr + p.MP + c, r2);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (c + j < p.M)
                        out[(size_t)(c + j) * WROWS] = fmaf(__uint_as_float(r2[j]), 0.0625f, __uint_as_float(r1[j]));
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

// y[m, n] = bf16(a_m * scale_n * sum over the slots of n's weight block + bias_n)
__global__ void direct_finalize_kernel(uint16_t* __restrict__ y, const float* __restrict__ partial,
                                       const float* __restrict__ scales, const float* __restrict__ bias,
                                       DirectParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the partial sums are complete
    const int total = p.M * p.N;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int m = e / p.N, n = e - m * p.N;
        const int nb = n / WROWS, nl = n - nb * WROWS;
        const int first = first_cta_of(nb, p.num_kb, p.quota);
        const int last = ((nb + 1) * p.num_kb - 1) / p.quota;
        const float* src = partial + ((size_t)(nb * p.pieces) * p.MP + m) * WROWS + nl;
        // the loads of up to four slots, the scales and the bias are independent and go out
        // together; the sum keeps the slot order
        const int np = last - first + 1;
        const size_t pitch = (size_t)p.MP * WROWS;
        const float p0 = src[0];
        const float p1 = np > 1 ? src[pitch] : 0.f;
        const float p2 = np > 2 ? src[2 * pitch] : 0.f;
        const float p3 = np > 3 ? src[3 * pitch] : 0.f;
        const float xs = p.xscale[m], sn = scales ? scales[n] : 1.f, bn = bias ? bias[n] : 0.f;
        float s = p0;
        if (np > 1) s = __fadd_rn(s, p1);
        if (np > 2) s = __fadd_rn(s, p2);
        if (np > 3) s = __fadd_rn(s, p3);
        for (int pc = 4; pc < np; pc++) s = __fadd_rn(s, src[(size_t)pc * pitch]);
        const float v = fmaf(__fmul_rn(s, xs), sn, bn);
        y[e] = (uint16_t)(pack_bf16(v, 0.f) & 0xFFFFu);
    }
}

struct Geometry { int MP, n_blocks, num_kb, ukb, k_blocks, total, grid, quota, pieces; size_t partial_bytes, x8_bytes; };
Geometry geometry(size_t M, size_t N, size_t K, int device) {
    Geometry g;
    g.MP = (int)((M + 15) / 16 * 16);
    g.n_blocks = (int)((N + WROWS - 1) / WROWS);
    g.ukb = unit_kblocks(g.MP);
    g.k_blocks = (int)((K + BKC - 1) / BKC);
    g.num_kb = (g.k_blocks + g.ukb - 1) / g.ukb;
    g.total = g.n_blocks * g.num_kb;
    g.grid = nvq_sm_count(device);
    if (g.grid > g.total) g.grid = g.total;
    g.quota = (g.total + g.grid - 1) / g.grid;
    g.grid = (g.total + g.quota - 1) / g.quota;
    g.pieces = (g.num_kb + g.quota - 1) / g.quota + 1;
    g.partial_bytes = ((size_t)g.n_blocks * g.pieces * g.MP * WROWS * sizeof(float) + 255) / 256 * 256;
    g.x8_bytes = ((size_t)2 * g.MP * K + 255) / 256 * 256;
    return g;
}


// ---------------------------------------------------------------- clustered form (M <= 32)
// For at most 32 rows and a weight that ONE wave of thread-block clusters covers, the fixed costs
// of the call (kernel boundaries, partial sums through HBM) outweigh the weight stream: 16 MB of
// codes stream in 2.5 us.  Here a cluster of S CTAs owns one 128-row weight block, each CTA
// takes 1/S of K, and the partial sums meet in distributed shared memory: after a cluster
// barrier CTA r of the cluster adds, in rank order, the S partial sums of the activation rows
// m = r, r + S, ... (so the reduction is spread over the cluster and deterministic), applies
// a_m, s_n, b_n and stores bf16.  No partial sum goes to HBM and no third kernel runs.
//
//   thread 0    barrier set-up, then at once the first ring of weight tiles (TMA); after the
//               wait for the activation-splitting kernel, the activation tiles
//   warp 1      TMEM allocation (off the producer's path), MMA issue (128 x 2 MP x 32), commit
//   warps 2-5   epilogue: TMEM -> p1 sum + p2 sum / 16 -> own shared memory; after the cluster
//               barrier the cross-CTA sums and the bf16 stores
// Every mbarrier wait is bounded; both cluster barriers are reached by every thread of every CTA
// whatever happened before them.
constexpr int CL_MAX_MP = 32;
constexpr int CL_STAGES = 8;                                 // ring slots at most; a CTA with fewer k-blocks takes fewer
constexpr int CL_TMEM_COLS = 64;
// Shared memory of a CTA: ring of `stages` slots (weight tile + activation tile), its partial sums
// [MP][128] fp32, the barriers.
__host__ __device__ constexpr int cl_slot_bytes(int MP) { return A_BYTES + 2 * MP * BKC; }
__host__ __device__ constexpr int cl_smem_bytes(int MP, int stages) {
    return 1024 + stages * cl_slot_bytes(MP) + MP * WROWS * 4 + 1024;
}

enum { ERR_CL_PRODUCER = 51, ERR_CL_MMA = 52, ERR_CL_EPILOGUE = 53 };

struct ClusterParams {
    uint16_t* y;            // M x N bf16
    const float* xscale;    // a_m, MP floats
    const float* scales;    // N or nullptr
    const float* bias;      // N or nullptr
    int M, MP, N, K;
    int S;                  // CTAs per cluster = K ranges per weight block
    int kb_per_cta, k_blocks;
    int stages;             // ring slots of this launch
    int* status;
};

struct ClusterShared {
    uint64_t full[CL_STAGES];
    uint64_t empty[CL_STAGES];
    uint64_t tmem_full;
    uint32_t tmem_base;
    int abort_flag;
};

// Not volatile on purpose: the loads of a thread's values are independent and must be in flight
// together (a remote shared-memory load takes a few hundred cycles).  They stay behind the
// cluster barrier through `token`, a zero that barrier's asm statement produces.
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr, uint32_t token) {
    float v;
    asm("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr + token));
    return v;
}
__device__ __forceinline__ uint32_t cluster_sync_token() {
    uint32_t z;
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;\n\tmov.u32 %0, 0;" : "=r"(z)::"memory");
    return z;
}


template <int FMT>
__global__ void __launch_bounds__(THREADS, 1)
linear_few_rows_cluster_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                               const ClusterParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    const int CL_SLOT = cl_slot_bytes(p.MP), STAGES_RT = p.stages;
    const uint32_t ring_bytes = (uint32_t)(STAGES_RT * CL_SLOT);
    const uint32_t part = tiles + ring_bytes;
    ClusterShared* sh = (ClusterShared*)(smem_raw + (tiles - raw) + ring_bytes + (uint32_t)p.MP * WROWS * 4u);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sh->abort_flag;
    const int rank = (int)tc::cluster_ctarank();          // this CTA's K range
    const int nb = (int)blockIdx.x / p.S;                 // this cluster's weight block
    const int kb0 = rank * p.kb_per_cta;
    const int nkb = max(0, min(p.kb_per_cta, p.k_blocks - kb0));
    const uint32_t NP = 2u * (uint32_t)p.MP;              // MMA N: p1 columns, then p2 columns
    const uint32_t X_BYTES = NP * BKC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < CL_STAGES; s++) {
            tc::mbar_init(tc::smem_u32(&sh->full[s]), 1);
            tc::mbar_init(tc::smem_u32(&sh->empty[s]), 1);
        }
        tc::mbar_init(tc::smem_u32(&sh->tmem_full), 1);
        sh->abort_flag = 0;
        tc::mbar_fence_init();
        // The weight does not depend on the kernel that splits the activations, which may still
        // be running: the first ring of weight tiles is requested right here, before anything
        // else exists; the activation tiles of those slots follow after the wait for that kernel.
        for (int i = 0; i < nkb && i < STAGES_RT; i++) {
            const uint32_t fbar = tc::smem_u32(&sh->full[i]);
            tc::mbar_arrive_expect_tx(fbar, A_BYTES + X_BYTES);
            tc::tma_load_2d(tiles + i * CL_SLOT, &map_w, fbar, (kb0 + i) * BKC, nb * WROWS);
        }
    }
    __syncthreads();                                      // the barriers exist

    float sn = 1.f, bn = 0.f, xs_mine[8];     // epilogue threads: channel scale, bias, a_m of the rows this CTA closes
#pragma unroll
    for (int q = 0; q < 8; q++) xs_mine[q] = 0.f;
    uint32_t tmem_base = 0;
    if (warp >= 1) {
        // TMEM allocation concerns the MMA warp and the epilogue warps only (named barrier 1, 160
        // threads); the producer is not held up by it
        if (warp == 1) {
            tc::tmem_alloc(tc::smem_u32(&sh->tmem_base), CL_TMEM_COLS);
            tc::tmem_relinquish();
        }
        tc::tc_fence_before();
        asm volatile("bar.sync 1, 160;" ::: "memory");
        tc::tc_fence_after();
        tmem_base = sh->tmem_base;
    }

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");   // the activation codes are complete and visible
            for (int i = 0; i < nkb && i < STAGES_RT; i++)
                tc::tma_load_2d(tiles + i * CL_SLOT + A_BYTES, &map_x, tc::smem_u32(&sh->full[i]), (kb0 + i) * BKC, 0);
            for (int i = STAGES_RT; i < nkb; i++) {
                const int stage = i % STAGES_RT;
                if (!tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), ((i / STAGES_RT) - 1) & 1, abort_flag, ERR_CL_PRODUCER))
                    break;
                const uint32_t fbar = tc::smem_u32(&sh->full[stage]);
                tc::mbar_arrive_expect_tx(fbar, A_BYTES + X_BYTES);
                tc::tma_load_2d(tiles + stage * CL_SLOT, &map_w, fbar, (kb0 + i) * BKC, nb * WROWS);
                tc::tma_load_2d(tiles + stage * CL_SLOT + A_BYTES, &map_x, fbar, (kb0 + i) * BKC, 0);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && nkb > 0) {
            // A = weight codes (E4M3 = 0, E5M2 = 1), B = activation codes (E4M3)
            const uint32_t idesc = tc::idesc_f16(WROWS, NP, FMT == NVQ_E5M2 ? 1u : 0u, 0u);
            bool ok = true;
            // The MMAs of a k-block are tiny (128 x 2 MP x 32, four of them); what costs is the
            // round around them (wait, fence, commit: ~250 ns).  The activation tiles arrive last
            // and together, so the slots are taken four at a time: one round per four k-blocks,
            // and a slot is only handed back when the ring will be walked again.
            const bool reuse = nkb > STAGES_RT;
            for (int i0 = 0; i0 < nkb && ok; i0 += 4) {
                const int i1 = min(nkb, i0 + 4);
                for (int i = i0; i < i1 && ok; i++)
                    ok = tc::mbar_wait(tc::smem_u32(&sh->full[i % STAGES_RT]), (i / STAGES_RT) & 1, abort_flag, ERR_CL_MMA);
                if (!ok) break;
                tc::tc_fence_after();
                for (int i = i0; i < i1; i++) {
                    const int stage = i % STAGES_RT;
                    const uint64_t a_desc = tc::smem_desc_k_sw128(tiles + stage * CL_SLOT);
                    const uint64_t b_desc = tc::smem_desc_k_sw128(tiles + stage * CL_SLOT + A_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; k++)      // four 32-byte k-steps of 32 codes
                        tc::tc_mma_f8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    if (reuse) tc::tc_commit(tc::smem_u32(&sh->empty[stage]));
                }
            }
            if (ok) tc::tc_commit(tc::smem_u32(&sh->tmem_full));
        }
    } else {
        // ------------------------------------------------------------ epilogue: own partial sums
        const int quarter = warp & 3;
        const int wrow = quarter * 32 + lane;             // weight row of this thread within the block
        // what the closing sums need from global memory is fetched now, while the MMAs run
        {
            const int n = nb * WROWS + wrow;
            sn = (p.scales && n < p.N) ? p.scales[n] : 1.f;
            bn = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            asm volatile("griddepcontrol.wait;" ::: "memory");   // xscale comes from the splitting kernel
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int m = rank + q * p.S;
                xs_mine[q] = m < p.M ? p.xscale[m] : 0.f;
            }
        }
        bool ok = nkb > 0 && tc::mbar_wait(tc::smem_u32(&sh->tmem_full), 0, abort_flag, ERR_CL_EPILOGUE);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (ok) tc::tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        // thread = weight row: for a fixed activation row a warp writes 32 consecutive floats
#pragma unroll
        for (int c = 0; c < CL_MAX_MP; c += 16) {
            if (c < p.MP) {
                uint32_t r1[16], r2[16];
                if (ok) {
                    tc::tmem_ld_32x16(taddr + c, r1);
                    tc::tmem_ld_32x16(taddr + p.MP + c, r2);
                    tc::tmem_ld_wait();
                }
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float v = ok ? fmaf(__uint_as_float(r2[j]), 0.0625f, __uint_as_float(r1[j])) : 0.f;
                    asm volatile("st.shared.f32 [%0], %1;" ::"r"(part + (uint32_t)((c + j) * WROWS + wrow) * 4u), "f"(v) : "memory");
                }
            }
        }
        if (ok) tc::tc_fence_before();
    }

    const uint32_t token = cluster_sync_token();          // every CTA's partial sums are in its shared memory
    if (warp >= 2) {
        // ------------------------------------------------------------ cross-CTA sums: rows m = rank, rank + S, ...
        const int wrow = (warp & 3) * 32 + lane;
        const int n = nb * WROWS + wrow;
        uint32_t peer[8];
#pragma unroll
        for (int r = 0; r < 8; r++) peer[r] = tc::mapa(part + (uint32_t)wrow * 4u, (uint32_t)(r < p.S ? r : 0));
        // rows rank, rank + S, ...: at most 32 / S of them, i.e. at most 8 for S >= 4; four at a time,
        // their S loads each all in flight together
#pragma unroll
        for (int q0 = 0; q0 < 8; q0 += 4) {
            const int m0 = rank + q0 * p.S;
            if (m0 >= p.M) break;
            float v[4][8];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int m = m0 + q * p.S;
#pragma unroll
                for (int r = 0; r < 8; r++)
                    v[q][r] = (m < p.M && r < p.S) ? ld_cluster_f32(peer[r] + (uint32_t)(m * WROWS) * 4u, token) : 0.f;
            }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int m = m0 + q * p.S;
                if (m < p.M && n < p.N) {
                    float s = v[q][0];
#pragma unroll
                    for (int r = 1; r < 8; r++)
                        if (r < p.S) s = __fadd_rn(s, v[q][r]);          // rank order: the same sum on every run
                    const float out = fmaf(__fmul_rn(s, xs_mine[q0 + q]), sn, bn);
                    p.y[(size_t)m * p.N + n] = (uint16_t)(pack_bf16(out, 0.f) & 0xFFFFu);
                }
            }
        }
    }
    if (warp >= 2) {
        // rows past the eight handled above (only for S < 4 with more than 8 S rows): plain loop
        const int wrow = (warp & 3) * 32 + lane;
        const int n = nb * WROWS + wrow;
        for (int m = rank + 8 * p.S; m < p.M; m += p.S) {
            float s = 0.f;
            for (int r = 0; r < p.S; r++) {
                const float t = ld_cluster_f32(tc::mapa(part + (uint32_t)(m * WROWS + wrow) * 4u, (uint32_t)r), token);
                s = r == 0 ? t : __fadd_rn(s, t);
            }
            if (n < p.N) p.y[(size_t)m * p.N + n] = (uint16_t)(pack_bf16(fmaf(__fmul_rn(s, p.xscale[m]), sn, bn), 0.f) & 0xFFFFu);
        }
    }
    tc::cluster_sync_all();          // nobody leaves while another CTA still reads its memory

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(20000);   // let copies in flight land
    }
    if (warp >= 1) {
        tc::tc_fence_before();
        asm volatile("bar.sync 1, 160;" ::: "memory");
        tc::tc_fence_after();
        if (warp == 1) tc::tmem_dealloc(tmem_base, CL_TMEM_COLS);
    }
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, 0, *abort_flag);
}

struct ClusterPlan { int S, kb_per_cta, stages, smem; };

// CTAs of the clustered kernel that can be resident at once in clusters of S (per device).
int cluster_resident_ctas(int S, int smem, int device) {
    static std::atomic<int> cache[64][4][256];       // S = 1, 2, 4, 8; shared memory in KB
    const int si = S == 1 ? 0 : (S == 2 ? 1 : (S == 4 ? 2 : 3));
    std::atomic<int>& slot = cache[device][si][(smem + 1023) / 1024 & 255];
    int v = slot.load(std::memory_order_relaxed);
    if (v) return v;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S * 64);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, linear_few_rows_cluster_kernel<NVQ_E4M3>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
    }
    v = clusters > 0 ? clusters * S : -1;
    slot.store(v, std::memory_order_relaxed);
    return v;
}

// The cluster size that puts the most CTAs to work in a single wave; S = 0 when the problem does
// not fit (more than 32 rows, or more weight blocks than one wave of clusters holds).
ClusterPlan cluster_plan(const Geometry& g, size_t M, int device) {
    ClusterPlan best = {0, 0, 0, 0};
    if (g.MP > CL_MAX_MP) return best;
    int best_ctas = 0;
    for (int S = 1; S <= 8; S *= 2) {
        const int kb = (g.k_blocks + S - 1) / S;
        if ((S - 1) * kb >= g.k_blocks) continue;            // every CTA gets at least one k-block
        // Always the full ring, i.e. one CTA per SM: with half-size rings two CTAs share an SM and a
        // cluster of 8 covers 4096 x 4096 in one wave, but that measured slower (10.9 against 9.7 us
        // per call for 16 x 4096 x 4096 from a CUDA graph) - twice the CTAs to launch and a wider
        // cluster barrier cost more than the halved MMA chain saves.
        const int stages = CL_STAGES;
        const int smem = cl_smem_bytes(g.MP, stages);
        const int cap = cluster_resident_ctas(S, smem, device);
        if (cap <= 0 || g.n_blocks * S > cap) continue;
        if (g.n_blocks * S > best_ctas) {
            best_ctas = g.n_blocks * S;
            best.S = S; best.kb_per_cta = kb; best.stages = stages; best.smem = smem;
        }
    }
    (void)M;
    return best;
}

}  // namespace

// workspace: [fp32 partial sums][activation codes, 2 MP x K bytes][a_m, MP floats]
size_t nvq_linear_small_m_direct_workspace(size_t M, size_t N, size_t K, int device) {
    const Geometry g = geometry(M, N, K, device);
    return g.partial_bytes + g.x8_bytes + (size_t)g.MP * sizeof(float);
}

nvq_status nvq_linear_launch_small_m_direct(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                            nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                            size_t M, size_t N, size_t K, void* d_workspace, int device,
                                            cudaStream_t st, bool use_cluster) {
    NVQ_REQUIRE(M >= 1 && M <= 128 && K % 16 == 0, "small-M Linear: needs 1 <= M <= 128 and K %% 16 == 0");
    NVQ_REQUIRE(fmt == NVQ_E4M3 || fmt == NVQ_E5M2, "small-M direct Linear: FP8 weight codes only");
    NVQ_REQUIRE(M * N < (1u << 31) && N < (1u << 24) && K < (1u << 24) && N * K < (1ull << 40),
                "small-M Linear: dimension too large");
    const Geometry g = geometry(M, N, K, device);
    uint8_t* ws = (uint8_t*)d_workspace;
    uint8_t* d_x8 = ws + g.partial_bytes;
    float* d_xscale = (float*)(ws + g.partial_bytes + g.x8_bytes);
    DirectParams p;
    p.partial = (float*)ws;
    p.xscale = d_xscale;
    p.M = (int)M;
    p.MP = g.MP;
    p.N = (int)N;
    p.K = (int)K;
    p.n_blocks = g.n_blocks;
    p.num_kb = g.num_kb;
    p.ukb = g.ukb;
    p.k_blocks = g.k_blocks;
    p.total = g.total;
    p.quota = g.quota;
    p.pieces = g.pieces;
    nvq_status s = nvq_status_word(device, &p.status);
    if (s != NVQ_OK) return s;
    CUtensorMap map_w, map_x;
    // both operands: rows of 128 codes, 128-byte swizzle; columns past K read as zero codes
    s = nvq_make_tmap_2d(&map_w, d_wq, N, K, WROWS, BKC, 1, 1);
    if (s != NVQ_OK) return s;
    s = nvq_make_tmap_2d(&map_x, d_x8, (uint64_t)2 * g.MP, K, (uint32_t)(2 * g.MP), BKC, 1, 1);
    if (s != NVQ_OK) return s;
    static std::atomic<bool> attr_set[64];   // per device; setting the attribute twice is harmless
    if (!attr_set[device]) {
        NVQ_CUDA(cudaFuncSetAttribute(linear_small_m_direct_kernel<NVQ_E4M3>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        NVQ_CUDA(cudaFuncSetAttribute(linear_small_m_direct_kernel<NVQ_E5M2>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        NVQ_CUDA(cudaFuncSetAttribute(linear_few_rows_cluster_kernel<NVQ_E4M3>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, cl_smem_bytes(CL_MAX_MP, CL_STAGES)));
        NVQ_CUDA(cudaFuncSetAttribute(linear_few_rows_cluster_kernel<NVQ_E5M2>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, cl_smem_bytes(CL_MAX_MP, CL_STAGES)));
        attr_set[device] = true;
    }
    split_activations_kernel<<<g.MP, 256, 0, st>>>(d_x8, d_xscale, d_x, (int)M, g.MP, (int)K);
    NVQ_LAUNCHED();
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // set up under the previous kernel's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    const ClusterPlan cp = use_cluster ? cluster_plan(g, M, device) : ClusterPlan{0, 0, 0, 0};
    if (cp.S > 0) {
        // two kernels: the split above, then the clustered stream with the reduction inside
        ClusterParams q;
        q.y = d_y;
        q.xscale = d_xscale;
        q.scales = d_scales;
        q.bias = d_bias;
        q.M = (int)M; q.MP = g.MP; q.N = (int)N; q.K = (int)K;
        q.S = cp.S; q.kb_per_cta = cp.kb_per_cta; q.k_blocks = g.k_blocks;
        q.stages = cp.stages;
        q.status = p.status;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = cp.S;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cudaLaunchConfig_t ccfg = {};
        ccfg.gridDim = dim3(g.n_blocks * cp.S);
        ccfg.blockDim = dim3(THREADS);
        ccfg.dynamicSmemBytes = cp.smem;
        ccfg.stream = st;
        ccfg.attrs = attr;
        ccfg.numAttrs = 2;
        if (fmt == NVQ_E4M3)
            NVQ_CUDA(cudaLaunchKernelEx(&ccfg, linear_few_rows_cluster_kernel<NVQ_E4M3>, map_w, map_x, q));
        else
            NVQ_CUDA(cudaLaunchKernelEx(&ccfg, linear_few_rows_cluster_kernel<NVQ_E5M2>, map_w, map_x, q));
        NVQ_LAUNCHED();
        return NVQ_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g.grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (fmt == NVQ_E4M3)
        NVQ_CUDA(cudaLaunchKernelEx(&cfg, linear_small_m_direct_kernel<NVQ_E4M3>, map_w, map_x, p));
    else
        NVQ_CUDA(cudaLaunchKernelEx(&cfg, linear_small_m_direct_kernel<NVQ_E5M2>, map_w, map_x, p));
    NVQ_LAUNCHED();
    const int total = p.M * p.N;
    int fgrid = (total + 255) / 256;
    const int cap = nvq_sm_count(device) * 8;
    if (fgrid > cap) fgrid = cap;
    cudaLaunchConfig_t fcfg = {};
    fcfg.gridDim = dim3(fgrid);
    fcfg.blockDim = dim3(256);
    fcfg.stream = st;
    fcfg.attrs = attr;
    fcfg.numAttrs = 1;
    NVQ_CUDA(cudaLaunchKernelEx(&fcfg, direct_finalize_kernel, d_y, (const float*)p.partial, d_scales, d_bias, p));
    NVQ_LAUNCHED();
    return NVQ_OK;
}
