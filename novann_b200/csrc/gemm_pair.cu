// Quantised-weight Linear forward, CTA-pair version: two CTAs on neighbouring SMs work on
// one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
//   CTA r of the pair holds rows [m0 + 128 r, +128) of X and rows [n0 + 128 r, +128) of the
//   expanded weight in ITS OWN shared memory; the leader (rank 0) issues one MMA of shape
//   256 x 256 x 16 that reads both CTAs' tiles and writes 128 accumulator rows into each CTA's
//   TMEM.  Per k-block every SM therefore pulls 32 KB through L2 instead of 48 KB, and the
//   shared-memory ring is six stages deep.
//
//   warp 0  producer (both CTAs): TMA loads into the CTA's own ring slot; the bytes of both
//           CTAs are counted on the LEADER's full barrier (no multicast anywhere)
//   warp 1  TMEM allocation (both CTAs, cta_group::2); in the leader one lane issues the MMAs
//           and commits: slot release and "accumulator ready" are multicast to both CTAs
//   warps 2-5 epilogue (both CTAs): own 128 rows; "accumulator drained" is signalled to the
//           leader's barrier, remotely from the peer
// Every wait is bounded; a cluster barrier before teardown keeps a CTA's shared memory alive
// until its partner has stopped signalling into it.
#include "gemm_common.cuh"

namespace {

constexpr int BM = 256;          // rows per pair tile (128 per CTA)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = 128 * BK * 2;      // per CTA
constexpr int B_BYTES = 128 * BK * 2;      // per CTA: half of the tile's weight rows
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 8192;

enum { ERR_PRODUCER = 11, ERR_MMA_FULL = 12, ERR_MMA_TMEM = 13, ERR_EPILOGUE = 14 };

struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    float scale[2][BN];
    float bias[2][BN];
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
linear_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const LinearParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    Shared* sh = (Shared*)(smem_raw + (tiles - raw) + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (p.K + BK - 1) / BK;
    volatile int* abort_flag = &sh->abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            tc::mbar_init(tc::smem_u32(&sh->full[s]), 1);
            tc::mbar_init(tc::smem_u32(&sh->empty[s]), 1);
        }
        for (int a = 0; a < 2; a++) {
            tc::mbar_init(tc::smem_u32(&sh->tmem_full[a]), 1);
            tc::mbar_init(tc::smem_u32(&sh->tmem_empty[a]), 8);   // 4 epilogue warps x 2 CTAs
        }
        sh->abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&map_a);
        tc::tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        tc::tmem_alloc_pair(tc::smem_u32(&sh->tmem_base), TMEM_COLS);
        tc::tmem_relinquish_pair();
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();          // the partner's barriers exist before anything targets them
    tc::tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int t = pair; t < p.num_items && ok; t += num_pairs) {
                const TileRef tr = tile_ref(p, t);
                const int bn = tr.is_half ? BN / 2 : BN;
                const int rows_b = bn / 2;                       // weight rows this CTA loads
                const int m0 = tr.m_blk * BM + (int)rank * 128;
                const int n0 = tr.n_blk * BN + tr.half * (BN / 2) + (int)rank * rows_b;
                for (int kb = 0; kb < num_kb; kb++) {
                    ok = tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_PRODUCER);
                    if (!ok) break;
                    const uint32_t dst = tiles + stage * STAGE_BYTES;
                    const uint32_t lead_full = tc::mapa(tc::smem_u32(&sh->full[stage]), 0);
                    if (rank == 0)   // the leader expects the bytes of both CTAs
                        tc::mbar_arrive_expect_tx(tc::smem_u32(&sh->full[stage]),
                                                  2 * (A_BYTES + rows_b * BK * 2));
                    tc::tma_load_2d_pair(dst, &map_a, lead_full, kb * BK, m0);
                    tc::tma_load_2d_pair(dst + A_BYTES, &map_b, lead_full, kb * BK, n0);
                    if (rows_b == 128)
                        tc::tma_load_2d_pair(dst + A_BYTES + B_BYTES / 2, &map_b, lead_full, kb * BK, n0 + 64);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int it = 0;
            for (int t = pair; t < p.num_items && ok; t += num_pairs, it++) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                const TileRef tr = tile_ref(p, t);
                const uint32_t idesc = tc::idesc_f16(BM, tr.is_half ? BN / 2 : BN, 1, 1);
                ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_empty[acc]), acc_phase ^ 1, abort_flag, ERR_MMA_TMEM);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; kb++) {
                    ok = tc::mbar_wait(tc::smem_u32(&sh->full[stage]), phase, abort_flag, ERR_MMA_FULL);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++)
                        tc::tc_mma_f16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                    tc::tc_commit_pair(tc::smem_u32(&sh->empty[stage]), 3);   // both CTAs' slots
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc::tc_commit_pair(tc::smem_u32(&sh->tmem_full[acc]), 3);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64;
        const bool vec32 = (p.N % 16) == 0;
        bool ok = true;
        int it = 0;
        for (int t = pair; t < p.num_items && ok; t += num_pairs, it++) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            const TileRef tr = tile_ref(p, t);
            const int bn = tr.is_half ? BN / 2 : BN;
            const int m0 = tr.m_blk * BM + (int)rank * 128;
            const int n0 = tr.n_blk * BN + tr.half * (BN / 2);
            for (int c = et; c < bn; c += 128) {
                int n = n0 + c;
                sh->scale[acc][c] = (p.scales && n < p.N) ? p.scales[n] : 1.f;
                sh->bias[acc][c] = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            }
            ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_full[acc]), acc_phase, abort_flag, ERR_EPILOGUE);
            ok = epilogue_all(ok);
            if (!ok) break;
            tc::tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            uint16_t* yrow = p.y + (size_t)row * p.N + n0;
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < bn; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c, r);
                tc::tmem_ld_wait();
                if (row < p.M)
                    store_chunk(r, &sh->scale[acc][c], &sh->bias[acc][c], yrow + c, n0 + c, p.N, vec32);
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_cluster(tc::mapa(tc::smem_u32(&sh->tmem_empty[acc]), 0));
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        for (int i = 0; i < 64; i++) __nanosleep(20000);
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::cluster_sync_all();          // partner no longer reads my tiles / signals my barriers
    tc::tc_fence_after();
    if (warp == 1) tc::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, 0, *abort_flag);
}

}  // namespace

nvq_status nvq_linear_launch_pair(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int device, cudaStream_t st) {
    CUtensorMap map_a, map_b;
    nvq_status s = nvq_make_tmap_2d(&map_a, d_x, M, K, 128, BK, 2);
    if (s != NVQ_OK) return s;
    s = nvq_make_tmap_2d(&map_b, d_w, N, K, 64, BK, 2);
    if (s != NVQ_OK) return s;
    static bool attr_set[64];
    if (!attr_set[device]) {
        NVQ_CUDA(cudaFuncSetAttribute(linear_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      SMEM_BYTES));
        attr_set[device] = true;
    }
    LinearParams p;
    p.y = d_y;
    p.scales = d_scales;
    p.bias = d_bias;
    p.M = (int)M;
    p.N = (int)N;
    p.K = (int)K;
    p.m_blocks = (int)((M + BM - 1) / BM);
    p.n_blocks = (int)((N + BN - 1) / BN);
    p.group_m = 8;
    s = nvq_status_word(device, &p.status);
    if (s != NVQ_OK) return s;
    int tiles = p.m_blocks * p.n_blocks;
    int pairs = nvq_sm_count(device) / 2;
    if (tiles < pairs) pairs = tiles;
    int rem = tiles % pairs;
    int split = (tiles > pairs && rem > 0 && 2 * rem <= pairs) ? rem : 0;
    p.num_big = tiles - split;
    p.num_items = p.num_big + 2 * split;
    linear_tc_pair_kernel<<<2 * pairs, THREADS, SMEM_BYTES, st>>>(map_a, map_b, p);
    NVQ_LAUNCHED();
    return NVQ_OK;
}
