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
//           and commits: slot release and "accumulator ready" are multicast to both CTAs;
//           accumulators: two of 256 TMEM columns, or four of 128 for outputs of <= 128 columns
//   warps 2-9 epilogue (both CTAs): own 128 rows, two warps per 32-row TMEM quarter taking
//           alternate 32-column chunks, the TMEM load of a warp's next chunk in flight while it
//           stores the current one; "accumulator drained" is signalled to the leader's barrier,
//           remotely from the peer
//   warps 10-17 (fused variant only) converters: the weight tile arrives by TMA as raw FP8
//           codes; these warps expand it to bf16 (exact) straight into the swizzled operand
//           slot, so no expanded copy of the weight ever exists in HBM.
// Every wait is bounded; a cluster barrier before teardown keeps a CTA's shared memory alive
// until its partner has stopped signalling into it.
#include "gemm_common.cuh"

namespace {

constexpr int BM = 256;          // rows per pair tile (128 per CTA)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = 128 * BK * 2;      // per CTA
constexpr int B_BYTES = 128 * BK * 2;      // per CTA: half of the tile's weight rows
constexpr int RAW_BYTES = 128 * BK;        // fused variant: the same rows as FP8 codes
constexpr int TMEM_COLS = 512;
constexpr int MAX_STAGES = 6;
constexpr int EPI_WARPS = 8;               // warps 2 .. 9
constexpr int FIRST_CONV_WARP = 2 + EPI_WARPS;
constexpr int PAIR_CONV_GROUPS = 2;        // fused variant: k-blocks expanded concurrently
static_assert(PAIR_CONV_GROUPS == 1 || PAIR_CONV_GROUPS == 2, "the five-slot ring feeds at most two groups");

// FUSED = 0: B comes expanded (bf16) from a workspace.  FUSED = NVQ_E4M3 / NVQ_E5M2: B comes as
// codes and is expanded in shared memory by four extra warps.
// FUSED = kW8A8: both operands arrive as E4M3 codes (activations quantised per row beforehand)
// and the MMAs are kind::f8f6f4: 128 codes per 128-byte row, so a k-block spans 128 elements.
// FUSED = kImplicitConv: A is gathered by 4-D TMA boxes from an NHWC activation tensor (one box
// per filter tap and 64-channel block), B is the expanded weight with columns ordered
// (kh, kw, c), and the epilogue writes fp32 NCHW.
constexpr int kW8A8 = -8;
constexpr int kImplicitConv = -16;
template <int FUSED>
struct Cfg {
    static constexpr bool CONV = FUSED > 0;
    static constexpr bool F8 = FUSED == kW8A8;
    static constexpr bool IMPL = FUSED == kImplicitConv;
    static constexpr int BKE = F8 ? 128 : BK;           // elements of K per k-block
    static constexpr int STAGES = CONV ? 5 : 6;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + (CONV ? RAW_BYTES : 0);
    static constexpr int THREADS = CONV ? 576 : 320;    // 2 + 8 epilogue warps; fused: + 8 converter warps
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 8192;
};

enum { ERR_PRODUCER = 11, ERR_MMA_FULL = 12, ERR_MMA_TMEM = 13, ERR_EPILOGUE = 14, ERR_CONVERT = 15 };

struct Shared {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t raw_full[MAX_STAGES];
    uint64_t tmem_full[4];
    uint64_t tmem_empty[4];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float scale[2][BN];   // read as float4 by the epilogue
    alignas(16) float bias[2][BN];
};

template <int FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg<FUSED>::THREADS, 1)
linear_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const LinearParams p) {
    constexpr int STAGES = Cfg<FUSED>::STAGES;
    constexpr int STAGE_BYTES = Cfg<FUSED>::STAGE_BYTES;
    constexpr bool CONV = Cfg<FUSED>::CONV;
    constexpr bool F8 = Cfg<FUSED>::F8;
    constexpr bool IMPL = Cfg<FUSED>::IMPL;
    constexpr int BKE = Cfg<FUSED>::BKE;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    Shared* sh = (Shared*)(smem_raw + (tiles - raw) + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_kb = (p.K + BKE - 1) / BKE;
    volatile int* abort_flag = &sh->abort_flag;
    // Accumulator buffers in TMEM: two of 256 columns, or four of 128 columns when the output has
    // at most 128 columns (every tile is then half-width).  Short tiles (few k-blocks) need the
    // deeper queue to hide the hand-off between the MMA warp and the epilogue warps.
    const bool narrow = p.N <= BN / 2;
    const uint32_t acc_cols = narrow ? BN / 2 : BN;
    auto acc_of = [&](int it, uint32_t& acc, uint32_t& acc_phase) {
        if (narrow) { acc = it & 3; acc_phase = (it >> 2) & 1; }
        else        { acc = it & 1; acc_phase = (it >> 1) & 1; }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            // fused: the leader's full barrier also collects one arrival per converter warp of
            // both CTAs (8 + 8) on top of the producer's
            tc::mbar_init(tc::smem_u32(&sh->full[s]), CONV ? 1 + 16 / PAIR_CONV_GROUPS : 1);
            tc::mbar_init(tc::smem_u32(&sh->empty[s]), 1);
            tc::mbar_init(tc::smem_u32(&sh->raw_full[s]), 1);
        }
        for (int a = 0; a < 4; a++) {
            tc::mbar_init(tc::smem_u32(&sh->tmem_full[a]), 1);
            tc::mbar_init(tc::smem_u32(&sh->tmem_empty[a]), 2 * EPI_WARPS);   // epilogue warps x 2 CTAs
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
    // Programmatic dependent launch: everything above ran while the kernel that fills the
    // weight workspace was still draining; from here on its output is needed.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            [[maybe_unused]] int img = 0, oh0 = 0, kh = 0, kw = 0, cb = 0;
            [[maybe_unused]] const int a_bytes = IMPL ? p.conv_bw * p.conv_bh * BK * 2 : 0;   // the box, padding included
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
                    if constexpr (CONV) {
                        if (rank == 0)   // the leader expects the X bytes of both CTAs
                            tc::mbar_arrive_expect_tx(tc::smem_u32(&sh->full[stage]), 2 * A_BYTES);
                        tc::tma_load_2d_pair(dst, &map_a, lead_full, kb * BK, m0);
                        // raw codes: own barrier, own CTA; consumed by the converter warps
                        const uint32_t rbar = tc::smem_u32(&sh->raw_full[stage]);
                        tc::mbar_arrive_expect_tx(rbar, rows_b * BK);
                        tc::tma_load_2d(dst + A_BYTES + B_BYTES, &map_b, rbar, kb * BK, n0);
                        if (rows_b == 128)
                            tc::tma_load_2d(dst + A_BYTES + B_BYTES + RAW_BYTES / 2, &map_b, rbar, kb * BK, n0 + 64);
                    } else if constexpr (IMPL) {
                        // this CTA's box: image and first output row of operand tile 2 * m_blk + rank;
                        // k-block kb = (tap (kh, kw), channel block), walked with counters (no
                        // divisions on the producer's per-k-block path)
                        if (kb == 0) {
                            const int cta_tile = tr.m_blk * 2 + (int)rank;
                            img = cta_tile / p.conv_th;
                            oh0 = (cta_tile % p.conv_th) * p.conv_bh;
                            kh = kw = cb = 0;
                        }
                        const int c0 = cb * BK;
                        if (rank == 0)
                            tc::mbar_arrive_expect_tx(tc::smem_u32(&sh->full[stage]),
                                                      2 * (a_bytes + rows_b * BK * 2));
                        // input pixel of output (oh, ow) under tap (kh, kw): (oh * sh + kh - ph, ow * sw + kw - pw),
                        // the strides being the tensor map's traversal strides;
                        // pixels outside the image (and images past the last) read as zeros
                        tc::tma_load_4d_pair(dst, &map_a, lead_full, c0, kw - p.conv_pw, oh0 * p.conv_sh + kh - p.conv_ph, img);
                        tc::tma_load_2d_pair(dst + A_BYTES, &map_b, lead_full, kb * BKE, n0);
                        if (rows_b == 128)
                            tc::tma_load_2d_pair(dst + A_BYTES + B_BYTES / 2, &map_b, lead_full, kb * BKE, n0 + 64);
                        if (++cb == p.conv_cpb) { cb = 0; if (++kw == p.conv_KW) { kw = 0; kh++; } }
                    } else {
                        if (rank == 0)   // the leader expects the bytes of both CTAs
                            tc::mbar_arrive_expect_tx(tc::smem_u32(&sh->full[stage]),
                                                      2 * (A_BYTES + rows_b * BK * 2));
                        tc::tma_load_2d_pair(dst, &map_a, lead_full, kb * BKE, m0);
                        tc::tma_load_2d_pair(dst + A_BYTES, &map_b, lead_full, kb * BKE, n0);
                        if (rows_b == 128)
                            tc::tma_load_2d_pair(dst + A_BYTES + B_BYTES / 2, &map_b, lead_full, kb * BKE, n0 + 64);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true, ready = false;
            int it = 0;
            for (int t = pair; t < p.num_items && ok; t += num_pairs, it++) {
                uint32_t acc, acc_phase;
                acc_of(it, acc, acc_phase);
                const TileRef tr = tile_ref(p, t);
                const uint32_t idesc = F8 ? tc::idesc_f16(BM, tr.is_half ? BN / 2 : BN, 0, 0)   // E4M3 x E4M3
                                          : tc::idesc_f16(BM, tr.is_half ? BN / 2 : BN, 1, 1);  // bf16 x bf16
                ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_empty[acc]), acc_phase ^ 1, abort_flag, ERR_MMA_TMEM);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_cols;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!ready) {
                        ok = tc::mbar_wait(tc::smem_u32(&sh->full[stage]), phase, abort_flag, ERR_MMA_FULL);
                        if (!ok) break;
                    }
                    tc::tc_fence_after();
                    const uint32_t nstage = stage + 1 == (uint32_t)STAGES ? 0u : stage + 1;
                    const uint32_t nphase = nstage == 0 ? phase ^ 1u : phase;
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {   // four 32-byte k-steps either way
                        if constexpr (F8)
                            tc::tc_mma_f8_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                        else
                            tc::tc_mma_f16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                        // look at the next slot's barrier while the MMAs are being taken up: the
                        // answer is there when this k-block's commit has been issued
                        if (k == 0) ready = tc::mbar_test_wait(tc::smem_u32(&sh->full[nstage]), nphase);
                    }
                    tc::tc_commit_pair(tc::smem_u32(&sh->empty[stage]), 3);   // both CTAs' slots
                    stage = nstage;
                    phase = nphase;
                }
                if (ok) tc::tc_commit_pair(tc::smem_u32(&sh->tmem_full[acc]), 3);
            }
        }
    } else if (CONV && warp >= FIRST_CONV_WARP) {
        // ------------------------------------------------------------ converters (both CTAs)
        if constexpr (CONV) {
            // The eight warps form PAIR_CONV_GROUPS groups that take alternate k-blocks, so that
            // many k-blocks are being expanded at any time (a group's wait -> load -> expand -> store
            // -> fence -> arrive chain is latency-bound).  A group reads the codes of its next
            // k-block into registers before it expands the current one.  Chunk i = 16 codes:
            // row i/4, quarter i%4 of the 64-byte raw row; rows past a half-width tile's extent are
            // read (inside the slot) and dropped.
            constexpr int G = PAIR_CONV_GROUPS, GT = 256 / G, CH = 512 / GT;
            const int cidx = threadIdx.x - 32 * FIRST_CONV_WARP;          // 0..255
            const int grp = cidx / GT, ct = cidx % GT;
            bool ok = true;
            uint4 nxt[CH];
            auto load_codes = [&](uint32_t st) {
                const uint32_t codes = tiles + st * STAGE_BYTES + A_BYTES + B_BYTES;
#pragma unroll
                for (int j = 0; j < CH; j++)
                    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(nxt[j].x), "=r"(nxt[j].y), "=r"(nxt[j].z), "=r"(nxt[j].w)
                                 : "r"(codes + (ct + GT * j) * 16));
            };
            const int my_tiles = pair < p.num_items ? (p.num_items - pair + num_pairs - 1) / num_pairs : 0;
            const int total_units = my_tiles * num_kb;
            // ring position of unit `unit` (all k-blocks of this CTA, in order)
            uint32_t stage = 0, phase = 0;
            auto step = [&](uint32_t& st, uint32_t& ph, int n) {
                st += n;
                if (st >= (uint32_t)STAGES) { st -= STAGES; ph ^= 1u; }
            };
            if (grp < total_units) {
                ok = tc::mbar_wait(tc::smem_u32(&sh->raw_full[grp]), 0, abort_flag, ERR_CONVERT);   // grp < STAGES
                if (ok) load_codes(grp);
            }
            int unit = 0;
            for (int t = pair; t < p.num_items && ok; t += num_pairs) {
                const TileRef tr = tile_ref(p, t);
                const int rows_b = (tr.is_half ? BN / 2 : BN) / 2;
                for (int kb = 0; kb < num_kb; kb++, unit++, step(stage, phase, 1)) {
                    if ((unit % G) != grp) continue;
                    uint4 in[CH];
#pragma unroll
                    for (int j = 0; j < CH; j++) in[j] = nxt[j];
                    if (unit + G < total_units) {
                        // the codes of this group's next k-block have landed (the producer runs ahead)
                        uint32_t nstage = stage, nphase = phase;
                        step(nstage, nphase, G);
                        ok = ok && tc::mbar_wait(tc::smem_u32(&sh->raw_full[nstage]), nphase, abort_flag, ERR_CONVERT);
                        if (ok) load_codes(nstage);
                    }
                    // the B slot is free once the MMAs of its previous use have completed
                    ok = ok && tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_CONVERT);
                    ok = __all_sync(0xFFFFFFFFu, ok);
                    if (!ok) break;
                    const uint32_t b_dst = tiles + stage * STAGE_BYTES + A_BYTES;
                    // 16 codes -> 16-byte chunks 2q, 2q+1 of the 128-byte operand row, placed by
                    // the 128-byte swizzle (chunk index XOR row mod 8)
#pragma unroll
                    for (int j = 0; j < CH; j++) {
                        const int i = ct + GT * j;
                        if (i < rows_b * 4) {
                            const int r = i >> 2, q = i & 3;
                            uint4 lo, hi;
                            if (p.codes_finite) expand16<FUSED, false>(in[j], lo, hi);
                            else expand16<FUSED, true>(in[j], lo, hi);
                            const uint32_t row_base = b_dst + (r >> 3) * 1024 + (r & 7) * 128;
                            const uint32_t c0 = (uint32_t)((2 * q) ^ (r & 7)), c1 = (uint32_t)((2 * q + 1) ^ (r & 7));
                            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(row_base + c0 * 16),
                                         "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w) : "memory");
                            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(row_base + c1 * 16),
                                         "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w) : "memory");
                        }
                    }
                    // make the generic-proxy writes visible to the tensor core's (async proxy)
                    // reads, then one arrival per warp on the leader's full barrier (CTA-scope
                    // release: a cluster-scope release here cost 2x in whole-kernel time)
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive_remote(tc::mapa(tc::smem_u32(&sh->full[stage]), 0));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int quarter = warp & 3;                 // the TMEM lanes this warp may read
        const int colgrp = (warp - 2) >> 2;           // 0 / 1: even / odd 32-column chunks
        const int et = threadIdx.x - 64;              // 0 .. 255
        const bool vec32 = (p.N % 16) == 0;
        bool ok = true;
        int it = 0;
        for (int t = pair; t < p.num_items && ok; t += num_pairs, it++) {
            uint32_t acc, acc_phase;
            acc_of(it, acc, acc_phase);
            const TileRef tr = tile_ref(p, t);
            const int bn = tr.is_half ? BN / 2 : BN;
            const int m0 = tr.m_blk * BM + (int)rank * 128;
            const int n0 = tr.n_blk * BN + tr.half * (BN / 2);
            // this buffer's scale and bias rows (2 x 256 or 4 x 128 floats)
            float* sc = &sh->scale[0][0] + acc * acc_cols;
            float* bi = &sh->bias[0][0] + acc * acc_cols;
            for (int c = et; c < bn; c += 32 * EPI_WARPS) {
                int n = n0 + c;
                sc[c] = (p.scales && n < p.N) ? p.scales[n] : 1.f;
                bi[c] = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            }
            ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_full[acc]), acc_phase, abort_flag, ERR_EPILOGUE);
            ok = epilogue_all<32 * EPI_WARPS>(ok);
            if (!ok) break;
            tc::tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * acc_cols + ((uint32_t)(quarter * 32) << 16);
            // implicit convolution: row r of this CTA's tile is output position oh0 * OW + r of
            // image img (the box spans whole output rows); each thread owns one position, so for a
            // fixed channel a warp writes 32 consecutive floats of the NCHW plane
            bool valid = row < p.M;
            float* obase = nullptr;
            int S = 0;
            if constexpr (IMPL) {
                const int cta_tile = tr.m_blk * 2 + (int)rank;
                const int img = cta_tile / p.conv_th, oh0 = (cta_tile % p.conv_th) * p.conv_bh;
                const int r_in = quarter * 32 + lane;
                S = p.conv_OH * p.conv_OW;
                const int pos = oh0 * p.conv_OW + r_in;
                valid = img < p.conv_images && r_in < p.conv_bw * p.conv_bh && pos < S;
                obase = (float*)p.y + ((size_t)img * p.N + n0) * S + pos;
            }
            auto emit = [&](uint32_t* r, int c) {      // one 32-column chunk of this thread's row
                if (!valid) return;
                if constexpr (IMPL) {
#pragma unroll
                    for (int j8 = 0; j8 < 32; j8 += 8) {
                        if (n0 + c + j8 >= p.N) break;      // N % 8 == 0: groups of 8 are in or out together
                        float s8[8], b8[8];
                        load8_f32(s8, sc + c + j8);
                        load8_f32(b8, bi + c + j8);
#pragma unroll
                        for (int j = 0; j < 8; j += 2) {
                            const float v0 = fmaf(__uint_as_float(r[j8 + j]), s8[j], b8[j]);
                            const float v1 = fmaf(__uint_as_float(r[j8 + j + 1]), s8[j + 1], b8[j + 1]);
                            const uint32_t pk = pack_bf16(v0, v1);     // the bf16 result, widened again
                            obase[(size_t)(c + j8 + j) * S] = __uint_as_float(pk << 16);
                            obase[(size_t)(c + j8 + j + 1) * S] = __uint_as_float(pk & 0xFFFF0000u);
                        }
                    }
                } else {
                    if (p.row_scales) {   // per-row activation scale (quantised activations)
                        const float rs = p.row_scales[row];
#pragma unroll
                        for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__fmul_rn(__uint_as_float(r[j]), rs));
                    }
                    store_row_chunk(p, r, &sc[c], &bi[c], row, n0 + c, vec32);
                }
            };
            // this warp's chunks: columns colgrp*32 + 64*i
            const int c_first = colgrp * 32;
            if constexpr (CONV) {
                // the fused variant runs 18 warps, which leaves 96 registers per thread: one chunk
                // buffer (a second one spilled, and the spill reloads stalled the converter warps)
#pragma unroll 1
                for (int c = c_first; c < bn; c += 64) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(taddr + c, r);
                    tc::tmem_ld_wait();
                    emit(r, c);
                }
            } else {
                // chunk i+1 is loaded from TMEM while chunk i is scaled and stored (tcgen05.wait::ld
                // waits for every load issued so far, so the next load is issued right after the wait)
                uint32_t ra[32], rb[32];
                tc::tmem_ld_32x32(taddr + c_first, ra);
#pragma unroll
                for (int i = 0; i < BN / 64; i += 2) {
                    const int c0 = c_first + 64 * i, c1 = c0 + 64, c2 = c1 + 64;
                    if (c0 < bn) {
                        tc::tmem_ld_wait();
                        if (c1 < bn) tc::tmem_ld_32x32(taddr + c1, rb);
                        emit(ra, c0);
                    }
                    if (c1 < bn) {
                        tc::tmem_ld_wait();
                        if (c2 < bn) tc::tmem_ld_32x32(taddr + c2, ra);
                        emit(rb, c1);
                    }
                }
            }
            tc::tc_fence_before();
            __syncwarp();
            // CTA-scope arrival: what it publishes is "the TMEM reads of this warp are complete"
            // (tcgen05.wait::ld above); a cluster-scope release would also wait for this warp's
            // global stores to be acknowledged, which costs microseconds per tile
            if (lane == 0) tc::mbar_arrive_remote(tc::mapa(tc::smem_u32(&sh->tmem_empty[acc]), 0));
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

template <int FUSED>
static nvq_status launch_pair(uint16_t* d_y, const void* d_x, const void* d_w,
                              const float* d_scales, const float* d_bias, size_t M, size_t N,
                              size_t K, int out_f32, int device, cudaStream_t st,
                              const float* row_scales = nullptr, int codes_finite = 0) {
    CUtensorMap map_a, map_b;
    constexpr bool F8 = Cfg<FUSED>::F8;
    // operand tiles: 128-byte rows with the 128-byte swizzle (64 bf16 or 128 FP8 codes)
    nvq_status s = F8 ? nvq_make_tmap_2d(&map_a, d_x, M, K, 128, 128, 1, 1)
                      : nvq_make_tmap_2d(&map_a, d_x, M, K, 128, BK, 2, 1);
    if (s != NVQ_OK) return s;
    // fused: codes, 64-byte rows, no swizzle (the converters read them linearly)
    s = F8 ? nvq_make_tmap_2d(&map_b, d_w, N, K, 64, 128, 1, 1)
           : (FUSED ? nvq_make_tmap_2d(&map_b, d_w, N, K, 64, BK, 1, 0)
                    : nvq_make_tmap_2d(&map_b, d_w, N, K, 64, BK, 2, 1));
    if (s != NVQ_OK) return s;
    static std::atomic<bool> attr_set[64];   // per device; setting the attribute twice is harmless
    if (!attr_set[device]) {
        NVQ_CUDA(cudaFuncSetAttribute(linear_tc_pair_kernel<FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg<FUSED>::SMEM_BYTES));
        attr_set[device] = true;
    }
    LinearParams p;
    p.y = d_y;
    p.out_f32 = out_f32;
    p.wq = nullptr;
    p.row_scales = row_scales;
    p.codes_finite = codes_finite;
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
    if (p.N <= BN / 2) split = 0;   // every tile is half-width already
    p.num_big = tiles - split;
    p.num_items = p.num_big + 2 * split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(Cfg<FUSED>::THREADS);
    cfg.dynamicSmemBytes = Cfg<FUSED>::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start under the tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;            // of the previous kernel
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NVQ_CUDA(cudaLaunchKernelEx(&cfg, linear_tc_pair_kernel<FUSED>, map_a, map_b, p));
    NVQ_LAUNCHED();
    return NVQ_OK;
}

static nvq_status launch_implicit_conv(float* d_out, const uint16_t* d_x_nhwc, const uint16_t* d_w,
                                       const float* d_scales, const float* d_bias, int N, int C, int H,
                                       int W, int Cout, int KH, int KW, int ph, int pw, int sh, int sw,
                                       int device, cudaStream_t st) {
    const int OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
    NVQ_REQUIRE(OH > 0 && OW > 0 && OW <= 128 && C % 64 == 0 && Cout % 8 == 0,
                "implicit convolution: needs OW <= 128, C %% 64 == 0, Cout %% 8 == 0");
    // box height: whole output rows, at most 128 positions, least padding over the image
    int bh = 1;
    long best = -1;
    for (int h = 1; h <= OH && h * OW <= 128; h++) {
        long tiles = (OH + h - 1) / h;
        if (best < 0 || tiles < best) { best = tiles; bh = h; }
    }
    const int th = (OH + bh - 1) / bh;
    const size_t K = (size_t)KH * KW * C;
    CUtensorMap map_a, map_b;
    nvq_status s = nvq_make_tmap_nhwc(&map_a, d_x_nhwc, N, H, W, C, OW, bh, sw, sh);
    if (s != NVQ_OK) return s;
    s = nvq_make_tmap_2d(&map_b, d_w, Cout, K, 64, BK, 2, 1);
    if (s != NVQ_OK) return s;
    static std::atomic<bool> attr_set[64];   // per device; setting the attribute twice is harmless
    if (!attr_set[device]) {
        NVQ_CUDA(cudaFuncSetAttribute(linear_tc_pair_kernel<kImplicitConv>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg<kImplicitConv>::SMEM_BYTES));
        attr_set[device] = true;
    }
    LinearParams p = {};
    p.y = (uint16_t*)d_out;
    p.out_f32 = 1;
    p.scales = d_scales;
    p.bias = d_bias;
    p.M = N * th * 128;
    p.N = Cout;
    p.K = (int)K;
    p.m_blocks = (N * th + 1) / 2;
    p.n_blocks = (Cout + BN - 1) / BN;
    p.group_m = 8;
    p.conv_bw = OW; p.conv_bh = bh; p.conv_th = th;
    p.conv_images = N; p.conv_OH = OH; p.conv_OW = OW;
    p.conv_KW = KW; p.conv_ph = ph; p.conv_pw = pw; p.conv_sh = sh; p.conv_cpb = C / 64;
    s = nvq_status_word(device, &p.status);
    if (s != NVQ_OK) return s;
    int tiles = p.m_blocks * p.n_blocks;
    int pairs = nvq_sm_count(device) / 2;
    if (tiles < pairs) pairs = tiles;
    int rem = tiles % pairs;
    int split = (tiles > pairs && rem > 0 && 2 * rem <= pairs) ? rem : 0;
    if (p.N <= BN / 2) split = 0;   // every tile is half-width already
    p.num_big = tiles - split;
    p.num_items = p.num_big + 2 * split;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(Cfg<kImplicitConv>::THREADS);
    cfg.dynamicSmemBytes = Cfg<kImplicitConv>::SMEM_BYTES;
    cfg.stream = st;
    NVQ_CUDA(cudaLaunchKernelEx(&cfg, linear_tc_pair_kernel<kImplicitConv>, map_a, map_b, p));
    NVQ_LAUNCHED();
    return NVQ_OK;
}

}  // namespace

nvq_status nvq_conv_launch_pair_implicit(float* d_out, const uint16_t* d_x_nhwc, const uint16_t* d_w,
                                         const float* d_scales, const float* d_bias, int N, int C,
                                         int H, int W, int Cout, int KH, int KW, int ph, int pw,
                                         int sh, int sw, int device, cudaStream_t st) {
    return launch_implicit_conv(d_out, d_x_nhwc, d_w, d_scales, d_bias, N, C, H, W, Cout, KH, KW, ph, pw,
                                sh, sw, device, st);
}

nvq_status nvq_linear_launch_pair(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int out_f32, int device, cudaStream_t st) {
    return launch_pair<0>(d_y, d_x, d_w, d_scales, d_bias, M, N, K, out_f32, device, st);
}

nvq_status nvq_linear_launch_pair_fused(uint16_t* d_y, const uint16_t* d_x, const uint8_t* d_wq,
                                        nvq_dtype fmt, const float* d_scales, const float* d_bias,
                                        size_t M, size_t N, size_t K, int out_f32, int device, cudaStream_t st,
                                        int codes_finite) {
    NVQ_REQUIRE(K % 16 == 0, "nvq_linear_fwd: K (%zu) must be a multiple of 16 for the fused FP8 path", K);
    if (fmt == NVQ_E4M3)
        return launch_pair<NVQ_E4M3>(d_y, d_x, d_wq, d_scales, d_bias, M, N, K, out_f32, device, st, nullptr,
                                     codes_finite);
    return launch_pair<NVQ_E5M2>(d_y, d_x, d_wq, d_scales, d_bias, M, N, K, out_f32, device, st, nullptr,
                                 codes_finite);
}

// W8A8: X and W both E4M3 codes, per-row and per-channel scales applied in the epilogue
nvq_status nvq_linear_launch_pair_w8a8(uint16_t* d_y, const uint8_t* d_xq, const float* d_x_scales,
                                       const uint8_t* d_wq, const float* d_w_scales,
                                       const float* d_bias, size_t M, size_t N, size_t K, int device,
                                       cudaStream_t st) {
    return launch_pair<kW8A8>(d_y, d_xq, d_wq, d_w_scales, d_bias, M, N, K, 0, device, st, d_x_scales);
}
