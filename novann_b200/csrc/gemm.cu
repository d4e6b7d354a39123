// Quantised-weight Linear forward on the tcgen05 tensor cores (the replacement for
// F.linear, novann/functional.py:147-163, when the weight is stored as FP8 / FP4):
//   Y[m,n] = bf16( s_n * sum_k X[m,k] * Wd[n,k] + b_n )
// X is M x K bf16 (K contiguous); Wd is the N x K weight whose codes were expanded to
// 16-bit values that represent them exactly (every E4M3 / E5M2 / E2M1 value is a bf16
// value), so the per-channel scale factors out of the K sum and is applied in the
// epilogue together with the bias and the bf16 rounding.
//
// Kernel: persistent, one CTA per SM, warp specialised.
//   warp 0      TMA producer: A (128 x 64) and B (BN x 64) tiles, 128-byte swizzle,
//               STAGES-deep ring of shared-memory slots guarded by full/empty mbarriers
//   warp 1      TMEM allocation, then one lane issues tcgen05.mma (128 x BN x 16, bf16 in,
//               fp32 accumulators in TMEM); tcgen05.commit frees the slot / publishes the tile
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp its own 32 TMEM lanes),
//               scale, bias, round, 32-byte global stores.  Two accumulators (2 x 256
//               TMEM columns) let the epilogue of tile i overlap the main loop of tile i+1.
// No TMA multicast and no peer memory anywhere: each CTA fetches its own tiles.
#include <stdlib.h>

#include <mutex>

#include "elementwise.cuh"
#include "gemm_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;          // 64 bf16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;  // two BN-column accumulators
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 8192 /*barriers, scales*/;

enum { ERR_PRODUCER = 1, ERR_MMA_FULL = 2, ERR_MMA_TMEM = 3, ERR_EPILOGUE = 4 };

struct Shared {            // lives after the tile ring
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float scale[2][BN];   // read as float4 by the epilogue
    alignas(16) float bias[2][BN];
};

__global__ void __launch_bounds__(THREADS, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const LinearParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;          // 1024-byte aligned tile ring
    Shared* sh = (Shared*)(smem_raw + (tiles - raw) + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.num_items;
    const int num_kb = (p.K + BK - 1) / BK;
    volatile int* abort_flag = &sh->abort_flag;

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
        tc::tma_prefetch_desc(&map_a);
        tc::tma_prefetch_desc(&map_b);
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
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const TileRef tr = tile_ref(p, t);
                const int bn = tr.is_half ? BN / 2 : BN;
                const int m0 = tr.m_blk * BM, n0 = tr.n_blk * BN + tr.half * (BN / 2);
                for (int kb = 0; kb < num_kb; kb++) {
                    ok = tc::mbar_wait(tc::smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, ERR_PRODUCER);
                    if (!ok) break;
                    const uint32_t bar = tc::smem_u32(&sh->full[stage]);
                    const uint32_t a_dst = tiles + stage * STAGE_BYTES;
                    // B arrives as 128-row boxes; 256 rows are two boxes back to back, which is
                    // the same shared-memory image as one 256-row tile
                    tc::mbar_arrive_expect_tx(bar, A_BYTES + (bn / 128) * (B_BYTES / 2));
                    tc::tma_load_2d(a_dst, &map_a, bar, kb * BK, m0);
                    tc::tma_load_2d(a_dst + A_BYTES, &map_b, bar, kb * BK, n0);
                    if (bn == BN)
                        tc::tma_load_2d(a_dst + A_BYTES + B_BYTES / 2, &map_b, bar, kb * BK, n0 + 128);
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
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it++) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_empty[acc]), acc_phase ^ 1, abort_flag, ERR_MMA_TMEM);
                if (!ok) break;
                tc::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const uint32_t idesc = tc::idesc_f16(BM, tile_ref(p, t).is_half ? BN / 2 : BN, 1, 1);
                for (int kb = 0; kb < num_kb; kb++) {
                    ok = tc::mbar_wait(tc::smem_u32(&sh->full[stage]), phase, abort_flag, ERR_MMA_FULL);
                    if (!ok) break;
                    tc::tc_fence_after();
                    const uint32_t a_addr = tiles + stage * STAGE_BYTES;
                    const uint64_t a_desc = tc::smem_desc_k_sw128(a_addr);
                    const uint64_t b_desc = tc::smem_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; k++) {
                        // advancing 16 elements along K = 32 bytes = 2 units of the address field
                        tc::tc_mma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
                    }
                    tc::tc_commit(tc::smem_u32(&sh->empty[stage]));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc::tc_commit(tc::smem_u32(&sh->tmem_full[acc]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quarter = warp & 3;               // the 32 TMEM lanes this warp may read
        const int et = threadIdx.x - 64;            // 0..127
        const bool vec32 = (p.N % 16) == 0;         // rows then start on 32-byte boundaries
        bool ok = true;
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it++) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            const TileRef tr = tile_ref(p, t);
            const int bn = tr.is_half ? BN / 2 : BN;
            const int m0 = tr.m_blk * BM, n0 = tr.n_blk * BN + tr.half * (BN / 2);
            // per-tile scale / bias into shared memory (two columns per thread)
            for (int c = et; c < bn; c += 128) {
                int n = n0 + c;
                sh->scale[acc][c] = (p.scales && n < p.N) ? p.scales[n] : 1.f;
                sh->bias[acc][c] = (p.bias && n < p.N) ? p.bias[n] : 0.f;
            }
            ok = tc::mbar_wait(tc::smem_u32(&sh->tmem_full[acc]), acc_phase, abort_flag, ERR_EPILOGUE);
            // barrier over the four epilogue warps: publishes scale/bias and makes the
            // go / give-up decision the same for all of them
            ok = epilogue_all(ok);
            if (!ok) break;
            tc::tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < bn; c += 32) {
                uint32_t r[32];
                tc::tmem_ld_32x32(taddr + c, r);
                tc::tmem_ld_wait();
                if (row < p.M)
                    store_row_chunk(p, r, &sh->scale[acc][c], &sh->bias[acc][c], row, n0 + c, vec32);
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tc::smem_u32(&sh->tmem_empty[acc]));
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        // a role gave up: let copies still in flight land before the CTA retires
        for (int i = 0; i < 64; i++) __nanosleep(20000);
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    if (warp == 1) tc::tmem_dealloc(tmem_base, TMEM_COLS);
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicCAS(p.status, 0, *abort_flag);
}

// ---- exact expansion of weight codes to bf16 (workspace fill) -------------------------
// 16 codes -> 16 bf16 per packet through the elementwise driver (several packets in flight per
// thread; the 32 MB it writes for a 4096 x 4096 weight stay in L2 for the GEMM that follows).
// Every E4M3 / E5M2 value is exactly a bf16 value.
template <int FMT>
struct ExpandOp {
    static constexpr int VEC = 16;
    static constexpr int UNROLL = 4;
    static constexpr int RESIDENT = 0;
    using In = uint4;
    // lets the GEMM that follows in the stream start its set-up (barriers, TMEM, descriptors)
    // while this kernel is still running; the GEMM waits for this grid before its first load
    __device__ __forceinline__ void init() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        return ldg_stream_128((const char*)src + p * 16);
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& in) const {
        // Bit placement + one bf16 multiply per pair of codes (integer / FMA pipes), non-finite
        // codes patched: exact for all 256 codes.  The hardware converters (e4m3x2 -> f16x2 -> f32
        // -> bf16x2) cost eight conversion-unit operations per four codes and made this pass
        // conversion-bound: 10.5 us for 16.8 M codes whose DRAM read takes 2.6 us.
        uint4 lo, hi;
        expand16<FMT, true>(in, lo, hi);
        u32x8 o;
        o.v[0] = lo.x; o.v[1] = lo.y; o.v[2] = lo.z; o.v[3] = lo.w;
        o.v[4] = hi.x; o.v[5] = hi.y; o.v[6] = hi.z; o.v[7] = hi.w;
        // plain (L2-allocating) store: the GEMM reads this back at once
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"((char*)dst + p * 32),
                     "r"(o.v[0]), "r"(o.v[1]), "r"(o.v[2]), "r"(o.v[3]), "r"(o.v[4]), "r"(o.v[5]),
                     "r"(o.v[6]), "r"(o.v[7])
                     : "memory");
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        uint32_t c = ((const uint8_t*)src)[i];
        uint32_t t = FMT == NVQ_E4M3 ? spec_fp8_to_f32<NVQ_E4M3>(c) : spec_fp8_to_f32<NVQ_E5M2>(c);
        ((uint16_t*)dst)[i] = (uint16_t)(t >> 16);   // exact: the low 16 bits are zero
    }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int* g_status_host[64];   // mapped pinned words, one per device
int* g_status_dev[64];

}  // namespace

// set by the allocation-free entry point for the duration of its launches (per thread)
static std::mutex g_status_mu;
static thread_local bool t_status_override = false;
static thread_local int* t_status_override_ptr = nullptr;

nvq_status nvq_status_word(int device, int** dev_ptr) {
    if (t_status_override) {
        *dev_ptr = t_status_override_ptr;
        return NVQ_OK;
    }
    std::lock_guard<std::mutex> lock(g_status_mu);
    if (!g_status_host[device]) {
        int* h = nullptr;
        NVQ_CUDA(cudaHostAlloc((void**)&h, sizeof(int), cudaHostAllocMapped));
        *h = 0;
        NVQ_CUDA(cudaHostGetDevicePointer((void**)&g_status_dev[device], h, 0));
        g_status_host[device] = h;
    }
    *dev_ptr = g_status_dev[device];
    return NVQ_OK;
}

static nvq_status ensure_encode() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        NVQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (!fn || q != cudaDriverEntryPointSuccess)
            NVQ_FAIL(NVQ_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
        g_encode = (EncodeTiledFn)fn;
    }
    return NVQ_OK;
}

nvq_status nvq_make_tmap_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                            uint32_t box_rows, uint32_t box_cols, int elem_bytes, int swizzle128) {
    nvq_status s0 = ensure_encode();
    if (s0 != NVQ_OK) return s0;
    NVQ_REQUIRE(nvq_aligned(base, 16), "tensor base must be 16-byte aligned");
    NVQ_REQUIRE((cols * elem_bytes) % 16 == 0, "row pitch (%llu bytes) must be a multiple of 16",
                (unsigned long long)(cols * elem_bytes));
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    // 16-bit operand tiles use the 128-byte swizzle the MMA descriptors name; byte tiles
    // (raw codes read by converter warps) are stored linearly
    CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) NVQ_FAIL(NVQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return NVQ_OK;
}

// fp32 NCHW output seen as (image, channel, position): box = 32 channels x 32 positions of one
// image, 128-byte rows with the 128-byte swizzle (the layout the storing warps write)
nvq_status nvq_make_tmap_nchw_out(CUtensorMap* map, const void* base, uint64_t N, uint64_t C, uint64_t S) {
    nvq_status s0 = ensure_encode();
    if (s0 != NVQ_OK) return s0;
    NVQ_REQUIRE(nvq_aligned(base, 16) && S % 4 == 0, "NCHW output map: base and plane size must be 16-byte multiples");
    cuuint64_t dims[3] = {S, C, N};
    cuuint64_t strides[2] = {S * 4, C * S * 4};
    cuuint32_t box[3] = {32, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) NVQ_FAIL(NVQ_ERR_CUDA, "cuTensorMapEncodeTiled (NCHW output) failed with %d", (int)r);
    return NVQ_OK;
}

nvq_status nvq_make_tmap_nhwc(CUtensorMap* map, const void* base, uint64_t N, uint64_t H, uint64_t W,
                              uint64_t C, uint32_t box_w, uint32_t box_h, uint32_t stride_w,
                              uint32_t stride_h) {
    nvq_status s0 = ensure_encode();
    if (s0 != NVQ_OK) return s0;
    NVQ_REQUIRE(nvq_aligned(base, 16), "tensor base must be 16-byte aligned");
    NVQ_REQUIRE(C % 64 == 0, "NHWC map: channels (%llu) must be a multiple of 64", (unsigned long long)C);
    NVQ_REQUIRE(box_w >= 1 && box_h >= 1 && box_w <= 256 && box_h <= 256 && box_w * box_h <= 256,
                "NHWC map: box %u x %u does not fit a 256-row operand tile", box_w, box_h);
    cuuint64_t dims[4] = {C, W, H, N};
    cuuint64_t strides[3] = {C * 2, W * C * 2, H * W * C * 2};
    NVQ_REQUIRE(stride_w >= 1 && stride_w <= 8 && stride_h >= 1 && stride_h <= 8 &&
                    box_w * stride_w <= 256 && box_h * stride_h <= 256,
                "NHWC map: strides %u x %u out of range for a box of %u x %u", stride_w, stride_h, box_w, box_h);
    // with a traversal stride s the box extent is given in pixels walked: n loaded pixels = n * s
    cuuint32_t box[4] = {64, box_w * stride_w, box_h * stride_h, 1};
    cuuint32_t estr[4] = {1, stride_w, stride_h, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) NVQ_FAIL(NVQ_ERR_CUDA, "cuTensorMapEncodeTiled (NHWC) failed with %d", (int)r);
    return NVQ_OK;
}

nvq_status nvq_linear_launch_single(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w_bf16,
                                    const float* d_scales, const float* d_bias, size_t M, size_t N,
                                    size_t K, int out_f32, int device, cudaStream_t st) {
    CUtensorMap map_a, map_b;
    nvq_status s = nvq_make_tmap_2d(&map_a, d_x, M, K, BM, BK, 2, 1);
    if (s != NVQ_OK) return s;
    s = nvq_make_tmap_2d(&map_b, d_w_bf16, N, K, BN / 2, BK, 2, 1);
    if (s != NVQ_OK) return s;
    static std::atomic<bool> attr_set[64];   // per device; setting the attribute twice is harmless
    if (!attr_set[device]) {
        NVQ_CUDA(cudaFuncSetAttribute(linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set[device] = true;
    }
    LinearParams p = {};
    p.y = d_y;
    p.out_f32 = out_f32;
    p.wq = nullptr;
    p.row_scales = nullptr;
    p.scales = d_scales;
    p.bias = d_bias;
    p.M = (int)M;
    p.N = (int)N;
    p.K = (int)K;
    p.m_blocks = (int)((M + BM - 1) / BM);
    p.n_blocks = (int)((N + BN - 1) / BN);
    p.group_m = 16;
    s = nvq_status_word(device, &p.status);
    if (s != NVQ_OK) return s;
    int tiles = p.m_blocks * p.n_blocks;
    int sms = nvq_sm_count(device);
    int grid = tiles < sms ? tiles : sms;
    // a partial last wave that would occupy at most half of the CTAs is cut into halves
    int rem = tiles % grid;
    int split = (tiles > grid && rem > 0 && 2 * rem <= grid) ? rem : 0;
    p.num_big = tiles - split;
    p.num_items = p.num_big + 2 * split;
    linear_tc_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(map_a, map_b, p);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

// Y = bf16(scale_n * X @ Wd^T + bias_n) with Wd already expanded to bf16 (N x K).
// More than 128 rows: CTA pairs on 256 x 256 tiles; otherwise one CTA per 128 x 256 tile.
// `kernel` (0 = by M, 1 = single CTA, 2 = CTA pair) carries the caller's path selector.
nvq_status nvq_linear_bf16_launch(uint16_t* d_y, const uint16_t* d_x, const uint16_t* d_w_bf16,
                                  const float* d_scales, const float* d_bias, size_t M, size_t N,
                                  size_t K, int out_f32, int device, cudaStream_t st, int kernel) {
    NVQ_REQUIRE(K % 8 == 0 && N % 8 == 0, "nvq_linear_fwd: K (%zu) and N (%zu) must be multiples of 8", K, N);
    NVQ_REQUIRE(nvq_aligned(d_y, 32), "nvq_linear_fwd: Y must be 32-byte aligned");
    NVQ_REQUIRE(M < (1u << 31) && N < (1u << 31) && K < (1u << 31), "nvq_linear_fwd: dimension too large");
    const bool pair = kernel == 2 || (kernel == 0 && M > 128);
    if (pair) return nvq_linear_launch_pair(d_y, d_x, d_w_bf16, d_scales, d_bias, M, N, K, out_f32, device, st);
    return nvq_linear_launch_single(d_y, d_x, d_w_bf16, d_scales, d_bias, M, N, K, out_f32, device, st);
}

extern "C" nvq_status nvq_linear_workspace_bytes(size_t N, size_t K, nvq_dtype w_fmt, size_t* bytes) {
    NVQ_REQUIRE(bytes, "null out pointer");
    NVQ_REQUIRE(w_fmt == NVQ_E4M3 || w_fmt == NVQ_E5M2 || w_fmt == NVQ_E2M1_B32,
                "nvq_linear_workspace_bytes: unsupported weight format %d", (int)w_fmt);
    *bytes = N * K * 2;
    return NVQ_OK;
}

// A wait that nothing will ever satisfy, with a 1 ms limit: exercises the give-up path of the
// bounded waits (record a code, leave, report) without faulting or hanging anything.
namespace {
__global__ void wait_selftest_kernel(int* status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        tc::mbar_init(tc::smem_u32(&bar), 1);
        abort_flag = 0;
        tc::mbar_fence_init();
    }
    __syncthreads();
    bool ok = tc::mbar_wait_limit(tc::smem_u32(&bar), 0, &abort_flag, 99, 1000000ull);
    __syncthreads();
    if (threadIdx.x == 0 && !ok && status) atomicCAS(status, 0, abort_flag);
}
}  // namespace

extern "C" nvq_status nvq_selftest_bounded_wait(int device, void* stream) {
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    int* status = nullptr;
    s = nvq_status_word(device, &status);
    if (s != NVQ_OK) return s;
    wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

// Frees the status words of every device (nvq_shutdown).
nvq_status nvq_gemm_release_status_words() {
    std::lock_guard<std::mutex> lock(g_status_mu);
    for (int d = 0; d < 64; d++) {
        if (!g_status_host[d]) continue;
        NVQ_CUDA(cudaFreeHost(g_status_host[d]));
        g_status_host[d] = nullptr;
        g_status_dev[d] = nullptr;
    }
    return NVQ_OK;
}

extern "C" nvq_status nvq_device_error_flag(int device, int* flag) {
    NVQ_REQUIRE(flag && device >= 0 && device < 64, "bad argument");
    *flag = 0;
    std::lock_guard<std::mutex> lock(g_status_mu);
    if (g_status_host[device]) {
        *flag = *(volatile int*)g_status_host[device];
        *(volatile int*)g_status_host[device] = 0;
    }
    return NVQ_OK;
}

extern "C" nvq_status nvq_linear_expand_weight(uint16_t* d_wd_bf16, const uint8_t* d_wq,
                                               nvq_dtype w_fmt, const float* d_w_scales, size_t N,
                                               size_t K, int device, void* stream) {
    NVQ_REQUIRE(d_wd_bf16 && d_wq && N > 0 && K > 0, "nvq_linear_expand_weight: bad argument");
    NVQ_REQUIRE(nvq_aligned(d_wd_bf16, 32), "nvq_linear_expand_weight: destination must be 32-byte aligned");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (w_fmt == NVQ_E2M1_B32) {
        // block scales vary along K, so they are folded into the expanded weight:
        // Wd = bf16(e2m1_value * scale_block); no per-channel factor is left
        NVQ_REQUIRE(K % 32 == 0 && d_w_scales, "nvq_linear_fwd: K (%zu) must be a multiple of 32 for E2M1_B32", K);
        return nvq_dequantize_fp4_b32(d_wd_bf16, d_wq, d_w_scales, N, K, device, stream);
    }
    NVQ_REQUIRE(w_fmt == NVQ_E4M3 || w_fmt == NVQ_E5M2, "nvq_linear_expand_weight: unsupported weight format %d", (int)w_fmt);
    NVQ_REQUIRE((N * K) % 16 == 0 && nvq_aligned(d_wq, 16),
                "nvq_linear_fwd: weight codes must be 16-byte aligned, N*K a multiple of 16");
    return w_fmt == NVQ_E4M3 ? ew_launch(ExpandOp<NVQ_E4M3>{}, d_wq, d_wd_bf16, N * K, device, st, 16, 32)
                             : ew_launch(ExpandOp<NVQ_E5M2>{}, d_wq, d_wd_bf16, N * K, device, st, 16, 32);
}

extern "C" nvq_status nvq_linear_fwd_expanded(uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                              const uint16_t* d_wd_bf16, const float* d_chan_scales,
                                              const float* d_bias, size_t M, size_t N, size_t K,
                                              int relu, int device, void* stream) {
    NVQ_REQUIRE(d_y_bf16 && d_x_bf16 && d_wd_bf16 && M > 0 && N > 0 && K > 0,
                "nvq_linear_fwd_expanded: bad argument");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    return nvq_linear_bf16_launch(d_y_bf16, d_x_bf16, d_wd_bf16, d_chan_scales, d_bias, M, N, K,
                                  relu ? 2 : 0, device, (cudaStream_t)stream);
}

// ---------------------------------------------------------------- expanded-weight cache
// A weight that stays fixed over many forwards (inference, or several forwards between two
// optimiser steps) is expanded once: the cache owns the N x K bf16 copy and remembers which
// (codes pointer, scales pointer, version) it was made from.
struct nvq_linear_cache {
    size_t N, K, bytes;
    nvq_dtype fmt;
    int device;
    void* d_buf;
    const void* codes;
    const void* scales;
    uint64_t version;
    bool valid;
};

extern "C" nvq_status nvq_linear_cache_create(nvq_linear_cache** out, size_t N, size_t K,
                                              nvq_dtype w_fmt, int device) {
    NVQ_REQUIRE(out && N > 0 && K > 0, "nvq_linear_cache_create: bad argument");
    *out = nullptr;
    size_t bytes = 0;
    nvq_status s = nvq_linear_workspace_bytes(N, K, w_fmt, &bytes);
    if (s != NVQ_OK) return s;
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    void* buf = nullptr;
    NVQ_CUDA(cudaMalloc(&buf, bytes));
    *out = new nvq_linear_cache{N, K, bytes, w_fmt, device, buf, nullptr, nullptr, 0, false};
    return NVQ_OK;
}

extern "C" nvq_status nvq_linear_cache_destroy(nvq_linear_cache* c) {
    if (!c) return NVQ_OK;
    nvq_status s = nvq_use_device(c->device);
    if (s == NVQ_OK && c->d_buf) cudaFree(c->d_buf);
    delete c;
    return s;
}

extern "C" nvq_status nvq_linear_cache_fwd(nvq_linear_cache* c, uint16_t* d_y_bf16,
                                           const uint16_t* d_x_bf16, const uint8_t* d_wq,
                                           const float* d_w_scales, const float* d_bias, size_t M,
                                           uint64_t version, int relu, int* expanded, void* stream) {
    NVQ_REQUIRE(c && d_y_bf16 && d_x_bf16 && d_wq && d_w_scales && M > 0, "nvq_linear_cache_fwd: bad argument");
    if (expanded) *expanded = 0;
    const bool fp8 = c->fmt == NVQ_E4M3 || c->fmt == NVQ_E5M2;
    if (M <= 128 && !relu) {
        // few rows: the weight-streaming kernels of nvq_linear_fwd read the codes once and keep
        // partial sums in the buffer, so the expanded copy (if any) is gone afterwards
        c->valid = false;
        return nvq_linear_fwd(d_y_bf16, d_x_bf16, d_wq, c->fmt, d_w_scales, d_bias, M, c->N, c->K, c->d_buf,
                              c->bytes, c->device, stream);
    }
    if (!c->valid || c->codes != d_wq || c->scales != d_w_scales || c->version != version) {
        c->valid = false;
        nvq_status s = nvq_linear_expand_weight((uint16_t*)c->d_buf, d_wq, c->fmt, d_w_scales, c->N, c->K,
                                                c->device, stream);
        if (s != NVQ_OK) return s;
        c->codes = d_wq;
        c->scales = d_w_scales;
        c->version = version;
        c->valid = true;
        if (expanded) *expanded = 1;
    }
    return nvq_linear_fwd_expanded(d_y_bf16, d_x_bf16, (const uint16_t*)c->d_buf, fp8 ? d_w_scales : nullptr,
                                   d_bias, M, c->N, c->K, relu, c->device, stream);
}

extern "C" nvq_status nvq_linear_fwd(uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                     const uint8_t* d_wq, nvq_dtype w_fmt, const float* d_w_scales,
                                     const float* d_bias, size_t M, size_t N, size_t K,
                                     void* d_workspace, size_t workspace_bytes, int device,
                                     void* stream) {
    return nvq_linear_fwd_opts(d_y_bf16, d_x_bf16, d_wq, w_fmt, d_w_scales, d_bias, M, N, K, d_workspace,
                               workspace_bytes, NVQ_LINEAR_AUTO, device, stream);
}

extern "C" nvq_status nvq_linear_fwd_opts(uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                          const uint8_t* d_wq, nvq_dtype w_fmt,
                                          const float* d_w_scales, const float* d_bias, size_t M,
                                          size_t N, size_t K, void* d_workspace,
                                          size_t workspace_bytes, uint32_t path, int device,
                                          void* stream) {
    NVQ_REQUIRE(d_y_bf16 && d_x_bf16 && d_wq && d_w_scales, "nvq_linear_fwd: null buffer");
    NVQ_REQUIRE(K % 8 == 0 && N % 8 == 0, "nvq_linear_fwd: K (%zu) and N (%zu) must be multiples of 8", K, N);
    const uint32_t kernel_bits = path & (NVQ_LINEAR_EXPAND_IN_KERNEL | NVQ_LINEAR_SINGLE_CTA | NVQ_LINEAR_CTA_PAIR);
    NVQ_REQUIRE((path & ~(uint32_t)(NVQ_LINEAR_BF16_ACTIVATIONS | NVQ_LINEAR_EXPAND_IN_KERNEL |
                                    NVQ_LINEAR_SINGLE_CTA | NVQ_LINEAR_CTA_PAIR | NVQ_LINEAR_CLUSTER_REDUCE |
                                    NVQ_LINEAR_CODES_FINITE)) == 0 &&
                    (kernel_bits & (kernel_bits - 1)) == 0,
                "nvq_linear_fwd_opts: unknown or contradictory path selector 0x%x", path);
    NVQ_REQUIRE(M > 0 && N > 0 && K > 0, "nvq_linear_fwd: empty problem");
    NVQ_REQUIRE(w_fmt == NVQ_E4M3 || w_fmt == NVQ_E5M2 || w_fmt == NVQ_E2M1_B32,
                "nvq_linear_fwd: unsupported weight format %d", (int)w_fmt);
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    // FP8 weights, more than one row block: the CTA-pair kernel can expand the codes in shared
    // memory itself, so no expanded copy of the weight is written to HBM and no workspace is
    // needed.  Measured on B200 it is slower than expansion pass + plain pair kernel (the
    // converter warps' shared-memory traffic competes with the tensor core's operand reads),
    // so it runs when the caller passes no workspace, or asks for it (NVQ_LINEAR_EXPAND_IN_KERNEL).
    bool can_fuse = w_fmt != NVQ_E2M1_B32 && M > 128 && K % 16 == 0 && nvq_aligned(d_wq, 16);
    bool fused = can_fuse && ((path & NVQ_LINEAR_EXPAND_IN_KERNEL) || (!kernel_bits && d_workspace == nullptr));
    if (fused) {
        NVQ_REQUIRE(K % 8 == 0 && N % 8 == 0, "nvq_linear_fwd: K (%zu) and N (%zu) must be multiples of 8", K, N);
        NVQ_REQUIRE(nvq_aligned(d_y_bf16, 32), "nvq_linear_fwd: Y must be 32-byte aligned");
        NVQ_REQUIRE(M < (1u << 31) && N < (1u << 31) && K < (1u << 31), "nvq_linear_fwd: dimension too large");
        return nvq_linear_launch_pair_fused(d_y_bf16, d_x_bf16, d_wq, w_fmt, d_w_scales, d_bias, M, N, K,
                                            0, device, st, (path & NVQ_LINEAR_CODES_FINITE) ? 1 : 0);
    }
    // Few rows: the time is the time to read the weight, so read it once, as codes.  The
    // workspace then holds fp32 partial sums instead of an expanded weight.
    if (M <= 128 && K % (w_fmt == NVQ_E2M1_B32 ? 32 : 16) == 0 && nvq_aligned(d_wq, 16) && nvq_aligned(d_x_bf16, 16) &&
        d_workspace && nvq_aligned(d_workspace, 16) && !kernel_bits && M * N < (1u << 31) && N < (1u << 24) &&
        K < (1u << 24) && N * K < (1ull << 40) &&
        workspace_bytes >= nvq_linear_small_m_workspace(M, N, K, device)) {
        // FP8 codes feed the tensor cores directly (activations split into two E4M3 rows);
        // NVQ_LINEAR_BF16_ACTIVATIONS keeps the kernel that expands the codes to bf16
        if (w_fmt != NVQ_E2M1_B32 && !(path & NVQ_LINEAR_BF16_ACTIVATIONS) &&
            workspace_bytes >= nvq_linear_small_m_direct_workspace(M, N, K, device))
            return nvq_linear_launch_small_m_direct(d_y_bf16, d_x_bf16, d_wq, w_fmt, d_w_scales, d_bias, M, N,
                                                    K, d_workspace, device, st,
                                                    (path & NVQ_LINEAR_CLUSTER_REDUCE) != 0);
        return nvq_linear_launch_small_m(d_y_bf16, d_x_bf16, d_wq, w_fmt, d_w_scales, d_bias, M, N, K,
                                         (float*)d_workspace, device, st);
    }
    NVQ_REQUIRE(d_workspace && workspace_bytes >= N * K * 2 && nvq_aligned(d_workspace, 32),
                "nvq_linear_fwd: workspace of %zu bytes (32-byte aligned) required", N * K * 2);
    s = nvq_linear_expand_weight((uint16_t*)d_workspace, d_wq, w_fmt, d_w_scales, N, K, device, stream);
    if (s != NVQ_OK) return s;
    uint16_t* wd = (uint16_t*)d_workspace;
    const float* chan_scales = w_fmt == NVQ_E2M1_B32 ? nullptr : d_w_scales;
    return nvq_linear_bf16_launch(d_y_bf16, d_x_bf16, wd, chan_scales, d_bias, M, N, K, 0, device, st,
                                  (path & NVQ_LINEAR_SINGLE_CTA) ? 1 : ((path & NVQ_LINEAR_CTA_PAIR) ? 2 : 0));
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for the expanded weight lives in the library image itself: one array per GPU that
// loads the library, held until the process exits.  NVQ_STATIC_WORKSPACE_BYTES bounds N * K.
static __device__ __align__(256) unsigned char g_static_workspace[NVQ_STATIC_WORKSPACE_BYTES];
static void* g_static_workspace_addr[64];   // device address of the array, per device

extern "C" nvq_status nvq_linear_fwd_static(uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                            const uint8_t* d_wq, nvq_dtype w_fmt,
                                            const float* d_w_scales, const float* d_bias, size_t M,
                                            size_t N, size_t K, int* d_status, int device,
                                            void* stream) {
    NVQ_REQUIRE(N > 0 && K > 0 && N * K * 2 <= (size_t)NVQ_STATIC_WORKSPACE_BYTES,
                "nvq_linear_fwd_static: N * K = %zu weights need %zu bytes of scratch; the built-in "
                "scratch holds %zu bytes (N * K <= %zu). Use nvq_linear_fwd with a caller workspace.",
                N * K, N * K * 2, (size_t)NVQ_STATIC_WORKSPACE_BYTES,
                (size_t)NVQ_STATIC_WORKSPACE_BYTES / 2);
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    if (!g_static_workspace_addr[device]) {
        // In host code the array's name is only a handle; the kernels need the address the
        // array has on THIS device, which the runtime reports with that device current.
        void* addr = nullptr;
        NVQ_CUDA(cudaGetSymbolAddress(&addr, g_static_workspace));
        if (!addr) NVQ_FAIL(NVQ_ERR_CUDA, "nvq_linear_fwd_static: no device address for the scratch array");
        g_static_workspace_addr[device] = addr;
    }
    t_status_override = true;
    t_status_override_ptr = d_status;
    s = nvq_linear_fwd(d_y_bf16, d_x_bf16, d_wq, w_fmt, d_w_scales, d_bias, M, N, K,
                       g_static_workspace_addr[device], NVQ_STATIC_WORKSPACE_BYTES, device, stream);
    t_status_override = false;
    t_status_override_ptr = nullptr;
    return s;
}

// ---------------------------------------------------------------- W8A8 variant
nvq_status nvq_quantize_e4m3_rows_bf16(uint8_t* d_dst, float* d_scales, const uint16_t* d_src,
                                       size_t rows, size_t cols, cudaStream_t st);

extern "C" nvq_status nvq_linear_w8a8_workspace_bytes(size_t M, size_t K, size_t* bytes) {
    NVQ_REQUIRE(bytes, "null out pointer");
    *bytes = (M * K + 255) / 256 * 256 + M * sizeof(float);
    return NVQ_OK;
}

extern "C" nvq_status nvq_linear_fwd_w8a8(uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                          const uint8_t* d_wq, const float* d_w_scales,
                                          const float* d_bias, size_t M, size_t N, size_t K,
                                          void* d_workspace, size_t workspace_bytes, int device,
                                          void* stream) {
    NVQ_REQUIRE(d_y_bf16 && d_x_bf16 && d_wq && d_w_scales && M > 0 && N > 0 && K > 0,
                "nvq_linear_fwd_w8a8: bad argument");
    NVQ_REQUIRE(K % 16 == 0 && N % 8 == 0, "nvq_linear_fwd_w8a8: K (%zu) must be a multiple of 16, N (%zu) of 8", K, N);
    NVQ_REQUIRE(nvq_aligned(d_y_bf16, 32) && nvq_aligned(d_wq, 16), "nvq_linear_fwd_w8a8: Y 32-byte, Wq 16-byte aligned");
    size_t need = 0;
    nvq_linear_w8a8_workspace_bytes(M, K, &need);
    NVQ_REQUIRE(d_workspace && workspace_bytes >= need && nvq_aligned(d_workspace, 256),
                "nvq_linear_fwd_w8a8: workspace of %zu bytes (256-byte aligned) required", need);
    NVQ_REQUIRE(M < (1u << 31) && N < (1u << 31) && K < (1u << 31), "nvq_linear_fwd_w8a8: dimension too large");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t* xq = (uint8_t*)d_workspace;
    float* xs = (float*)((char*)d_workspace + (M * K + 255) / 256 * 256);
    s = nvq_quantize_e4m3_rows_bf16(xq, xs, d_x_bf16, M, K, st);
    if (s != NVQ_OK) return s;
    return nvq_linear_launch_pair_w8a8(d_y_bf16, xq, xs, d_wq, d_w_scales, d_bias, M, N, K, device, st);
}
