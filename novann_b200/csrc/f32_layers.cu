// fp32 pieces of the reference's training step (novann/utils/train/train.py:60-75):
// Linear forward / backward, ReLU, softmax cross-entropy, SGD, plus the fp32 im2col
// convolution forward.  These are the small, latency-bound kernels of the
// "MLP train step" configuration (batch 128, 784-256-128-10): plain fp32 FMA on the
// CUDA cores, no tensor cores, so results differ from NumPy's sgemm only by summation
// order.  Elementwise steps reproduce the reference's roundings exactly (separate
// multiply and add where NumPy performs two operations).
#include <math.h>
#include <stdlib.h>

#include <algorithm>

#include "nvq_common.cuh"
#include "gemm_common.cuh"

namespace {

// ---- generic strided fp32 GEMM ------------------------------------------------------
//   C(i,j) = sum_l A(i,l) * B(l,j),  A(i,l) = a[i*a_si + l*a_sl],  B(l,j) = b[l*b_sl + j*b_sj]
// One T x T output tile per 256-thread block (T = 32 or 16), 64-deep k chunks staged in shared
// memory.  Loads walk the unit-stride index fastest, whichever it is.

struct GemmArgs {
    const float* a; long long a_si, a_sl;
    const float* b; long long b_sl, b_sj;
    float* c;
    int I, J, L;
    // epilogue
    const float* bias;      // added per column j (bias_per_row = 0) or per row i (= 1)
    int bias_per_row;
    int relu;               // out = v * (v > 0); mask (same indexing as c) optional
    float* mask_out;
    const float* mask_in;   // out = v * mask_in[c index]
    // output indexing: 0 = row-major I x J; 1 = "NCHW": j = (n, s) with s < inner:
    //   c[(n * I + i) * inner + s]
    int out_mode, inner;
    // split-K (epilogue-free calls only): block z covers k in [z * l_per_split, (z+1) * l_per_split)
    // and stores its raw sums to partial[z][I][J]; splitk_reduce_kernel adds them in z order
    int splits, l_per_split;
    float* partial;
    // optional by-product: rowsum[i] = sum_l A(i, l), added in l order by the blocks of the first
    // tile column (Linear.backward's bias gradient = column sums of grad = row sums of grad^T)
    float* rowsum;
};

constexpr int kSplitChunk = 64;   // split-k ranges are multiples of the deepest chunk

// element e of a T x TK tile -> (row-in-tile, k-in-chunk); the index that has unit stride in
// memory runs fastest across threads so global loads coalesce
template <int T, int TK>
__device__ __forceinline__ void tile_coord(int e, bool k_contiguous, int& r, int& l) {
    if (k_contiguous) { l = e & (TK - 1); r = e / TK; }
    else              { r = e & (T - 1); l = e / T; }
}

// T x T output tile per 256-thread block: T = 32 (2 x 2 outputs per thread) for large outputs,
// T = 16 (one output per thread) when the output is so small that 32 x 32 tiles would leave
// most SMs idle - these GEMMs are latency-bound, so more blocks means more loads in flight.
// TK = k depth of one staged chunk: 64, or 16 for shallow contractions (the first convolution
// has k = 9; a 64-deep chunk would multiply 55 rows of zeros).
template <int T, int TK = 64>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const GemmArgs g) {
    nvq_chain_sync();
    constexpr int R = T / 16;                 // outputs per thread per dimension
    constexpr int LD = T * TK / 256;          // tile elements each thread stages per chunk
    // double-buffered tiles: chunk c+1 is fetched into registers while chunk c is multiplied
    __shared__ float As[2][TK][T + 1];   // [buf][l][i]
    __shared__ float Bs[2][TK][T + 1];   // [buf][l][j]
    const int i0 = blockIdx.y * T, j0 = blockIdx.x * T;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const bool a_kc = g.a_sl == 1, b_kc = g.b_sl == 1;
    float acc[R][R];
    float rs[R];
#pragma unroll
    for (int u = 0; u < R; u++) {
        rs[u] = 0.f;
#pragma unroll
        for (int v = 0; v < R; v++) acc[u][v] = 0.f;
    }
    const bool do_rowsum = g.rowsum != nullptr && blockIdx.x == 0 && tx == 0;
    float ra[LD], rb[LD];
    const int l_lo = g.splits > 1 ? blockIdx.z * g.l_per_split : 0;
    const int l_hi = g.splits > 1 ? min(g.L, l_lo + g.l_per_split) : g.L;
    auto fetch = [&](int l0) {
#pragma unroll
        for (int r = 0; r < LD; r++) {
            int e = threadIdx.x + 256 * r, ii, ll;
            tile_coord<T, TK>(e, a_kc, ii, ll);
            int i = i0 + ii, l = l0 + ll;
            ra[r] = (i < g.I && l < l_hi) ? g.a[i * g.a_si + l * g.a_sl] : 0.f;
            int jj;
            tile_coord<T, TK>(e, b_kc, jj, ll);
            int j = j0 + jj;
            l = l0 + ll;
            rb[r] = (j < g.J && l < l_hi) ? g.b[l * g.b_sl + j * g.b_sj] : 0.f;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int r = 0; r < LD; r++) {
            int e = threadIdx.x + 256 * r, ii, ll;
            tile_coord<T, TK>(e, a_kc, ii, ll);
            As[buf][ll][ii] = ra[r];
            tile_coord<T, TK>(e, b_kc, ii, ll);
            Bs[buf][ll][ii] = rb[r];
        }
    };
    fetch(l_lo);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int l0 = l_lo; l0 < l_hi; l0 += TK) {
        const bool more = l0 + TK < l_hi;
        if (more) fetch(l0 + TK);
#pragma unroll 16
        for (int l = 0; l < TK; l++) {
            float a[R], b[R];
#pragma unroll
            for (int u = 0; u < R; u++) { a[u] = As[buf][l][ty + 16 * u]; b[u] = Bs[buf][l][tx + 16 * u]; }
#pragma unroll
            for (int u = 0; u < R; u++)
#pragma unroll
                for (int v = 0; v < R; v++) acc[u][v] = fmaf(a[u], b[v], acc[u][v]);
            if (do_rowsum) {
#pragma unroll
                for (int u = 0; u < R; u++) rs[u] = __fadd_rn(rs[u], a[u]);
            }
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
    if (do_rowsum) {
#pragma unroll
        for (int u = 0; u < R; u++)
            if (i0 + ty + 16 * u < g.I) g.rowsum[i0 + ty + 16 * u] = rs[u];
    }
#pragma unroll
    for (int u = 0; u < R; u++) {
#pragma unroll
        for (int v = 0; v < R; v++) {
            int i = i0 + ty + 16 * u, j = j0 + tx + 16 * v;
            if (i >= g.I || j >= g.J) continue;
            float val = acc[u][v];
            if (g.splits > 1) {
                g.partial[((size_t)blockIdx.z * g.I + i) * g.J + j] = val;
                continue;
            }
            if (g.bias) val = __fadd_rn(val, g.bias_per_row ? g.bias[i] : g.bias[j]);
            size_t idx = g.out_mode == 0 ? (size_t)i * g.J + j
                                         : ((size_t)(j / g.inner) * g.I + i) * g.inner + (j % g.inner);
            if (g.relu) {
                float m = val > 0.f ? 1.f : 0.f;
                if (g.mask_out) g.mask_out[idx] = m;
                val = __fmul_rn(val, m);
            }
            if (g.mask_in) val = __fmul_rn(val, g.mask_in[idx]);
            g.c[idx] = val;
        }
    }
}

// A small output with a deep contraction (the MLP's first layer: 128 x 256 outputs, k = 784).  The
// one-output-per-thread kernel above walks 13 chunks in a row at ~0.85 us per chunk: every
// multiply-add of a warp costs two shared-memory wavefronts (its A values, its B values), and the
// chunks of a tile are strictly one after the other (load, barrier, multiply, barrier).  Here a
// block has four groups of 256 threads that take every fourth chunk of the same 16 x 16 tile (own
// shared-memory tiles, own named barrier), so one group's loads and barriers run under the
// others' multiplies; the four sums of an output are added in group order by group 0, which runs
// the epilogue.  Warm, first layer of the MLP: 15.7 -> 13.9 us, whole step 48.1 -> 45.4 us.
constexpr int kSliceGroups = 4;
__global__ void __launch_bounds__(256 * kSliceGroups) gemm_f32_ksplit_kernel(const GemmArgs g) {
    nvq_chain_sync();
    constexpr int T = 16, TK = 64, LD = T * TK / 256;
    __shared__ float As[kSliceGroups][TK][T + 1];
    __shared__ float Bs[kSliceGroups][TK][T + 1];
    const int grp = threadIdx.x >> 8, tid = threadIdx.x & 255;
    const int i0 = blockIdx.y * T, j0 = blockIdx.x * T;
    const int tx = tid & 15, ty = tid >> 4;
    const bool a_kc = g.a_sl == 1, b_kc = g.b_sl == 1;
    float acc = 0.f;
    float ra[LD], rb[LD];
    auto fetch = [&](int l0) {
#pragma unroll
        for (int r = 0; r < LD; r++) {
            int e = tid + 256 * r, ii, ll;
            tile_coord<T, TK>(e, a_kc, ii, ll);
            int i = i0 + ii, l = l0 + ll;
            ra[r] = (i < g.I && l < g.L) ? g.a[i * g.a_si + l * g.a_sl] : 0.f;
            int jj;
            tile_coord<T, TK>(e, b_kc, jj, ll);
            int j = j0 + jj;
            l = l0 + ll;
            rb[r] = (j < g.J && l < g.L) ? g.b[l * g.b_sl + j * g.b_sj] : 0.f;
        }
    };
    auto group_barrier = [&]() { asm volatile("bar.sync %0, 256;" ::"r"(grp + 1) : "memory"); };
    const int n_chunks = (g.L + TK - 1) / TK;
    if (grp < n_chunks) fetch(grp * TK);
    for (int c = grp; c < n_chunks; c += kSliceGroups) {
#pragma unroll
        for (int r = 0; r < LD; r++) {
            int e = tid + 256 * r, ii, ll;
            tile_coord<T, TK>(e, a_kc, ii, ll);
            As[grp][ll][ii] = ra[r];
            tile_coord<T, TK>(e, b_kc, ii, ll);
            Bs[grp][ll][ii] = rb[r];
        }
        group_barrier();
        if (c + kSliceGroups < n_chunks) fetch((c + kSliceGroups) * TK);    // in flight during the multiply
#pragma unroll 16
        for (int l = 0; l < TK; l++) acc = fmaf(As[grp][l][ty], Bs[grp][l][tx], acc);
        group_barrier();           // the group is done with its tiles before they are overwritten
    }
    // the four partial sums of every output, added in group order
    __syncthreads();
    float* red = &As[0][0][0];     // 4 x 64 x 17 floats: room for 3 x 256
    if (grp > 0) red[(grp - 1) * 256 + tid] = acc;
    __syncthreads();
    if (grp != 0) return;
    for (int s = 0; s < kSliceGroups - 1; s++) acc = __fadd_rn(acc, red[s * 256 + tid]);
    const int i = i0 + ty, j = j0 + tx;
    if (i >= g.I || j >= g.J) return;
    float val = acc;
    if (g.bias) val = __fadd_rn(val, g.bias_per_row ? g.bias[i] : g.bias[j]);
    const size_t idx = g.out_mode == 0 ? (size_t)i * g.J + j
                                       : ((size_t)(j / g.inner) * g.I + i) * g.inner + (j % g.inner);
    if (g.relu) {
        const float m = val > 0.f ? 1.f : 0.f;
        if (g.mask_out) g.mask_out[idx] = m;
        val = __fmul_rn(val, m);
    }
    if (g.mask_in) val = __fmul_rn(val, g.mask_in[idx]);
    g.c[idx] = val;
}

// Linear forward with both operands contiguous along k (X (M, K), W (N, K)) and an output too small
// to fill the GPU with shared-memory tiles: no shared memory at all.  A warp owns a 4 x 4 block of
// outputs; its lanes split k (lane t takes elements 4 t .. 4 t + 3 of every 128), so the four rows
// of X and the four rows of W are read as fully coalesced 128-bit loads (rows shared with the
// block's other warps come from L1), 64 multiply-adds per eight loads, and the 16 sums are
// combined over the lanes by a fixed butterfly at the end (the same bits on every run; another
// order than the tile kernels, within their 1e-5 of the reference's sgemm).
__global__ void __launch_bounds__(256) linear_fwd_klanes_kernel(const GemmArgs g) {
    nvq_chain_sync();
    const int lane = threadIdx.x & 31;
    const int wj_count = (g.J + 3) / 4;
    const int w = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int i0 = (w / wj_count) * 4, j0 = (w % wj_count) * 4;
    if (i0 >= g.I) return;
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) acc[u][v] = 0.f;
    const float* arow[4];
    const float* brow[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
        arow[u] = g.a + (long long)min(i0 + u, g.I - 1) * g.a_si;     // rows past the end repeat the last one
        brow[u] = g.b + (long long)min(j0 + u, g.J - 1) * g.b_sj;     // (their results are not stored)
    }
    for (int l = 4 * lane; l < g.L; l += 128) {
        float4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            a[u] = *reinterpret_cast<const float4*>(arow[u] + l);
            b[u] = *reinterpret_cast<const float4*>(brow[u] + l);
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int v = 0; v < 4; v++) {
                acc[u][v] = fmaf(a[u].x, b[v].x, acc[u][v]);
                acc[u][v] = fmaf(a[u].y, b[v].y, acc[u][v]);
                acc[u][v] = fmaf(a[u].z, b[v].z, acc[u][v]);
                acc[u][v] = fmaf(a[u].w, b[v].w, acc[u][v]);
            }
    }
    // all lanes end up with the 16 sums; lane 4 u + v stores output (i0 + u, j0 + v)
    float mine = 0.f;
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) {
            float x = acc[u][v];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) x = __fadd_rn(x, __shfl_xor_sync(0xFFFFFFFFu, x, o));
            if (lane == 4 * u + v) mine = x;
        }
    if (lane >= 16) return;
    const int i = i0 + (lane >> 2), j = j0 + (lane & 3);
    if (i >= g.I || j >= g.J) return;
    float val = mine;
    if (g.bias) val = __fadd_rn(val, g.bias_per_row ? g.bias[i] : g.bias[j]);
    const size_t idx = (size_t)i * g.J + j;
    if (g.relu) {
        const float m = val > 0.f ? 1.f : 0.f;
        if (g.mask_out) g.mask_out[idx] = m;
        val = __fmul_rn(val, m);
    }
    if (g.mask_in) val = __fmul_rn(val, g.mask_in[idx]);
    g.c[idx] = val;
}

// Register-tiled form for large outputs: a 16 x 16 thread grid, each thread RI x RJ outputs
// (RJ consecutive columns, read from shared memory as float4), 16-deep chunks, double
// buffered.  Per k step a thread issues RI + RJ/4 shared loads for RI * RJ multiply-adds,
// against 4 loads for 4 multiply-adds in the 32 x 32 kernel above.  The additions of one output
// run in the same k order as there, so both kernels return the same bits.
#ifndef NVQ_GEMM_BIG_TK
#define NVQ_GEMM_BIG_TK 16
#endif
template <int RI, int RJ>
__global__ void __launch_bounds__(256) gemm_f32_big_kernel(const GemmArgs g) {
    nvq_chain_sync();
    constexpr int TI = 16 * RI, TJ = 16 * RJ, TKB = NVQ_GEMM_BIG_TK;
    constexpr int LDA = TI * TKB / 256, LDB = TJ * TKB / 256;
    __shared__ __align__(16) float As[2][TKB][TI + 4];
    __shared__ __align__(16) float Bs[2][TKB][TJ + 4];
    const int i0 = blockIdx.y * TI, j0 = blockIdx.x * TJ;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const bool a_kc = g.a_sl == 1, b_kc = g.b_sl == 1;
    float acc[RI][RJ];
    float rs[RI];
#pragma unroll
    for (int u = 0; u < RI; u++) {
        rs[u] = 0.f;
#pragma unroll
        for (int v = 0; v < RJ; v++) acc[u][v] = 0.f;
    }
    const bool do_rowsum = g.rowsum != nullptr && blockIdx.x == 0 && tx == 0;
    float ra[LDA], rb[LDB];
    const int l_lo = g.splits > 1 ? blockIdx.z * g.l_per_split : 0;
    const int l_hi = g.splits > 1 ? min(g.L, l_lo + g.l_per_split) : g.L;
    // Each thread stages the same tile positions in every chunk: their addresses at l_lo, their
    // k offsets and their row / column validity are worked out once; a chunk then costs one
    // compare, one load and one pointer bump per element.
    const float* pa[LDA];
    const float* pb[LDB];
    int ka[LDA], kb[LDB];          // k offset inside a chunk, or a huge value for rows outside
#pragma unroll
    for (int r = 0; r < LDA; r++) {
        int ii, ll;
        tile_coord<TI, TKB>(threadIdx.x + 256 * r, a_kc, ii, ll);
        const int i = i0 + ii;
        ka[r] = i < g.I ? ll : (1 << 30);
        pa[r] = g.a + (long long)min(i, g.I - 1) * g.a_si + (long long)(l_lo + ll) * g.a_sl;
    }
#pragma unroll
    for (int r = 0; r < LDB; r++) {
        int jj, ll;
        tile_coord<TJ, TKB>(threadIdx.x + 256 * r, b_kc, jj, ll);
        const int j = j0 + jj;
        kb[r] = j < g.J ? ll : (1 << 30);
        pb[r] = g.b + (long long)(l_lo + ll) * g.b_sl + (long long)min(j, g.J - 1) * g.b_sj;
    }
    const long long a_step = (long long)TKB * g.a_sl, b_step = (long long)TKB * g.b_sl;
    auto fetch = [&](int l0) {
        const int room = l_hi - l0;           // elements with k offset < room exist
#pragma unroll
        for (int r = 0; r < LDA; r++) {
            ra[r] = ka[r] < room ? *pa[r] : 0.f;
            pa[r] += a_step;
        }
#pragma unroll
        for (int r = 0; r < LDB; r++) {
            rb[r] = kb[r] < room ? *pb[r] : 0.f;
            pb[r] += b_step;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int r = 0; r < LDA; r++) {
            int ii, ll;
            tile_coord<TI, TKB>(threadIdx.x + 256 * r, a_kc, ii, ll);
            As[buf][ll][ii] = ra[r];
        }
#pragma unroll
        for (int r = 0; r < LDB; r++) {
            int jj, ll;
            tile_coord<TJ, TKB>(threadIdx.x + 256 * r, b_kc, jj, ll);
            Bs[buf][ll][jj] = rb[r];
        }
    };
    fetch(l_lo);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int l0 = l_lo; l0 < l_hi; l0 += TKB) {
        const bool more = l0 + TKB < l_hi;
        if (more) fetch(l0 + TKB);
#pragma unroll
        for (int l = 0; l < TKB; l++) {
            float a[RI], b[RJ];
#pragma unroll
            for (int u = 0; u < RI; u++) a[u] = As[buf][l][ty * RI + u];
#pragma unroll
            for (int v = 0; v < RJ; v += 4) {
                const float4 t = *reinterpret_cast<const float4*>(&Bs[buf][l][tx * RJ + v]);
                b[v] = t.x; b[v + 1] = t.y; b[v + 2] = t.z; b[v + 3] = t.w;
            }
#pragma unroll
            for (int u = 0; u < RI; u++)
#pragma unroll
                for (int v = 0; v < RJ; v++) acc[u][v] = fmaf(a[u], b[v], acc[u][v]);
            if (do_rowsum) {
#pragma unroll
                for (int u = 0; u < RI; u++) rs[u] = __fadd_rn(rs[u], a[u]);
            }
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
    if (do_rowsum) {
#pragma unroll
        for (int u = 0; u < RI; u++)
            if (i0 + ty * RI + u < g.I) g.rowsum[i0 + ty * RI + u] = rs[u];
    }
#pragma unroll
    for (int u = 0; u < RI; u++) {
#pragma unroll
        for (int v = 0; v < RJ; v++) {
            const int i = i0 + ty * RI + u, j = j0 + tx * RJ + v;
            if (i >= g.I || j >= g.J) continue;
            float val = acc[u][v];
            if (g.splits > 1) {
                g.partial[((size_t)blockIdx.z * g.I + i) * g.J + j] = val;
                continue;
            }
            if (g.bias) val = __fadd_rn(val, g.bias_per_row ? g.bias[i] : g.bias[j]);
            size_t idx = g.out_mode == 0 ? (size_t)i * g.J + j
                                         : ((size_t)(j / g.inner) * g.I + i) * g.inner + (j % g.inner);
            if (g.relu) {
                float m = val > 0.f ? 1.f : 0.f;
                if (g.mask_out) g.mask_out[idx] = m;
                val = __fmul_rn(val, m);
            }
            if (g.mask_in) val = __fmul_rn(val, g.mask_in[idx]);
            g.c[idx] = val;
        }
    }
}

// c[e] = sum over z of partial[z][e]: one warp per output, lane t adds z = t, t+32, ... in
// order and the 32 lane sums are combined by a fixed butterfly (same result on every run)
__global__ void splitk_reduce_kernel(float* __restrict__ c, const float* __restrict__ partial,
                                     int n, int splits) {
    nvq_chain_sync();
    const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (e >= n) return;
    float s = 0.f;
    for (int z = lane; z < splits; z += 32) s = __fadd_rn(s, partial[(size_t)z * n + e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xFFFFFFFFu, s, o));
    if (lane == 0) c[e] = s;
}

// A small output with a very deep contraction (the convolution weight gradient: Cout x CKK
// outputs, k = every output position of the batch) is split along k over enough blocks to fill
// the GPU; `scratch` must hold scratch_elems floats.
nvq_status launch_gemm_splitk(GemmArgs g, float* scratch, size_t scratch_elems, int device,
                              cudaStream_t st) {
    if (g.I <= 0 || g.J <= 0) return NVQ_OK;
    // tile shape by the number of rows, as in launch_gemm; 16 x 16 tiles for tiny outputs
    int ti, tj, kind;
    if (g.I > 32)                  { ti = 64; tj = 64; kind = 44; }
    else if (g.I > 16)             { ti = 32; tj = 128; kind = 28; }
    else if (g.J >= 64)            { ti = 16; tj = 128; kind = 18; }
    else                           { ti = 16; tj = 16; kind = 0; }
    const dim3 tiles2((g.J + tj - 1) / tj, (g.I + ti - 1) / ti);
    auto launch = [&](unsigned z) {
        const dim3 grid(tiles2.x, tiles2.y, z);
        if (kind == 44) nvq_launch_chained(gemm_f32_big_kernel<4, 4>, grid, 256, 0, st, g);
        else if (kind == 28) nvq_launch_chained(gemm_f32_big_kernel<2, 8>, grid, 256, 0, st, g);
        else if (kind == 18) nvq_launch_chained(gemm_f32_big_kernel<1, 8>, grid, 256, 0, st, g);
        else nvq_launch_chained(gemm_f32_kernel<16>, grid, 256, 0, st, g);
    };
    const long long tiles = (long long)tiles2.x * tiles2.y;
    const long long out = (long long)g.I * g.J;
    long long want = (4LL * nvq_sm_count(device) + tiles - 1) / tiles;
    want = std::min<long long>(want, g.L / 64);
    if (scratch) want = std::min<long long>(want, (long long)(scratch_elems / (size_t)out));
    if (!scratch || want < 2 || g.bias || g.relu || g.mask_in || g.out_mode != 0) {
        g.splits = 1;
        launch(1);
        NVQ_LAUNCHED();
        return NVQ_OK;
    }
    int lps = (int)((g.L + want - 1) / want);
    lps = (lps + kSplitChunk - 1) / kSplitChunk * kSplitChunk;
    g.l_per_split = lps;
    g.splits = (g.L + lps - 1) / lps;
    g.partial = scratch;
    launch((unsigned)g.splits);
    NVQ_LAUNCHED();
    nvq_launch_chained(splitk_reduce_kernel, dim3((unsigned)((out + 7) / 8)), 256, 0, st, g.c, (const float*)scratch, (int)out, g.splits);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status launch_gemm(const GemmArgs& g, cudaStream_t st) {
    if (g.I <= 0 || g.J <= 0) return NVQ_OK;
    // large outputs with a contraction worth tiling in registers: 64 x 64, 32 x 128 or 16 x 128
    // tiles by the number of rows, as long as there are blocks for about half of the SMs
    if (g.L > 16) {
        const long long b44 = (long long)((g.J + 63) / 64) * ((g.I + 63) / 64);
        const long long b28 = (long long)((g.J + 127) / 128) * ((g.I + 31) / 32);
        const long long b18 = (long long)((g.J + 127) / 128) * ((g.I + 15) / 16);
        if (g.I > 32 && b44 >= 64) {
            nvq_launch_chained(gemm_f32_big_kernel<4, 4>, dim3((g.J + 63) / 64, (g.I + 63) / 64), 256, 0, st, g);
            NVQ_LAUNCHED();
            return NVQ_OK;
        }
        if (g.I > 16 && g.I <= 32 && b28 >= 64) {
            nvq_launch_chained(gemm_f32_big_kernel<2, 8>, dim3((g.J + 127) / 128, (g.I + 31) / 32), 256, 0, st, g);
            NVQ_LAUNCHED();
            return NVQ_OK;
        }
        if (g.I <= 16 && b18 >= 64) {
            nvq_launch_chained(gemm_f32_big_kernel<1, 8>, dim3((g.J + 127) / 128, (g.I + 15) / 16), 256, 0, st, g);
            NVQ_LAUNCHED();
            return NVQ_OK;
        }
    }
    const long long big_blocks = (long long)((g.J + 31) / 32) * ((g.I + 31) / 32);
    if (big_blocks >= 148 && g.L <= 16) {
        // shallow contraction: 16-deep chunks; 16-row tiles when the output has few rows
        if (g.I <= 16) {
            dim3 grid((g.J + 15) / 16, (g.I + 15) / 16);
            nvq_launch_chained(gemm_f32_kernel<16, 16>, grid, 256, 0, st, g);
        } else {
            dim3 grid((g.J + 31) / 32, (g.I + 31) / 32);
            nvq_launch_chained(gemm_f32_kernel<32, 16>, grid, 256, 0, st, g);
        }
    } else if (big_blocks >= 148) {
        dim3 grid((g.J + 31) / 32, (g.I + 31) / 32);
        nvq_launch_chained(gemm_f32_kernel<32>, grid, 256, 0, st, g);
    } else {
        dim3 grid((g.J + 15) / 16, (g.I + 15) / 16);
        const bool k_rows = g.a_sl == 1 && g.b_sl == 1 && g.L % 4 == 0 && g.a_si % 4 == 0 && g.b_sj % 4 == 0 &&
                            nvq_aligned(g.a, 16) && nvq_aligned(g.b, 16) && g.out_mode == 0 && !g.rowsum &&
                            g.splits <= 1;
        if (k_rows && g.L >= 128) {
            const long long warps = (long long)((g.I + 3) / 4) * ((g.J + 3) / 4);
            nvq_launch_chained(linear_fwd_klanes_kernel, dim3((unsigned)((warps + 7) / 8)), 256, 0, st, g);
        } else if (g.L >= 256 && !g.rowsum && g.splits <= 1)
            nvq_launch_chained(gemm_f32_ksplit_kernel, grid, 256 * kSliceGroups, 0, st, g);
        else
            nvq_launch_chained(gemm_f32_kernel<16>, grid, 256, 0, st, g);
    }
    NVQ_LAUNCHED();
    return NVQ_OK;
}

// column sums of an M x N matrix: out[n] = sum_m g[m, n].  A block covers 32 columns with 8
// row groups; each thread adds its rows in order, the 8 partial sums are combined in order.
__global__ void __launch_bounds__(256)
colsum_kernel(const float* __restrict__ g, float* __restrict__ out, int M, int N) {
    nvq_chain_sync();
    __shared__ float part[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (n < N)
        for (int m = ty; m < M; m += 8) s = __fadd_rn(s, g[(size_t)m * N + n]);
    part[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && n < N) {
        float t = part[0][tx];
#pragma unroll
        for (int r = 1; r < 8; r++) t = __fadd_rn(t, part[r][tx]);
        out[n] = t;
    }
}

__global__ void relu_kernel(float* __restrict__ out, float* __restrict__ mask,
                            const float* __restrict__ x, size_t n) {
    nvq_chain_sync();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = x[i];
        float m = v > 0.f ? 1.f : 0.f;
        if (mask) mask[i] = m;
        out[i] = __fmul_rn(v, m);
    }
}

__global__ void mul_kernel(float* __restrict__ out, const float* __restrict__ a,
                           const float* __restrict__ b, size_t n) {
    nvq_chain_sync();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = __fmul_rn(a[i], b[i]);
}

// One block; thread per row for the softmax, then a block reduction for the loss.
//   y_hat = softmax(logits, axis 1) in fp32; grad = float((double(y_hat) - onehot) / M)
//   loss  = -sum(onehot * log(p2 + 1e-8)) / M with p2 = softmax(y_hat, axis 0): the value the
//   reference reports (it applies softmax a second time, along the batch axis).
__device__ void ce_loss_from_yhat(float* __restrict__ loss, const float* __restrict__ yhat_scratch,
                                  const int* __restrict__ labels, int M, int C, double* red);

__global__ void softmax_ce_kernel(float* __restrict__ grad, float* __restrict__ loss,
                                  const float* __restrict__ logits, const int* __restrict__ labels,
                                  float* __restrict__ yhat_scratch, int M, int C) {
    nvq_chain_sync();
    extern __shared__ double red[];
    for (int m = threadIdx.x; m < M; m += blockDim.x) {
        const float* z = logits + (size_t)m * C;
        float mx = z[0];
        for (int c = 1; c < C; c++) mx = fmaxf(mx, z[c]);
        float s = 0.f;
        for (int c = 0; c < C; c++) s = __fadd_rn(s, expf(__fsub_rn(z[c], mx)));
        int lab = labels[m];
        for (int c = 0; c < C; c++) {
            float y = __fdiv_rn(expf(__fsub_rn(z[c], mx)), s);
            yhat_scratch[(size_t)m * C + c] = y;
            double d = ((double)y - (c == lab ? 1.0 : 0.0)) / (double)M;
            grad[(size_t)m * C + c] = (float)d;
        }
    }
    __syncthreads();
    if (!loss) return;
    ce_loss_from_yhat(loss, yhat_scratch, labels, M, C, red);
}

// loss = -sum(onehot * log(p2 + 1e-8)) / M with p2 = softmax(y_hat, axis 0), from the y_hat the
// kernel above left in yhat_scratch.  Nothing in the step depends on the value, so a training
// step runs this beside its backward pass instead of in front of it.
__global__ void ce_loss_kernel(float* __restrict__ loss, const float* __restrict__ yhat,
                               const int* __restrict__ labels, int M, int C) {
    nvq_chain_sync();
    extern __shared__ double red[];
    ce_loss_from_yhat(loss, yhat, labels, M, C, red);
}

__device__ void ce_loss_from_yhat(float* __restrict__ loss, const float* __restrict__ yhat_scratch,
                                  const int* __restrict__ labels, int M, int C, double* red) {
    // second softmax along the batch axis: one warp per class column, lanes stride over the
    // rows; only the labelled entries enter the loss
    double part = 0.0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int c = warp; c < C; c += nwarps) {
        float mx = -INFINITY;
        for (int m = lane; m < M; m += 32) mx = fmaxf(mx, yhat_scratch[(size_t)m * C + c]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        float s = 0.f;
        for (int m = lane; m < M; m += 32) s += expf(__fsub_rn(yhat_scratch[(size_t)m * C + c], mx));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        for (int m = lane; m < M; m += 32) {
            if (labels[m] == c) {
                float p2 = __fdiv_rn(expf(__fsub_rn(yhat_scratch[(size_t)m * C + c], mx)), s);
                part += (double)logf(__fadd_rn(p2, 1e-8f));
            }
        }
    }
    // fixed butterfly inside each warp, then the warp sums in order: the same value on every run
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
    if (lane == 0) red[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int i = 0; i < nwarps; i++) tot += red[i];
        *loss = (float)(-tot / (double)M);
    }
}

__global__ void sgd_kernel(float* __restrict__ p, const float* __restrict__ g, size_t n, float lr,
                           float grad_scale) {
    nvq_chain_sync();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float gr = g[i];
        if (grad_scale != 1.f) gr = __fmul_rn(gr, grad_scale);
        p[i] = __fsub_rn(p[i], __fmul_rn(lr, gr));   // two roundings, as p -= lr * g in NumPy
    }
}

// AdamW.step (novann/optim/adamw.py:41-65), every product, sum, quotient and root rounded
// separately in fp32 exactly where NumPy rounds them.
struct AdamWArgs { float b1, c1, b2, c2, bc1, bc2, lr, eps, lr_wd; int decay; };
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, size_t n, AdamWArgs a) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float gi = g[i];
        float mi = __fadd_rn(__fmul_rn(a.b1, m[i]), __fmul_rn(a.c1, gi));
        float vi = __fadd_rn(__fmul_rn(a.b2, v[i]), __fmul_rn(a.c2, __fmul_rn(gi, gi)));
        m[i] = mi;
        v[i] = vi;
        float mh = __fdiv_rn(mi, a.bc1), vh = __fdiv_rn(vi, a.bc2);
        float upd = __fdiv_rn(__fmul_rn(a.lr, mh), __fadd_rn(__fsqrt_rn(vh), a.eps));
        float pi = __fsub_rn(p[i], upd);
        if (a.decay) pi = __fsub_rn(pi, __fmul_rn(a.lr_wd, pi));
        p[i] = pi;
    }
}

// ---- im2col ---------------------------------------------------------------------------
__device__ __forceinline__ int pad_index(int idx, int size, int mode, bool& zero) {
    zero = false;
    if (idx >= 0 && idx < size) return idx;
    if (mode == NVQ_PAD_ZEROS) { zero = true; return 0; }
    if (mode == NVQ_PAD_REPLICATE) return idx < 0 ? 0 : size - 1;
    if (mode == NVQ_PAD_CIRCULAR) { int r = idx % size; return r < 0 ? r + size : r; }
    // reflect without repeating the edge; a length-1 axis repeats its only value
    if (size == 1) return 0;
    int period = 2 * (size - 1);
    int r = idx % period;
    if (r < 0) r += period;
    return r < size ? r : period - r;
}

struct ConvGeom { int N, C, H, W, KH, KW, sh, sw, ph, pw, OH, OW, mode; };

// fp32 col, rows (c,kh,kw), columns (n,oh,ow): the reference's layout
// Idx = uint32_t whenever every element count fits 31 bits (64-bit divisions are several times
// dearer and these kernels are bound by their index arithmetic), size_t otherwise.
template <class Idx>
__global__ void im2col_f32_kernel(float* __restrict__ col, const float* __restrict__ x, ConvGeom g) {
    const Idx L = (Idx)g.N * g.OH * g.OW, total = (Idx)g.C * g.KH * g.KW * L;
    Idx stride = (Idx)gridDim.x * blockDim.x;
    for (Idx e = (Idx)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        Idx row = e / L, colj = e - row * L;
        int kw = row % g.KW, kh = (row / g.KW) % g.KH, c = row / (g.KW * g.KH);
        int ow = colj % g.OW, oh = (colj / g.OW) % g.OH, n = colj / ((Idx)g.OW * g.OH);
        bool z1, z2;
        int ih = pad_index(oh * g.sh + kh - g.ph, g.H, g.mode, z1);
        int iw = pad_index(ow * g.sw + kw - g.pw, g.W, g.mode, z2);
        col[e] = (z1 || z2) ? 0.f : x[(((Idx)n * g.C + c) * g.H + ih) * g.W + iw];
    }
}

// bf16 patches for the tensor-core path: rows (n,oh,ow), columns (c,kh,kw) padded with zeros
// to Kpad; values rounded to nearest even
__global__ void im2col_bf16_rows_kernel(uint16_t* __restrict__ col, const float* __restrict__ x,
                                        ConvGeom g, int Kpad) {
    const size_t L = (size_t)g.N * g.OH * g.OW, total = L * Kpad;
    const int CKK = g.C * g.KH * g.KW;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t rowj = e / Kpad;
        int kk = e % Kpad;
        float v = 0.f;
        if (kk < CKK) {
            int kw = kk % g.KW, kh = (kk / g.KW) % g.KH, c = kk / (g.KW * g.KH);
            int ow = rowj % g.OW, oh = (rowj / g.OW) % g.OH, n = rowj / ((size_t)g.OW * g.OH);
            bool z1, z2;
            int ih = pad_index(oh * g.sh + kh - g.ph, g.H, g.mode, z1);
            int iw = pad_index(ow * g.sw + kw - g.pw, g.W, g.mode, z2);
            if (!(z1 || z2)) v = x[(((size_t)n * g.C + c) * g.H + ih) * g.W + iw];
        }
        col[e] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v));
    }
}

// Y (L x Cout, bf16, rows (n,oh,ow)) -> out (N, Cout, OH, OW) fp32
__global__ void rows_bf16_to_nchw_kernel(float* __restrict__ out, const uint16_t* __restrict__ y,
                                         int N, int Cout, int S) {
    size_t total = (size_t)N * Cout * S, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        int s = e % S, c = (e / S) % Cout, n = e / ((size_t)S * Cout);
        out[e] = __uint_as_float((uint32_t)y[((size_t)n * S + s) * Cout + c] << 16);
    }
}

// Tiled forms of the two kernels above, used whenever the geometry fits their tables.
// Patches: a block takes 32 consecutive rows (n,oh,ow) and walks the columns (c,kh,kw) in
// chunks of 64.  Reads: one warp per column, lanes = rows, so a warp reads 32 consecutive
// pixels of one input plane; writes: 128 contiguous bytes per row through shared memory.
constexpr int kImRows = 32, kImK = 64, kImLut = 4096;

__global__ void __launch_bounds__(256)
im2col_bf16_tiled_kernel(uint16_t* __restrict__ col, const float* __restrict__ x, ConvGeom g,
                         int Kpad, int L) {
    __shared__ uint16_t tile[kImRows][kImK + 2];     // 33-word rows: conflict-free column writes
    __shared__ uint32_t lut[kImLut];                 // column -> c << 16 | kh << 8 | kw
    const int CKK = g.C * g.KH * g.KW;
    for (int kk = threadIdx.x; kk < CKK; kk += 256) {
        int kw = kk % g.KW, kh = (kk / g.KW) % g.KH, c = kk / (g.KW * g.KH);
        lut[kk] = ((uint32_t)c << 16) | ((uint32_t)kh << 8) | (uint32_t)kw;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wr = threadIdx.x >> 3, wseg = threadIdx.x & 7;      // write role: row, 8-column group
    for (int row0 = blockIdx.x * kImRows; row0 < L; row0 += gridDim.x * kImRows) {
        const int row = row0 + lane;
        const bool valid = row < L;
        int ow = row % g.OW, oh = (row / g.OW) % g.OH, n = row / (g.OW * g.OH);
        const int base_h = oh * g.sh - g.ph, base_w = ow * g.sw - g.pw;
        const float* xn = x + (size_t)n * g.C * g.H * g.W;
        for (int k0 = 0; k0 < Kpad; k0 += kImK) {
#pragma unroll
            for (int i = 0; i < kImK / 8; i++) {
                const int kc = warp + 8 * i, kk = k0 + kc;
                float v = 0.f;
                if (valid && kk < CKK) {
                    const uint32_t e = lut[kk];
                    bool z1, z2;
                    int ih = pad_index(base_h + (int)((e >> 8) & 0xFFu), g.H, g.mode, z1);
                    int iw = pad_index(base_w + (int)(e & 0xFFu), g.W, g.mode, z2);
                    if (!(z1 || z2)) v = xn[((size_t)(e >> 16) * g.H + ih) * g.W + iw];
                }
                tile[lane][kc] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v));
            }
            __syncthreads();
            const int kk = k0 + wseg * 8;
            if (row0 + wr < L && kk < Kpad) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(&tile[wr][wseg * 8]);
                uint4 o = make_uint4(src[0], src[1], src[2], src[3]);
                *reinterpret_cast<uint4*>(col + (size_t)(row0 + wr) * Kpad + kk) = o;
            }
            __syncthreads();
        }
    }
}

// Y (N*S x Cout, bf16) -> out (N, Cout, S) fp32 through a 32 x 64 shared tile: 128-byte reads
// along Cout, 128-byte writes along S.
__global__ void __launch_bounds__(256)
rows_bf16_to_nchw_tiled_kernel(float* __restrict__ out, const uint16_t* __restrict__ y, int N,
                               int Cout, int S) {
    __shared__ float tile[64][33];
    const int s_tiles = (S + 31) / 32, c_tiles = (Cout + 63) / 64;
    const long long total = (long long)N * s_tiles * c_tiles;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rr = threadIdx.x >> 3, seg = threadIdx.x & 7;
    for (long long t = blockIdx.x; t < total; t += gridDim.x) {
        const int ct = (int)(t % c_tiles), stl = (int)((t / c_tiles) % s_tiles), n = (int)(t / ((long long)c_tiles * s_tiles));
        const int s0 = stl * 32, c0 = ct * 64;
        if (s0 + rr < S && c0 + seg * 8 < Cout) {
            const uint4 v = *reinterpret_cast<const uint4*>(y + ((size_t)n * S + s0 + rr) * Cout + c0 + seg * 8);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                tile[seg * 8 + 2 * q][rr] = __uint_as_float(w[q] << 16);
                tile[seg * 8 + 2 * q + 1][rr] = __uint_as_float(w[q] & 0xFFFF0000u);
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int c = c0 + warp + 8 * i;
            if (c < Cout && s0 + lane < S)
                out[((size_t)n * Cout + c) * S + s0 + lane] = tile[warp + 8 * i][lane];
        }
        __syncthreads();
    }
}

// ---- pre-passes of the implicit-GEMM convolution ---------------------------------------
// x (N, C, S) fp32 -> (N, S, C) bf16 (round to nearest even): 32 pixels x 64 channels per tile,
// 128-byte reads along S, 128-byte writes along C.
__global__ void __launch_bounds__(256)
nchw_f32_to_nhwc_bf16_kernel(uint16_t* __restrict__ out, const float* __restrict__ x, int N, int C,
                             int S) {
    __shared__ uint16_t tile[32][64 + 2];
    const int s_tiles = (S + 31) / 32, c_tiles = C / 64;
    const long long total = (long long)N * s_tiles * c_tiles;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wr = threadIdx.x >> 3, wseg = threadIdx.x & 7;
    for (long long t = blockIdx.x; t < total; t += gridDim.x) {
        const int ct = (int)(t % c_tiles), stl = (int)((t / c_tiles) % s_tiles);
        const int n = (int)(t / ((long long)c_tiles * s_tiles));
        const int s0 = stl * 32, c0 = ct * 64;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int c = warp + 8 * i;
            float v = s0 + lane < S ? x[((size_t)n * C + c0 + c) * S + s0 + lane] : 0.f;
            tile[lane][c] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v));
        }
        __syncthreads();
        if (s0 + wr < S) {
            const uint32_t* src = reinterpret_cast<const uint32_t*>(&tile[wr][wseg * 8]);
            *reinterpret_cast<uint4*>(out + ((size_t)n * S + s0 + wr) * C + c0 + wseg * 8) =
                make_uint4(src[0], src[1], src[2], src[3]);
        }
        __syncthreads();
    }
}

// Same for S % 4 == 0: 64 pixels x 64 channels per tile, four 16-byte loads in flight per thread
// (one channel, four consecutive pixels each), two 16-byte stores (one pixel, eight channels each).
__global__ void __launch_bounds__(256)
nchw_f32_to_nhwc_bf16_v4_kernel(uint16_t* __restrict__ out, const float* __restrict__ x, int N, int C,
                                int S) {
    __shared__ uint16_t tile[64][64 + 2];
    const int s_tiles = (S + 63) / 64, c_tiles = C / 64;
    const long long total = (long long)N * s_tiles * c_tiles;
    const int lc = threadIdx.x >> 4, lp = threadIdx.x & 15;       // load role: channel row, pixel quad
    const int wr = threadIdx.x >> 3, wseg = threadIdx.x & 7;      // store role: pixel, 8-channel group
    for (long long t = blockIdx.x; t < total; t += gridDim.x) {
        const int ct = (int)(t % c_tiles), stl = (int)((t / c_tiles) % s_tiles);
        const int n = (int)(t / ((long long)c_tiles * s_tiles));
        const int s0 = stl * 64, c0 = ct * 64;
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = lc + 16 * i, s = s0 + 4 * lp;
            v[i] = s < S ? *reinterpret_cast<const float4*>(x + ((size_t)n * C + c0 + c) * S + s)
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = lc + 16 * i;
            tile[4 * lp + 0][c] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v[i].x));
            tile[4 * lp + 1][c] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v[i].y));
            tile[4 * lp + 2][c] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v[i].z));
            tile[4 * lp + 3][c] = (uint16_t)spec_f32_to_bf16(__float_as_uint(v[i].w));
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int px = wr + 32 * i;
            if (s0 + px < S) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(&tile[px][wseg * 8]);
                *reinterpret_cast<uint4*>(out + ((size_t)n * S + s0 + px) * C + c0 + wseg * 8) =
                    make_uint4(src[0], src[1], src[2], src[3]);
            }
        }
        __syncthreads();
    }
}

// FP8 weight codes (Cout x Kpad, columns (c, kh, kw)) -> bf16 (Cout x KH*KW*C, columns
// (kh, kw, c)), exact
template <int FMT>
__global__ void expand_permute_weight_kernel(uint16_t* __restrict__ out, const uint8_t* __restrict__ wq,
                                             int Cout, int C, int KH, int KW, int Kpad) {
    const int K = C * KH * KW, total = Cout * K;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int co = e / K, k = e - co * K;
        const int c = k % C, tap = k / C, kh = tap / KW, kw = tap - kh * KW;
        const uint32_t code = wq[(size_t)co * Kpad + (c * KH + kh) * KW + kw];
        out[e] = (uint16_t)(spec_fp8_to_f32<FMT>(code) >> 16);   // the low 16 bits are zero
    }
}

// FP4 E2M1 block-32 weight (Cout x Kpad/2 packed bytes, Kpad/32 fp32 scales per row, columns
// (c, kh, kw)) -> bf16(value * scale) (Cout x KH*KW*C, columns (kh, kw, c)): the block scale
// varies along k, so it is folded into the expanded weight (same rule as the FP4 dequantiser)
__global__ void expand_permute_weight_fp4_kernel(uint16_t* __restrict__ out, const uint8_t* __restrict__ wq,
                                                 const float* __restrict__ scales, int Cout, int C,
                                                 int KH, int KW, int Kpad) {
    const int K = C * KH * KW, total = Cout * K;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int co = e / K, k = e - co * K;
        const int c = k % C, tap = k / C, kh = tap / KW, kw = tap - kh * KW;
        const int ko = (c * KH + kh) * KW + kw;
        const uint32_t code = (wq[(size_t)co * (Kpad / 2) + (ko >> 1)] >> (4 * (ko & 1))) & 0xFu;
        const uint32_t m = code & 7u;   // {0, .5, 1, 1.5, 2, 3, 4, 6} as fp32 patterns
        const uint32_t vb = (m == 0 ? 0u : m == 1 ? 0x3F000000u : (((m >> 1) + 126u) << 23) | ((m & 1u) << 22)) |
                            ((code & 8u) << 28);
        const uint32_t su = __float_as_uint(scales[(size_t)co * (Kpad / 32) + (ko >> 5)]);
        out[e] = (uint16_t)spec_f32_to_bf16(spec_mul_bits(vb, su));
    }
}

// grad (N, Cout, S) -> g_r (Cout, N*S): the reference's grad.transpose(1,0,2,3).reshape(Cout,-1)
template <class Idx>
__global__ void nchw_to_crows_kernel(float* __restrict__ out, const float* __restrict__ g, int N,
                                     int Cout, int S) {
    Idx total = (Idx)N * Cout * S, stride = (Idx)gridDim.x * blockDim.x;
    for (Idx e = (Idx)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        int s = e % S, n = (e / S) % N, c = e / ((Idx)S * N);
        out[e] = g[((size_t)n * Cout + c) * S + s];
    }
}

// row sums: out[r] = sum_l a[r, l]; one warp per row
__global__ void rowsum_kernel(const float* __restrict__ a, float* __restrict__ out, int R, size_t L) {
    int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= R) return;
    float s = 0.f;
    for (size_t l = lane; l < L; l += 32) s += a[(size_t)r * L + l];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    if (lane == 0) out[r] = s;
}

// col2im as a gather (Conv2d._col2im, novann/layers/convolutional/conv2d.py:117-148): every input
// element sums the dcol entries of the windows that cover it, in (kh, kw) order, which is the
// order np.add.at applies them in.  As in the reference, gradient that falls on padding is dropped
// whatever the padding mode.
// ST = the stride when it is 1 or 2 in both directions (divisions fold away), 0 = read it from g.
template <class Idx, int ST>
__global__ void col2im_kernel(float* __restrict__ dx, const float* __restrict__ dcol, ConvGeom g) {
    const int sh = ST ? ST : g.sh, sw = ST ? ST : g.sw;
    const Idx L = (Idx)g.N * g.OH * g.OW, total = (Idx)g.N * g.C * g.H * g.W;
    Idx stride = (Idx)gridDim.x * blockDim.x;
    for (Idx e = (Idx)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        int w = e % g.W, h = (e / g.W) % g.H, c = (e / ((Idx)g.W * g.H)) % g.C;
        int n = e / ((Idx)g.W * g.H * g.C);
        float s = 0.f;
        for (int kh = 0; kh < g.KH; kh++) {
            int t = h + g.ph - kh;
            if (t < 0 || t % sh) continue;
            int oh = t / sh;
            if (oh >= g.OH) continue;
            for (int kw = 0; kw < g.KW; kw++) {
                int u = w + g.pw - kw;
                if (u < 0 || u % sw) continue;
                int ow = u / sw;
                if (ow >= g.OW) continue;
                Idx row = ((Idx)c * g.KH + kh) * g.KW + kw;
                s = __fadd_rn(s, dcol[row * L + ((Idx)n * g.OH + oh) * g.OW + ow]);
            }
        }
        dx[e] = s;
    }
}

nvq_status geom(ConvGeom& g, int N, int C, int H, int W, int KH, int KW, int sh, int sw, int ph,
                int pw, nvq_pad_mode mode) {
    NVQ_REQUIRE(N > 0 && C > 0 && H > 0 && W > 0 && KH > 0 && KW > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0,
                "conv2d: bad geometry");
    NVQ_REQUIRE(mode >= NVQ_PAD_ZEROS && mode <= NVQ_PAD_CIRCULAR,
                "padding_mode Only accept ('zeros', 'reflect', 'replicate', 'circular')");
    NVQ_REQUIRE(H + 2 * ph >= KH && W + 2 * pw >= KW, "conv2d: kernel larger than the padded input");
    g = ConvGeom{N, C, H, W, KH, KW, sh, sw, ph, pw, (H + 2 * ph - KH) / sh + 1, (W + 2 * pw - KW) / sw + 1, (int)mode};
    return NVQ_OK;
}

unsigned ew_grid(size_t n, int device) {
    size_t want = (n + 255) / 256, cap = (size_t)nvq_sm_count(device) * 8;
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace

extern "C" nvq_status nvq_linear_fwd_f32(float* d_y, const float* d_x, const float* d_w,
                                         const float* d_bias, int M, int N, int K, int relu,
                                         float* d_mask, int device, void* stream) {
    NVQ_REQUIRE(d_y && d_x && d_w && M >= 0 && N > 0 && K > 0, "nvq_linear_fwd_f32: bad argument");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    GemmArgs g{};
    g.a = d_x; g.a_si = K; g.a_sl = 1;          // X[m,k]
    g.b = d_w; g.b_sl = 1; g.b_sj = K;          // W^T: B(k,n) = W[n,k]
    g.c = d_y; g.I = M; g.J = N; g.L = K;
    g.bias = d_bias; g.bias_per_row = 0;
    g.relu = relu; g.mask_out = relu ? d_mask : nullptr;
    return launch_gemm(g, (cudaStream_t)stream);
}

extern "C" nvq_status nvq_linear_bwd_f32(float* d_dw, float* d_db, float* d_dx, const float* d_g,
                                         const float* d_x, const float* d_w, const float* d_mask,
                                         int M, int N, int K, int device, void* stream) {
    NVQ_REQUIRE(d_g && M > 0 && N > 0 && K > 0, "nvq_linear_bwd_f32: bad argument");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (d_dw) {   // dW[n,k] = sum_m G[m,n] X[m,k]
        NVQ_REQUIRE(d_x, "nvq_linear_bwd_f32: dW needs x");
        GemmArgs g{};
        g.a = d_g; g.a_si = 1; g.a_sl = N;
        g.b = d_x; g.b_sl = K; g.b_sj = 1;
        g.c = d_dw; g.I = N; g.J = K; g.L = M;
        g.rowsum = d_db;          // db[n] = sum_m G[m,n]: the row sums of the A operand, for free
        s = launch_gemm(g, st);
        if (s != NVQ_OK) return s;
    } else if (d_db) {
        nvq_launch_chained(colsum_kernel, dim3((N + 31) / 32), 256, 0, st, d_g, d_db, M, N);
        NVQ_LAUNCHED();
    }
    if (d_dx) {   // dX[m,k] = sum_n G[m,n] W[n,k]
        NVQ_REQUIRE(d_w, "nvq_linear_bwd_f32: dX needs w");
        GemmArgs g{};
        g.a = d_g; g.a_si = N; g.a_sl = 1;
        g.b = d_w; g.b_sl = K; g.b_sj = 1;
        g.c = d_dx; g.I = M; g.J = K; g.L = N;
        g.mask_in = d_mask;
        s = launch_gemm(g, st);
        if (s != NVQ_OK) return s;
    }
    return NVQ_OK;
}

extern "C" nvq_status nvq_relu_fwd_f32(float* d_out, float* d_mask, const float* d_x, size_t n,
                                       int device, void* stream) {
    if (n == 0) return NVQ_OK;
    NVQ_REQUIRE(d_out && d_x, "nvq_relu_fwd_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    nvq_launch_chained(relu_kernel, dim3(ew_grid(n, device)), 256, 0, (cudaStream_t)stream, d_out, d_mask, d_x, n);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_mul_f32(float* d_out, const float* d_a, const float* d_b, size_t n,
                                  int device, void* stream) {
    if (n == 0) return NVQ_OK;
    NVQ_REQUIRE(d_out && d_a && d_b, "nvq_mul_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    nvq_launch_chained(mul_kernel, dim3(ew_grid(n, device)), 256, 0, (cudaStream_t)stream, d_out, d_a, d_b, n);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_softmax_ce_f32(float* d_grad, float* d_loss, const float* d_logits,
                                         const int32_t* d_labels, float* d_yhat, int M, int C,
                                         int device, void* stream) {
    NVQ_REQUIRE(d_grad && d_logits && d_labels && d_yhat && M > 0 && C > 0,
                "nvq_softmax_ce_f32: bad argument");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    nvq_launch_chained(softmax_ce_kernel, dim3(1), 256, 256 * sizeof(double), (cudaStream_t)stream, d_grad, d_loss,
                   d_logits, (const int*)d_labels, d_yhat, M, C);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_ce_loss_f32(float* d_loss, const float* d_yhat, const int32_t* d_labels, int M,
                                      int C, int device, void* stream) {
    NVQ_REQUIRE(d_loss && d_yhat && d_labels && M > 0 && C > 0, "nvq_ce_loss_f32: bad argument");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    nvq_launch_chained(ce_loss_kernel, dim3(1), 256, 256 * sizeof(double), (cudaStream_t)stream, d_loss, d_yhat,
                       (const int*)d_labels, M, C);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_sgd_step_f32(float* d_param, const float* d_grad, size_t n, float lr,
                                       float grad_scale, int device, void* stream) {
    if (n == 0) return NVQ_OK;
    NVQ_REQUIRE(d_param && d_grad, "nvq_sgd_step_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    nvq_launch_chained(sgd_kernel, dim3(ew_grid(n, device)), 256, 0, (cudaStream_t)stream, d_param, d_grad, n, lr, grad_scale);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_conv2d_out_size(int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
                                          int* OH, int* OW) {
    NVQ_REQUIRE(OH && OW && sh > 0 && sw > 0, "nvq_conv2d_out_size: bad argument");
    *OH = (H + 2 * ph - KH) / sh + 1;
    *OW = (W + 2 * pw - KW) / sw + 1;
    return NVQ_OK;
}

extern "C" nvq_status nvq_im2col_f32(float* d_col, const float* d_x, int N, int C, int H, int W,
                                     int KH, int KW, int sh, int sw, int ph, int pw,
                                     nvq_pad_mode mode, int device, void* stream) {
    ConvGeom g;
    nvq_status s = geom(g, N, C, H, W, KH, KW, sh, sw, ph, pw, mode);
    if (s != NVQ_OK) return s;
    NVQ_REQUIRE(d_col && d_x, "nvq_im2col_f32: null buffer");
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    size_t total = (size_t)C * KH * KW * N * g.OH * g.OW;
    if (total < (1u << 31) && (size_t)N * C * H * W < (1u << 31))
        im2col_f32_kernel<uint32_t><<<ew_grid(total, device), 256, 0, (cudaStream_t)stream>>>(d_col, d_x, g);
    else
        im2col_f32_kernel<size_t><<<ew_grid(total, device), 256, 0, (cudaStream_t)stream>>>(d_col, d_x, g);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_conv2d_fwd_f32(float* d_out, const float* d_x, const float* d_w,
                                         const float* d_bias, float* d_col, int N, int C, int H,
                                         int W, int Cout, int KH, int KW, int sh, int sw, int ph,
                                         int pw, nvq_pad_mode mode, int device, void* stream) {
    NVQ_REQUIRE(d_out && d_w && d_col && Cout > 0, "nvq_conv2d_fwd_f32: bad argument");
    nvq_status s = nvq_im2col_f32(d_col, d_x, N, C, H, W, KH, KW, sh, sw, ph, pw, mode, device, stream);
    if (s != NVQ_OK) return s;
    ConvGeom gm;
    geom(gm, N, C, H, W, KH, KW, sh, sw, ph, pw, mode);
    const int CKK = C * KH * KW, L = N * gm.OH * gm.OW;
    GemmArgs g{};
    g.a = d_w; g.a_si = CKK; g.a_sl = 1;        // w_col[cout, ckk]
    g.b = d_col; g.b_sl = L; g.b_sj = 1;        // col[ckk, l]
    g.c = d_out; g.I = Cout; g.J = L; g.L = CKK;
    g.bias = d_bias; g.bias_per_row = 1;
    g.out_mode = 1; g.inner = gm.OH * gm.OW;    // (n, cout, oh, ow) contiguous
    return launch_gemm(g, (cudaStream_t)stream);
}

extern "C" nvq_status nvq_conv2d_q_sizes(int N, int C, int H, int W, int Cout, int KH, int KW, int sh,
                                         int sw, int ph, int pw, size_t* rows, size_t* kpad) {
    NVQ_REQUIRE(rows && kpad && sh > 0 && sw > 0, "nvq_conv2d_q_sizes: bad argument");
    int OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
    *rows = (size_t)N * OH * OW;
    *kpad = ((size_t)C * KH * KW + 15) / 16 * 16;
    (void)Cout;
    return NVQ_OK;
}

extern "C" nvq_status nvq_conv2d_fwd_q(float* d_out, const float* d_x, const uint8_t* d_wq,
                                       nvq_dtype w_fmt, const float* d_w_scales, const float* d_bias,
                                       uint16_t* d_col_bf16, uint16_t* d_y_bf16, void* d_workspace,
                                       size_t workspace_bytes, int N, int C, int H, int W, int Cout,
                                       int KH, int KW, int sh, int sw, int ph, int pw,
                                       nvq_pad_mode mode, int device, void* stream) {
    return nvq_conv2d_fwd_q_opts(d_out, d_x, d_wq, w_fmt, d_w_scales, d_bias, d_col_bf16, d_y_bf16,
                                 d_workspace, workspace_bytes, N, C, H, W, Cout, KH, KW, sh, sw, ph, pw,
                                 mode, NVQ_CONV_AUTO, device, stream);
}

extern "C" nvq_status nvq_conv2d_fwd_q_opts(float* d_out, const float* d_x, const uint8_t* d_wq,
                                            nvq_dtype w_fmt, const float* d_w_scales,
                                            const float* d_bias, uint16_t* d_col_bf16,
                                            uint16_t* d_y_bf16, void* d_workspace,
                                            size_t workspace_bytes, int N, int C, int H, int W,
                                            int Cout, int KH, int KW, int sh, int sw, int ph, int pw,
                                            nvq_pad_mode mode, uint32_t path, int device,
                                            void* stream) {
    NVQ_REQUIRE(path == NVQ_CONV_AUTO || path == NVQ_CONV_PATCH_MATRIX || path == NVQ_CONV_CTA_PAIR,
                "nvq_conv2d_fwd_q_opts: unknown path selector 0x%x", path);
    ConvGeom g;
    nvq_status s = geom(g, N, C, H, W, KH, KW, sh, sw, ph, pw, mode);
    if (s != NVQ_OK) return s;
    NVQ_REQUIRE(d_out && d_x && d_wq && d_w_scales && d_col_bf16 && d_y_bf16, "nvq_conv2d_fwd_q: null buffer");
    NVQ_REQUIRE(Cout % 8 == 0, "nvq_conv2d_fwd_q: Cout (%d) must be a multiple of 8", Cout);
    NVQ_REQUIRE(w_fmt == NVQ_E4M3 || w_fmt == NVQ_E5M2 || w_fmt == NVQ_E2M1_B32,
                "nvq_conv2d_fwd_q: weight format must be E4M3, E5M2 or E2M1_B32");
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t L = (size_t)N * g.OH * g.OW;
    const int kq = w_fmt == NVQ_E2M1_B32 ? 32 : 16;          // FP4 blocks are 32 columns
    const int Kpad = (C * KH * KW + kq - 1) / kq * kq;
    // Implicit GEMM (no patch matrix): strides 1 or 2, zero padding, channels in blocks of 64, output
    // rows of at most 256 positions (and at most 256 input pixels walked per row).  d_col_bf16 holds x as bf16 NHWC, d_workspace the weight with
    // its columns reordered to (kh, kw, c).  NVQ_CONV_PATCH_MATRIX forces the patch-matrix path.
    const bool pair_only = path == NVQ_CONV_CTA_PAIR;     // the pair kernel's tiles hold 128 positions per CTA
    const bool implicit_ok = sh >= 1 && sh <= 2 && sw >= 1 && sw <= 2 && mode == NVQ_PAD_ZEROS && C % 64 == 0 &&
                             (g.OW <= 128 || (!pair_only && g.OW * sw <= 256)) &&
                             L < (1u << 31) && (size_t)Cout * C * KH * KW < (1u << 31) &&
                             workspace_bytes >= (size_t)Cout * C * KH * KW * 2 && d_workspace &&
                             (size_t)H * W <= (size_t)g.OH * g.OW * KH * KW &&
                             path != NVQ_CONV_PATCH_MATRIX;
    if (implicit_ok) {
        const int S_in = H * W;
        const size_t cap = (size_t)nvq_sm_count(device) * 16;
        if (S_in % 4 == 0 && nvq_aligned(d_x, 16)) {
            const size_t want = (size_t)N * ((S_in + 63) / 64) * (C / 64);
            nchw_f32_to_nhwc_bf16_v4_kernel<<<(unsigned)std::min(want, cap), 256, 0, st>>>(d_col_bf16, d_x, N, C, S_in);
        } else {
            const size_t want = (size_t)N * ((S_in + 31) / 32) * (C / 64);
            nchw_f32_to_nhwc_bf16_kernel<<<(unsigned)std::min(want, cap), 256, 0, st>>>(d_col_bf16, d_x, N, C, S_in);
        }
        NVQ_LAUNCHED();
        const int wtotal = Cout * C * KH * KW;
        if (w_fmt == NVQ_E4M3)
            expand_permute_weight_kernel<NVQ_E4M3><<<ew_grid(wtotal, device), 256, 0, st>>>(
                (uint16_t*)d_workspace, d_wq, Cout, C, KH, KW, Kpad);
        else if (w_fmt == NVQ_E5M2)
            expand_permute_weight_kernel<NVQ_E5M2><<<ew_grid(wtotal, device), 256, 0, st>>>(
                (uint16_t*)d_workspace, d_wq, Cout, C, KH, KW, Kpad);
        else
            expand_permute_weight_fp4_kernel<<<ew_grid(wtotal, device), 256, 0, st>>>(
                (uint16_t*)d_workspace, d_wq, d_w_scales, Cout, C, KH, KW, Kpad);
        NVQ_LAUNCHED();
        // FP4 block scales are already in the expanded weight; FP8 channel scales go to the epilogue.
        // The operand-swapped kernel is the default: measured 4-13 % faster than the CTA-pair kernel
        // at 256 and 512 output channels and 25 % faster at 128 ([128, 64, 56, 56] -> 128: 0.106 ms
        // against 0.139 ms).  NVQ_CONV_CTA_PAIR selects the pair kernel.
        if (g.OW * sw <= 256 && !pair_only)
            return nvq_conv_launch_swapped(d_out, d_col_bf16, (const uint16_t*)d_workspace,
                                           w_fmt == NVQ_E2M1_B32 ? nullptr : d_w_scales, d_bias, N, C, H, W,
                                           Cout, KH, KW, ph, pw, sh, sw, device, st);
        return nvq_conv_launch_pair_implicit(d_out, d_col_bf16, (const uint16_t*)d_workspace,
                                             w_fmt == NVQ_E2M1_B32 ? nullptr : d_w_scales, d_bias, N, C, H, W,
                                             Cout, KH, KW, ph, pw, sh, sw, device, st);
    }
    const bool tiled = C * KH * KW <= kImLut && KH < 256 && KW < 256 && C < 65536 && L < (1u << 31);
    if (tiled) {
        const size_t want = (L + kImRows - 1) / kImRows, cap = (size_t)nvq_sm_count(device) * 8;
        im2col_bf16_tiled_kernel<<<(unsigned)std::min(want, cap), 256, 0, st>>>(d_col_bf16, d_x, g, Kpad, (int)L);
    } else {
        im2col_bf16_rows_kernel<<<ew_grid(L * Kpad, device), 256, 0, st>>>(d_col_bf16, d_x, g, Kpad);
    }
    NVQ_LAUNCHED();
    s = nvq_linear_fwd(d_y_bf16, d_col_bf16, d_wq, w_fmt, d_w_scales, d_bias, L, (size_t)Cout,
                       (size_t)Kpad, d_workspace, workspace_bytes, device, stream);
    if (s != NVQ_OK) return s;
    if (tiled) {
        const int S = g.OH * g.OW;
        const size_t want = (size_t)N * ((S + 31) / 32) * ((Cout + 63) / 64), cap = (size_t)nvq_sm_count(device) * 16;
        rows_bf16_to_nchw_tiled_kernel<<<(unsigned)std::min(want, cap), 256, 0, st>>>(d_out, d_y_bf16, N, Cout, S);
    } else {
        rows_bf16_to_nchw_kernel<<<ew_grid(L * Cout, device), 256, 0, st>>>(d_out, d_y_bf16, N, Cout, g.OH * g.OW);
    }
    NVQ_LAUNCHED();
    return NVQ_OK;
}

// ---- activations kept bf16 NHWC between chained quantised layers -------------------------------
extern "C" nvq_status nvq_nchw_f32_to_nhwc_bf16(uint16_t* d_dst, const float* d_src, int N, int C, int S,
                                                int device, void* stream) {
    NVQ_REQUIRE(d_dst && d_src && N > 0 && C > 0 && S > 0, "nvq_nchw_f32_to_nhwc_bf16: bad argument");
    NVQ_REQUIRE(C % 64 == 0, "nvq_nchw_f32_to_nhwc_bf16: C (%d) must be a multiple of 64", C);
    NVQ_REQUIRE(nvq_aligned(d_dst, 16), "nvq_nchw_f32_to_nhwc_bf16: destination must be 16-byte aligned");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t cap = (size_t)nvq_sm_count(device) * 16;
    if (S % 4 == 0 && nvq_aligned(d_src, 16)) {
        const size_t want = (size_t)N * ((S + 63) / 64) * (C / 64);
        nchw_f32_to_nhwc_bf16_v4_kernel<<<(unsigned)std::min(want, cap), 256, 0, st>>>(d_dst, d_src, N, C, S);
    } else {
        const size_t want = (size_t)N * ((S + 31) / 32) * (C / 64);
        nchw_f32_to_nhwc_bf16_kernel<<<(unsigned)std::min(want, cap), 256, 0, st>>>(d_dst, d_src, N, C, S);
    }
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_nhwc_bf16_to_nchw_f32(float* d_dst, const uint16_t* d_src, int N, int C, int S,
                                                int device, void* stream) {
    NVQ_REQUIRE(d_dst && d_src && N > 0 && C > 0 && S > 0, "nvq_nhwc_bf16_to_nchw_f32: bad argument");
    NVQ_REQUIRE(C % 8 == 0 && nvq_aligned(d_src, 16), "nvq_nhwc_bf16_to_nchw_f32: C (%d) must be a multiple of 8, source 16-byte aligned", C);
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    const size_t want = (size_t)N * ((S + 31) / 32) * ((C + 63) / 64), cap = (size_t)nvq_sm_count(device) * 16;
    rows_bf16_to_nchw_tiled_kernel<<<(unsigned)std::min(want, cap), 256, 0, (cudaStream_t)stream>>>(d_dst, d_src, N, C, S);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_conv2d_fwd_q_nhwc(uint16_t* d_out_bf16, const uint16_t* d_x_bf16,
                                            const uint8_t* d_wq, nvq_dtype w_fmt,
                                            const float* d_w_scales, const float* d_bias,
                                            void* d_workspace, size_t workspace_bytes, int N, int C,
                                            int H, int W, int Cout, int KH, int KW, int sh, int sw,
                                            int ph, int pw, int relu, int device, void* stream) {
    ConvGeom g;
    nvq_status s = geom(g, N, C, H, W, KH, KW, sh, sw, ph, pw, NVQ_PAD_ZEROS);
    if (s != NVQ_OK) return s;
    NVQ_REQUIRE(d_out_bf16 && d_x_bf16 && d_wq && d_w_scales && d_workspace, "nvq_conv2d_fwd_q_nhwc: null buffer");
    NVQ_REQUIRE(Cout % 8 == 0, "nvq_conv2d_fwd_q_nhwc: Cout (%d) must be a multiple of 8", Cout);
    NVQ_REQUIRE(w_fmt == NVQ_E4M3 || w_fmt == NVQ_E5M2 || w_fmt == NVQ_E2M1_B32,
                "nvq_conv2d_fwd_q_nhwc: weight format must be E4M3, E5M2 or E2M1_B32");
    NVQ_REQUIRE(nvq_aligned(d_out_bf16, 16) && nvq_aligned(d_x_bf16, 16) && nvq_aligned(d_workspace, 16),
                "nvq_conv2d_fwd_q_nhwc: buffers must be 16-byte aligned");
    const size_t L = (size_t)N * g.OH * g.OW;
    if (!(sh >= 1 && sh <= 2 && sw >= 1 && sw <= 2 && C % 64 == 0 && g.OW * sw <= 256 && L < (1u << 31) &&
          (size_t)Cout * C * KH * KW < (1u << 31)))
        NVQ_FAIL(NVQ_ERR_UNSUPPORTED, "nvq_conv2d_fwd_q_nhwc: needs strides 1 or 2, C %% 64 == 0 and OW * stride <= 256 "
                                      "(got stride %d x %d, C = %d, OW = %d); use nvq_conv2d_fwd_q", sh, sw, C, g.OW);
    NVQ_REQUIRE(workspace_bytes >= (size_t)Cout * C * KH * KW * 2,
                "nvq_conv2d_fwd_q_nhwc: workspace of %zu bytes required", (size_t)Cout * C * KH * KW * 2);
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const int kq = w_fmt == NVQ_E2M1_B32 ? 32 : 16;
    const int Kpad = (C * KH * KW + kq - 1) / kq * kq;
    const int wtotal = Cout * C * KH * KW;
    if (w_fmt == NVQ_E4M3)
        expand_permute_weight_kernel<NVQ_E4M3><<<ew_grid(wtotal, device), 256, 0, st>>>(
            (uint16_t*)d_workspace, d_wq, Cout, C, KH, KW, Kpad);
    else if (w_fmt == NVQ_E5M2)
        expand_permute_weight_kernel<NVQ_E5M2><<<ew_grid(wtotal, device), 256, 0, st>>>(
            (uint16_t*)d_workspace, d_wq, Cout, C, KH, KW, Kpad);
    else
        expand_permute_weight_fp4_kernel<<<ew_grid(wtotal, device), 256, 0, st>>>(
            (uint16_t*)d_workspace, d_wq, d_w_scales, Cout, C, KH, KW, Kpad);
    NVQ_LAUNCHED();
    return nvq_conv_launch_swapped(nullptr, d_x_bf16, (const uint16_t*)d_workspace,
                                   w_fmt == NVQ_E2M1_B32 ? nullptr : d_w_scales, d_bias, N, C, H, W, Cout, KH, KW,
                                   ph, pw, sh, sw, device, st, d_out_bf16, relu ? 1 : 0);
}

extern "C" nvq_status nvq_conv2d_bwd_f32(float* d_dw, float* d_db, float* d_dx, const float* d_grad,
                                         const float* d_col, const float* d_w, float* d_gr,
                                         float* d_dcol, int N, int C, int H, int W, int Cout, int KH,
                                         int KW, int sh, int sw, int ph, int pw, int device,
                                         void* stream) {
    ConvGeom gm;
    nvq_status s = geom(gm, N, C, H, W, KH, KW, sh, sw, ph, pw, NVQ_PAD_ZEROS);
    if (s != NVQ_OK) return s;
    NVQ_REQUIRE(d_grad && d_gr && Cout > 0, "nvq_conv2d_bwd_f32: bad argument");
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    const int S = gm.OH * gm.OW, CKK = C * KH * KW;
    const size_t L = (size_t)N * S;
    NVQ_REQUIRE(L < (1u << 31), "nvq_conv2d_bwd_f32: too many output positions");
    const bool small = (size_t)CKK * L < (1u << 31) && L * Cout < (1u << 31) &&
                       (size_t)N * C * H * W < (1u << 31);
    if (small) nchw_to_crows_kernel<uint32_t><<<ew_grid(L * Cout, device), 256, 0, st>>>(d_gr, d_grad, N, Cout, S);
    else nchw_to_crows_kernel<size_t><<<ew_grid(L * Cout, device), 256, 0, st>>>(d_gr, d_grad, N, Cout, S);
    NVQ_LAUNCHED();
    if (d_dw) {   // dW = g_r @ col^T
        NVQ_REQUIRE(d_col, "nvq_conv2d_bwd_f32: dW needs col");
        GemmArgs g{};
        g.a = d_gr; g.a_si = (long long)L; g.a_sl = 1;
        g.b = d_col; g.b_sl = 1; g.b_sj = (long long)L;
        g.c = d_dw; g.I = Cout; g.J = CKK; g.L = (int)L;
        // d_dcol (free until the dX pass below) holds the split-k partial sums
        s = launch_gemm_splitk(g, d_dcol, d_dcol ? (size_t)CKK * L : 0, device, st);
        if (s != NVQ_OK) return s;
    }
    if (d_db) {
        rowsum_kernel<<<(Cout + 7) / 8, 256, 0, st>>>(d_gr, d_db, Cout, L);
        NVQ_LAUNCHED();
    }
    if (d_dx) {   // dcol = w_col^T @ g_r, then gather back onto the input
        NVQ_REQUIRE(d_w && d_dcol, "nvq_conv2d_bwd_f32: dX needs w and the dcol scratch");
        GemmArgs g{};
        g.a = d_w; g.a_si = 1; g.a_sl = CKK;
        g.b = d_gr; g.b_sl = (long long)L; g.b_sj = 1;
        g.c = d_dcol; g.I = CKK; g.J = (int)L; g.L = Cout;
        s = launch_gemm(g, st);
        if (s != NVQ_OK) return s;
        const unsigned grid = ew_grid((size_t)N * C * H * W, device);
        if (small && sh == 1 && sw == 1) col2im_kernel<uint32_t, 1><<<grid, 256, 0, st>>>(d_dx, d_dcol, gm);
        else if (small && sh == 2 && sw == 2) col2im_kernel<uint32_t, 2><<<grid, 256, 0, st>>>(d_dx, d_dcol, gm);
        else if (small) col2im_kernel<uint32_t, 0><<<grid, 256, 0, st>>>(d_dx, d_dcol, gm);
        else col2im_kernel<size_t, 0><<<grid, 256, 0, st>>>(d_dx, d_dcol, gm);
        NVQ_LAUNCHED();
    }
    return NVQ_OK;
}

extern "C" nvq_status nvq_adamw_step_f32(float* d_param, const float* d_grad, float* d_m, float* d_v,
                                         size_t n, float beta1, float one_minus_beta1, float beta2,
                                         float one_minus_beta2, float bias_corr1, float bias_corr2,
                                         float lr, float eps, float lr_times_wd, int apply_decay,
                                         int device, void* stream) {
    if (n == 0) return NVQ_OK;
    NVQ_REQUIRE(d_param && d_grad && d_m && d_v, "nvq_adamw_step_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    AdamWArgs a{beta1, one_minus_beta1, beta2, one_minus_beta2, bias_corr1, bias_corr2, lr, eps,
                lr_times_wd, apply_decay};
    adamw_kernel<<<ew_grid(n, device), 256, 0, (cudaStream_t)stream>>>(d_param, d_grad, d_m, d_v, n, a);
    NVQ_LAUNCHED();
    return NVQ_OK;
}
