// The layers either side of the GEMMs in NovaNN's CNN: BatchNorm (1-D and 2-D), MaxPool2d,
// GlobalAvgPool2d, Dropout, and the float64 AdamW step the BatchNorm parameters need.
//
// NovaNN creates gamma / beta / running statistics as float64 arrays
// (novann/layers/batchnorm/batchnorm2d.py:41-48), so a BatchNorm output there is float64 and
// every consumer narrows it with astype(np.float32) (conv2d.py:159, maxpool2d forward, the
// global average pool, linear.py:81).  These kernels evaluate the float64 expression and emit
// the narrowed fp32 value directly.  Batch statistics are accumulated in float64 (NumPy sums
// pairwise in fp32), so results agree with the reference to fp32 rounding of the statistics,
// not bit for bit; everything downstream of the statistics follows NumPy's operation order.
#include "nvq_common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxSplits = 32;   // blocks that share one channel's reduction

// Activations are (N, C, S) row-major: S = H*W for BatchNorm2d, the sequence length for
// BatchNorm1d on 3-D input, 1 for 2-D input.  Element j of channel c (j in [0, N*S)):
__device__ __forceinline__ size_t chan_index(int j, int c, int C, int S) {
    int n = j / S, s = j - n * S;
    return ((size_t)n * C + c) * S + s;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// Sum of up to four per-thread doubles over the block; result valid in thread 0.
template <int NV>
__device__ __forceinline__ void block_sum(double (&v)[NV], double (*sh)[kThreads / 32]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        v[i] = warp_sum(v[i]);
        if (lane == 0) sh[i][warp] = v[i];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            double t = lane < kThreads / 32 ? sh[i][lane] : 0.0;
            v[i] = warp_sum(t);
        }
    }
}

struct BnGeom { int N, C, S, P; };

// ---- forward, training: pass 1 -- per-channel partial sums of x and x^2 in float64
__global__ void __launch_bounds__(kThreads)
bn_stats_partial_kernel(double* __restrict__ partial, const float* __restrict__ x, BnGeom g) {
    __shared__ double sh[2][kThreads / 32];
    const int c = blockIdx.y, p = blockIdx.x, m = g.N * g.S;
    double v[2] = {0.0, 0.0};
    for (int j = p * kThreads + threadIdx.x; j < m; j += g.P * kThreads) {
        double xv = (double)x[chan_index(j, c, g.C, g.S)];
        v[0] += xv;
        v[1] += xv * xv;
    }
    block_sum<2>(v, sh);
    if (threadIdx.x == 0) {
        partial[((size_t)c * g.P + p) * 2 + 0] = v[0];
        partial[((size_t)c * g.P + p) * 2 + 1] = v[1];
    }
}

struct BnFwdArgs { double one_minus_momentum; float momentum32; float eps32; float bessel32; };

// pass 2 -- finish the statistics (every block of a channel repeats the tiny reduction),
// normalise, scale and shift; block 0 of a channel also writes the saved statistics and the
// running averages.
//   mu   = float32(mean);  var = float32(biased var) * float32(m/(m-1))      (fp32, as NumPy)
//   xhat = (x - mu) / sqrt(var + eps)                                        (fp32)
//   y    = float32(gamma * xhat + beta)                                      (float64 inside)
//   running = (1-momentum) * running + float64(float32(momentum) * stat)
__global__ void __launch_bounds__(kThreads)
bn_apply_train_kernel(float* __restrict__ y, const float* __restrict__ x,
                      const double* __restrict__ partial, const double* __restrict__ gamma,
                      const double* __restrict__ beta, double* __restrict__ run_mean,
                      double* __restrict__ run_var, float* __restrict__ save_stats, BnGeom g,
                      BnFwdArgs a) {
    __shared__ float s_mu, s_den;
    const int c = blockIdx.y, p = blockIdx.x, m = g.N * g.S;
    if (threadIdx.x < 32) {
        double s = 0.0, q = 0.0;
        if ((int)threadIdx.x < g.P) {
            s = partial[((size_t)c * g.P + threadIdx.x) * 2 + 0];
            q = partial[((size_t)c * g.P + threadIdx.x) * 2 + 1];
        }
        s = warp_sum(s);
        q = warp_sum(q);
        if (threadIdx.x == 0) {
            double mean = s / m;
            double var = q / m - mean * mean;
            if (var < 0.0) var = 0.0;
            float mu32 = (float)mean;
            float var32 = (float)var;
            if (m > 1) var32 = __fmul_rn(var32, a.bessel32);
            s_mu = mu32;
            s_den = __fsqrt_rn(__fadd_rn(var32, a.eps32));
            if (p == 0) {
                save_stats[c] = mu32;
                save_stats[g.C + c] = var32;
                run_mean[c] = __dadd_rn(__dmul_rn(a.one_minus_momentum, run_mean[c]),
                                        (double)__fmul_rn(a.momentum32, mu32));
                run_var[c] = __dadd_rn(__dmul_rn(a.one_minus_momentum, run_var[c]),
                                       (double)__fmul_rn(a.momentum32, var32));
            }
        }
    }
    __syncthreads();
    const float mu = s_mu, den = s_den;
    const double ga = gamma[c], be = beta[c];
    for (int j = p * kThreads + threadIdx.x; j < m; j += g.P * kThreads) {
        size_t i = chan_index(j, c, g.C, g.S);
        float xhat = __fdiv_rn(__fsub_rn(x[i], mu), den);
        y[i] = (float)__dadd_rn(__dmul_rn(ga, (double)xhat), be);
    }
}

// ---- forward, evaluation: y = float32(gamma * ((x - running_mean) / sqrt(running_var + eps)) + beta),
// all in float64 as NumPy promotes it (batchnorm2d.py:98-101)
__global__ void __launch_bounds__(kThreads)
bn_apply_eval_kernel(float* __restrict__ y, const float* __restrict__ x,
                     const double* __restrict__ gamma, const double* __restrict__ beta,
                     const double* __restrict__ run_mean, const double* __restrict__ run_var,
                     BnGeom g, double eps) {
    const int c = blockIdx.y, p = blockIdx.x, m = g.N * g.S;
    const double rm = run_mean[c], den = __dsqrt_rn(__dadd_rn(run_var[c], eps));
    const double ga = gamma[c], be = beta[c];
    for (int j = p * kThreads + threadIdx.x; j < m; j += g.P * kThreads) {
        size_t i = chan_index(j, c, g.C, g.S);
        double xhat = __ddiv_rn(__dsub_rn((double)x[i], rm), den);
        y[i] = (float)__dadd_rn(__dmul_rn(ga, xhat), be);
    }
}

// ---- backward: pass 1 -- partial sums of grad, grad*xhat, grad*(x-mu), (x-mu)
__global__ void __launch_bounds__(kThreads)
bn_bwd_partial_kernel(double* __restrict__ partial, const float* __restrict__ grad,
                      const float* __restrict__ x, const float* __restrict__ save_stats, BnGeom g,
                      float eps32) {
    __shared__ double sh[4][kThreads / 32];
    const int c = blockIdx.y, p = blockIdx.x, m = g.N * g.S;
    const float mu = save_stats[c];
    const float den = __fsqrt_rn(__fadd_rn(save_stats[g.C + c], eps32));
    double v[4] = {0.0, 0.0, 0.0, 0.0};
    for (int j = p * kThreads + threadIdx.x; j < m; j += g.P * kThreads) {
        size_t i = chan_index(j, c, g.C, g.S);
        float xmu = __fsub_rn(x[i], mu);
        float xhat = __fdiv_rn(xmu, den);
        double gr = (double)grad[i];
        v[0] += gr;
        v[1] += gr * (double)xhat;
        v[2] += gr * (double)xmu;
        v[3] += (double)xmu;
    }
    block_sum<4>(v, sh);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int k = 0; k < 4; k++) partial[((size_t)c * g.P + p) * 4 + k] = v[k];
    }
}

// pass 2 -- BatchNorm2d.backward (batchnorm2d.py:104-146) in float64, narrowed on store:
//   dgamma = sum(grad*xhat);  dbeta = sum(grad);  dxhat = grad*gamma
//   inv_std = (var+eps)^-1/2, inv_std3 = (var+eps)^-3/2      (fp32 values, as NumPy holds them)
//   dvar = sum(dxhat * xmu * -0.5 * inv_std3);  dmu = sum(dxhat * -inv_std) + dvar * sum(-2 xmu) / m
//   dx   = dxhat*inv_std + dvar*(2 xmu)/m + dmu/m
__global__ void __launch_bounds__(kThreads)
bn_bwd_apply_kernel(float* __restrict__ dx, double* __restrict__ dgamma, double* __restrict__ dbeta,
                    const float* __restrict__ grad, const float* __restrict__ x,
                    const double* __restrict__ partial, const float* __restrict__ save_stats,
                    const double* __restrict__ gamma, BnGeom g, float eps32) {
    __shared__ double s_dvar, s_dmu_m;
    __shared__ float s_inv;
    const int c = blockIdx.y, p = blockIdx.x, m = g.N * g.S;
    const float mu = save_stats[c];
    const float base = __fadd_rn(save_stats[g.C + c], eps32);
    if (threadIdx.x < 32) {
        double v[4] = {0.0, 0.0, 0.0, 0.0};
        if ((int)threadIdx.x < g.P) {
#pragma unroll
            for (int k = 0; k < 4; k++) v[k] = partial[((size_t)c * g.P + threadIdx.x) * 4 + k];
        }
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] = warp_sum(v[k]);
        if (threadIdx.x == 0) {
            const double b = (double)base, r = 1.0 / sqrt(b);
            const float inv_std = (float)r, inv_std3 = (float)(r / b);
            const double ga = gamma[c];
            const double dvar = ga * v[2] * (-0.5) * (double)inv_std3;
            const double dmu = ga * v[0] * (-(double)inv_std) + dvar * (-2.0 * v[3]) / m;
            s_dvar = dvar;
            s_dmu_m = dmu / m;
            s_inv = inv_std;
            if (p == 0) {
                if (dgamma) dgamma[c] = v[1];
                if (dbeta) dbeta[c] = v[0];
            }
        }
    }
    __syncthreads();
    if (!dx) return;
    const double dvar = s_dvar, dmu_m = s_dmu_m, inv = (double)s_inv, ga = gamma[c], md = (double)m;
    for (int j = p * kThreads + threadIdx.x; j < m; j += g.P * kThreads) {
        size_t i = chan_index(j, c, g.C, g.S);
        double xmu = (double)__fsub_rn(x[i], mu);
        double t1 = __dmul_rn(__dmul_rn((double)grad[i], ga), inv);
        double t2 = __ddiv_rn(__dmul_rn(dvar, __dmul_rn(2.0, xmu)), md);
        dx[i] = (float)__dadd_rn(__dadd_rn(t1, t2), dmu_m);
    }
}

// ---- MaxPool2d ---------------------------------------------------------------------------
__device__ __forceinline__ int pool_pad_index(int idx, int size, int mode, bool& zero) {
    zero = false;
    if (idx >= 0 && idx < size) return idx;
    if (mode == NVQ_PAD_ZEROS) { zero = true; return 0; }
    if (mode == NVQ_PAD_REPLICATE) return idx < 0 ? 0 : size - 1;
    if (mode == NVQ_PAD_CIRCULAR) { int r = idx % size; return r < 0 ? r + size : r; }
    if (size == 1) return 0;
    int period = 2 * (size - 1);
    int r = idx % period;
    if (r < 0) r += period;
    return r < size ? r : period - r;
}

struct PoolGeom { int N, C, H, W, KH, KW, sh, sw, ph, pw, OH, OW, mode; };

// value of the padded plane at padded coordinates (hp, wp)
__device__ __forceinline__ float padded_at(const float* plane, const PoolGeom& g, int hp, int wp) {
    bool zh, zw;
    int h = pool_pad_index(hp - g.ph, g.H, g.mode, zh);
    int w = pool_pad_index(wp - g.pw, g.W, g.mode, zw);
    return (zh || zw) ? 0.f : plane[h * g.W + w];
}

// window maximum as np.max gives it (a NaN in the window makes the maximum NaN) and the
// number of entries equal to it.  A window holding both zeros yields +0 (IEEE maximum); NumPy's
// sign there depends on its reduction order, and the two zeros count as equal either way.
__device__ __forceinline__ float window_max(const float* plane, const PoolGeom& g, int oh, int ow,
                                            int* count) {
    float mx = 0.f;
    bool first = true, nan = false;
    int cnt = 0;
    for (int kh = 0; kh < g.KH; kh++)
        for (int kw = 0; kw < g.KW; kw++) {
            float v = padded_at(plane, g, oh * g.sh + kh, ow * g.sw + kw);
            if (v != v) nan = true;
            if (first || v > mx) { mx = v; cnt = 1; first = false; }
            else if (v == mx) { cnt++; if (__float_as_uint(mx) == 0x80000000u) mx = v; }
        }
    if (nan) { mx = __int_as_float(0x7FC00000); cnt = 0; }
    if (count) *count = cnt;
    return mx;
}

__global__ void maxpool_fwd_kernel(float* __restrict__ out, const float* __restrict__ x, PoolGeom g) {
    const size_t total = (size_t)g.N * g.C * g.OH * g.OW, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        int ow = e % g.OW, oh = (e / g.OW) % g.OH;
        size_t nc = e / ((size_t)g.OW * g.OH);
        out[e] = window_max(x + nc * g.H * g.W, g, oh, ow, nullptr);
    }
}

// MaxPool2d.backward (maxpool2d.py backward): every entry equal to its window's maximum receives
// grad / (number of such entries); the reference adds the windows in (oh, ow) order into the
// padded plane and crops it, which this gather reproduces addition by addition.
__global__ void maxpool_bwd_kernel(float* __restrict__ dx, const float* __restrict__ grad,
                                   const float* __restrict__ x, PoolGeom g) {
    const size_t total = (size_t)g.N * g.C * g.H * g.W, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        int w = e % g.W, h = (e / g.W) % g.H;
        size_t nc = e / ((size_t)g.W * g.H);
        const float* plane = x + nc * g.H * g.W;
        const float* gp = grad + nc * g.OH * g.OW;
        const int hp = h + g.ph, wp = w + g.pw;
        const float v = plane[h * g.W + w];
        int i0 = hp - g.KH + 1 <= 0 ? 0 : (hp - g.KH + g.sh) / g.sh;   // ceil((hp-KH+1)/sh)
        int j0 = wp - g.KW + 1 <= 0 ? 0 : (wp - g.KW + g.sw) / g.sw;
        int i1 = min(hp / g.sh, g.OH - 1), j1 = min(wp / g.sw, g.OW - 1);
        float acc = 0.f;
        for (int i = i0; i <= i1; i++)
            for (int j = j0; j <= j1; j++) {
                int cnt;
                float mx = window_max(plane, g, i, j, &cnt);
                float share = __fdiv_rn(gp[i * g.OW + j], cnt > 0 ? (float)cnt : 1.f);
                acc = __fadd_rn(acc, (v == mx) ? share : __fmul_rn(0.f, share));
            }
        dx[e] = acc;
    }
}

// ---- GlobalAvgPool2d: one warp per (n, c) plane -----------------------------------------
__global__ void gap_fwd_kernel(float* __restrict__ out, const float* __restrict__ x, size_t planes,
                               int S) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (size_t pl = warp; pl < planes; pl += n_warps) {
        double s = 0.0;
        for (int i = lane; i < S; i += 32) s += (double)x[pl * S + i];
        s = warp_sum(s);
        if (lane == 0) out[pl] = (float)(s / S);
    }
}

// GlobalAvgPool2d.backward: ones * (grad * float32(1/(H*W)))
__global__ void gap_bwd_kernel(float* __restrict__ dx, const float* __restrict__ grad, size_t total,
                               int S, float factor) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride)
        dx[e] = __fmul_rn(1.0f, __fmul_rn(grad[e / S], factor));
}

// Dropout forward and backward (dropout.py): (x * mask) / keep_prob
__global__ void dropout_kernel(float* __restrict__ out, const float* __restrict__ x,
                               const float* __restrict__ mask, size_t n, float keep) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride)
        out[e] = __fdiv_rn(__fmul_rn(x[e], mask[e]), keep);
}

// AdamW.step on float64 tensors (the BatchNorm parameters), each operation rounded separately
struct AdamW64Args { double b1, c1, b2, c2, bc1, bc2, lr, eps, lr_wd; int decay; };
__global__ void adamw_f64_kernel(double* __restrict__ p, const double* __restrict__ g,
                                 double* __restrict__ m, double* __restrict__ v, size_t n,
                                 AdamW64Args a) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        double gi = g[i];
        double mi = __dadd_rn(__dmul_rn(a.b1, m[i]), __dmul_rn(a.c1, gi));
        double vi = __dadd_rn(__dmul_rn(a.b2, v[i]), __dmul_rn(a.c2, __dmul_rn(gi, gi)));
        m[i] = mi;
        v[i] = vi;
        double mh = __ddiv_rn(mi, a.bc1), vh = __ddiv_rn(vi, a.bc2);
        double upd = __ddiv_rn(__dmul_rn(a.lr, mh), __dadd_rn(__dsqrt_rn(vh), a.eps));
        double pi = __dsub_rn(p[i], upd);
        if (a.decay) pi = __dsub_rn(pi, __dmul_rn(a.lr_wd, pi));
        p[i] = pi;
    }
}

unsigned flat_grid(size_t n, int device) {
    size_t want = (n + kThreads - 1) / kThreads, cap = (size_t)nvq_sm_count(device) * 8;
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

// blocks per channel: enough for about eight blocks per SM (the loops are latency-bound), at most kMaxSplits, and no more
// than the channel has 256-element slices
int bn_splits(int N, int C, int S, int device) {
    long m = (long)N * S;
    long by_size = (m + kThreads - 1) / kThreads;
    long by_sm = (8L * nvq_sm_count(device) + C - 1) / C;
    long p = by_size < by_sm ? by_size : by_sm;
    if (p > kMaxSplits) p = kMaxSplits;
    return (int)(p < 1 ? 1 : p);
}

nvq_status pool_geom(PoolGeom& g, int N, int C, int H, int W, int KH, int KW, int sh, int sw, int ph,
                     int pw, nvq_pad_mode mode, const char* who) {
    NVQ_REQUIRE(N >= 0 && C > 0 && H > 0 && W > 0 && KH > 0 && KW > 0 && sh > 0 && sw > 0 &&
                    ph >= 0 && pw >= 0, "%s: bad geometry", who);
    NVQ_REQUIRE(mode >= NVQ_PAD_ZEROS && mode <= NVQ_PAD_CIRCULAR, "%s: unknown padding mode", who);
    NVQ_REQUIRE(H + 2 * ph >= KH && W + 2 * pw >= KW, "%s: window larger than the padded input", who);
    if (mode == NVQ_PAD_REFLECT)
        NVQ_REQUIRE(ph < H && pw < W, "%s: reflect padding must be smaller than the input", who);
    if (mode == NVQ_PAD_CIRCULAR)
        NVQ_REQUIRE(ph <= H && pw <= W, "%s: circular padding must not exceed the input", who);
    g = PoolGeom{N, C, H, W, KH, KW, sh, sw, ph, pw, (H + 2 * ph - KH) / sh + 1,
                 (W + 2 * pw - KW) / sw + 1, (int)mode};
    return NVQ_OK;
}

}  // namespace

extern "C" {

size_t nvq_batchnorm_scratch_bytes(int C) {
    return C > 0 ? (size_t)C * kMaxSplits * 4 * sizeof(double) : 0;
}

nvq_status nvq_batchnorm_fwd_f32(float* d_y, const float* d_x, const double* d_gamma,
                                 const double* d_beta, double* d_running_mean,
                                 double* d_running_var, float* d_save_stats, double* d_scratch,
                                 int N, int C, int S, double momentum, double eps, int training,
                                 int device, void* stream) {
    NVQ_REQUIRE(N >= 0 && C > 0 && S > 0, "nvq_batchnorm_fwd_f32: bad shape");
    NVQ_REQUIRE((long)N * S < (1L << 31), "nvq_batchnorm_fwd_f32: more than 2^31 elements per channel");
    if (N == 0) return NVQ_OK;
    NVQ_REQUIRE(d_y && d_x && d_gamma && d_beta && d_running_mean && d_running_var,
                "nvq_batchnorm_fwd_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    BnGeom g{N, C, S, bn_splits(N, C, S, device)};
    dim3 grid(g.P, C);
    cudaStream_t st = (cudaStream_t)stream;
    if (!training) {
        bn_apply_eval_kernel<<<grid, kThreads, 0, st>>>(d_y, d_x, d_gamma, d_beta, d_running_mean,
                                                        d_running_var, g, eps);
        NVQ_LAUNCHED();
        return NVQ_OK;
    }
    NVQ_REQUIRE(d_save_stats && d_scratch, "nvq_batchnorm_fwd_f32: training needs save_stats and scratch");
    const long m = (long)N * S;
    BnFwdArgs a{1.0 - momentum, (float)momentum, (float)eps,
                m > 1 ? (float)((double)m / (double)(m - 1)) : 1.0f};
    bn_stats_partial_kernel<<<grid, kThreads, 0, st>>>(d_scratch, d_x, g);
    NVQ_LAUNCHED();
    bn_apply_train_kernel<<<grid, kThreads, 0, st>>>(d_y, d_x, d_scratch, d_gamma, d_beta,
                                                     d_running_mean, d_running_var, d_save_stats, g, a);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_batchnorm_bwd_f32(float* d_dx, double* d_dgamma, double* d_dbeta, const float* d_grad,
                                 const float* d_x, const float* d_save_stats, const double* d_gamma,
                                 double* d_scratch, int N, int C, int S, double eps, int device,
                                 void* stream) {
    NVQ_REQUIRE(N >= 0 && C > 0 && S > 0, "nvq_batchnorm_bwd_f32: bad shape");
    NVQ_REQUIRE((long)N * S < (1L << 31), "nvq_batchnorm_bwd_f32: more than 2^31 elements per channel");
    if (N == 0) return NVQ_OK;
    NVQ_REQUIRE(d_grad && d_x && d_save_stats && d_gamma && d_scratch,
                "nvq_batchnorm_bwd_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    BnGeom g{N, C, S, bn_splits(N, C, S, device)};
    dim3 grid(g.P, C);
    cudaStream_t st = (cudaStream_t)stream;
    bn_bwd_partial_kernel<<<grid, kThreads, 0, st>>>(d_scratch, d_grad, d_x, d_save_stats, g, (float)eps);
    NVQ_LAUNCHED();
    bn_bwd_apply_kernel<<<grid, kThreads, 0, st>>>(d_dx, d_dgamma, d_dbeta, d_grad, d_x, d_scratch,
                                                   d_save_stats, d_gamma, g, (float)eps);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_maxpool2d_fwd_f32(float* d_out, const float* d_x, int N, int C, int H, int W, int KH,
                                 int KW, int sh, int sw, int ph, int pw, nvq_pad_mode mode,
                                 int device, void* stream) {
    PoolGeom g;
    nvq_status s = pool_geom(g, N, C, H, W, KH, KW, sh, sw, ph, pw, mode, "nvq_maxpool2d_fwd_f32");
    if (s != NVQ_OK) return s;
    size_t total = (size_t)N * C * g.OH * g.OW;
    if (total == 0) return NVQ_OK;
    NVQ_REQUIRE(d_out && d_x, "nvq_maxpool2d_fwd_f32: null buffer");
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    maxpool_fwd_kernel<<<flat_grid(total, device), kThreads, 0, (cudaStream_t)stream>>>(d_out, d_x, g);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_maxpool2d_bwd_f32(float* d_dx, const float* d_grad, const float* d_x, int N, int C,
                                 int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
                                 nvq_pad_mode mode, int device, void* stream) {
    PoolGeom g;
    nvq_status s = pool_geom(g, N, C, H, W, KH, KW, sh, sw, ph, pw, mode, "nvq_maxpool2d_bwd_f32");
    if (s != NVQ_OK) return s;
    size_t total = (size_t)N * C * H * W;
    if (total == 0) return NVQ_OK;
    NVQ_REQUIRE(d_dx && d_grad && d_x, "nvq_maxpool2d_bwd_f32: null buffer");
    s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    maxpool_bwd_kernel<<<flat_grid(total, device), kThreads, 0, (cudaStream_t)stream>>>(d_dx, d_grad,
                                                                                       d_x, g);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_gap2d_fwd_f32(float* d_out, const float* d_x, size_t planes, int S, int device,
                             void* stream) {
    NVQ_REQUIRE(S > 0, "nvq_gap2d_fwd_f32: empty plane");
    if (planes == 0) return NVQ_OK;
    NVQ_REQUIRE(d_out && d_x, "nvq_gap2d_fwd_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    gap_fwd_kernel<<<flat_grid(planes * 32, device), kThreads, 0, (cudaStream_t)stream>>>(d_out, d_x,
                                                                                         planes, S);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_gap2d_bwd_f32(float* d_dx, const float* d_grad, size_t planes, int S, int device,
                             void* stream) {
    NVQ_REQUIRE(S > 0, "nvq_gap2d_bwd_f32: empty plane");
    if (planes == 0) return NVQ_OK;
    NVQ_REQUIRE(d_dx && d_grad, "nvq_gap2d_bwd_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    gap_bwd_kernel<<<flat_grid(planes * S, device), kThreads, 0, (cudaStream_t)stream>>>(
        d_dx, d_grad, planes * S, S, (float)(1.0 / (double)S));
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_dropout_f32(float* d_out, const float* d_x, const float* d_mask, size_t n,
                           float keep_prob, int device, void* stream) {
    NVQ_REQUIRE(keep_prob > 0.f && keep_prob <= 1.f, "nvq_dropout_f32: keep_prob must be in (0, 1]");
    if (n == 0) return NVQ_OK;
    NVQ_REQUIRE(d_out && d_x && d_mask, "nvq_dropout_f32: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    dropout_kernel<<<flat_grid(n, device), kThreads, 0, (cudaStream_t)stream>>>(d_out, d_x, d_mask, n,
                                                                               keep_prob);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

nvq_status nvq_adamw_step_f64(double* d_param, const double* d_grad, double* d_m, double* d_v,
                              size_t n, double beta1, double one_minus_beta1, double beta2,
                              double one_minus_beta2, double bias_corr1, double bias_corr2, double lr,
                              double eps, double lr_times_wd, int apply_decay, int device,
                              void* stream) {
    if (n == 0) return NVQ_OK;
    NVQ_REQUIRE(d_param && d_grad && d_m && d_v, "nvq_adamw_step_f64: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    AdamW64Args a{beta1, one_minus_beta1, beta2, one_minus_beta2, bias_corr1, bias_corr2, lr, eps,
                  lr_times_wd, apply_decay};
    adamw_f64_kernel<<<flat_grid(n, device), kThreads, 0, (cudaStream_t)stream>>>(d_param, d_grad, d_m,
                                                                                 d_v, n, a);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

}  // extern "C"
