// Backward of the quantised-weight Linear on the tensor cores (the rules of Linear.backward,
// novann/layers/linear/linear.py:85-108, with the weight held as FP8 codes):
//   dX = G @ dequant(Wq)        (M x N) . (N x K)
//   dW = G^T @ X                (N x M) . (M x K)   -> fp32, for the master weight
//   db = column sums of G       (fp32, exact order-of-rows sum)
// Both contractions reuse the forward kernel (bf16 operands, K-major, fp32 accumulate, fp32
// output); what differs is how the operands are laid out, so this file only holds the
// transposing converters that produce them:
//   G  fp32 (M x N) -> bf16 (M x N)  and  bf16 G^T (N x M)
//   X  fp32 (M x K) -> bf16 X^T (K x M)
//   Wq codes (N x K) with per-channel scales -> bf16 (K x N) holding bf16(value * s_n): the
//   scale runs along the contraction here, so it has to be folded into the operand.
#include "gemm_common.cuh"

namespace {

// dst (C x R) bf16 = transpose(src (R x C) fp32), 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
transpose_f32_to_bf16_kernel(uint16_t* __restrict__ dst, const float* __restrict__ src, int R, int C) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int r = r0 + ty + 8 * i, c = c0 + tx;
        tile[ty + 8 * i][tx] = (r < R && c < C) ? src[(size_t)r * C + c] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int c = c0 + ty + 8 * i, r = r0 + tx;
        if (c < C && r < R)
            dst[(size_t)c * R + r] = (uint16_t)spec_f32_to_bf16(__float_as_uint(tile[tx][ty + 8 * i]));
    }
}

// dst (K x N) bf16 = bf16(value(code[n, k]) * scale[n])
template <int FMT>
__global__ void __launch_bounds__(256)
expand_transpose_kernel(uint16_t* __restrict__ dst, const uint8_t* __restrict__ codes,
                        const float* __restrict__ scales, int N, int K) {
    __shared__ float tile[32][33];
    const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int n = n0 + ty + 8 * i, k = k0 + tx;
        float v = 0.f;
        if (n < N && k < K)
            v = __fmul_rn(__uint_as_float(spec_fp8_to_f32<FMT>(codes[(size_t)n * K + k])), scales[n]);
        tile[ty + 8 * i][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int k = k0 + ty + 8 * i, n = n0 + tx;
        if (k < K && n < N)
            dst[(size_t)k * N + n] = (uint16_t)spec_f32_to_bf16(__float_as_uint(tile[tx][ty + 8 * i]));
    }
}

__global__ void colsum_rows_kernel(const float* __restrict__ g, float* __restrict__ out, int M, int N) {
    int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float s = 0.f;
    for (int m = 0; m < M; m++) s = __fadd_rn(s, g[(size_t)m * N + n]);
    out[n] = s;
}

size_t align256(size_t b) { return (b + 255) / 256 * 256; }

}  // namespace

extern "C" nvq_status nvq_linear_bwd_q_workspace_bytes(size_t M, size_t N, size_t K, size_t* bytes) {
    NVQ_REQUIRE(bytes, "null out pointer");
    // bf16 G, bf16 G^T, bf16 X^T, bf16 scaled W^T
    *bytes = 2 * align256(M * N * 2) + align256(M * K * 2) + align256(N * K * 2);
    return NVQ_OK;
}

extern "C" nvq_status nvq_linear_bwd_q(float* d_dx, float* d_dw, float* d_db, const float* d_g,
                                       const float* d_x, const uint8_t* d_wq, nvq_dtype w_fmt,
                                       const float* d_w_scales, size_t M, size_t N, size_t K,
                                       void* d_workspace, size_t workspace_bytes, int device,
                                       void* stream) {
    NVQ_REQUIRE(d_g && M > 0 && N > 0 && K > 0, "nvq_linear_bwd_q: bad argument");
    NVQ_REQUIRE(w_fmt == NVQ_E4M3 || w_fmt == NVQ_E5M2, "nvq_linear_bwd_q: weight format must be E4M3 or E5M2");
    NVQ_REQUIRE(M % 8 == 0 && N % 8 == 0 && K % 8 == 0,
                "nvq_linear_bwd_q: M (%zu), N (%zu) and K (%zu) must be multiples of 8", M, N, K);
    size_t need = 0;
    nvq_linear_bwd_q_workspace_bytes(M, N, K, &need);
    NVQ_REQUIRE(d_workspace && workspace_bytes >= need && nvq_aligned(d_workspace, 256),
                "nvq_linear_bwd_q: workspace of %zu bytes (256-byte aligned) required", need);
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    char* ws = (char*)d_workspace;
    uint16_t* gb = (uint16_t*)ws;                          ws += align256(M * N * 2);
    uint16_t* gbt = (uint16_t*)ws;                         ws += align256(M * N * 2);
    uint16_t* xbt = (uint16_t*)ws;                         ws += align256(M * K * 2);
    uint16_t* wdt = (uint16_t*)ws;
    const int Mi = (int)M, Ni = (int)N, Ki = (int)K;
    if (d_db) {
        colsum_rows_kernel<<<(Ni + 127) / 128, 128, 0, st>>>(d_g, d_db, Mi, Ni);
        NVQ_LAUNCHED();
    }
    if (d_dx) {
        NVQ_REQUIRE(d_wq && d_w_scales, "nvq_linear_bwd_q: dX needs the weight codes and scales");
        s = nvq_cast(gb, NVQ_BF16, d_g, NVQ_F32, M * N, device, stream);
        if (s != NVQ_OK) return s;
        dim3 grid((Ki + 31) / 32, (Ni + 31) / 32);
        if (w_fmt == NVQ_E4M3)
            expand_transpose_kernel<NVQ_E4M3><<<grid, 256, 0, st>>>(wdt, d_wq, d_w_scales, Ni, Ki);
        else
            expand_transpose_kernel<NVQ_E5M2><<<grid, 256, 0, st>>>(wdt, d_wq, d_w_scales, Ni, Ki);
        NVQ_LAUNCHED();
        // dX (M x K) = G (M x N) @ (W^T (K x N))^T
        s = nvq_linear_bf16_launch((uint16_t*)d_dx, gb, wdt, nullptr, nullptr, M, K, N, 1, device, st);
        if (s != NVQ_OK) return s;
    }
    if (d_dw) {
        NVQ_REQUIRE(d_x, "nvq_linear_bwd_q: dW needs x");
        dim3 g1((Ni + 31) / 32, (Mi + 31) / 32), g2((Ki + 31) / 32, (Mi + 31) / 32);
        transpose_f32_to_bf16_kernel<<<g1, 256, 0, st>>>(gbt, d_g, Mi, Ni);   // (N x M)
        NVQ_LAUNCHED();
        transpose_f32_to_bf16_kernel<<<g2, 256, 0, st>>>(xbt, d_x, Mi, Ki);   // (K x M)
        NVQ_LAUNCHED();
        // dW (N x K) = G^T (N x M) @ (X^T (K x M))^T
        s = nvq_linear_bf16_launch((uint16_t*)d_dw, gbt, xbt, nullptr, nullptr, N, K, M, 1, device, st);
        if (s != NVQ_OK) return s;
    }
    return NVQ_OK;
}
