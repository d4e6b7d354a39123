/*
 * nvq.h -- C ABI of the B200 (sm_100a) cast / quantise / quantised-GEMM library.
 *
 * NovaNN (the reference framework) is pure Python over NumPy and has no native
 * boundary of its own; what this library replaces are the NumPy calls on its hot
 * path.  Each entry point names the reference call it stands in for as
 * file:line inside the reference project.  The Python package novann_b200 binds
 * these symbols with ctypes and presents the reference's Layer / functional API.
 *
 * Conventions
 *  - every function returns an nvq_status (0 = ok, negative = failure); nothing
 *    throws or aborts.  nvq_last_error() gives a thread-local message.
 *  - all pointers named d_* are DEVICE pointers on `device`; h_* are host pointers.
 *  - compute calls are asynchronous on `stream` (a cudaStream_t passed as void*,
 *    NULL = the default stream of `device`); the caller synchronises.
 *  - the library allocates nothing inside compute calls except where a function
 *    says otherwise; buffers come from nvq_malloc or any other CUDA allocator.
 *  - there is no CPU fallback anywhere: without a CUDA device every call fails.
 */
#ifndef NVQ_H
#define NVQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t nvq_status;
enum {
    NVQ_OK = 0,
    NVQ_ERR_INVALID = -1,     /* bad argument (null, size, alignment, dtype, scale) */
    NVQ_ERR_CUDA = -2,        /* a CUDA runtime / driver call failed */
    NVQ_ERR_UNSUPPORTED = -3, /* valid request this build cannot serve (shape rule) */
    NVQ_ERR_TIMEOUT = -4,     /* a bounded device-side wait gave up (kernel self check) */
    NVQ_ERR_NCCL = -5         /* an NCCL call failed */
};

typedef enum {
    NVQ_F32 = 0,
    NVQ_F16 = 1,
    NVQ_BF16 = 2,
    NVQ_E4M3 = 3,     /* FP8 E4M3 "fn": bias 7, no inf, NaN 0x7f/0xff, max 448 */
    NVQ_E5M2 = 4,     /* FP8 E5M2: bias 15, max finite 57344 */
    NVQ_E2M1_B32 = 5, /* FP4 E2M1, two codes per byte (low nibble first), one fp32
                         scale per 32 consecutive elements of a row */
    NVQ_F64 = 6       /* float64: what NovaNN's BatchNorm emits (float64 gamma / beta) */
} nvq_dtype;

typedef enum {
    NVQ_PAD_ZEROS = 0,
    NVQ_PAD_REFLECT = 1,
    NVQ_PAD_REPLICATE = 2,
    NVQ_PAD_CIRCULAR = 3
} nvq_pad_mode;

/* ---------------------------------------------------------------- runtime */

const char* nvq_last_error(void);
const char* nvq_version(void);
nvq_status nvq_device_count(int* count);
/* SM count and total memory of a device (grid sizing / shard sizing). */
nvq_status nvq_device_info(int device, int* sm_count, size_t* total_bytes, int* cc_major,
                           int* cc_minor);
/* Frees what the library allocated lazily on every device: the staging buffers and streams of
 * the host-array calls (nvq_cast_host), and the words behind nvq_device_error_flag.  Buffers,
 * streams, events, graphs and communicators handed to the caller stay the caller's to free.
 * No other call of the library may be in flight; later calls allocate again on demand. */
nvq_status nvq_shutdown(void);

nvq_status nvq_malloc(int device, size_t bytes, void** d_ptr);
nvq_status nvq_free(int device, void* d_ptr);
nvq_status nvq_host_alloc(size_t bytes, void** h_ptr); /* pinned */
nvq_status nvq_host_free(void* h_ptr);
nvq_status nvq_memcpy_h2d(void* d_dst, const void* h_src, size_t bytes, int device, void* stream);
nvq_status nvq_memcpy_d2h(void* h_dst, const void* d_src, size_t bytes, int device, void* stream);
nvq_status nvq_memcpy_d2d(void* d_dst, const void* d_src, size_t bytes, int device, void* stream);
nvq_status nvq_memset(void* d_dst, int value, size_t bytes, int device, void* stream);

nvq_status nvq_stream_create(int device, void** stream);
nvq_status nvq_stream_destroy(int device, void* stream);
nvq_status nvq_stream_sync(int device, void* stream);
nvq_status nvq_device_sync(int device);
nvq_status nvq_event_create(int device, void** event);
nvq_status nvq_event_destroy(int device, void* event);
nvq_status nvq_event_record(int device, void* event, void* stream);
/* work enqueued on `stream` after this call waits for what `event` recorded (also inside a stream
 * capture, where it forks / joins branches of the graph) */
nvq_status nvq_stream_wait_event(int device, void* stream, void* event);
nvq_status nvq_event_sync(int device, void* event);
nvq_status nvq_event_elapsed_ms(void* start, void* stop, float* ms);

/* CUDA graphs for launch-bound sequences (the fp32 train step is ~13 small kernels): every
 * compute call of this library may be captured once it has run at least once on the device
 * (first calls query attributes).  nvq_launch_count() counts launches at capture time only. */
nvq_status nvq_graph_begin_capture(int device, void* stream);
nvq_status nvq_graph_end_capture(int device, void* stream, void** graph_exec);
nvq_status nvq_graph_launch(int device, void* graph_exec, void* stream);
nvq_status nvq_graph_destroy(int device, void* graph_exec);

/* Number of kernels this library has launched in the calling process so far. */
uint64_t nvq_launch_count(void);

/* ---------------------------------------------------------------- casts
 * Replaces ndarray.astype at novann/layers/linear/linear.py:81,96 and
 * novann/layers/convolutional/conv2d.py:159,188 (NumPy round-to-nearest-even
 * narrowing, overflow to +-inf, exact widening), extended to bf16.
 *   f32->f16: bit-identical to NumPy astype(float16), NaN payload rule included.
 *   f32->bf16: RNE, any NaN -> sign|0x7fc0.   f16/bf16->f32: exact.
 *   f64->f32 (the narrowing NovaNN really performs, on BatchNorm's float64 output):
 *   bit-identical to NumPy astype(float32): RNE, overflow to +-inf, subnormal results kept,
 *   NaN -> sign | 0x7fc00000 | (payload >> 29).   f32->f64: exact, NaN quiet with its
 *   payload shifted left 29.
 * Supported pairs: {f32}<->{f16,bf16,f64}.  n elements, any alignment (pointers aligned to
 * 16 bytes on the narrow side and 32 on the wide side take the vectorised path).
 */
nvq_status nvq_cast(void* d_dst, nvq_dtype dst_dtype, const void* d_src, nvq_dtype src_dtype,
                    size_t n, int device, void* stream);

/* Host-buffer variant of nvq_cast: h_src/h_dst are host arrays; the data is streamed through
 * device staging buffers in chunks with H2D, kernel and D2H overlapped.  Page-locked arrays
 * (nvq_host_alloc) move at full PCIe rate; plain (pageable) arrays of 8 MiB and more are
 * staged through page-locked buffers of the library by a few host threads (about half that
 * rate, three times what the driver's own handling of pageable copies gives).  Synchronous.  This is the call that
 * sits exactly where ndarray.astype sat (host array in, host array out).  The staging
 * buffers (6 x 64 MiB per device, and as much page-locked host memory once a pageable array
 * was seen) are allocated by the first call on a device and kept
 * until nvq_shutdown; calls on one device are serialised, calls on different devices
 * run concurrently. */
nvq_status nvq_cast_host(void* h_dst, nvq_dtype dst_dtype, const void* h_src,
                         nvq_dtype src_dtype, size_t n, int device);

/* ---------------------------------------------------------------- FP8, per tensor
 * No reference counterpart (NovaNN has no quantisation); semantics follow the
 * written rules: amax exact with NaNs ignored; scale = amax/FMAX and
 * inv_scale = FMAX/amax, one fp32 division each (both 1 when amax == 0);
 * q = cvt_sat_rne(x * inv_scale) with one fp32 multiply; x' = float(q) * scale.
 */
/* *d_amax = max|x| (fp32).  d_amax is written, not accumulated. */
nvq_status nvq_amax_f32(const float* d_src, size_t n, float* d_amax, int device, void* stream);
/* fmt = NVQ_E4M3 or NVQ_E5M2; inv_scale must be finite and > 0. */
nvq_status nvq_quantize_fp8(uint8_t* d_dst, const float* d_src, size_t n, nvq_dtype fmt,
                            float inv_scale, int device, void* stream);
nvq_status nvq_dequantize_fp8(float* d_dst, const uint8_t* d_src, size_t n, nvq_dtype fmt,
                              float scale, int device, void* stream);
/* amax + scale computation + quantise without a host round trip.
 * d_amax_scale_inv: 3 floats written {amax, scale, inv_scale}.  If d_amax_in is not
 * NULL it holds an already combined amax (e.g. the max over all row shards) and the
 * reduction over d_src is skipped. */
nvq_status nvq_quantize_fp8_tensor(uint8_t* d_dst, float* d_amax_scale_inv, const float* d_src,
                                   size_t n, nvq_dtype fmt, const float* d_amax_in, int device,
                                   void* stream);

/* Per-row (per output channel) quantisation of a rows x cols fp32 weight matrix:
 * d_scales[r] = amax_r / FMAX (1 for an all-zero row); codes = cvt_sat_rne(w * (FMAX/amax_r)). */
nvq_status nvq_quantize_fp8_rows(uint8_t* d_dst, float* d_scales, const float* d_src, size_t rows,
                                 size_t cols, nvq_dtype fmt, int device, void* stream);

/* ---------------------------------------------------------------- FP4 E2M1, block 32
 * No reference counterpart.  rows x cols bf16, cols % 32 == 0.
 * d_packed: rows x cols/2 bytes; d_scales: rows x cols/32 fp32.
 */
nvq_status nvq_quantize_fp4_b32(uint8_t* d_packed, float* d_scales, const uint16_t* d_src_bf16,
                                size_t rows, size_t cols, int device, void* stream);
nvq_status nvq_dequantize_fp4_b32(uint16_t* d_dst_bf16, const uint8_t* d_packed,
                                  const float* d_scales, size_t rows, size_t cols, int device,
                                  void* stream);

/* ---------------------------------------------------------------- quantised Linear
 * Replaces F.linear, novann/functional.py:147-163 (out = input @ weight.T; out +=
 * bias) for a weight stored as FP8 / FP4 codes:
 *   Y[m,n] = bf16_rne( s_n * sum_k X[m,k] * dequant(Wq[n,k]) + b_n )
 * X: M x K bf16 row-major.  Wq: N x K codes.  E4M3 / E5M2: one byte per weight and
 * d_w_scales holds N per-output-channel fp32 scales.  E2M1_B32: N x K/2 packed bytes
 * and d_w_scales holds N x K/32 block scales (K % 32 == 0).  d_bias: N fp32 or NULL.
 * Y: M x N bf16, 32-byte aligned.  K % 8 == 0, N % 8 == 0; M, N, K tails are handled.
 * fp32 accumulation on the tcgen05 tensor cores.
 * d_workspace: scratch of nvq_linear_workspace_bytes(N, K, fmt) bytes (32-byte
 * aligned) that receives the weight expanded to 16-bit tensor-core operands; it is
 * rewritten by every call, so calls that share a workspace must be stream ordered.
 * d_workspace may be NULL for E4M3 / E5M2 weights when M > 128 and K % 16 == 0: the
 * codes are then expanded inside the GEMM kernel, in shared memory (slower than the
 * workspace form on large problems, but nothing is written to HBM).
 * M <= 128 (few rows): the weight is read once, as codes, and the workspace holds
 * partial sums instead.  FP8 codes are then the tensor cores' operand as they are
 * (kind::f8f6f4) and each activation row is carried as two rows of E4M3 codes,
 * x = a_m * (p1 + p2 / 16) with a_m a power of two: exact for every element down to
 * 2^-13 of its row's largest, an absolute error <= 2^-21 of the row's largest below
 * that; a non-finite activation makes its output row NaN, and an E5M2 infinity code
 * in the weight gives NaN (the quantiser never emits one).  A caller that needs the bf16
 * activations taken as they are passes NVQ_LINEAR_BF16_ACTIVATIONS to nvq_linear_fwd_opts:
 * the kernel that expands the codes to bf16 in shared memory then runs (also the FP4 path).
 */
nvq_status nvq_linear_workspace_bytes(size_t N, size_t K, nvq_dtype w_fmt, size_t* bytes);
nvq_status nvq_linear_fwd(uint16_t* d_y_bf16, const uint16_t* d_x_bf16, const uint8_t* d_wq,
                          nvq_dtype w_fmt, const float* d_w_scales, const float* d_bias,
                          size_t M, size_t N, size_t K, void* d_workspace, size_t workspace_bytes,
                          int device, void* stream);
/* nvq_linear_fwd with the kernel path chosen by the caller instead of by the shape rules above.
 * `path` is NVQ_LINEAR_AUTO (= nvq_linear_fwd), NVQ_LINEAR_BF16_ACTIVATIONS or
 * NVQ_LINEAR_CLUSTER_REDUCE, optionally or-ed with at most one of the three kernel selectors.  A kernel selector switches the
 * few-rows kernels off; NVQ_LINEAR_EXPAND_IN_KERNEL falls back to the expansion pass where the
 * in-kernel form does not apply (FP4 weights, M <= 128, K % 16 != 0). */
enum {
    NVQ_LINEAR_AUTO = 0,
    NVQ_LINEAR_BF16_ACTIVATIONS = 1 << 0, /* M <= 128: no two-piece E4M3 carrier for the activations */
    NVQ_LINEAR_EXPAND_IN_KERNEL = 1 << 1, /* FP8 codes expanded in shared memory, nothing written to HBM */
    NVQ_LINEAR_SINGLE_CTA = 1 << 2,       /* expansion pass + one CTA per 128 x 256 tile */
    NVQ_LINEAR_CTA_PAIR = 1 << 3,         /* expansion pass + CTA pair per 256 x 256 tile */
    NVQ_LINEAR_CODES_FINITE = 1 << 5,     /* the caller vouches that no weight code is NaN or inf (true of
                                             every code nvq_quantize_fp8_rows makes from finite weights):
                                             the in-kernel expansion leaves its test for such codes out;
                                             a NaN / inf code would then expand to the finite value its
                                             bits spell */
    NVQ_LINEAR_CLUSTER_REDUCE = 1 << 4    /* M <= 32, FP8 codes, a weight that one wave of thread-block
                                             clusters covers: the CTAs of a cluster split K and add
                                             their partial sums through distributed shared memory
                                             (two kernels, nothing through HBM) instead of the
                                             split / stream / reduce kernels; same carrier, same
                                             scales; measured no faster, so not the default */
};
nvq_status nvq_linear_fwd_opts(uint16_t* d_y_bf16, const uint16_t* d_x_bf16, const uint8_t* d_wq,
                               nvq_dtype w_fmt, const float* d_w_scales, const float* d_bias,
                               size_t M, size_t N, size_t K, void* d_workspace,
                               size_t workspace_bytes, uint32_t path, int device, void* stream);
/* W8A8 VARIANT (outside the 1e-2 parity bound; offered for throughput, labelled as such):
 * the bf16 activations are quantised to E4M3 per row (scale_m = amax_m / 448) inside the call and
 * the contraction runs as FP8 x FP8 (tcgen05 kind::f8f6f4), Y = bf16(sx_m * sw_n * sum + b_n).
 * E4M3 weights only.  K % 16 == 0, N % 8 == 0.  Workspace: nvq_linear_w8a8_workspace_bytes(M, K)
 * bytes, 256-byte aligned (activation codes and row scales). */
nvq_status nvq_linear_w8a8_workspace_bytes(size_t M, size_t K, size_t* bytes);
nvq_status nvq_linear_fwd_w8a8(uint16_t* d_y_bf16, const uint16_t* d_x_bf16, const uint8_t* d_wq,
                               const float* d_w_scales, const float* d_bias, size_t M, size_t N,
                               size_t K, void* d_workspace, size_t workspace_bytes, int device,
                               void* stream);

/* Backward of the quantised-weight Linear on the tensor cores (Linear.backward,
 * novann/layers/linear/linear.py:85-108, with the weight held as FP8 codes):
 *   dX (M x K fp32) = bf16(G) @ bf16(dequant(Wq) * s)      G: M x N fp32 gradient of the output
 *   dW (N x K fp32) = bf16(G)^T @ bf16(X)                  X: M x K fp32 forward input
 *   db (N fp32)     = column sums of G, rows added in order
 * bf16 operands, fp32 accumulation and fp32 results; any of d_dx, d_dw, d_db may be NULL.
 * M, N, K multiples of 8.  d_workspace: nvq_linear_bwd_q_workspace_bytes bytes, 256-byte
 * aligned (bf16 copies / transposes of G, X and the scaled weight). */
nvq_status nvq_linear_bwd_q_workspace_bytes(size_t M, size_t N, size_t K, size_t* bytes);
nvq_status nvq_linear_bwd_q(float* d_dx, float* d_dw, float* d_db, const float* d_g,
                            const float* d_x, const uint8_t* d_wq, nvq_dtype w_fmt,
                            const float* d_w_scales, size_t M, size_t N, size_t K,
                            void* d_workspace, size_t workspace_bytes, int device, void* stream);

/* Allocation-free form of nvq_linear_fwd.  It has no counterpart in the reference.
 *
 * Some hosts of this library may not allocate device memory at the point where they need a
 * Linear: code running between the capture-safe phases of a serving loop, plugins that were
 * handed a fixed memory budget by their framework and must not grow it, and runtimes in which
 * cudaMalloc would synchronise the whole device in the middle of a latency-critical step.  For
 * them the scratch that receives the expanded weight is an array compiled into the library:
 * NVQ_STATIC_WORKSPACE_BYTES bytes per GPU that loads the library, held until the process exits.
 * The call allocates nothing (no cudaMalloc / cudaFree / cudaHostAlloc, no allocating library
 * routine) and takes the same inputs and outputs as nvq_linear_fwd, minus the workspace.
 *
 *  - Limit: N * K * 2 <= NVQ_STATIC_WORKSPACE_BYTES (N * K <= 4 Mi weights, e.g. 2048 x 2048);
 *    larger weights are rejected with NVQ_ERR_INVALID and a message naming the limit.
 *  - The first call on each device looks up the array's address on that device (a host-side
 *    query, no allocation).  Make that first call before any stream capture begins.
 *  - For M <= 128 the array holds what the few-rows kernels keep in a workspace instead of an
 *    expanded weight: fp32 partial sums, the activations' E4M3 codes and their row scales;
 *    a problem whose partial sums do not fit takes the expanded-weight path.
 *  - Every call on a device shares the one array, and it keeps the previous call's contents.
 *    Each call rewrites every byte it later reads, so nothing needs clearing, but two calls
 *    that overlap on the GPU (different streams, or threads racing on one device) corrupt each
 *    other: order them on one stream.
 *  - d_status: optional device word (may be NULL) that receives a non-zero code if a bounded
 *    device-side wait gave up; the caller zeroes it.  (nvq_device_error_flag does not cover
 *    this entry point, because its word is allocated on first use.)
 */
#define NVQ_STATIC_WORKSPACE_BYTES (8u << 20)
nvq_status nvq_linear_fwd_static(uint16_t* d_y_bf16, const uint16_t* d_x_bf16, const uint8_t* d_wq,
                                 nvq_dtype w_fmt, const float* d_w_scales, const float* d_bias,
                                 size_t M, size_t N, size_t K, int* d_status, int device,
                                 void* stream);

/* The two halves of nvq_linear_fwd, for callers whose weight codes stay unchanged over many
 * calls (inference, or several forwards between optimiser steps) and who can afford 2 bytes per
 * weight: expand once, then run the contraction alone.
 *   nvq_linear_expand_weight: Wd (N x K bf16, 32-byte aligned) = exact value of every E4M3 / E5M2
 *     code (d_w_scales unused), or bf16(value * block scale) for E2M1_B32.
 *   nvq_linear_fwd_expanded: Y = bf16(act(s_n * X @ Wd^T + b_n)); d_chan_scales = the N per-channel
 *     scales for FP8 weights, NULL for an E2M1_B32 weight (scales already folded in); relu != 0
 *     fuses F.relu (novann/functional.py:8-22: v * (v > 0)) into the epilogue before rounding. */
nvq_status nvq_linear_expand_weight(uint16_t* d_wd_bf16, const uint8_t* d_wq, nvq_dtype w_fmt,
                                    const float* d_w_scales, size_t N, size_t K, int device,
                                    void* stream);
nvq_status nvq_linear_fwd_expanded(uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                   const uint16_t* d_wd_bf16, const float* d_chan_scales,
                                   const float* d_bias, size_t M, size_t N, size_t K, int relu,
                                   int device, void* stream);

/* The same, with the expanded copy owned by a handle.  nvq_linear_cache_create allocates the
 * N x K bf16 copy (nvq_linear_workspace_bytes) on `device`; nvq_linear_cache_fwd expands the codes
 * only when (d_wq, d_w_scales, version) differ from what the copy was made from, then runs the
 * contraction alone.  The caller bumps `version` whenever it rewrites the codes in place (a
 * quantised layer does after every optimiser step); *expanded (may be NULL) reports whether this
 * call ran the expansion pass.  M <= 128 without relu runs the few-rows kernels of nvq_linear_fwd
 * on the codes (the buffer then holds partial sums and the next larger call expands again).
 * Calls on one handle must be stream ordered.  With relu == 0 results equal nvq_linear_fwd's bit
 * for bit. */
typedef struct nvq_linear_cache nvq_linear_cache;
nvq_status nvq_linear_cache_create(nvq_linear_cache** out, size_t N, size_t K, nvq_dtype w_fmt, int device);
nvq_status nvq_linear_cache_fwd(nvq_linear_cache* cache, uint16_t* d_y_bf16, const uint16_t* d_x_bf16,
                                const uint8_t* d_wq, const float* d_w_scales, const float* d_bias,
                                size_t M, uint64_t version, int relu, int* expanded, void* stream);
nvq_status nvq_linear_cache_destroy(nvq_linear_cache* cache);

/* Tensor-core kernels bound every device-side wait; a wait that gives up records a
 * non-zero code here (read and cleared by this call) instead of hanging. */
nvq_status nvq_device_error_flag(int device, int* flag);
/* Launches a one-warp kernel that waits (limit 1 ms) on a barrier nothing arrives at: the wait
 * gives up, the kernel returns, and nvq_device_error_flag then reports code 99.  A check of the
 * give-up path that faults and hangs nothing. */
nvq_status nvq_selftest_bounded_wait(int device, void* stream);

/* ---------------------------------------------------------------- fp32 train step
 * The pieces of the reference's training step (novann/utils/train/train.py:60-75) in fp32
 * on the CUDA cores (no tensor cores: results differ from NumPy's sgemm only by summation
 * order; elementwise steps round exactly as NumPy does).
 */
/* F.linear (novann/functional.py:147-163): Y = X @ W^T + b; X MxK, W NxK, b N or NULL.
 * relu != 0 additionally applies F.relu (novann/functional.py:8-22): mask = (Y > 0),
 * Y = Y * mask; d_mask (MxN, may be NULL) receives the mask. */
nvq_status nvq_linear_fwd_f32(float* d_y, const float* d_x, const float* d_w, const float* d_bias,
                              int M, int N, int K, int relu, float* d_mask, int device,
                              void* stream);
/* Linear.backward (novann/layers/linear/linear.py:85-108): dW = G^T @ X (assigned, NxK),
 * db = sum over rows of G (N), dX = G @ W (MxK).  Any of d_dw, d_db, d_dx may be NULL.  If
 * d_mask (MxK) is not NULL, dX is multiplied by it (ReLU.backward,
 * novann/layers/activations/relu.py:36-45). */
nvq_status nvq_linear_bwd_f32(float* d_dw, float* d_db, float* d_dx, const float* d_g,
                              const float* d_x, const float* d_w, const float* d_mask, int M,
                              int N, int K, int device, void* stream);
/* F.relu (novann/functional.py:8-22): mask = (x > 0) as fp32, out = x * mask. */
nvq_status nvq_relu_fwd_f32(float* d_out, float* d_mask, const float* d_x, size_t n, int device,
                            void* stream);
/* ReLU.backward (novann/layers/activations/relu.py:36-45): out = grad * mask, elementwise. */
nvq_status nvq_mul_f32(float* d_out, const float* d_a, const float* d_b, size_t n, int device,
                       void* stream);
/* CrossEntropyLoss (novann/losses/loss_functions.py:29-75): d_yhat (MxC) = softmax(logits,
 * axis 1); grad = float32((double(y_hat) - onehot) / M); *d_loss (may be NULL) = the value the
 * reference reports, i.e. softmax applied a second time along the batch axis inside
 * F.cross_entropy (novann/functional.py:108-128), eps 1e-8.  labels int32 in [0, C). */
nvq_status nvq_softmax_ce_f32(float* d_grad, float* d_loss, const float* d_logits,
                              const int32_t* d_labels, float* d_yhat, int M, int C, int device,
                              void* stream);
/* The loss value alone, from the y_hat that nvq_softmax_ce_f32 left in d_yhat (call that one with
 * d_loss = NULL): nothing in a training step depends on the number, so a step can run this beside
 * its backward pass.  Same arithmetic, same bits as the one-call form. */
nvq_status nvq_ce_loss_f32(float* d_loss, const float* d_yhat, const int32_t* d_labels, int M, int C,
                           int device, void* stream);
/* SGD.step, vanilla path (novann/optim/sgd.py:58-82): p = p - lr * (g * grad_scale), each
 * product and the subtraction rounded separately (grad_scale == 1 skips its multiply). */
nvq_status nvq_sgd_step_f32(float* d_param, const float* d_grad, size_t n, float lr,
                            float grad_scale, int device, void* stream);

/* AdamW.step (novann/optim/adamw.py:41-65) on one tensor, in place on p, m, v:
 *   m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;  p -= lr*(m/bc1) / (sqrt(v/bc2) + eps);
 *   if apply_decay: p -= (lr*wd) * p.   bc1 = 1 - b1^t, bc2 = 1 - b2^t.
 * The caller passes the derived scalars already rounded to fp32 (as NumPy rounds the Python
 * floats); every operation is a separately rounded fp32 operation, so results are bit-exact. */
nvq_status nvq_adamw_step_f32(float* d_param, const float* d_grad, float* d_m, float* d_v, size_t n,
                              float beta1, float one_minus_beta1, float beta2, float one_minus_beta2,
                              float bias_corr1, float bias_corr2, float lr, float eps,
                              float lr_times_wd, int apply_decay, int device, void* stream);

/* ---------------------------------------------------------------- Conv2d forward
 * Replaces F.conv2d, novann/functional.py:275-385: pad (zeros / reflect / replicate /
 * circular = np.pad constant / reflect / edge / wrap) -> im2col with rows ordered (c,kh,kw)
 * and columns (n,oh,ow) -> w_col @ col + bias -> (N,Cout,OH,OW).
 */
/* _calc_out_size (novann/functional.py:319-323) */
nvq_status nvq_conv2d_out_size(int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
                               int* OH, int* OW);
/* _im2col (novann/functional.py:346-368): d_col is (C*KH*KW) x (N*OH*OW) fp32, row-major. */
nvq_status nvq_im2col_f32(float* d_col, const float* d_x, int N, int C, int H, int W, int KH,
                          int KW, int sh, int sw, int ph, int pw, nvq_pad_mode mode, int device,
                          void* stream);
/* fp32 convolution forward: x NCHW, w (Cout,C,KH,KW), bias Cout or NULL, out NCHW contiguous.
 * d_col: scratch of C*KH*KW*N*OH*OW floats (the reference's `col`, kept for backward). */
nvq_status nvq_conv2d_fwd_f32(float* d_out, const float* d_x, const float* d_w,
                              const float* d_bias, float* d_col, int N, int C, int H, int W,
                              int Cout, int KH, int KW, int sh, int sw, int ph, int pw,
                              nvq_pad_mode mode, int device, void* stream);
/* Conv2d.backward (novann/layers/convolutional/conv2d.py:179-207, _col2im :117-148):
 * dW (Cout,C,KH,KW) = g_r @ col^T, db (Cout) = row sums of g_r, dX (N,C,H,W) = col2im(w_col^T @ g_r)
 * with g_r = grad.transpose(1,0,2,3).reshape(Cout,-1).  d_col is the im2col matrix of the forward
 * pass.  Scratch: d_gr Cout*N*OH*OW floats, d_dcol C*KH*KW*N*OH*OW floats (it also holds the
 * partial sums of the split-k weight-gradient GEMM; it may be NULL when d_dx is NULL, at the
 * price of an unsplit dW contraction).  Any of d_dw, d_db, d_dx may be NULL.  As in the reference, gradient falling on padding is dropped for every padding mode. */
nvq_status nvq_conv2d_bwd_f32(float* d_dw, float* d_db, float* d_dx, const float* d_grad,
                              const float* d_col, const float* d_w, float* d_gr, float* d_dcol,
                              int N, int C, int H, int W, int Cout, int KH, int KW, int sh, int sw,
                              int ph, int pw, int device, void* stream);
/* Quantised-weight convolution forward on the tensor cores; Wq holds the codes of
 * w.reshape(Cout, C*KH*KW) zero padded to kpad columns: E4M3 / E5M2 - Cout x kpad bytes, kpad =
 * C*KH*KW rounded up to 16 (nvq_conv2d_q_sizes), Cout per-channel scales; E2M1_B32 - Cout x kpad/2
 * packed bytes, kpad rounded up to 32, scales Cout x kpad/32 (the layout of nvq_quantize_fp4_b32).
 * out is fp32 NCHW holding the bf16-rounded results.  Cout % 8 == 0.
 *   Strides 1 or 2, zero padding, C % 64 == 0, OW * stride <= 256: implicit GEMM.  x is rewritten as bf16 NHWC
 *   (into d_col_bf16), the codes are expanded with their columns reordered to (kh, kw, c) (into
 *   d_workspace), and a tcgen05 kernel gathers the input operand with one 4-D TMA box per
 *   filter tap and 64-channel block (padding = out-of-range box = zeros, stride = the tensor
 *   map's traversal stride) and writes NCHW fp32 from its epilogue (TMA stores where planes
 *   and tiles are multiples of four positions).  No patch matrix exists.
 *   Otherwise: patches of x are gathered (padding mode applied) and rounded to bf16 into
 *   d_col_bf16 (rows x kpad, rows = N*OH*OW), the contraction is nvq_linear_fwd, and d_y_bf16
 *   (rows x Cout) is transposed to NCHW.
 * Scratch for either path: d_col_bf16 rows*kpad uint16, d_y_bf16 rows*Cout uint16, d_workspace
 * as for nvq_linear_fwd with N=Cout, K=kpad. */
nvq_status nvq_conv2d_q_sizes(int N, int C, int H, int W, int Cout, int KH, int KW, int sh, int sw,
                              int ph, int pw, size_t* rows, size_t* kpad);
nvq_status nvq_conv2d_fwd_q(float* d_out, const float* d_x, const uint8_t* d_wq, nvq_dtype w_fmt,
                            const float* d_w_scales, const float* d_bias, uint16_t* d_col_bf16,
                            uint16_t* d_y_bf16, void* d_workspace, size_t workspace_bytes, int N,
                            int C, int H, int W, int Cout, int KH, int KW, int sh, int sw, int ph,
                            int pw, nvq_pad_mode mode, int device, void* stream);

/* nvq_conv2d_fwd_q with the path chosen by the caller: NVQ_CONV_AUTO (= nvq_conv2d_fwd_q),
 * NVQ_CONV_PATCH_MATRIX (always gather patches and run nvq_linear_fwd) or NVQ_CONV_CTA_PAIR
 * (implicit GEMM on the CTA-pair kernel where the shape allows an implicit GEMM at all). */
enum { NVQ_CONV_AUTO = 0, NVQ_CONV_PATCH_MATRIX = 1, NVQ_CONV_CTA_PAIR = 2 };
nvq_status nvq_conv2d_fwd_q_opts(float* d_out, const float* d_x, const uint8_t* d_wq,
                                 nvq_dtype w_fmt, const float* d_w_scales, const float* d_bias,
                                 uint16_t* d_col_bf16, uint16_t* d_y_bf16, void* d_workspace,
                                 size_t workspace_bytes, int N, int C, int H, int W, int Cout,
                                 int KH, int KW, int sh, int sw, int ph, int pw, nvq_pad_mode mode,
                                 uint32_t path, int device, void* stream);

/* Quantised convolution between chained quantised layers: the activations stay in HBM as bf16
 * NHWC ((N*H*W) x C, channels contiguous), which is the tensor cores' operand layout, so the
 * per-call layout pass of nvq_conv2d_fwd_q and the fp32 NCHW output (four times the bytes) are
 * gone.  Same contraction as F.conv2d (novann/functional.py:275-385) with zero padding:
 *   out[(n, oh, ow), co] = bf16( act( s_co * sum x[n, oh*sh+kh-ph, ow*sw+kw-pw, c] * dequant(Wq)[co, (c,kh,kw)] + b_co ) )
 * act = F.relu's v * (v > 0) when relu != 0 (novann/functional.py:8-22), identity otherwise.
 * Wq / scales as for nvq_conv2d_fwd_q.  Strides 1 or 2, C % 64 == 0, OW * stride <= 256,
 * Cout % 8 == 0; other shapes return NVQ_ERR_UNSUPPORTED (use nvq_conv2d_fwd_q).
 * d_workspace: Cout * C * KH * KW * 2 bytes (the tap-ordered expanded weight), 16-byte aligned.
 * The two converters sit at the ends of such a chain (S = H * W; C % 64 == 0 for the first,
 * C % 8 == 0 for the second). */
nvq_status nvq_conv2d_fwd_q_nhwc(uint16_t* d_out_bf16, const uint16_t* d_x_bf16, const uint8_t* d_wq,
                                 nvq_dtype w_fmt, const float* d_w_scales, const float* d_bias,
                                 void* d_workspace, size_t workspace_bytes, int N, int C, int H, int W,
                                 int Cout, int KH, int KW, int sh, int sw, int ph, int pw, int relu,
                                 int device, void* stream);
nvq_status nvq_nchw_f32_to_nhwc_bf16(uint16_t* d_dst, const float* d_src, int N, int C, int S,
                                     int device, void* stream);
nvq_status nvq_nhwc_bf16_to_nchw_f32(float* d_dst, const uint16_t* d_src, int N, int C, int S,
                                     int device, void* stream);

/* ---------------------------------------------------------------- BatchNorm, pooling, Dropout
 * The layers either side of the GEMMs in NovaNN's CNN.  Activations are fp32 (N, C, S)
 * row-major with S = H*W (BatchNorm2d), the sequence length (BatchNorm1d, 3-D input) or 1
 * (BatchNorm1d, 2-D input).  NovaNN keeps gamma, beta and the running statistics as float64
 * arrays, so they are float64 here; the fp32 output is the value every consumer in NovaNN
 * obtains with astype(np.float32) from the float64 result.  Batch statistics are summed in
 * float64, so they match NumPy's fp32 pairwise sums to rounding, not bit for bit.
 */
/* Bytes of float64 scratch the two BatchNorm calls need for C channels. */
size_t nvq_batchnorm_scratch_bytes(int C);
/* BatchNorm2d.forward (novann/layers/batchnorm/batchnorm2d.py:57-102) and BatchNorm1d.forward
 * (batchnorm1d.py:96-141).  training != 0: batch mean and Bessel-corrected variance, running
 * statistics updated in place, d_save_stats (2*C floats: mean, variance) kept for backward.
 * training == 0: running statistics, float64 arithmetic; d_save_stats / d_scratch unused. */
nvq_status nvq_batchnorm_fwd_f32(float* d_y, const float* d_x, const double* d_gamma,
                                 const double* d_beta, double* d_running_mean,
                                 double* d_running_var, float* d_save_stats, double* d_scratch,
                                 int N, int C, int S, double momentum, double eps, int training,
                                 int device, void* stream);
/* BatchNorm2d.backward (batchnorm2d.py:104-146) / BatchNorm1d.backward: d_dgamma, d_dbeta
 * (C float64 each; either may be NULL) and d_dx (may be NULL) from the forward input d_x and the
 * statistics saved by the training forward. */
nvq_status nvq_batchnorm_bwd_f32(float* d_dx, double* d_dgamma, double* d_dbeta, const float* d_grad,
                                 const float* d_x, const float* d_save_stats, const double* d_gamma,
                                 double* d_scratch, int N, int C, int S, double eps, int device,
                                 void* stream);
/* F.max_pool2d (novann/functional.py:450-536): pad (np.pad modes; zero padding takes part in the
 * maximum), windows KHxKW at stride (sh, sw), np.max per window.  out is (N, C, OH, OW). */
nvq_status nvq_maxpool2d_fwd_f32(float* d_out, const float* d_x, int N, int C, int H, int W, int KH,
                                 int KW, int sh, int sw, int ph, int pw, nvq_pad_mode mode,
                                 int device, void* stream);
/* MaxPool2d.backward (novann/layers/pooling/maxpool/maxpool2d.py backward): the gradient of a
 * window is split evenly over the entries equal to its maximum, windows are added in (oh, ow)
 * order, gradient on padding is dropped.  Bit-exact with the reference. */
nvq_status nvq_maxpool2d_bwd_f32(float* d_dx, const float* d_grad, const float* d_x, int N, int C,
                                 int H, int W, int KH, int KW, int sh, int sw, int ph, int pw,
                                 nvq_pad_mode mode, int device, void* stream);
/* F.avg_pool2d (novann/functional.py:550-559): mean over each of `planes` = N*C planes of S
 * elements; GlobalAvgPool2d.backward (novann/layers/pooling/gap/gap2d.py backward):
 * dx = ones * (grad * float32(1/S)). */
nvq_status nvq_gap2d_fwd_f32(float* d_out, const float* d_x, size_t planes, int S, int device,
                             void* stream);
nvq_status nvq_gap2d_bwd_f32(float* d_dx, const float* d_grad, size_t planes, int S, int device,
                             void* stream);
/* Dropout.forward / backward (novann/layers/regularization/dropout.py:40-70):
 * out = (x * mask) / keep_prob with the 0/1 mask drawn by the caller (the reference draws it
 * from NumPy's global generator, which only the host can reproduce). */
nvq_status nvq_dropout_f32(float* d_out, const float* d_x, const float* d_mask, size_t n,
                           float keep_prob, int device, void* stream);
/* AdamW.step (novann/optim/adamw.py:41-65) on a float64 tensor (BatchNorm's gamma / beta);
 * same operation order as nvq_adamw_step_f32, in float64. */
nvq_status nvq_adamw_step_f64(double* d_param, const double* d_grad, double* d_m, double* d_v,
                              size_t n, double beta1, double one_minus_beta1, double beta2,
                              double one_minus_beta2, double bias_corr1, double bias_corr2, double lr,
                              double eps, double lr_times_wd, int apply_decay, int device,
                              void* stream);

/* ---------------------------------------------------------------- data-parallel step
 * NCCL communicator for the gradient all-reduce of the data-parallel training step (no
 * reference counterpart: NovaNN is single process).  One process per GPU; rank 0 makes the
 * unique id and hands it to the others over the launcher's side channel.
 */
#define NVQ_UNIQUE_ID_BYTES 128
nvq_status nvq_comm_unique_id(uint8_t id[NVQ_UNIQUE_ID_BYTES]);
nvq_status nvq_comm_init(const uint8_t id[NVQ_UNIQUE_ID_BYTES], int rank, int world, int device,
                         void** comm);
nvq_status nvq_comm_destroy(void* comm);
/* in-place sum over ranks of an fp32 bucket */
nvq_status nvq_allreduce_sum_f32(void* comm, float* d_buf, size_t n, int device, void* stream);
/* Watchdog for the collective: waits on the host until everything enqueued on `stream` has
 * finished, polling the communicator's asynchronous error state (ncclCommGetAsyncError) every
 * few hundred microseconds.  Returns NVQ_OK when the stream drained, NVQ_ERR_NCCL when NCCL
 * reported an error, NVQ_ERR_TIMEOUT when timeout_ms passed first (a peer that never joined
 * the collective).  After a failure the communicator is unusable: call nvq_comm_abort. */
nvq_status nvq_comm_wait(void* comm, int device, void* stream, uint32_t timeout_ms);
/* ncclCommAbort: tears the communicator down without waiting for outstanding collectives
 * (nvq_comm_destroy waits for them).  The handle is invalid afterwards. */
nvq_status nvq_comm_abort(void* comm);

/* The same step without NCCL: gradient all-reduce fused with the SGD update over NVLink peer
 * memory (CUDA IPC, plain peer loads and stores; one process per GPU, at most 8 ranks).
 *   nvq_peer_create   allocates, on `device`, two gradient buffers of n_floats and a flag array;
 *   nvq_peer_export   writes this rank's handle (nvq_peer_handle_bytes bytes) for the launcher's
 *                     side channel; nvq_peer_connect takes the handles of all ranks, in rank order
 *                     (an all-zero handle marks a rank that is absent: it is never heard from, which
 *                     is how a test makes the bounded wait run out);
 *   nvq_peer_grad_buffer  where the backward pass writes this rank's gradients; steps alternate
 *                     between buffer 0 and buffer 1 (`parity`), starting with 0, on every rank alike;
 *   nvq_peer_allreduce_sgd  one kernel: announces the step to every rank, waits (at most timeout_ms,
 *                     default 2000) until every rank has announced it, adds the gradients of all
 *                     ranks in rank order and applies p -= lr * (sum / world).  A wait that runs out
 *                     leaves the parameters untouched and records code 61 for nvq_device_error_flag;
 *                     nothing hangs.  The step number is kept on the device, so the launch can be
 *                     captured into a CUDA graph (one graph per parity) and replayed.
 * All ranks must call it the same number of times; destroy only after a host-side rendezvous
 * (a peer may still be reading this rank's buffers until its own step has completed). */
typedef struct nvq_peer_group nvq_peer_group;
nvq_status nvq_peer_handle_bytes(size_t* bytes);
nvq_status nvq_peer_create(nvq_peer_group** out, int rank, int world, size_t n_floats, uint32_t timeout_ms,
                           int device);
nvq_status nvq_peer_export(nvq_peer_group* group, void* handle);
nvq_status nvq_peer_connect(nvq_peer_group* group, const void* handles);
nvq_status nvq_peer_grad_buffer(nvq_peer_group* group, int parity, float** d_ptr);
nvq_status nvq_peer_allreduce_sgd(nvq_peer_group* group, int parity, float* d_params, float lr, void* stream);
nvq_status nvq_peer_destroy(nvq_peer_group* group);

#ifdef __cplusplus
}
#endif
#endif /* NVQ_H */
