// fp32 <-> fp16 / bf16 / fp64 casts: the replacement for ndarray.astype on NovaNN's layer
// entry (novann/layers/linear/linear.py:81,96).  HBM-bound: 6 bytes per element for the
// 16-bit pairs, 12 for the fp64 pair.  fp64 -> fp32 is the one conversion NovaNN really
// performs: BatchNorm holds float64 gamma / beta (novann/layers/batchnorm/batchnorm2d.py:40-41),
// so its output is float64 and the next layer's astype(np.float32) narrows it.
//
// Finite and infinite values go through the hardware converters (cvt.rn.*), which
// implement round-to-nearest-even with subnormals; a packet that holds a NaN takes
// the integer path so the NaN payload rules hold bit for bit.
#include <sched.h>
#include <string.h>
#if defined(__x86_64__)
#include <emmintrin.h>
#endif

#include <condition_variable>
#include <mutex>
#include <thread>

#include "elementwise.cuh"

namespace {

__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t cvt_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float cvt_f32_f16(uint16_t h) {
    float r;
    asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"(h));
    return r;
}

// ---- fp32 -> 16-bit: 8 elements per packet, 256-bit load, 128-bit store ----------
template <bool BF16>
struct NarrowOp {
    static constexpr int VEC = 8;
    static constexpr int UNROLL = 4;
    static constexpr int RESIDENT = 3;
    using In = u32x8;
    __device__ __forceinline__ void init() {}
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        return ldg_stream_256((const char*)src + p * 32);
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& a) const {
        uint32_t w[4];
        if (!any_nonfinite8(a)) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float lo = __uint_as_float(a.v[2 * i]), hi = __uint_as_float(a.v[2 * i + 1]);
                w[i] = BF16 ? cvt_bf16x2(lo, hi) : cvt_f16x2(lo, hi);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t lo = BF16 ? spec_f32_to_bf16(a.v[2 * i]) : spec_f32_to_f16(a.v[2 * i]);
                uint32_t hi = BF16 ? spec_f32_to_bf16(a.v[2 * i + 1]) : spec_f32_to_f16(a.v[2 * i + 1]);
                w[i] = lo | (hi << 16);
            }
        }
        stg_stream_128((char*)dst + p * 16, make_uint4(w[0], w[1], w[2], w[3]));
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        uint32_t u = ((const uint32_t*)src)[i];
        ((uint16_t*)dst)[i] = (uint16_t)(BF16 ? spec_f32_to_bf16(u) : spec_f32_to_f16(u));
    }
};

// ---- 16-bit -> fp32: 8 elements per packet, 128-bit load, 256-bit store ----------
template <bool BF16>
struct WidenOp {
    static constexpr int VEC = 8;
    static constexpr int UNROLL = 4;
    static constexpr int RESIDENT = 2;
    using In = uint4;
    __device__ __forceinline__ void init() {}
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        return ldg_stream_128((const char*)src + p * 16);
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& a) const {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
        u32x8 o;
        if (BF16) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                o.v[2 * i] = w[i] << 16;
                o.v[2 * i + 1] = w[i] & 0xFFFF0000u;
            }
        } else {
            // any half with all exponent bits set (inf / NaN) -> integer path
            uint32_t special = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) special |= ((w[i] & 0x7FFF7FFFu) + 0x04000400u);
            if (!(special & 0x80008000u)) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    o.v[2 * i] = __float_as_uint(cvt_f32_f16((uint16_t)(w[i] & 0xFFFFu)));
                    o.v[2 * i + 1] = __float_as_uint(cvt_f32_f16((uint16_t)(w[i] >> 16)));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    o.v[2 * i] = spec_f16_to_f32(w[i] & 0xFFFFu);
                    o.v[2 * i + 1] = spec_f16_to_f32(w[i] >> 16);
                }
            }
        }
        stg_stream_256((char*)dst + p * 32, o);
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        uint32_t h = ((const uint16_t*)src)[i];
        ((uint32_t*)dst)[i] = BF16 ? (h << 16) : spec_f16_to_f32(h);
    }
};

// ---- fp64 -> fp32: 4 elements per packet, 256-bit load, 128-bit store ----------------
// NumPy narrows with the C cast (double -> float): RNE, overflow to +-inf, subnormal results
// kept.  A NaN keeps its sign and the top 22 payload bits and comes out quiet
// (sign | 0x7fc00000 | payload >> 29).  Finite and infinite lanes use cvt.rn.f32.f64.
__device__ __forceinline__ uint32_t spec_f64_to_f32(uint32_t lo, uint32_t hi) {
    uint32_t a = hi & 0x7FFFFFFFu;
    if (a > 0x7FF00000u || (a == 0x7FF00000u && lo != 0u))
        return (hi & 0x80000000u) | 0x7FC00000u | ((a & 0xFFFFFu) << 3) | (lo >> 29);
    return __float_as_uint(__double2float_rn(__hiloint2double((int)hi, (int)lo)));
}
struct NarrowF64Op {
    static constexpr int VEC = 4;
    static constexpr int UNROLL = 4;
    static constexpr int RESIDENT = 3;
    using In = u32x8;
    __device__ __forceinline__ void init() {}
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        return ldg_stream_256((const char*)src + p * 32);
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& a) const {
        uint32_t w[4];
        uint32_t special = 0;   // a lane with all exponent bits set (inf / NaN)
#pragma unroll
        for (int i = 0; i < 4; i++) special |= ((a.v[2 * i + 1] & 0x7FF00000u) + 0x00100000u);
        if (!(special & 0x80000000u)) {
#pragma unroll
            for (int i = 0; i < 4; i++)
                w[i] = __float_as_uint(__double2float_rn(
                    __hiloint2double((int)a.v[2 * i + 1], (int)a.v[2 * i])));
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] = spec_f64_to_f32(a.v[2 * i], a.v[2 * i + 1]);
        }
        stg_stream_128((char*)dst + p * 16, make_uint4(w[0], w[1], w[2], w[3]));
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        uint2 u = ((const uint2*)src)[i];
        ((uint32_t*)dst)[i] = spec_f64_to_f32(u.x, u.y);
    }
};

// ---- fp32 -> fp64: exact; a NaN comes out quiet with its payload shifted left 29 ------
__device__ __forceinline__ uint2 spec_f32_to_f64(uint32_t u) {
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
        uint32_t m = u & 0x7FFFFFu;
        return make_uint2(m << 29, (u & 0x80000000u) | 0x7FF80000u | (m >> 3));
    }
    double d = (double)__uint_as_float(u);
    return make_uint2((uint32_t)__double2loint(d), (uint32_t)__double2hiint(d));
}
struct WidenF64Op {
    static constexpr int VEC = 4;
    static constexpr int UNROLL = 4;
    static constexpr int RESIDENT = 2;
    using In = uint4;
    __device__ __forceinline__ void init() {}
    __device__ __forceinline__ In load(const void* src, size_t p) const {
        return ldg_stream_128((const char*)src + p * 16);
    }
    __device__ __forceinline__ void store(void* dst, size_t p, const In& a) const {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
        u32x8 o;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint2 d = spec_f32_to_f64(w[i]);
            o.v[2 * i] = d.x;
            o.v[2 * i + 1] = d.y;
        }
        stg_stream_256((char*)dst + p * 32, o);
    }
    __device__ __forceinline__ void scalar(const void* src, void* dst, size_t i) const {
        ((uint2*)dst)[i] = spec_f32_to_f64(((const uint32_t*)src)[i]);
    }
};

}  // namespace

extern "C" nvq_status nvq_cast(void* d_dst, nvq_dtype dst_dtype, const void* d_src,
                               nvq_dtype src_dtype, size_t n, int device, void* stream) {
    NVQ_REQUIRE(n == 0 || (d_dst && d_src), "nvq_cast: null buffer");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    cudaStream_t st = (cudaStream_t)stream;
    if (src_dtype == NVQ_F32 && dst_dtype == NVQ_BF16)
        return ew_launch(NarrowOp<true>{}, d_src, d_dst, n, device, st, 32, 16);
    if (src_dtype == NVQ_F32 && dst_dtype == NVQ_F16)
        return ew_launch(NarrowOp<false>{}, d_src, d_dst, n, device, st, 32, 16);
    if (src_dtype == NVQ_BF16 && dst_dtype == NVQ_F32)
        return ew_launch(WidenOp<true>{}, d_src, d_dst, n, device, st, 16, 32);
    if (src_dtype == NVQ_F16 && dst_dtype == NVQ_F32)
        return ew_launch(WidenOp<false>{}, d_src, d_dst, n, device, st, 16, 32);
    if (src_dtype == NVQ_F64 && dst_dtype == NVQ_F32)
        return ew_launch(NarrowF64Op{}, d_src, d_dst, n, device, st, 32, 16);
    if (src_dtype == NVQ_F32 && dst_dtype == NVQ_F64)
        return ew_launch(WidenF64Op{}, d_src, d_dst, n, device, st, 16, 32);
    NVQ_FAIL(NVQ_ERR_INVALID, "nvq_cast: unsupported dtype pair %d -> %d", (int)src_dtype,
             (int)dst_dtype);
}

// ---- host-buffer variant ------------------------------------------------------------
// Streams a host array through per-device staging buffers in chunks.  Three slots,
// each with its own stream, keep one chunk uploading, one converting and one
// downloading at any time, so the PCIe link runs in both directions at once.  In-stream
// ordering alone makes the reuse of a slot's buffers safe.
//
// Page-locked arrays (nvq_host_alloc) are the copies' source and destination as they are.
// A plain (pageable) array - what ndarray.astype is handed - cannot be: the driver stages such
// copies itself through one small buffer and one thread (about 15 GB/s here for the cast sweep).
// Those arrays go through page-locked staging buffers of the library instead, filled and
// drained by a few host threads while the previous chunk is on the link.
namespace {
constexpr int kSlots = 3;
constexpr size_t kChunkBytes = (size_t)64 << 20;  // per staging buffer: 64 MiB on the wide side
constexpr int kMaxDev = 64;
constexpr size_t kStageMinBytes = (size_t)8 << 20;   // smaller pageable arrays: the plain path

struct Staging {
    std::mutex mu;            // one transfer at a time per device; devices are independent
    bool ready = false;
    bool host_ready = false;
    cudaStream_t stream[kSlots];
    cudaEvent_t done[kSlots];
    void* d_in[kSlots];
    void* d_out[kSlots];
    void* h_in[kSlots];       // page-locked staging for pageable arrays (allocated on first need)
    void* h_out[kSlots];
};
Staging g_staging[kMaxDev];

size_t dtype_size(nvq_dtype t) { return t == NVQ_F64 ? 8 : (t == NVQ_F32 ? 4 : 2); }

// ---- a small pool of host threads that copy memory in parallel ------------------------
// Never destroyed: the workers are detached and sleep on a condition variable between jobs, so
// a process that exits without nvq_shutdown just ends them.
// Host copy of one piece with non-temporal stores: the destination (a staging buffer the DMA
// engine reads next, or the caller's output array) is not read first and does not push the
// source out of the cache.  Eight threads on an 8-core host: 27.8 GB/s against 19.4 for memcpy;
// the pageable cast sweep on a B200 box: 31.2 -> 34.0 GB/s.
static void stream_copy(char* dst, const char* src, size_t n) {
#if defined(__x86_64__)
    size_t i = 0;
    for (; i < n && ((uintptr_t)(dst + i) & 15); i++) dst[i] = src[i];
    for (; i + 64 <= n; i += 64) {
        const __m128i a = _mm_loadu_si128((const __m128i*)(src + i));
        const __m128i b = _mm_loadu_si128((const __m128i*)(src + i + 16));
        const __m128i c = _mm_loadu_si128((const __m128i*)(src + i + 32));
        const __m128i d = _mm_loadu_si128((const __m128i*)(src + i + 48));
        _mm_stream_si128((__m128i*)(dst + i), a);
        _mm_stream_si128((__m128i*)(dst + i + 16), b);
        _mm_stream_si128((__m128i*)(dst + i + 32), c);
        _mm_stream_si128((__m128i*)(dst + i + 48), d);
    }
    for (; i < n; i++) dst[i] = src[i];
    _mm_sfence();
#else
    memcpy(dst, src, n);
#endif
}

class CopyPool {
  public:
    static CopyPool& get() {
        static CopyPool* pool = new CopyPool();
        return *pool;
    }
    // dst[0, bytes) = src[0, bytes), split over the workers and the calling thread
    void copy(void* dst, const void* src, size_t bytes) {
        if (bytes < ((size_t)1 << 20) || workers_ == 0) {
            memcpy(dst, src, bytes);
            return;
        }
        std::unique_lock<std::mutex> call_lock(call_mu_);      // one parallel copy at a time
        const int parts = workers_ + 1;
        const size_t piece = ((bytes + parts - 1) / parts + 4095) & ~(size_t)4095;
        {
            std::lock_guard<std::mutex> lk(mu_);
            dst_ = (char*)dst; src_ = (const char*)src; bytes_ = bytes; piece_ = piece;
            pending_ = workers_;
            generation_++;
        }
        cv_.notify_all();
        run_piece(workers_);                                    // the caller takes the last piece
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [&] { return pending_ == 0; });
    }

  private:
    CopyPool() {
        int n = 8;
        cpu_set_t set;
        if (sched_getaffinity(0, sizeof(set), &set) == 0) {
            const int avail = CPU_COUNT(&set);
            if (avail - 1 < n) n = avail - 1;
        }
        if (n < 0) n = 0;
        workers_ = n;
        for (int w = 0; w < n; w++) std::thread([this, w] { loop(w); }).detach();
    }
    void run_piece(int idx) {
        const size_t off = (size_t)idx * piece_;
        if (off < bytes_) stream_copy(dst_ + off, src_ + off, bytes_ - off < piece_ ? bytes_ - off : piece_);
    }
    void loop(int idx) {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
            }
            run_piece(idx);
            std::lock_guard<std::mutex> lk(mu_);
            if (--pending_ == 0) done_cv_.notify_all();
        }
    }
    std::mutex call_mu_, mu_;
    std::condition_variable cv_, done_cv_;
    uint64_t generation_ = 0;
    int workers_ = 0, pending_ = 0;
    char* dst_ = nullptr;
    const char* src_ = nullptr;
    size_t bytes_ = 0, piece_ = 0;
};

bool is_pinned(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeHost || a.type == cudaMemoryTypeManaged;
}
}  // namespace

// Frees the staging buffers and streams of every device (nvq_shutdown).
nvq_status nvq_cast_release_staging() {
    for (int d = 0; d < kMaxDev; d++) {
        Staging& sg = g_staging[d];
        std::lock_guard<std::mutex> lock(sg.mu);
        if (!sg.ready) continue;
        NVQ_CUDA(cudaSetDevice(d));
        for (int i = 0; i < kSlots; i++) {
            NVQ_CUDA(cudaStreamSynchronize(sg.stream[i]));
            NVQ_CUDA(cudaFree(sg.d_in[i]));
            NVQ_CUDA(cudaFree(sg.d_out[i]));
            if (sg.host_ready) {
                NVQ_CUDA(cudaFreeHost(sg.h_in[i]));
                NVQ_CUDA(cudaFreeHost(sg.h_out[i]));
            }
            NVQ_CUDA(cudaEventDestroy(sg.done[i]));
            NVQ_CUDA(cudaStreamDestroy(sg.stream[i]));
        }
        sg.ready = sg.host_ready = false;
    }
    return NVQ_OK;
}

extern "C" nvq_status nvq_cast_host(void* h_dst, nvq_dtype dst_dtype, const void* h_src,
                                    nvq_dtype src_dtype, size_t n, int device) {
    NVQ_REQUIRE(n == 0 || (h_dst && h_src), "nvq_cast_host: null buffer");
    bool narrow = src_dtype == NVQ_F32 && (dst_dtype == NVQ_F16 || dst_dtype == NVQ_BF16);
    bool widen = dst_dtype == NVQ_F32 && (src_dtype == NVQ_F16 || src_dtype == NVQ_BF16);
    bool f64 = (src_dtype == NVQ_F64 && dst_dtype == NVQ_F32) || (src_dtype == NVQ_F32 && dst_dtype == NVQ_F64);
    NVQ_REQUIRE(narrow || widen || f64, "nvq_cast_host: unsupported dtype pair %d -> %d", (int)src_dtype,
                (int)dst_dtype);
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    Staging& sg = g_staging[device];
    std::lock_guard<std::mutex> lock(sg.mu);
    if (!sg.ready) {
        for (int i = 0; i < kSlots; i++) {
            NVQ_CUDA(cudaStreamCreateWithFlags(&sg.stream[i], cudaStreamNonBlocking));
            NVQ_CUDA(cudaEventCreateWithFlags(&sg.done[i], cudaEventDisableTiming));
            NVQ_CUDA(cudaMalloc(&sg.d_in[i], kChunkBytes));
            NVQ_CUDA(cudaMalloc(&sg.d_out[i], kChunkBytes));
        }
        sg.ready = true;
    }
    const size_t ss = dtype_size(src_dtype), ds = dtype_size(dst_dtype);
    const size_t chunk = kChunkBytes / (ss > ds ? ss : ds);
    const bool stage_in = n * ss >= kStageMinBytes && !is_pinned(h_src);
    const bool stage_out = n * ds >= kStageMinBytes && !is_pinned(h_dst);
    if ((stage_in || stage_out) && !sg.host_ready) {
        for (int i = 0; i < kSlots; i++) {
            NVQ_CUDA(cudaHostAlloc(&sg.h_in[i], kChunkBytes, cudaHostAllocPortable));
            NVQ_CUDA(cudaHostAlloc(&sg.h_out[i], kChunkBytes, cudaHostAllocPortable));
        }
        sg.host_ready = true;
    }
    if (!stage_in && !stage_out) {
        int slot = 0;
        for (size_t off = 0; off < n; off += chunk, slot = (slot + 1) % kSlots) {
            size_t m = n - off < chunk ? n - off : chunk;
            cudaStream_t st = sg.stream[slot];
            NVQ_CUDA(cudaMemcpyAsync(sg.d_in[slot], (const char*)h_src + off * ss, m * ss,
                                     cudaMemcpyHostToDevice, st));
            s = nvq_cast(sg.d_out[slot], dst_dtype, sg.d_in[slot], src_dtype, m, device, st);
            if (s != NVQ_OK) return s;
            NVQ_CUDA(cudaMemcpyAsync((char*)h_dst + off * ds, sg.d_out[slot], m * ds,
                                     cudaMemcpyDeviceToHost, st));
        }
        for (int i = 0; i < kSlots; i++) NVQ_CUDA(cudaStreamSynchronize(sg.stream[i]));
        return NVQ_OK;
    }
    // Staged form.  Iteration i fills the staging buffer of chunk i and puts its copies and its
    // kernel on the slot's stream, then drains chunk i - 1, whose transfer ran meanwhile; a slot
    // comes round again only after its chunk was drained.
    CopyPool& pool = CopyPool::get();
    const size_t n_chunks = (n + chunk - 1) / chunk;
    for (size_t i = 0; i <= n_chunks; i++) {
        if (i < n_chunks) {
            const int slot = (int)(i % kSlots);
            const size_t off = i * chunk, m = n - off < chunk ? n - off : chunk;
            cudaStream_t st = sg.stream[slot];
            const void* src = (const char*)h_src + off * ss;
            if (stage_in) {
                pool.copy(sg.h_in[slot], src, m * ss);
                src = sg.h_in[slot];
            }
            NVQ_CUDA(cudaMemcpyAsync(sg.d_in[slot], src, m * ss, cudaMemcpyHostToDevice, st));
            s = nvq_cast(sg.d_out[slot], dst_dtype, sg.d_in[slot], src_dtype, m, device, st);
            if (s != NVQ_OK) return s;
            NVQ_CUDA(cudaMemcpyAsync(stage_out ? sg.h_out[slot] : (void*)((char*)h_dst + off * ds), sg.d_out[slot],
                                     m * ds, cudaMemcpyDeviceToHost, st));
            NVQ_CUDA(cudaEventRecord(sg.done[slot], st));
        }
        if (i >= 1) {
            const size_t j = i - 1;
            const int slot = (int)(j % kSlots);
            const size_t off = j * chunk, m = n - off < chunk ? n - off : chunk;
            NVQ_CUDA(cudaEventSynchronize(sg.done[slot]));
            if (stage_out) pool.copy((char*)h_dst + off * ds, sg.h_out[slot], m * ds);
        }
    }
    return NVQ_OK;
}
