// fp32 <-> fp16 / bf16 / fp64 casts: the replacement for ndarray.astype on NovaNN's layer
// entry (novann/layers/linear/linear.py:81,96).  HBM-bound: 6 bytes per element for the
// 16-bit pairs, 12 for the fp64 pair.  fp64 -> fp32 is the one conversion NovaNN really
// performs: BatchNorm holds float64 gamma / beta (novann/layers/batchnorm/batchnorm2d.py:40-41),
// so its output is float64 and the next layer's astype(np.float32) narrows it.
//
// Finite and infinite values go through the hardware converters (cvt.rn.*), which
// implement round-to-nearest-even with subnormals; a packet that holds a NaN takes
// the integer path so the NaN payload rules hold bit for bit.
#include <mutex>

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
namespace {
constexpr int kSlots = 3;
constexpr size_t kChunkBytes = (size_t)64 << 20;  // per staging buffer: 64 MiB on the wide side
constexpr int kMaxDev = 64;

struct Staging {
    std::mutex mu;            // one transfer at a time per device; devices are independent
    bool ready = false;
    cudaStream_t stream[kSlots];
    void* d_in[kSlots];
    void* d_out[kSlots];
};
Staging g_staging[kMaxDev];

size_t dtype_size(nvq_dtype t) { return t == NVQ_F64 ? 8 : (t == NVQ_F32 ? 4 : 2); }
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
            NVQ_CUDA(cudaStreamDestroy(sg.stream[i]));
        }
        sg.ready = false;
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
            NVQ_CUDA(cudaMalloc(&sg.d_in[i], kChunkBytes));
            NVQ_CUDA(cudaMalloc(&sg.d_out[i], kChunkBytes));
        }
        sg.ready = true;
    }
    const size_t ss = dtype_size(src_dtype), ds = dtype_size(dst_dtype);
    const size_t chunk = kChunkBytes / (ss > ds ? ss : ds);
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
