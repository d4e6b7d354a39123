// Gradient all-reduce fused with the SGD update over NVLink peer memory, for the data-parallel
// training step (one process per GPU; NovaNN itself is single process, so there is no reference
// counterpart).  Every rank keeps two gradient buffers and a small flag array in its own HBM and
// maps the other ranks' copies through CUDA IPC.  One kernel per step and rank:
//
//   1. announce: block 0 writes the step number into flag [my rank] of EVERY rank (release, system
//      scope).  The backward kernels precede this kernel in the stream, so the number says "the
//      gradients of this step are complete in my buffer";
//   2. wait: every block polls its own GPU's flag array until all ranks have announced the step
//      (acquire, system scope; bounded by a time limit, after which the kernel records a code,
//      leaves the parameters untouched and returns);
//   3. reduce + update: each rank reads the gradient of every rank (its own from HBM, the others'
//      with plain loads over NVLink), adds them in rank order - the same order on every rank, so
//      all ranks compute the same bits - and applies p -= lr * (sum / world).
//
// 0.94 MB per rank is latency-bound: NCCL needs 14 us (2 ranks) to 30 us (8 ranks) for the sum
// alone; here the exchange is one flag round plus (world - 1) x 0.94 MB of peer reads per rank,
// and the SGD kernel is gone.  Gradients alternate between the two buffers from step to step: a
// rank overwrites buffer b again two steps later, and by then every peer has announced the step
// in between, which it does only after its kernel that read buffer b has completed.
// No multicast, no TMA, no NCCL: plain peer loads and stores.
#include <string.h>

#include "nvq_common.cuh"

nvq_status nvq_status_word(int device, int** dev_ptr);

namespace {

constexpr int MAX_RANKS = 8;
constexpr int ERR_PEER_WAIT = 61;
constexpr size_t FLAG_BYTES = 256;   // MAX_RANKS x 8 bytes of flags, the step counter (+64), the block ticket (+72)

struct PeerArgs {
    const float* grads[MAX_RANKS];            // rank r's gradient buffer of this step's parity
    unsigned long long* announce[MAX_RANKS];  // &flags_of_rank_r[my rank]; nullptr = absent peer
    const unsigned long long* flags;          // my own flag array: [r] is written by rank r
    float* params;
    size_t n;
    float lr, inv_world;
    unsigned long long timeout_ns;
    // The step number lives on the device so that the kernel can be replayed from a CUDA graph:
    // every block reads *step_ctr + 1 as this launch's step; the last block to finish stores it back.
    unsigned long long* step_ctr;
    unsigned int* arrived;
    int rank, world;
    int* status;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer_v4(const float* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_peer_f32(const float* p) {
    float v;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(256) peer_allreduce_sgd_kernel(const PeerArgs a) {
    __shared__ int s_abort;
    __shared__ unsigned long long s_step;
    if (threadIdx.x == 0) {
        s_abort = 0;
        s_step = *(volatile unsigned long long*)a.step_ctr + 1;
    }
    __syncthreads();
    const unsigned long long step = s_step;
    // every block leaves through here: the last one publishes the step number for the next launch
    auto leave = [&]() {
        if (threadIdx.x == 0) {
            if (atomicAdd(a.arrived, 1u) == gridDim.x - 1) {
                *a.arrived = 0;
                *(volatile unsigned long long*)a.step_ctr = step;
            }
        }
    };
    if (blockIdx.x == 0 && threadIdx.x < a.world && a.announce[threadIdx.x])
        st_release_sys(a.announce[threadIdx.x], step);
    if (threadIdx.x < a.world) {
        const unsigned long long t0 = global_ns();
        while (ld_acquire_sys(a.flags + threadIdx.x) < step) {
            if (global_ns() - t0 > a.timeout_ns) {
                atomicExch(&s_abort, 1);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (s_abort) {
        // a rank never announced the step: nothing is read, nothing is updated
        if (threadIdx.x == 0 && a.status) atomicCAS(a.status, 0, ERR_PEER_WAIT);
        leave();
        return;
    }
    const size_t n4 = a.n / 4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 g[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; r++)
            if (r < a.world) g[r] = ld_peer_v4(a.grads[r] + 4 * i);
        float4 s = g[0];
#pragma unroll
        for (int r = 1; r < MAX_RANKS; r++)
            if (r < a.world) {
                s.x = __fadd_rn(s.x, g[r].x); s.y = __fadd_rn(s.y, g[r].y);
                s.z = __fadd_rn(s.z, g[r].z); s.w = __fadd_rn(s.w, g[r].w);
            }
        float4 p = reinterpret_cast<const float4*>(a.params)[i];
        // gradient = sum / world, then p -= lr * gradient: the roundings of the NCCL + SGD form
        p.x = __fsub_rn(p.x, __fmul_rn(a.lr, __fmul_rn(s.x, a.inv_world)));
        p.y = __fsub_rn(p.y, __fmul_rn(a.lr, __fmul_rn(s.y, a.inv_world)));
        p.z = __fsub_rn(p.z, __fmul_rn(a.lr, __fmul_rn(s.z, a.inv_world)));
        p.w = __fsub_rn(p.w, __fmul_rn(a.lr, __fmul_rn(s.w, a.inv_world)));
        reinterpret_cast<float4*>(a.params)[i] = p;
    }
    // the last n % 4 elements
    for (size_t i = 4 * n4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
        float s = ld_peer_f32(a.grads[0] + i);
        for (int r = 1; r < a.world; r++) s = __fadd_rn(s, ld_peer_f32(a.grads[r] + i));
        a.params[i] = __fsub_rn(a.params[i], __fmul_rn(a.lr, __fmul_rn(s, a.inv_world)));
    }
    leave();
}

size_t padded_floats(size_t n) { return (n + 63) / 64 * 64; }

}  // namespace

struct nvq_peer_group {
    int rank, world, device;
    size_t n, buf_bytes;         // floats per gradient buffer; bytes of one buffer (padded)
    char* base;                  // own allocation: [grad 0][grad 1][flags]
    char* peer_base[MAX_RANKS];  // mapped allocations of the others (own = base, absent = nullptr)
    bool connected;
    unsigned long long timeout_ns;
};

extern "C" nvq_status nvq_peer_handle_bytes(size_t* bytes) {
    NVQ_REQUIRE(bytes, "null out pointer");
    *bytes = sizeof(cudaIpcMemHandle_t);
    return NVQ_OK;
}

extern "C" nvq_status nvq_peer_create(nvq_peer_group** out, int rank, int world, size_t n_floats,
                                      uint32_t timeout_ms, int device) {
    NVQ_REQUIRE(out && world >= 1 && world <= MAX_RANKS && rank >= 0 && rank < world && n_floats > 0,
                "nvq_peer_create: bad argument (at most %d ranks)", MAX_RANKS);
    *out = nullptr;
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    nvq_peer_group* g = new nvq_peer_group();
    g->rank = rank; g->world = world; g->device = device;
    g->n = n_floats;
    g->buf_bytes = padded_floats(n_floats) * sizeof(float);
    g->connected = world == 1;
    g->timeout_ns = (unsigned long long)(timeout_ms ? timeout_ms : 2000) * 1000000ull;
    for (int r = 0; r < MAX_RANKS; r++) g->peer_base[r] = nullptr;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, 2 * g->buf_bytes + FLAG_BYTES);
    if (e != cudaSuccess) {
        delete g;
        NVQ_FAIL(NVQ_ERR_CUDA, "nvq_peer_create: cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    g->base = (char*)p;
    g->peer_base[rank] = g->base;
    e = cudaMemset(p, 0, 2 * g->buf_bytes + FLAG_BYTES);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();   // the flags are zero before anyone can map them
    if (e != cudaSuccess) {
        cudaFree(p);
        delete g;
        NVQ_FAIL(NVQ_ERR_CUDA, "nvq_peer_create: clearing the buffers failed: %s", cudaGetErrorString(e));
    }
    *out = g;
    return NVQ_OK;
}

extern "C" nvq_status nvq_peer_export(nvq_peer_group* g, void* handle) {
    NVQ_REQUIRE(g && handle, "nvq_peer_export: bad argument");
    nvq_status s = nvq_use_device(g->device);
    if (s != NVQ_OK) return s;
    cudaIpcMemHandle_t h;
    NVQ_CUDA(cudaIpcGetMemHandle(&h, g->base));
    memcpy(handle, &h, sizeof(h));
    return NVQ_OK;
}

extern "C" nvq_status nvq_peer_connect(nvq_peer_group* g, const void* handles) {
    NVQ_REQUIRE(g && handles, "nvq_peer_connect: bad argument");
    NVQ_REQUIRE(!g->connected || g->world == 1, "nvq_peer_connect: already connected");
    nvq_status s = nvq_use_device(g->device);
    if (s != NVQ_OK) return s;
    const char* hb = (const char*)handles;
    static const char zero[sizeof(cudaIpcMemHandle_t)] = {0};
    for (int r = 0; r < g->world; r++) {
        if (r == g->rank) continue;
        const char* hr = hb + (size_t)r * sizeof(cudaIpcMemHandle_t);
        if (memcmp(hr, zero, sizeof(zero)) == 0) continue;   // absent peer: never announces
        cudaIpcMemHandle_t h;
        memcpy(&h, hr, sizeof(h));
        void* p = nullptr;
        NVQ_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        g->peer_base[r] = (char*)p;
    }
    g->connected = true;
    return NVQ_OK;
}

extern "C" nvq_status nvq_peer_grad_buffer(nvq_peer_group* g, int parity, float** d_ptr) {
    NVQ_REQUIRE(g && d_ptr && (parity == 0 || parity == 1), "nvq_peer_grad_buffer: bad argument");
    *d_ptr = (float*)(g->base + (size_t)parity * g->buf_bytes);
    return NVQ_OK;
}

extern "C" nvq_status nvq_peer_allreduce_sgd(nvq_peer_group* g, int parity, float* d_params, float lr,
                                             void* stream) {
    NVQ_REQUIRE(g && d_params && (parity == 0 || parity == 1), "nvq_peer_allreduce_sgd: bad argument");
    NVQ_REQUIRE(g->connected, "nvq_peer_allreduce_sgd: nvq_peer_connect has not run");
    NVQ_REQUIRE(nvq_aligned(d_params, 16), "nvq_peer_allreduce_sgd: parameters must be 16-byte aligned");
    nvq_status s = nvq_use_device(g->device);
    if (s != NVQ_OK) return s;
    PeerArgs a = {};
    for (int r = 0; r < g->world; r++) {
        // an absent peer contributes this rank's own buffer (its flag is what never arrives)
        const char* b = g->peer_base[r] ? g->peer_base[r] : g->base;
        a.grads[r] = (const float*)(b + (size_t)parity * g->buf_bytes);
        a.announce[r] = g->peer_base[r]
                            ? (unsigned long long*)(g->peer_base[r] + 2 * g->buf_bytes) + g->rank
                            : nullptr;
    }
    a.flags = (const unsigned long long*)(g->base + 2 * g->buf_bytes);
    a.params = d_params;
    a.n = g->n;
    a.lr = lr;
    a.inv_world = 1.0f / (float)g->world;
    a.step_ctr = (unsigned long long*)(g->base + 2 * g->buf_bytes + 64);
    a.arrived = (unsigned int*)(g->base + 2 * g->buf_bytes + 72);
    a.timeout_ns = g->timeout_ns;
    a.rank = g->rank;
    a.world = g->world;
    s = nvq_status_word(g->device, &a.status);
    if (s != NVQ_OK) return s;
    const size_t n4 = (g->n + 3) / 4;
    size_t blocks = (n4 + 255) / 256;
    const size_t cap = 2 * (size_t)nvq_sm_count(g->device);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    peer_allreduce_sgd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a);
    NVQ_LAUNCHED();
    return NVQ_OK;
}

extern "C" nvq_status nvq_peer_destroy(nvq_peer_group* g) {
    if (!g) return NVQ_OK;
    nvq_status s = nvq_use_device(g->device);
    if (s == NVQ_OK) {
        for (int r = 0; r < g->world; r++)
            if (r != g->rank && g->peer_base[r]) cudaIpcCloseMemHandle(g->peer_base[r]);
        if (g->base) cudaFree(g->base);
    }
    delete g;
    return s;
}
