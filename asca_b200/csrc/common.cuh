// Shared internals of libasca_b200: the context object, error plumbing, launch accounting.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "../../include/asca_b200.h"

struct asca_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    size_t smem_optin = 0;
    std::string err;
    std::string desc;
    int64_t launches = 0;
    // Programmatic dependent launch: while set, launches made through asca_launch may start their prologue before the
    // previous kernel on the stream has finished (only kernels that execute pdl_wait() first are launched that way).
    bool pdl = false;
    // size-class cache of freed blocks (the role of the reference's DevBuf pool,
    // rust/src/cuda/mod.rs:104-174): key = rounded size.
    std::multimap<size_t, void*> pool;
    std::map<void*, size_t> live;
    // lazily grown scratch owned by the context (partials, tile tables, error words)
    void* ws = nullptr;
    size_t ws_bytes = 0;
    int* err_word = nullptr;  // device int the kernels with bounded waits write to
    // Dynamic tile claims of the persistent tensor-core products (gemm_tc.cu; ASCA_GEMM_DYNAMIC=0 turns them off).
    // dyn_buf: two counters + the walkers' claim rings.
    void* dyn_buf = nullptr;
    uint32_t dyn_seq = 0;
    // tiles of the tensor-core delta forwards that wrote checkpoints, kept for their backwards: one entry per
    // checkpoint buffer (a model keeps one per block), least recently used evicted beyond 32 entries / dtiles_cap bytes
    struct DeltaTiles {
        const void* ckpt = nullptr;   // key: the checkpoint buffer the forward filled (null: contents invalid)
        const void *q = nullptr, *k = nullptr, *v = nullptr, *alpha = nullptr, *beta = nullptr;   // and its inputs
        int64_t B = 0, T = 0, H = 0;
        void* buf = nullptr;
        size_t bytes = 0;
        uint64_t stamp = 0;
    };
    std::vector<DeltaTiles> dtiles;
    uint64_t dtiles_clock = 0;
    size_t dtiles_cap = (size_t)32 << 30;   // bytes of kept tiles beyond which the least recently used set is reused
    // Adam moments kept on the device between optimizer calls of the host-pointer API, keyed by the caller's
    // (host address of m, length) as the reference keys them (rust/src/cuda/mod.rs:36-73)
    std::map<std::pair<uintptr_t, size_t>, std::pair<float*, float*>> resident;
    // optional per-kernel timing (asca_ctx_profile): CUDA events around selected launches
    bool profiling = false;
    struct Span {
        const char* name;
        cudaEvent_t e0, e1;
        double work;   // algorithmic FLOPs (products) or bytes of the launch; 0 = not stated
    };
    std::vector<Span> spans;
};

// Brackets one kernel launch with CUDA events on the context's stream when profiling is on.
struct asca_span {
    asca_ctx* ctx;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    const char* name;
    double work;
    asca_span(asca_ctx* c, const char* n, double w = 0.0) : ctx(c), name(n), work(w) {
        if (!ctx->profiling) return;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        cudaEventRecord(e0, ctx->stream);
    }
    ~asca_span() {
        if (!e0) return;
        cudaEventRecord(e1, ctx->stream);
        ctx->spans.push_back({name, e0, e1, work});
    }
};

int asca_fail(asca_ctx* ctx, int code, const char* fmt, ...);

#ifdef __CUDACC__
// Programmatic dependent launch, device side. pdl_wait() returns once every kernel this launch depends on has
// finished and its writes are visible (immediately when the launch was an ordinary one); nothing before it may
// touch global memory that another kernel writes or reads. pdl_launch_dependents() lets the next kernel on the
// stream be scheduled. Most kernels call it after pdl_wait(), so that at most one kernel is resident ahead of the running
// one; the few-row product triggers BEFORE its wait when its caller sets b_early (gemm_tc.cuh), so several of a decode
// step's products can be resident behind one running kernel, each having read only weights, dispatch offsets and state
// that were final before the nearest preceding kernel that waits before it triggers.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launches `kern` on the context's stream; with ctx->pdl set, as a programmatic dependent of the previous kernel.
// Only for kernels whose every thread calls pdl_wait() before its first global memory access.
template <typename... KArgs, typename... Args>
inline cudaError_t asca_launch(asca_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
#endif
// Returns scratch of at least `bytes` (256-byte aligned); contents are undefined.
int asca_workspace(asca_ctx* ctx, size_t bytes, void** out);

#define ASCA_CUDA(ctx, call)                                                                  \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess)                                                               \
            return asca_fail((ctx), e__ == cudaErrorMemoryAllocation ? ASCA_ERR_OOM : ASCA_ERR_CUDA, \
                             "CUDA error %d (%s) at %s:%d", (int)e__, cudaGetErrorString(e__),\
                             __FILE__, __LINE__);                                             \
    } while (0)

#define ASCA_CHECK_LAUNCH(ctx)                                                                \
    do {                                                                                      \
        (ctx)->launches++;                                                                    \
        ASCA_CUDA((ctx), cudaGetLastError());                                                 \
    } while (0)

#define ASCA_REQUIRE(ctx, cond, ...)                                                          \
    do {                                                                                      \
        if (!(cond)) return asca_fail((ctx), ASCA_ERR_ARG, __VA_ARGS__);                      \
    } while (0)

#define ASCA_TRY(expr)                                                                        \
    do {                                                                                      \
        int rc__ = (expr);                                                                    \
        if (rc__ != ASCA_OK) return rc__;                                                     \
    } while (0)

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- small device helpers shared by several kernels
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Deterministic block-wide sum (fixed tree), result broadcast to all threads.
// `red` must hold at least 33 floats. blockDim.x must be a multiple of 32.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
