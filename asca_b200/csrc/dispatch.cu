// Hash-MoE dispatch as a stable integer counting sort.
//
// expert(t) = hash_route(ids[t], E)  (rust/src/model.rs:69-77), and the permutation is the
// concatenation of the reference's buckets (rust/src/model.rs:190-193): inside an expert,
// tokens keep ascending token order. Three small kernels, integer only:
//   1. each warp histograms its contiguous 1024-token segment            -> counts[seg][E]
//   2. one CTA turns counts into segment start positions (expert-major scan) + offsets[E+1]
//   3. each warp replays its segment 32 tokens at a time; match_any gives every lane its rank
//      among equal experts in the group, a per-warp running counter gives the base.
// Integer adds in any order give the same histogram, and the ranking is by construction the
// token order, so the result is bit-exact and run-to-run identical.
#include "common.cuh"

namespace {

constexpr int SEG = 1024;      // tokens per warp segment
constexpr int WARPS = 4;       // warps per CTA
constexpr int MAX_E = 2048;    // experts supported (smem: WARPS*E ints)

__device__ __forceinline__ uint32_t hash_route_dev(uint32_t id, uint32_t n_experts) {
    uint32_t h = id * 0x9E3779B1u;
    h ^= h >> 15;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    return h % n_experts;
}

__global__ void __launch_bounds__(WARPS * 32) hist_kernel(const uint32_t* __restrict__ ids, int64_t N, int E,
                                                          int32_t* __restrict__ counts,
                                                          int32_t* __restrict__ route) {
    extern __shared__ int32_t sh[];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* cnt = sh + w * E;
    for (int e = lane; e < E; e += 32) cnt[e] = 0;
    __syncwarp();
    const int64_t seg = (int64_t)blockIdx.x * WARPS + w;
    const int64_t lo = seg * SEG;
    if (lo < N) {
        const int64_t hi = lo + SEG < N ? lo + SEG : N;
        for (int64_t t = lo + lane; t < hi; t += 32) {
            uint32_t e = hash_route_dev(ids[t], (uint32_t)E);
            if (route) route[t] = (int32_t)e;
            atomicAdd(&cnt[e], 1);  // integer, shared memory: order-independent result
        }
        __syncwarp();
        for (int e = lane; e < E; e += 32) counts[seg * E + e] = cnt[e];
    }
}

// counts[seg][e] -> start[seg][e] = offsets[e] + sum_{seg' < seg} counts[seg'][e]; one CTA.
__global__ void __launch_bounds__(1024) scan_kernel(int32_t* __restrict__ counts, int n_seg, int E,
                                                    int32_t* __restrict__ offsets) {
    __shared__ int32_t tot[MAX_E];
    __shared__ int32_t ex[MAX_E];
    __shared__ int32_t wsum[32];
    // per-expert totals and in-place exclusive scan over segments (thread per expert)
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int32_t run = 0;
        for (int s = 0; s < n_seg; ++s) {
            int32_t c = counts[(int64_t)s * E + e];
            counts[(int64_t)s * E + e] = run;
            run += c;
        }
        tot[e] = run;
    }
    __syncthreads();
    // exclusive scan of totals over experts (E <= MAX_E, blockDim = 1024, two items/thread)
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int i0 = threadIdx.x * 2;
    int32_t a = i0 < E ? tot[i0] : 0, b = i0 + 1 < E ? tot[i0 + 1] : 0;
    int32_t s = a + b, inc = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int32_t n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    if (lane == 31) wsum[w] = inc;
    __syncthreads();
    if (w == 0) {
        int32_t v = wsum[lane], iv = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int32_t n = __shfl_up_sync(0xffffffffu, iv, o);
            if (lane >= o) iv += n;
        }
        wsum[lane] = iv - v;
    }
    __syncthreads();
    const int32_t excl = wsum[w] + inc - s;
    if (i0 < E) ex[i0] = excl;
    if (i0 + 1 < E) ex[i0 + 1] = excl + a;
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) offsets[e] = ex[e];
    if (threadIdx.x == 0) offsets[E] = ex[E - 1] + tot[E - 1];
    for (int64_t i = threadIdx.x; i < (int64_t)n_seg * E; i += blockDim.x) counts[i] += ex[i % E];
}

__global__ void __launch_bounds__(WARPS * 32) place_kernel(const uint32_t* __restrict__ ids, int64_t N, int E,
                                                           const int32_t* __restrict__ start,
                                                           int32_t* __restrict__ perm) {
    extern __shared__ int32_t sh[];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* run = sh + w * E;
    const int64_t seg = (int64_t)blockIdx.x * WARPS + w;
    const int64_t lo = seg * SEG;
    if (lo >= N) return;
    for (int e = lane; e < E; e += 32) run[e] = start[seg * E + e];
    __syncwarp();
    const int64_t hi = lo + SEG < N ? lo + SEG : N;
    for (int64_t base = lo; base < hi; base += 32) {
        const int64_t t = base + lane;
        const bool live = t < hi;
        const unsigned act = __ballot_sync(0xffffffffu, live);
        if (live) {
            const uint32_t e = hash_route_dev(ids[t], (uint32_t)E);
            const unsigned peers = __match_any_sync(act, e);
            const int rank = __popc(peers & ((1u << lane) - 1u));
            const int32_t pos = run[e] + rank;
            perm[pos] = (int32_t)t;
            __syncwarp(act);
            if (rank == 0) run[e] += __popc(peers);  // one leader per distinct expert
        }
        __syncwarp();
    }
}

}  // namespace

extern "C" int asca_moe_dispatch(asca_ctx* ctx, const uint32_t* ids, int64_t N, int64_t E, int32_t* perm,
                                 int32_t* offsets, int32_t* route) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, ids && perm && offsets && N >= 0 && E >= 1, "moe_dispatch: bad arguments");
    ASCA_REQUIRE(ctx, E <= MAX_E, "moe_dispatch: at most %d experts", MAX_E);
    ASCA_REQUIRE(ctx, N < ((int64_t)1 << 31), "moe_dispatch: N must fit int32");
    if (N == 0) {
        ASCA_CUDA(ctx, cudaMemsetAsync(offsets, 0, (size_t)(E + 1) * 4, ctx->stream));
        return ASCA_OK;
    }
    const int64_t n_seg = ceil_div64(N, SEG);
    const int64_t n_blk = ceil_div64(n_seg, WARPS);
    void* ws;
    ASCA_TRY(asca_workspace(ctx, (size_t)(n_blk * WARPS) * E * 4 + 256, &ws));
    int32_t* counts = (int32_t*)ws;
    const size_t smem = (size_t)WARPS * E * 4;
    hist_kernel<<<(unsigned)n_blk, WARPS * 32, smem, ctx->stream>>>(ids, N, (int)E, counts, route);
    ASCA_CHECK_LAUNCH(ctx);
    scan_kernel<<<1, 1024, 0, ctx->stream>>>(counts, (int)n_seg, (int)E, offsets);
    ASCA_CHECK_LAUNCH(ctx);
    place_kernel<<<(unsigned)n_blk, WARPS * 32, smem, ctx->stream>>>(ids, N, (int)E, counts, perm);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

// ------------------------------------------------------------------ allocation-free variant
// Scratch for asca_moe_dispatch_noalloc: the per-segment expert histogram that the three
// kernels above pass between each other. It lives in the library's device image, so every GPU
// that loads the library carries these 256 KiB until the process exits.
constexpr int NOALLOC_MAX_INTS = 65536;  // (segments rounded up to a multiple of 4) * E
static __device__ __align__(256) int32_t g_dispatch_scratch[NOALLOC_MAX_INTS];

namespace {
constexpr int MAX_DEVICES = 64;
int32_t* g_scratch_addr[MAX_DEVICES];  // device address of g_dispatch_scratch, per device ordinal
}  // namespace

extern "C" int asca_moe_dispatch_noalloc(asca_ctx* ctx, const uint32_t* ids, int64_t N, int64_t E, int32_t* perm,
                                         int32_t* offsets, int32_t* route) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, ids && perm && offsets && N >= 0 && E >= 1, "moe_dispatch_noalloc: bad arguments");
    ASCA_REQUIRE(ctx, E <= MAX_E, "moe_dispatch_noalloc: at most %d experts", MAX_E);
    ASCA_REQUIRE(ctx, N < ((int64_t)1 << 31), "moe_dispatch_noalloc: N must fit int32");
    ASCA_REQUIRE(ctx, ctx->device >= 0 && ctx->device < MAX_DEVICES, "moe_dispatch_noalloc: device ordinal out of range");
    const int64_t n_seg = ceil_div64(N, SEG);
    const int64_t n_blk = ceil_div64(n_seg, WARPS);
    if (n_blk * WARPS * E > NOALLOC_MAX_INTS)
        return asca_fail(ctx, ASCA_ERR_ARG,
                         "moe_dispatch_noalloc: ceil(N/%d) rounded up to a multiple of %d, times E, is %lld and must "
                         "not exceed %d (N=%lld, E=%lld); use asca_moe_dispatch for larger problems",
                         SEG, WARPS, (long long)(n_blk * WARPS * E), NOALLOC_MAX_INTS, (long long)N, (long long)E);
    if (N == 0) {
        ASCA_CUDA(ctx, cudaMemsetAsync(offsets, 0, (size_t)(E + 1) * 4, ctx->stream));
        return ASCA_OK;
    }
    // One-time set-up per device: the array's name is only a host-side stand-in here, so ask the
    // runtime for its address on this device, with this device current.
    if (!g_scratch_addr[ctx->device]) {
        int cur = -1;
        ASCA_CUDA(ctx, cudaGetDevice(&cur));
        if (cur != ctx->device) ASCA_CUDA(ctx, cudaSetDevice(ctx->device));
        void* addr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&addr, g_dispatch_scratch);
        if (cur != ctx->device) cudaSetDevice(cur);
        if (e != cudaSuccess || !addr)
            return asca_fail(ctx, ASCA_ERR_CUDA, "moe_dispatch_noalloc: cudaGetSymbolAddress failed: %s",
                             cudaGetErrorString(e));
        g_scratch_addr[ctx->device] = (int32_t*)addr;
    }
    int32_t* counts = g_scratch_addr[ctx->device];
    // Nothing in the scratch has to start at zero: hist_kernel overwrites every entry that
    // scan_kernel and place_kernel read (segments 0 .. n_seg-1), whatever the last call left.
    const size_t smem = (size_t)WARPS * E * 4;
    hist_kernel<<<(unsigned)n_blk, WARPS * 32, smem, ctx->stream>>>(ids, N, (int)E, counts, route);
    ASCA_CHECK_LAUNCH(ctx);
    scan_kernel<<<1, 1024, 0, ctx->stream>>>(counts, (int)n_seg, (int)E, offsets);
    ASCA_CHECK_LAUNCH(ctx);
    place_kernel<<<(unsigned)n_blk, WARPS * 32, smem, ctx->stream>>>(ids, N, (int)E, counts, perm);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}
