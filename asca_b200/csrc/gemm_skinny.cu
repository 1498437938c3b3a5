// bf16 products with few rows (a decode step's 256 streams, a handful of tokens per expert) on tcgen05.
//
// With few rows the product is a stream of weights: every weight byte is used once. The 128-row instruction
// shape is therefore given to the WEIGHTS -- the kernel computes C^T tiles of 128 output features x NT tokens
// (NT = 32 or 64 is the instruction's N) -- so that a shared-memory stage holds 16 KiB of weights and only
// NT x 128 bytes of activations, where the row-tiled kernel spends half of every stage on 128 activation rows
// of which an expert owns a dozen. Operands: the weight tile W[k0.., f0..] (memory K x features, feature
// contiguous) is the MN-major A operand; the token tile X[t0.., k0..] (memory tokens x K) is the K-major B
// operand; neither is copied or transposed.
//
// Persistent, roles as in the row-tiled kernel: warp 0 = TMA producer through a ring of mbarriers, warp 1 =
// TMEM allocation + one thread issuing tcgen05.mma into one of two accumulator buffers, warps 2-5 = epilogue.
// An accumulator lane is an output feature and a column is a token: the epilogue turns 16 tokens x 32 features
// at a time through shared memory, so that global memory sees 16-byte accesses with 8 lanes on each token's
// 128 bytes. Bias, SiLU (bf16 second output), accumulation and the row map of the MoE combine are applied there.
//
// Every mbarrier wait is bounded; a wait that runs out raises the error word and the CTA frees its TMEM and exits.
#include "gemm_tc.cuh"

#include <algorithm>
#include "tc_common.cuh"

namespace gemm_tc {
namespace {

constexpr int BF = 128, BK = 64, THREADS = 192;
constexpr int W_BYTES = BF * BK * 2;
constexpr int SK_MAX_GROUPS = 512;

template <int NT, int ST> struct SkShape {
    static constexpr int STAGES = ST;                          // 10 x 20 KiB (NT 32) or 8 x 24 KiB (NT 64): one CTA per SM
    static constexpr int X_BYTES = NT * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;      // 20 / 24 KiB: every stage starts 1024-byte aligned
    static constexpr int TMEM_COLS = 2 * NT;                   // two accumulator buffers
    static constexpr int CTAS_PER_SM = ST * STAGE_BYTES <= 102 * 1024 ? 2 : 1;
    static constexpr size_t SMEM_FIXED = (size_t)STAGES * STAGE_BYTES + 4 * 2048 /*epilogue staging*/ + 1024 /*alignment slack*/ +
                                         256 /*barriers*/;
};

struct SkP {
    float* C;
    int64_t ldc;
    int M, N, K;
    const float* bias;
    int accumulate;
    const int32_t* c_idx;
    const int32_t* offsets;
    int n_groups, grouped;
    int w_goff_inner, w_goff_outer;
    int64_t bias_gstride;
    int epi;
    __nv_bfloat16* C2;
    int64_t ldc2;
    int c2_mapped;
    int w_packed;
    int early;
    int* err_word;
};

__device__ __forceinline__ float sk_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int NT, int ST>
__global__ void __launch_bounds__(THREADS, SkShape<NT, ST>::CTAS_PER_SM) gemm_skinny_kernel(const __grid_constant__ CUtensorMap mapW,
                                                                                       const __grid_constant__ CUtensorMap mapX,
                                                                                       const SkP p) {
    constexpr int STAGES = ST, STAGE_BYTES = SkShape<NT, ST>::STAGE_BYTES, TMEM_COLS = SkShape<NT, ST>::TMEM_COLS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = tiles + STAGES * STAGE_BYTES;                 // 4 epilogue warps x 2 KiB
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + 4 * 2048);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* prefix = const_cast<int*>(abort_flag) + 1;   // [n_groups + 1] first tile of every group

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_f = (p.N + BF - 1) / BF;
    const int num_k = (p.K + BK - 1) / BK;
    const int n_groups = p.grouped ? p.n_groups : 1;

    // ---- what does not read another kernel's output: barriers, TMEM, descriptor prefetch
    if (warp == 0 && lane == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 4);
        }
        tc::mbar_fence_init();
        tc::prefetch_tensormap(&mapW);
        tc::prefetch_tensormap(&mapX);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, TMEM_COLS);
    if (!p.early) pdl_wait();
    // ---- tile table: group g owns tiles [prefix[g], prefix[g+1]); within it tile = token_tile * tiles_f + feature_tile
    if (warp == 0) {
        int base = 0;
        for (int g0 = 0; g0 < n_groups; g0 += 32) {
            const int g = g0 + lane;
            int cnt = 0;
            if (g < n_groups) {
                const int rows = p.grouped ? p.offsets[g + 1] - p.offsets[g] : p.M;
                cnt = ((rows + NT - 1) / NT) * tiles_f;
            }
            int inc = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int nb = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += nb;
            }
            if (g < n_groups) prefix[g] = base + inc - cnt;
            base += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) prefix[n_groups] = base;
    }
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    pdl_launch_dependents();   // after this CTA holds its TMEM: a dependent that becomes resident early cannot take it
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[n_groups];

    struct Tile {
        int g, f0, row0, rows, w_in, w_out;   // row0: first memory row of the token tile; rows: live tokens in it
        int pk_row;                           // packed weights: row of the tile's first k-tile
    };
    auto locate = [&](int t) {
        int lo = 0, hi = n_groups - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= t) lo = mid; else hi = mid - 1;
        }
        Tile x;
        x.g = lo;
        const int in = t - prefix[lo];
        const int t0 = (in / tiles_f) * NT;
        x.f0 = (in % tiles_f) * BF;
        int seg_lo = 0, seg_n = p.M;
        if (p.grouped) {
            seg_lo = p.offsets[lo];
            seg_n = p.offsets[lo + 1] - seg_lo;
        }
        x.row0 = seg_lo + t0;
        x.rows = min(NT, seg_n - t0);
        x.w_in = lo * p.w_goff_inner;
        x.w_out = lo * p.w_goff_outer;
        x.pk_row = (lo * tiles_f + in % tiles_f) * num_k * BF;
        return x;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            const auto load_w = [&](const Tile& x, int kt, int s) {
                uint8_t* w_s = tiles + s * STAGE_BYTES;
                tc::mbar_expect_tx(&full[s], STAGE_BYTES);   // the stage's weights and tokens
                if (p.w_packed) {   // the stage's 16 KiB are contiguous in memory: one box of 128 rows x 128 bytes
                    tc::tma_load_2d(w_s, &mapW, 0, x.pk_row + kt * BF, &full[s]);
                } else {
                    tc::tma_load_2d(w_s, &mapW, x.f0 + x.w_in, kt * BK + x.w_out, &full[s]);          // 64 features x 64 k rows
                    tc::tma_load_2d(w_s + 8192, &mapW, x.f0 + 64 + x.w_in, kt * BK + x.w_out, &full[s]);
                }
            };
            // Weights that do not depend on the previous kernel: the ring is filled with them while that kernel is still
            // running (this CTA is resident early under programmatic dependent launch); the tokens follow after the wait.
            uint32_t n_pre = 0;
            if (p.early) {
                for (int t = blockIdx.x; t < total_tiles && n_pre < STAGES; t += gridDim.x) {
                    const Tile x = locate(t);
                    for (int kt = 0; kt < num_k && n_pre < STAGES; ++kt, ++n_pre) load_w(x, kt, n_pre);
                }
                pdl_wait();
            }
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const Tile x = locate(t);
                for (int kt = 0; kt < num_k; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (it >= n_pre) {
                        if (it >= STAGES && !tc::mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag, p.err_word, 111)) {
                            ok = false;
                            break;
                        }
                        load_w(x, kt, s);
                    }
                    tc::tma_load_2d(tiles + s * STAGE_BYTES + W_BYTES, &mapX, kt * BK, x.row0, &full[s]);   // 64 k x NT token rows
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (one thread)
        constexpr uint32_t IDESC = tc::idesc_bf16_f32(BF, NT, 1, 0);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version 1, 128-byte swizzle
        constexpr uint32_t W_LBO = 8192u >> 4, X_LBO = 16u >> 4;
        constexpr uint32_t W_K16 = 2048u >> 4, X_K16 = 32u >> 4;               // per k16 step, in 16-byte units
        const uint32_t w_lo0 = ((tc::smem_u32(tiles) >> 4) & 0x3FFF) | (W_LBO << 16);
        const uint32_t x_lo0 = (((tc::smem_u32(tiles) + W_BYTES) >> 4) & 0x3FFF) | (X_LBO << 16);
        if (lane == 0) {
            bool ok = true;
            uint32_t it = 0;
            int tl = 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tl) {
                const int buf = tl & 1;
                const uint32_t tmem_acc = tmem_base + buf * NT;
                if (tl >= 2) ok = tc::mbar_wait(&acc_empty[buf], ((tl >> 1) - 1) & 1, abort_flag, p.err_word, 114);
                tc::tcgen05_fence_after();
                for (int kt = 0; kt < num_k && ok; ++kt, ++it) {
                    const uint32_t s = it % STAGES;
                    ok = tc::mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, p.err_word, 112);
                    if (!ok) break;
                    tc::tcgen05_fence_after();
                    const uint32_t w_lo = w_lo0 + s * (STAGE_BYTES >> 4), x_lo = x_lo0 + s * (STAGE_BYTES >> 4);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16)
                        tc::umma_bf16(tmem_acc, ((uint64_t)DESC_HI << 32) | (w_lo + k16 * W_K16),
                                      ((uint64_t)DESC_HI << 32) | (x_lo + k16 * X_K16), IDESC, (kt > 0 || k16 > 0) ? 1u : 0u);
                    tc::umma_commit(&empty[s]);
                    if (kt == num_k - 1) tc::umma_commit(&acc_full[buf]);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        // A warp owns the 32 features of its TMEM lane quarter. 16 tokens at a time: tcgen05.ld (a feature per lane) ->
        // the warp's 2 KiB of shared memory as [token][feature] -> global memory with 8 lanes on each token's 128 bytes
        // (16-byte accesses), where bias, activation, accumulation and the row map are applied.
        const int q = warp & 3;
        if (p.early) pdl_wait();   // the output rows may be the previous kernel's (accumulate) or its inputs'
        float* stg = reinterpret_cast<float*>(staging + q * 2048);
        const int col4 = lane & 7, rsub = lane >> 3;   // store phase: features 4 col4 .. + 3 of token row 4 i + rsub
        const bool vec_c = p.C && (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
        const bool vec_c2 = p.C2 && (p.ldc2 & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C2) & 7) == 0;
        bool ok = true;
        int tl = 0;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tl) {
            const Tile x = locate(t);
            const int buf = tl & 1;
            const uint32_t tmem_acc = tmem_base + buf * NT;
            const int fb = x.f0 + q * 32 + col4 * 4;   // this lane's first feature in the store phase
            const bool full4 = fb + 4 <= p.N;
            float b4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (p.bias) {
                const float* bias = p.bias + (int64_t)x.g * p.bias_gstride;
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (fb + e < p.N) b4[e] = bias[fb + e];
            }
            int got = 0;
            if (lane == 0) got = tc::mbar_wait(&acc_full[buf], (tl >> 1) & 1, abort_flag, p.err_word, 113) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, got, 0) != 0;
            if (!ok) break;
            tc::tcgen05_fence_after();
#pragma unroll 1
            for (int c = 0; c < NT / 16; ++c) {
                uint32_t r[16];
                tc::tmem_ld_32x16(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 16), r);
                // lanes 0..15: memory row of token 16 c + lane of this tile (-1: past the end of the segment)
                const int tk = c * 16 + (lane & 15);
                int my_row = -1;
                if (tk < x.rows) my_row = p.c_idx ? p.c_idx[x.row0 + tk] : x.row0 + tk;
                tc::tmem_ld_wait();
                if (c == NT / 16 - 1) {   // this warp's quarter of the buffer is free for the tile after next
                    tc::tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) stg[e * 32 + lane] = __uint_as_float(r[e]);
                __syncwarp();
                int rows_m[4];
                float4 acc4[4], old4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {   // every load of the pass is issued before any is used
                    const int rr = 4 * i + rsub;
                    rows_m[i] = __shfl_sync(0xffffffffu, my_row, rr);
                    acc4[i] = *reinterpret_cast<const float4*>(stg + rr * 32 + col4 * 4);
                    old4[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (p.accumulate && p.C && rows_m[i] >= 0 && fb < p.N) {
                        const float* crow = p.C + (int64_t)rows_m[i] * p.ldc + fb;
                        if (vec_c && full4) old4[i] = *reinterpret_cast<const float4*>(crow);
                        else {
                            old4[i].x = crow[0];
                            if (fb + 1 < p.N) old4[i].y = crow[1];
                            if (fb + 2 < p.N) old4[i].z = crow[2];
                            if (fb + 3 < p.N) old4[i].w = crow[3];
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (rows_m[i] < 0 || fb >= p.N) continue;
                    float v[4] = {acc4[i].x + b4[0] + old4[i].x, acc4[i].y + b4[1] + old4[i].y, acc4[i].z + b4[2] + old4[i].z,
                                  acc4[i].w + b4[3] + old4[i].w};
                    if (p.C) {
                        float* crow = p.C + (int64_t)rows_m[i] * p.ldc + fb;
                        if (vec_c && full4) *reinterpret_cast<float4*>(crow) = make_float4(v[0], v[1], v[2], v[3]);
                        else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (fb + e < p.N) crow[e] = v[e];
                        }
                    }
                    if (p.C2) {
                        if (p.epi == EPI_SILU) {
#pragma unroll
                            for (int e = 0; e < 4; ++e) v[e] = sk_silu(v[e]);
                        }
                        const int64_t row2 = p.c2_mapped ? rows_m[i] : x.row0 + c * 16 + 4 * i + rsub;
                        __nv_bfloat16* c2 = p.C2 + row2 * p.ldc2 + fb;
                        if (vec_c2 && full4) {
                            const __nv_bfloat162 lo2 = __floats2bfloat162_rn(v[0], v[1]), hi2 = __floats2bfloat162_rn(v[2], v[3]);
                            *reinterpret_cast<uint2*>(c2) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo2),
                                                                       *reinterpret_cast<const uint32_t*>(&hi2));
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                if (fb + e < p.N) c2[e] = __float2bfloat16(v[e]);
                        }
                    }
                }
                __syncwarp();   // every lane is done with the staging rows before the next pass overwrites them
            }
        }
    }
    // ---- teardown
    tc::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(20000);   // let copies already in flight land before the CTA exits
    if (warp == 1) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

// one thread per 8 elements of the packed buffer
__global__ void __launch_bounds__(256) skinny_pack_kernel(const __nv_bfloat16* __restrict__ src, int64_t ld, int goff_in, int goff_out,
                                                          int K, int N, int tiles_f, int num_k, int64_t total8,
                                                          __nv_bfloat16* __restrict__ dst) {
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total8) return;
    const int64_t row = idx >> 3;
    const int c8 = (int)(idx & 7), kr = (int)(row & 63), half = (int)((row >> 6) & 1);
    int64_t t = row >> 7;
    const int kt = (int)(t % num_k);
    t /= num_k;
    const int ft = (int)(t % tiles_f), g = (int)(t / tiles_f);
    const int k = kt * BK + kr, f = ft * BF + half * 64 + c8 * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (k < K && f < N) {
        const __nv_bfloat16* s = src + ((int64_t)g * goff_out + k) * ld + (int64_t)g * goff_in + f;
        if (f + 8 <= N && (reinterpret_cast<uintptr_t>(s) & 15) == 0) v = *reinterpret_cast<const uint4*>(s);
        else {
            __nv_bfloat16 e[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) e[j] = f + j < N ? s[j] : __float2bfloat16(0.0f);
            v = *reinterpret_cast<const uint4*>(e);
        }
    }
    reinterpret_cast<uint4*>(dst)[idx] = v;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn sk_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

bool sk_make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows) {
    EncodeTiledFn fn = sk_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT, int ST>
int sk_launch_shape(asca_ctx* ctx, const Args& a, int64_t tiles) {
    CUtensorMap mapW, mapX;
    const bool w_ok = a.b_packed ? sk_make_map(&mapW, a.B, a.b_rows, 64, 64, 64, 128) : sk_make_map(&mapW, a.B, a.b_rows, a.b_cols, a.ldb, 64, 64);
    if (!w_ok || !sk_make_map(&mapX, a.A, a.a_rows, a.a_cols, a.lda, 64, NT))
        return asca_fail(ctx, ASCA_ERR_CUDA, "gemm_skinny: cuTensorMapEncodeTiled failed");
    SkP p{};
    p.C = a.C; p.ldc = a.ldc; p.M = a.M; p.N = a.N; p.K = a.K;
    p.bias = a.bias; p.accumulate = a.accumulate; p.c_idx = a.c_idx;
    p.offsets = a.offsets; p.n_groups = a.n_groups; p.grouped = a.group_dim == GROUP_M;
    p.w_goff_inner = a.b_goff_inner; p.w_goff_outer = a.b_goff_outer;
    p.bias_gstride = a.bias_gstride; p.epi = a.epi; p.C2 = a.C2; p.ldc2 = a.ldc2; p.c2_mapped = a.c2_mapped;
    p.w_packed = a.b_packed;
    p.early = a.b_early;
    p.err_word = ctx->err_word;
    const int n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int64_t grid = std::min<int64_t>(tiles, (int64_t)n_sm * SkShape<NT, ST>::CTAS_PER_SM);
    const size_t smem = SkShape<NT, ST>::SMEM_FIXED + (size_t)((p.grouped ? a.n_groups : 1) + 2) * 4;
    auto kern = gemm_skinny_kernel<NT, ST>;
    ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)(SkShape<NT, ST>::SMEM_FIXED + (SK_MAX_GROUPS + 2) * 4)));
    ASCA_CUDA(ctx, asca_launch(ctx, kern, dim3((unsigned)grid), dim3(THREADS), smem, mapW, mapX, p));
    ctx->launches++;
    return ASCA_OK;
}

}  // namespace

// Problems the few-row kernel takes: C = A B (+ bias) with A (rows x K) and B (K x features) as stored, dense or
// with A's rows grouped by expert, and at most 64 rows per group on average.
bool skinny_wanted(const Args& a) {
    if (a.mode != ASCA_NN || (a.group_dim != GROUP_NONE && a.group_dim != GROUP_M)) return false;
    if (a.epi != EPI_NONE && a.epi != EPI_SILU) return false;
    if (a.aux || a.c_gstride != 0 || a.K <= 0 || a.N <= 0) return false;
    if (a.group_dim == GROUP_NONE) return a.M > 0 && a.M <= 256;
    if (a.n_groups <= 0 || a.n_groups > SK_MAX_GROUPS || a.total_rows <= 0 || a.total_rows > 64 * (int64_t)a.n_groups) return false;
    // an expert's tile must not reach into its neighbour's weights: whole feature tiles and whole k-tiles
    if (!a.b_packed && a.b_goff_inner != 0 && (a.N % BF) != 0) return false;
    if (!a.b_packed && a.b_goff_outer != 0 && (a.K % BK) != 0) return false;
    return true;
}

int launch_skinny(asca_ctx* ctx, const Args& a) {
    const int64_t tiles_f = (a.N + BF - 1) / BF;
    // measurement harnesses: the weight bytes the product must stream go with the timed span
    asca_span sp(ctx, a.group_dim == GROUP_NONE ? "gemm_skinny_kernel (dense)" : "gemm_skinny_kernel (expert-grouped)",
                 2.0 * (double)a.K * (double)a.N * (a.group_dim == GROUP_NONE ? 1.0 : (double)a.n_groups));
    // One CTA per SM with the whole shared memory as its ring: a CTA's k-loop is one latency-bound stream, and what
    // keeps HBM busy is the bytes in flight per SM (10 stages of 20 KiB, or 8 of 24 KiB).
    if (a.group_dim == GROUP_NONE) {
        const int n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
        // token tiles of 32 while they still fit one wave: more CTAs streaming, and 10 of a tile's k-tiles in its ring
        if (a.M <= 32 || ((a.M + 31) / 32) * tiles_f <= n_sm) return sk_launch_shape<32, 10>(ctx, a, ((a.M + 31) / 32) * tiles_f);
        return sk_launch_shape<64, 8>(ctx, a, ((a.M + 63) / 64) * tiles_f);
    }
    return sk_launch_shape<32, 10>(ctx, a, (a.total_rows / 32 + a.n_groups) * tiles_f);
}

// Rows of a packed weight buffer (64 bf16 each) for `groups` matrices of K x N.
int64_t skinny_packed_rows(int64_t groups, int64_t K, int64_t N) {
    return groups * ((N + BF - 1) / BF) * ((K + BK - 1) / BK) * BF;
}

int skinny_pack(asca_ctx* ctx, const __nv_bfloat16* src, int64_t ld, int64_t groups, int64_t goff_inner, int64_t goff_outer,
                int64_t K, int64_t N, __nv_bfloat16* dst) {
    const int64_t total8 = skinny_packed_rows(groups, K, N) * 8;
    if (total8 == 0) return ASCA_OK;
    skinny_pack_kernel<<<(unsigned)((total8 + 255) / 256), 256, 0, ctx->stream>>>(src, ld, (int)goff_inner, (int)goff_outer, (int)K, (int)N,
                                                                                (int)((N + BF - 1) / BF), (int)((K + BK - 1) / BK), total8, dst);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // namespace gemm_tc
