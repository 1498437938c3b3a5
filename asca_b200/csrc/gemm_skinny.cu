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
// An accumulator lane is an output feature and a column is a token, so the epilogue's stores are coalesced
// as they come out of tcgen05.ld: for each token the 32 lanes of a warp write 32 consecutive features.
// Bias, SiLU (bf16 second output), accumulation and the row map of the MoE combine are applied there.
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

template <int NT> struct SkShape {
    static constexpr int STAGES = NT == 32 ? 5 : 8;            // 100 KiB x 2 CTAs per SM, or 192 KiB x 1
    static constexpr int X_BYTES = NT * BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;      // 20 / 24 KiB: every stage starts 1024-byte aligned
    static constexpr int TMEM_COLS = 2 * NT;                   // two accumulator buffers
    static constexpr int CTAS_PER_SM = NT == 32 ? 2 : 1;
    static constexpr size_t SMEM_FIXED = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
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
    int* err_word;
};

__device__ __forceinline__ float sk_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

template <int NT>
__global__ void __launch_bounds__(THREADS, SkShape<NT>::CTAS_PER_SM) gemm_skinny_kernel(const __grid_constant__ CUtensorMap mapW,
                                                                                       const __grid_constant__ CUtensorMap mapX,
                                                                                       const SkP p) {
    constexpr int STAGES = SkShape<NT>::STAGES, STAGE_BYTES = SkShape<NT>::STAGE_BYTES, TMEM_COLS = SkShape<NT>::TMEM_COLS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* prefix = const_cast<int*>(abort_flag) + 1;   // [n_groups + 1] first tile of every group

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_f = (p.N + BF - 1) / BF;
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
    pdl_wait();
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
    const int num_k = (p.K + BK - 1) / BK;

    struct Tile {
        int g, f0, row0, rows, w_in, w_out;   // row0: first memory row of the token tile; rows: live tokens in it
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
        return x;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const Tile x = locate(t);
                for (int kt = 0; kt < num_k; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !tc::mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag, p.err_word, 111)) {
                        ok = false;
                        break;
                    }
                    uint8_t* w_s = tiles + s * STAGE_BYTES;
                    tc::mbar_expect_tx(&full[s], STAGE_BYTES);
                    const int k0 = kt * BK;
                    tc::tma_load_2d(w_s, &mapW, x.f0 + x.w_in, k0 + x.w_out, &full[s]);              // 64 features x 64 k rows
                    tc::tma_load_2d(w_s + 8192, &mapW, x.f0 + 64 + x.w_in, k0 + x.w_out, &full[s]);
                    tc::tma_load_2d(w_s + W_BYTES, &mapX, k0, x.row0, &full[s]);                     // 64 k x NT token rows
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
        const int q = warp & 3;   // TMEM lane quarter: features f0 + 32 q + lane
        bool ok = true;
        int tl = 0;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tl) {
            const Tile x = locate(t);
            const int buf = tl & 1;
            const uint32_t tmem_acc = tmem_base + buf * NT;
            int got = 0;
            if (lane == 0) got = tc::mbar_wait(&acc_full[buf], (tl >> 1) & 1, abort_flag, p.err_word, 113) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, got, 0) != 0;
            if (!ok) break;
            tc::tcgen05_fence_after();
            const int f = x.f0 + q * 32 + lane;
            const bool f_ok = f < p.N;
            const float bias = (p.bias && f_ok) ? p.bias[(int64_t)x.g * p.bias_gstride + f] : 0.0f;
#pragma unroll 1
            for (int c = 0; c < NT / 32; ++c) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
                // memory row of token c * 32 + lane of this tile (-1: past the end of the segment)
                const int tk = c * 32 + lane;
                int my_row = -1;
                if (tk < x.rows) my_row = p.c_idx ? p.c_idx[x.row0 + tk] : x.row0 + tk;
                tc::tmem_ld_wait();
                if (c == NT / 32 - 1) {   // this warp's quarter of the buffer is free for the tile after next
                    tc::tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
                }
                float old[32];
                if (p.accumulate && p.C) {   // every load of the pass is issued before any is used
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int row = __shfl_sync(0xffffffffu, my_row, j);
                        old[j] = (row >= 0 && f_ok) ? p.C[(int64_t)row * p.ldc + f] : 0.0f;
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int row = __shfl_sync(0xffffffffu, my_row, j);
                    if (row < 0 || !f_ok) continue;
                    float v = __uint_as_float(r[j]) + bias;
                    if (p.C) {
                        if (p.accumulate) v += old[j];
                        p.C[(int64_t)row * p.ldc + f] = v;
                    }
                    if (p.C2) {
                        const float y = p.epi == EPI_SILU ? sk_silu(v) : v;
                        p.C2[(int64_t)(p.c2_mapped ? row : x.row0 + c * 32 + j) * p.ldc2 + f] = __float2bfloat16(y);
                    }
                }
            }
        }
    }
    // ---- teardown
    tc::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(20000);   // let copies already in flight land before the CTA exits
    if (warp == 1) tc::tmem_dealloc(tmem_base, TMEM_COLS);
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

template <int NT>
int sk_launch_shape(asca_ctx* ctx, const Args& a, int64_t tiles) {
    CUtensorMap mapW, mapX;
    if (!sk_make_map(&mapW, a.B, a.b_rows, a.b_cols, a.ldb, 64, 64) || !sk_make_map(&mapX, a.A, a.a_rows, a.a_cols, a.lda, 64, NT))
        return asca_fail(ctx, ASCA_ERR_CUDA, "gemm_skinny: cuTensorMapEncodeTiled failed");
    SkP p{};
    p.C = a.C; p.ldc = a.ldc; p.M = a.M; p.N = a.N; p.K = a.K;
    p.bias = a.bias; p.accumulate = a.accumulate; p.c_idx = a.c_idx;
    p.offsets = a.offsets; p.n_groups = a.n_groups; p.grouped = a.group_dim == GROUP_M;
    p.w_goff_inner = a.b_goff_inner; p.w_goff_outer = a.b_goff_outer;
    p.bias_gstride = a.bias_gstride; p.epi = a.epi; p.C2 = a.C2; p.ldc2 = a.ldc2; p.c2_mapped = a.c2_mapped;
    p.err_word = ctx->err_word;
    const int n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int64_t grid = std::min<int64_t>(tiles, (int64_t)n_sm * SkShape<NT>::CTAS_PER_SM);
    const size_t smem = SkShape<NT>::SMEM_FIXED + (size_t)((p.grouped ? a.n_groups : 1) + 2) * 4;
    auto kern = gemm_skinny_kernel<NT>;
    ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)(SkShape<NT>::SMEM_FIXED + (SK_MAX_GROUPS + 2) * 4)));
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
    if (a.b_goff_inner != 0 && (a.N % BF) != 0) return false;
    if (a.b_goff_outer != 0 && (a.K % BK) != 0) return false;
    return true;
}

int launch_skinny(asca_ctx* ctx, const Args& a) {
    const int64_t tiles_f = (a.N + BF - 1) / BF;
    if (a.group_dim == GROUP_NONE) {
        if (a.M <= 32) return sk_launch_shape<32>(ctx, a, tiles_f);
        return sk_launch_shape<64>(ctx, a, ((a.M + 63) / 64) * tiles_f);
    }
    return sk_launch_shape<32>(ctx, a, (a.total_rows / 32 + a.n_groups) * tiles_f);
}

}  // namespace gemm_tc
