// f32-accurate SIMT GEMM (FFMA, f32 accumulate) with optional row gather / scatter maps and
// expert grouping. It is the exact-mode (1e-5) engine behind asca_matmul / asca_gemm and the
// grouped expert products of the hash-MoE; operands may be f32 or bf16 and are widened to f32
// on the way into shared memory.
//
// Tiling: 128 x 128 x 16 per CTA, 256 threads, 8 x 8 outputs per thread held in registers;
// operands are staged in shared memory k-major ([k][m] and [k][n]) so the inner product reads
// two float4 per operand per k. The next k-slab is prefetched into registers while the current
// one is multiplied.
#pragma once
#include "common.cuh"

namespace gemm {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256, PAD = 4;

enum { EPI_NONE = 0, EPI_SILU = 1, EPI_SILU_BWD = 2 };
enum { GROUP_NONE = 0, GROUP_M = 1, GROUP_K = 2 };

struct Params {
    const void* A;
    const void* B;
    float* C;
    int64_t lda, ldb, ldc;
    int M, N, K;
    const float* bias;      // per output column, nullable
    int accumulate;         // C += result
    // optional maps from a logical "token" row to a memory row (int32), nullable:
    //   a_idx: rows of A's memory layout; b_idx: rows of B's memory layout (TN only);
    //   c_idx: rows of C.
    const int32_t* a_idx;
    const int32_t* b_idx;
    const int32_t* c_idx;
    // grouping (hash-MoE experts): offsets[n_groups+1] are row ranges in the permuted order.
    //   GROUP_M: group g owns logical rows [offsets[g], offsets[g+1]) of A and C (M varies).
    //   GROUP_K: group g owns memory rows  [offsets[g], offsets[g+1]) of A and B (K varies).
    // The operand that is not token-indexed moves by *_gstride elements per group.
    const int32_t* offsets;
    int n_groups;
    int group_dim;
    int64_t a_gstride, b_gstride, c_gstride, bias_gstride;
    // epilogue: EPI_SILU writes the pre-activation to C and silu to C2 (type TC2);
    // EPI_SILU_BWD multiplies by silu'(aux[row][col]) (aux rows follow the logical row).
    int epi;
    const float* aux;
    int64_t ldaux;
    void* C2;
    int64_t ldc2;
};

template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec_ok, int valid, float out[4]);

template <>
__device__ __forceinline__ void load4<float>(const float* p, bool vec_ok, int valid, float out[4]) {
    if (vec_ok && valid == 4) {
        float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = j < valid ? p[j] : 0.0f;
    }
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, bool vec_ok, int valid, float out[4]) {
    if (vec_ok && valid == 4) {
        uint2 raw = *reinterpret_cast<const uint2*>(p);
        __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
        out[0] = __low2float(a); out[1] = __high2float(a); out[2] = __low2float(b); out[3] = __high2float(b);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = j < valid ? __bfloat162float(p[j]) : 0.0f;
    }
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float p) {
    float sg = 1.0f / (1.0f + expf(-p));
    return sg * (1.0f + p * (1.0f - sg));
}

// MODE: ASCA_NN / ASCA_TN / ASCA_NT as in the public header.
template <int MODE, typename TA, typename TB, typename TC2>
__global__ void __launch_bounds__(THREADS) gemm_kernel(Params p) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Bs[BK][BN + PAD];
    __shared__ int sh_group[4];

    int M = p.M, N = p.N, K = p.K;
    int tile_m, tile_n;
    int64_t row_base = 0;   // logical row offset of this group (GROUP_M) or k offset (GROUP_K)
    const TA* A = reinterpret_cast<const TA*>(p.A);
    const TB* B = reinterpret_cast<const TB*>(p.B);
    float* C = p.C;
    const float* bias = p.bias;
    const int tiles_n = (N + BN - 1) / BN;

    if (p.group_dim == GROUP_NONE) {
        tile_n = blockIdx.x % tiles_n;
        tile_m = blockIdx.x / tiles_n;
    } else {
        // locate (group, tile) for this CTA: warp 0 scans the per-group tile counts
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            int found_g = -1, found_t = 0, base = 0;
            for (int g0 = 0; g0 < p.n_groups && found_g < 0; g0 += 32) {
                int g = g0 + lane;
                int cnt = 0;
                if (g < p.n_groups) {
                    int n_g = p.offsets[g + 1] - p.offsets[g];
                    cnt = p.group_dim == GROUP_M ? ((n_g + BM - 1) / BM) * tiles_n : ((M + BM - 1) / BM) * tiles_n;
                }
                int inc = cnt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int n = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += n;
                }
                int start = base + inc - cnt;
                bool mine = (int)blockIdx.x >= start && (int)blockIdx.x < start + cnt;
                unsigned m = __ballot_sync(0xffffffffu, mine);
                if (m) {
                    int src = __ffs(m) - 1;
                    found_g = __shfl_sync(0xffffffffu, g, src);
                    found_t = (int)blockIdx.x - __shfl_sync(0xffffffffu, start, src);
                }
                base += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (lane == 0) {
                sh_group[0] = found_g;
                sh_group[1] = found_t;
            }
        }
        __syncthreads();
        const int g = sh_group[0];
        if (g < 0) return;  // surplus CTA of the upper-bound grid
        const int t = sh_group[1];
        tile_n = t % tiles_n;
        tile_m = t / tiles_n;
        const int lo = p.offsets[g], n_g = p.offsets[g + 1] - lo;
        row_base = lo;
        if (p.group_dim == GROUP_M) {
            M = n_g;
            B += (int64_t)g * p.b_gstride;
        } else {
            K = n_g;
            C += (int64_t)g * p.c_gstride;
        }
        if (bias) bias += (int64_t)g * p.bias_gstride;
        (void)A;
    }

    const int m0 = tile_m * BM, n0 = tile_n * BN;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;

    // ---- global -> register staging descriptors
    // "k-contiguous" operand (A in NN/NT, B in NT): thread loads rows r = tid/4 + {0,64},
    // 4 consecutive k at kq = (tid%4)*4. "row-contiguous" operand (A in TN, B in NN/TN):
    // thread loads k rows kr = tid/32 + {0,8}, 4 consecutive columns at (tid%32)*4.
    constexpr bool A_KCONT = (MODE != ASCA_TN);
    constexpr bool B_KCONT = (MODE == ASCA_NT);
    const bool a_vec = ((p.lda & 3) == 0) && ((reinterpret_cast<uintptr_t>(A) & (sizeof(TA) * 4 - 1)) == 0);
    const bool b_vec = ((p.ldb & 3) == 0) && ((reinterpret_cast<uintptr_t>(B) & (sizeof(TB) * 4 - 1)) == 0);

    float ra[2][4], rb[2][4];
    int64_t a_row_off[2];  // element offset of the memory row this thread reads (k-contiguous A)
    bool a_row_ok[2];
    int64_t b_row_off[2];
    bool b_row_ok[2];
    if (A_KCONT) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int m = m0 + (tid >> 2) + h * 64;
            a_row_ok[h] = m < M;
            int64_t lr = row_base * (p.group_dim == GROUP_M) + m;
            int64_t mr = a_row_ok[h] ? (p.a_idx ? (int64_t)p.a_idx[lr] : lr) : 0;
            a_row_off[h] = mr * p.lda;
        }
    }
    if (B_KCONT) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int n = n0 + (tid >> 2) + h * 64;
            b_row_ok[h] = n < N;
            b_row_off[h] = (int64_t)(b_row_ok[h] ? n : 0) * p.ldb;
        }
    }

    auto fetch = [&](int k0) {
        if (A_KCONT) {
            const int kq = k0 + (tid & 3) * 4;
            const int valid = K - kq < 0 ? 0 : (K - kq > 4 ? 4 : K - kq);
#pragma unroll
            for (int h = 0; h < 2; ++h)
                load4<TA>(A + a_row_off[h] + kq, a_vec, a_row_ok[h] ? valid : 0, ra[h]);
        } else {  // TN: A memory is (K x M); rows are k (token rows under GROUP_K)
            const int mc = m0 + (tid & 31) * 4;
            const int valid = M - mc < 0 ? 0 : (M - mc > 4 ? 4 : M - mc);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int k = k0 + (tid >> 5) + h * 8;
                bool ok = k < K;
                int64_t lr = row_base * (p.group_dim == GROUP_K) + k;
                int64_t mr = ok ? (p.a_idx ? (int64_t)p.a_idx[lr] : lr) : 0;
                load4<TA>(A + mr * p.lda + mc, a_vec, ok ? valid : 0, ra[h]);
            }
        }
        if (B_KCONT) {
            const int kq = k0 + (tid & 3) * 4;
            const int valid = K - kq < 0 ? 0 : (K - kq > 4 ? 4 : K - kq);
#pragma unroll
            for (int h = 0; h < 2; ++h)
                load4<TB>(B + b_row_off[h] + kq, b_vec, b_row_ok[h] ? valid : 0, rb[h]);
        } else {  // B memory is (K x N)
            const int nc = n0 + (tid & 31) * 4;
            const int valid = N - nc < 0 ? 0 : (N - nc > 4 ? 4 : N - nc);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int k = k0 + (tid >> 5) + h * 8;
                bool ok = k < K;
                int64_t lr = (MODE == ASCA_TN ? row_base * (p.group_dim == GROUP_K) : 0) + k;
                int64_t mr = ok ? ((MODE == ASCA_TN && p.b_idx) ? (int64_t)p.b_idx[lr] : lr) : 0;
                load4<TB>(B + mr * p.ldb + nc, b_vec, ok ? valid : 0, rb[h]);
            }
        }
    };
    auto stash = [&]() {
        if (A_KCONT) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) As[(tid & 3) * 4 + j][(tid >> 2) + h * 64] = ra[h][j];
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
                *reinterpret_cast<float4*>(&As[(tid >> 5) + h * 8][(tid & 31) * 4]) =
                    make_float4(ra[h][0], ra[h][1], ra[h][2], ra[h][3]);
        }
        if (B_KCONT) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 4; ++j) Bs[(tid & 3) * 4 + j][(tid >> 2) + h * 64] = rb[h][j];
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
                *reinterpret_cast<float4*>(&Bs[(tid >> 5) + h * 8][(tid & 31) * 4]) =
                    make_float4(rb[h][0], rb[h][1], rb[h][2], rb[h][3]);
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    if (K > 0) {
        fetch(0);
        for (int k0 = 0; k0 < K; k0 += BK) {
            __syncthreads();
            stash();
            __syncthreads();
            if (k0 + BK < K) fetch(k0 + BK);
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                float a[8], b[8];
                float4 t;
                t = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
                a[0] = t.x; a[1] = t.y; a[2] = t.z; a[3] = t.w;
                t = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
                a[4] = t.x; a[5] = t.y; a[6] = t.z; a[7] = t.w;
                t = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
                b[0] = t.x; b[1] = t.y; b[2] = t.z; b[3] = t.w;
                t = *reinterpret_cast<const float4*>(&Bs[kk][64 + tx * 4]);
                b[4] = t.x; b[5] = t.y; b[6] = t.z; b[7] = t.w;
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
        }
    }

    // ---- epilogue
    TC2* C2 = reinterpret_cast<TC2*>(p.C2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= M) continue;
        const int64_t lr = row_base * (p.group_dim == GROUP_M) + m;
        const int64_t cr = p.c_idx ? (int64_t)p.c_idx[lr] : lr;
        float* crow = C + cr * p.ldc;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            if (p.epi == EPI_SILU_BWD) v *= silu_grad_f(p.aux[lr * p.ldaux + n]);
            if (p.accumulate) v += crow[n];
            crow[n] = v;
            if (p.epi == EPI_SILU) C2[lr * p.ldc2 + n] = from_f32<TC2>(silu_f(v));
        }
    }
}

// Number of CTAs for a launch (upper bound for GROUP_M: every group can add one ragged tile).
inline int64_t grid_size(const Params& p, int64_t total_token_rows) {
    const int64_t tn = (p.N + BN - 1) / BN;
    if (p.group_dim == GROUP_NONE) return ((p.M + BM - 1) / BM) * tn;
    if (p.group_dim == GROUP_M) return (total_token_rows / BM + p.n_groups) * tn;
    return (int64_t)p.n_groups * ((p.M + BM - 1) / BM) * tn;
}

template <typename TC2 = float>
inline cudaError_t launch(const Params& p, int mode, int a_bf16, int b_bf16, int64_t total_token_rows,
                          cudaStream_t s) {
    const int64_t g = grid_size(p, total_token_rows);
    if (g <= 0) return cudaSuccess;
    dim3 grid((unsigned)g), block(THREADS);
#define ASCA_GEMM_CASE(MD, TA_, TB_) gemm_kernel<MD, TA_, TB_, TC2><<<grid, block, 0, s>>>(p)
#define ASCA_GEMM_MODE(MD)                                                       \
    if (!a_bf16 && !b_bf16) ASCA_GEMM_CASE(MD, float, float);                    \
    else if (a_bf16 && b_bf16) ASCA_GEMM_CASE(MD, __nv_bfloat16, __nv_bfloat16); \
    else if (a_bf16) ASCA_GEMM_CASE(MD, __nv_bfloat16, float);                   \
    else ASCA_GEMM_CASE(MD, float, __nv_bfloat16)
    if (mode == ASCA_NN) { ASCA_GEMM_MODE(ASCA_NN); }
    else if (mode == ASCA_TN) { ASCA_GEMM_MODE(ASCA_TN); }
    else { ASCA_GEMM_MODE(ASCA_NT); }
#undef ASCA_GEMM_MODE
#undef ASCA_GEMM_CASE
    return cudaGetLastError();
}

}  // namespace gemm
