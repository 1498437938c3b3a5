// Dense GEMM entry points (NN / TN / NT), the device side of Gpu::matmul and Gpu::matmul_ta
// (rust/src/cuda/mod.rs:286-344) and of Mat::matmul_t (rust/src/tensor.rs:180-201).
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"

#include <algorithm>

#include <cstdlib>

// ASCA_B200_NO_TC=1 keeps bf16 problems on the SIMT kernel (A/B comparisons).
bool asca_tc_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("ASCA_B200_NO_TC");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

namespace {

__global__ void splitk_offsets_kernel(int32_t* offs, int n_split, int chunk, int K) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= n_split) offs[i] = min(i * chunk, K);
}
// C = (accumulate ? C : 0) + bias + sum over the k-slices' partial products, slices added in order
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int n_split, int64_t mn, int N, float* __restrict__ C,
                                                            int64_t ldc, const float* __restrict__ bias, int accumulate) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= mn) return;
    const int64_t r = i / N;
    const int c = (int)(i % N);
    float acc = 0.0f;
    for (int s = 0; s < n_split; ++s) acc += part[(int64_t)s * mn + i];
    if (bias) acc += bias[c];
    float* dst = C + r * ldc + c;
    *dst = accumulate ? *dst + acc : acc;
}

// A^T B with few output tiles and a very long k (a weight gradient over all tokens of a micro-batch for a narrow
// layer: the gates, the head): the k range is cut into slices that run as the groups of the kernel's grouped-k
// form into a scratch buffer, and a second pass adds the slices in order. Returns ASCA_ERR_UNSUPPORTED when the
// shape does not call for it.
int gemm_tn_split_k(asca_ctx* ctx, gemm_tc::Args t) {
    const int n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int64_t tiles = ((int64_t)(t.M + 127) / 128) * ((t.N + 127) / 128);
    if (t.mode != ASCA_TN || tiles * 4 > n_sm || t.K < 16384) return ASCA_ERR_UNSUPPORTED;
    int n_split = (int)std::min<int64_t>(2 * n_sm / tiles, t.K / 4096);
    if (n_split < 2) return ASCA_ERR_UNSUPPORTED;
    const int chunk = (int)(((t.K + n_split - 1) / n_split + 63) / 64 * 64);
    n_split = (t.K + chunk - 1) / chunk;
    const int64_t mn = (int64_t)t.M * t.N;
    void *part = nullptr, *offs = nullptr;
    ASCA_TRY(asca_malloc(ctx, (size_t)n_split * mn * 4, &part));
    if (asca_malloc(ctx, (size_t)(n_split + 1) * 4, &offs) != ASCA_OK) {
        asca_free(ctx, part);
        return ASCA_ERR_OOM;
    }
    float* C = t.C;
    const int64_t ldc = t.ldc;
    const float* bias = t.bias;
    const int accumulate = t.accumulate;
    t.C = (float*)part; t.ldc = t.N; t.bias = nullptr; t.accumulate = 0;
    t.group_dim = gemm_tc::GROUP_K; t.offsets = (const int32_t*)offs; t.n_groups = n_split; t.total_rows = t.K;
    t.c_gstride = mn;
    int rc = gemm_tc::supported(t) ? ASCA_OK : ASCA_ERR_UNSUPPORTED;
    if (rc == ASCA_OK) {
        splitk_offsets_kernel<<<1, 256, 0, ctx->stream>>>((int32_t*)offs, n_split, chunk, t.K);
        ctx->launches++;
        rc = gemm_tc::launch(ctx, t);
    }
    if (rc == ASCA_OK) {
        splitk_reduce_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, ctx->stream>>>((const float*)part, n_split, mn, t.N, C, ldc, bias, accumulate);
        ctx->launches++;
        if (cudaGetLastError() != cudaSuccess) rc = ASCA_ERR_CUDA;
    }
    asca_free(ctx, offs);
    asca_free(ctx, part);
    return rc;
}

}  // namespace

extern "C" {

int asca_gemm(asca_ctx* ctx, int mode, int64_t M, int64_t N, int64_t K, const void* A, int64_t lda, const void* B,
              int64_t ldb, void* C, int64_t ldc, const float* bias, int accumulate, int dtype) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, mode == ASCA_NN || mode == ASCA_TN || mode == ASCA_NT, "gemm: unknown mode %d", mode);
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "gemm: unknown dtype %d", dtype);
    ASCA_REQUIRE(ctx, M >= 0 && N >= 0 && K >= 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
                 "gemm: bad shape %lld x %lld x %lld", (long long)M, (long long)N, (long long)K);
    if (M == 0 || N == 0) return ASCA_OK;
    ASCA_REQUIRE(ctx, C && (K == 0 || (A && B)), "gemm: null operand");
    const int64_t a_cols = mode == ASCA_TN ? M : K, b_cols = mode == ASCA_NT ? K : N;
    ASCA_REQUIRE(ctx, lda >= a_cols && ldb >= b_cols && ldc >= N, "gemm: leading dimension too small");
    if (dtype == ASCA_BF16 && asca_tc_enabled() && K > 0) {
        gemm_tc::Args t{};
        t.mode = mode; t.A = A; t.B = B; t.lda = lda; t.ldb = ldb;
        t.a_rows = mode == ASCA_TN ? K : M; t.a_cols = a_cols;
        t.b_rows = mode == ASCA_NT ? N : K; t.b_cols = b_cols;
        t.C = (float*)C; t.ldc = ldc; t.M = (int)M; t.N = (int)N; t.K = (int)K;
        t.bias = bias; t.accumulate = accumulate;
        t.group_dim = gemm_tc::GROUP_NONE; t.epi = gemm_tc::EPI_NONE;
        if (gemm_tc::supported(t)) {
            const int rc = gemm_tn_split_k(ctx, t);
            if (rc != ASCA_ERR_UNSUPPORTED) return rc;
            return gemm_tc::launch(ctx, t);
        }
    }
    gemm::Params p{};
    p.A = A; p.B = B; p.C = (float*)C;
    p.lda = lda; p.ldb = ldb; p.ldc = ldc;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.bias = bias;
    p.accumulate = accumulate;
    p.group_dim = gemm::GROUP_NONE;
    p.epi = gemm::EPI_NONE;
    const int bf = dtype == ASCA_BF16;
    ASCA_CUDA(ctx, gemm::launch<float>(p, mode, bf, bf, 0, ctx->stream));
    ctx->launches++;
    return ASCA_OK;
}

int asca_matmul(asca_ctx* ctx, const void* A, const void* B, void* C, int64_t M, int64_t K, int64_t N, int mode,
                int dtype) {
    const int64_t lda = mode == ASCA_TN ? M : K, ldb = mode == ASCA_NT ? K : N;
    return asca_gemm(ctx, mode, M, N, K, A, lda, B, ldb, C, N, nullptr, 0, dtype);
}

}  // extern "C"
