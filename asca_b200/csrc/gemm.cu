// Dense GEMM entry points (NN / TN / NT), the device side of Gpu::matmul and Gpu::matmul_ta
// (rust/src/cuda/mod.rs:286-344) and of Mat::matmul_t (rust/src/tensor.rs:180-201).
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"

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
        if (gemm_tc::supported(t)) return gemm_tc::launch(ctx, t);
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
