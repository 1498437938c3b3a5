// Hash-MoE expert FFN: grouped forward and backward products over the dispatch permutation,
// and the per-token decode step. Math of rust/src/model.rs:237-293 (forward), :417-495
// (backward), :309-337 (step); replaces Gpu::moe_forward_dev / moe_bwd_dev
// (rust/src/cuda/mod.rs:523-607, :745-824), which loop over experts with 7 + 10 launches and
// fresh allocations per expert. Here every product is ONE grouped launch over all experts:
// the row gather is fused into the operand load, bias + SiLU (forward) and SiLU' (backward)
// into the epilogue, and the un-permute scatter into the output store.
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"

bool asca_tc_enabled();  // gemm.cu

namespace {

// Column sums of a (rows x cols) f32 matrix, optionally per expert segment of the permuted
// order and optionally through a row map. Deterministic: each CTA owns 32 columns of one
// segment and reduces rows in a fixed order. out[g*out_gstride + c].
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ src, int64_t ld,
                                                     const int32_t* __restrict__ row_idx,
                                                     const int32_t* __restrict__ offsets, int64_t rows_total,
                                                     int cols, float* __restrict__ out, int64_t out_gstride, int accumulate) {
    __shared__ float part[8][33];
    const int g = blockIdx.y;
    const int64_t lo = offsets ? offsets[g] : 0, hi = offsets ? offsets[g + 1] : rows_total;
    const int c = blockIdx.x * 32 + (threadIdx.x & 31);
    const int w = threadIdx.x >> 5;
    float acc = 0.0f;
    if (c < cols)
        for (int64_t r = lo + w; r < hi; r += 8) {
            int64_t mr = row_idx ? (int64_t)row_idx[r] : r;
            acc += src[mr * ld + c];
        }
    part[w][threadIdx.x & 31] = acc;
    __syncthreads();
    if (w == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += part[i][threadIdx.x];
        float* o = out + (int64_t)g * out_gstride + c;
        *o = accumulate ? *o + t : t;
    }
}

// The same sums for a bf16 matrix grouped by expert segment: each CTA owns 64 columns (a lane two) of one segment.
__global__ void __launch_bounds__(256) colsum_bf16_seg_kernel(const __nv_bfloat16* __restrict__ src, int64_t ld,
                                                              const int32_t* __restrict__ offsets, int cols,
                                                              float* __restrict__ out, int64_t out_gstride, int accumulate) {
    __shared__ float2 part[8][32];
    const int g = blockIdx.y, lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t lo = offsets[g], hi = offsets[g + 1];
    const int c = blockIdx.x * 64 + 2 * lane;
    float2 acc = make_float2(0.0f, 0.0f);
    if (c < cols) {
        int64_t r = lo + w;
        for (; r + 24 < hi; r += 32) {   // four rows in flight per thread
            __nv_bfloat162 v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const __nv_bfloat162*>(src + (r + 8 * i) * ld + c);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc.x += __low2float(v[i]);
                acc.y += __high2float(v[i]);
            }
        }
        for (; r < hi; r += 8) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(src + r * ld + c);
            acc.x += __low2float(v);
            acc.y += __high2float(v);
        }
    }
    part[w][lane] = acc;
    __syncthreads();
    if (w == 0 && c < cols) {
        float2 t = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            t.x += part[i][lane].x;
            t.y += part[i][lane].y;
        }
        float* o = out + (int64_t)g * out_gstride + c;
        o[0] = accumulate ? o[0] + t.x : t.x;
        if (c + 1 < cols) o[1] = accumulate ? o[1] + t.y : t.y;
    }
}

// Decode step: one CTA per token. rmsnorm -> pre = b1[e] + xn W1[:, e] -> silu -> out = b2 + h W2[e].
template <typename T>
__global__ void __launch_bounds__(256) moe_step_kernel(const float* __restrict__ x, const uint32_t* __restrict__ ids,
                                                       const T* __restrict__ w1, const float* __restrict__ b1,
                                                       const T* __restrict__ w2, const float* __restrict__ b2, int d,
                                                       int F, int E, float* __restrict__ out) {
    extern __shared__ float sh[];  // xn[d] | hid[F] | red[33]
    float* xn = sh;
    float* hid = sh + d;
    float* red = hid + F;
    const int s = blockIdx.x;
    uint32_t h = ids[s] * 0x9E3779B1u;
    h ^= h >> 15;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    const int e = (int)(h % (uint32_t)E);
    const float* xr = x + (int64_t)s * d;
    float acc = 0.0f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) acc += xr[c] * xr[c];
    const float ss = block_sum(acc, red);
    const float inv = 1.0f / sqrtf(ss / (float)d + 1e-6f);
    for (int c = threadIdx.x; c < d; c += blockDim.x) xn[c] = xr[c] * inv;
    __syncthreads();
    const int64_t EF = (int64_t)E * F;
    for (int j = threadIdx.x; j < F; j += blockDim.x) {  // coalesced over j
        float a = b1[(int64_t)e * F + j];
        const T* col = w1 + (int64_t)e * F + j;
        for (int c = 0; c < d; ++c) a = fmaf(xn[c], to_f32<T>(col[(int64_t)c * EF]), a);
        hid[j] = a / (1.0f + expf(-a));
    }
    __syncthreads();
    for (int c = threadIdx.x; c < d; c += blockDim.x) {  // coalesced over c
        float a = b2[c];
        const T* col = w2 + (int64_t)e * F * d + c;
        for (int j = 0; j < F; ++j) a = fmaf(hid[j], to_f32<T>(col[(int64_t)j * d]), a);
        out[(int64_t)s * d + c] = a;
    }
}


// dst[r,:] = src[idx[r],:] for bf16 rows (cols % 8 == 0): 16-byte copies, one warp per row.
__global__ void __launch_bounds__(256) gather_rows_bf16_kernel(const __nv_bfloat16* __restrict__ src,
                                                               const int32_t* __restrict__ idx,
                                                               __nv_bfloat16* __restrict__ dst, int64_t n_rows,
                                                               int cols) {
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + w;
    pdl_wait();
    pdl_launch_dependents();
    if (r >= n_rows) return;
    const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)idx[r] * cols);
    uint4* d = reinterpret_cast<uint4*>(dst + r * cols);
    for (int c = lane; c < cols / 8; c += 32) d[c] = s[c];
}
// dst[r,:] = bf16(src[idx[r],:]) for f32 rows (cols % 4 == 0).
__global__ void __launch_bounds__(256) gather_rows_f32_to_bf16_kernel(const float* __restrict__ src,
                                                                      const int32_t* __restrict__ idx,
                                                                      __nv_bfloat16* __restrict__ dst, int64_t n_rows,
                                                                      int cols) {
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + w;
    if (r >= n_rows) return;
    const float4* s = reinterpret_cast<const float4*>(src + (int64_t)idx[r] * cols);
    uint2* d = reinterpret_cast<uint2*>(dst + r * cols);
    for (int c = lane; c < cols / 4; c += 32) {
        const float4 v = s[c];
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        d[c] = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    }
}

inline bool tc_shapes_ok(int64_t d, int64_t F) { return asca_tc_enabled() && d % 64 == 0 && F % 64 == 0; }

inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Tensor-core forward: permute xn once, then two grouped tcgen05 GEMMs.
int moe_fwd_tc(asca_ctx* ctx, const __nv_bfloat16* xn, const __nv_bfloat16* w1, const float* b1,
               const __nv_bfloat16* w2, const float* b2, const int32_t* perm, const int32_t* offsets, int64_t N,
               int64_t d, int64_t F, int64_t E, float* out, float* pre_p, __nv_bfloat16* hid_p) {
    void* ws;
    ASCA_TRY(asca_workspace(ctx, align256((size_t)N * d * 2) + 256, &ws));
    __nv_bfloat16* xp = (__nv_bfloat16*)ws;
    gemm_tc::Args a{};
    a.mode = ASCA_NN;
    a.A = xp; a.lda = d; a.a_rows = N; a.a_cols = d;
    a.B = w1; a.ldb = E * F; a.b_rows = d; a.b_cols = E * F; a.b_goff_inner = (int)F;
    a.C = pre_p; a.ldc = F; a.N = (int)F; a.K = (int)d;
    a.bias = b1; a.bias_gstride = F;
    a.offsets = offsets; a.n_groups = (int)E; a.group_dim = gemm_tc::GROUP_M; a.total_rows = N;
    a.epi = gemm_tc::EPI_SILU; a.C2 = hid_p; a.ldc2 = F;
    gemm_tc::Args b{};
    b.mode = ASCA_NN;
    b.A = hid_p; b.lda = F; b.a_rows = N; b.a_cols = F;
    b.B = w2; b.ldb = d; b.b_rows = E * F; b.b_cols = d; b.b_goff_outer = (int)F;
    b.C = out; b.ldc = d; b.N = (int)d; b.K = (int)F; b.c_idx = perm;
    b.bias = b2; b.bias_gstride = 0;
    b.offsets = offsets; b.n_groups = (int)E; b.group_dim = gemm_tc::GROUP_M; b.total_rows = N;
    // nothing is launched unless every product can run here: the caller falls back as a whole
    if (!gemm_tc::supported(a) || !gemm_tc::supported(b)) return ASCA_ERR_UNSUPPORTED;
    ASCA_CUDA(ctx, asca_launch(ctx, gather_rows_bf16_kernel, dim3((unsigned)ceil_div64(N, 8)), dim3(256), 0, xn, perm, xp, N, (int)d));
    ctx->launches++;
    ASCA_TRY(gemm_tc::launch(ctx, a));
    return gemm_tc::launch(ctx, b);
}

// Tensor-core backward: permuted bf16 copies of xn and dout, then four grouped tcgen05 GEMMs.
int moe_bwd_tc(asca_ctx* ctx, const __nv_bfloat16* xn, const __nv_bfloat16* w1, const __nv_bfloat16* w2,
               const float* pre_p, const __nv_bfloat16* hid_p, const float* dout, const int32_t* perm,
               const int32_t* offsets, int64_t N, int64_t d, int64_t F, int64_t E, float* d_w1, float* d_b1,
               float* d_w2, float* d_b2, float* dxn, int acc) {
    cudaStream_t s = ctx->stream;
    const size_t b_xp = align256((size_t)N * d * 2), b_dp16 = align256((size_t)N * F * 2);
    void* ws;
    ASCA_TRY(asca_workspace(ctx, 2 * b_xp + b_dp16 + 256, &ws));
    char* w = (char*)ws;
    __nv_bfloat16* xp = (__nv_bfloat16*)w;
    __nv_bfloat16* dout_p = (__nv_bfloat16*)(w + b_xp);
    __nv_bfloat16* dpre16 = (__nv_bfloat16*)(w + 2 * b_xp);
    gemm_tc::Args g1{}, g2{}, g3{}, g4{};
    // d_w2[eF+j, c] = sum_r hid_p[r,j] dout_p[r,c]
    g1.mode = ASCA_TN;
    g1.A = hid_p; g1.lda = F; g1.a_rows = N; g1.a_cols = F;
    g1.B = dout_p; g1.ldb = d; g1.b_rows = N; g1.b_cols = d;
    g1.C = d_w2; g1.ldc = d; g1.c_gstride = F * d; g1.M = (int)F; g1.N = (int)d; g1.accumulate = acc;
    g1.offsets = offsets; g1.n_groups = (int)E; g1.group_dim = gemm_tc::GROUP_K; g1.total_rows = N;
    // dpre16[r,j] = (sum_c dout_p[r,c] W2[eF+j,c]) * silu'(pre_p[r,j]), written as bf16 only: the weight-gradient product
    // below reads bf16, and the bias gradient sums the same rounded values
    g2.mode = ASCA_NT;
    g2.A = dout_p; g2.lda = d; g2.a_rows = N; g2.a_cols = d;
    g2.B = w2; g2.ldb = d; g2.b_rows = E * F; g2.b_cols = d; g2.b_goff_outer = (int)F;
    g2.C = nullptr; g2.ldc = F; g2.N = (int)F; g2.K = (int)d; g2.c2_only = 1;
    g2.offsets = offsets; g2.n_groups = (int)E; g2.group_dim = gemm_tc::GROUP_M; g2.total_rows = N;
    g2.epi = gemm_tc::EPI_SILU_BWD; g2.aux = pre_p; g2.ldaux = F; g2.C2 = dpre16; g2.ldc2 = F;
    // d_w1[c, eF+j] = sum_r xp[r,c] dpre16[r,j]
    g3.mode = ASCA_TN;
    g3.A = xp; g3.lda = d; g3.a_rows = N; g3.a_cols = d;
    g3.B = dpre16; g3.ldb = F; g3.b_rows = N; g3.b_cols = F;
    g3.C = d_w1; g3.ldc = E * F; g3.c_gstride = F; g3.M = (int)d; g3.N = (int)F; g3.accumulate = acc;
    g3.offsets = offsets; g3.n_groups = (int)E; g3.group_dim = gemm_tc::GROUP_K; g3.total_rows = N;
    // dxn[perm[r], c] = sum_j dpre16[r,j] W1[c, eF+j]
    g4.mode = ASCA_NT;
    g4.A = dpre16; g4.lda = F; g4.a_rows = N; g4.a_cols = F;
    g4.B = w1; g4.ldb = E * F; g4.b_rows = d; g4.b_cols = E * F; g4.b_goff_inner = (int)F;
    g4.C = dxn; g4.ldc = d; g4.N = (int)d; g4.K = (int)F; g4.c_idx = perm;
    g4.offsets = offsets; g4.n_groups = (int)E; g4.group_dim = gemm_tc::GROUP_M; g4.total_rows = N;
    // nothing is launched unless every product can run here: the caller falls back as a whole, and with
    // `acc` a partial run followed by the fallback would add some gradients twice
    if (!gemm_tc::supported(g1) || !gemm_tc::supported(g2) || !gemm_tc::supported(g3) || !gemm_tc::supported(g4))
        return ASCA_ERR_UNSUPPORTED;
    gather_rows_bf16_kernel<<<(unsigned)ceil_div64(N, 8), 256, 0, s>>>(xn, perm, xp, N, (int)d);
    ASCA_CHECK_LAUNCH(ctx);
    gather_rows_f32_to_bf16_kernel<<<(unsigned)ceil_div64(N, 8), 256, 0, s>>>(dout, perm, dout_p, N, (int)d);
    ASCA_CHECK_LAUNCH(ctx);
    ASCA_TRY(asca_colsum(ctx, dout, d, N, d, d_b2, acc));   // row-sliced, deterministic
    ASCA_TRY(gemm_tc::launch(ctx, g1));
    ASCA_TRY(gemm_tc::launch(ctx, g2));
    colsum_bf16_seg_kernel<<<dim3((unsigned)ceil_div64(F, 64), (unsigned)E), 256, 0, s>>>(dpre16, F, offsets, (int)F, d_b1, F, acc);
    ASCA_CHECK_LAUNCH(ctx);
    ASCA_TRY(gemm_tc::launch(ctx, g3));
    return gemm_tc::launch(ctx, g4);
}

}  // namespace

// Decode-step form of the layer, on bf16 rows already in expert order: x[perm[r], :] += silu(xp[r] W1_e + b1_e) W2_e + b2
// in place on the f32 residual rows, with a bf16 copy of the updated rows in x16. Two launches of the few-row
// kernel; ASCA_ERR_UNSUPPORTED (nothing launched) when that kernel does not take the shapes. check_only: launch nothing.
// packed: w1 and w2 point to the experts' weights in the kernel's streaming order (gemm_tc::skinny_pack).
int asca_moe_fwd_sorted_residual(asca_ctx* ctx, const __nv_bfloat16* xp, const __nv_bfloat16* w1, const float* b1,
                                 const __nv_bfloat16* w2, const float* b2, const int32_t* perm, const int32_t* offsets, int64_t N,
                                 int64_t d, int64_t F, int64_t E, float* x, __nv_bfloat16* x16, __nv_bfloat16* hid_p, int check_only,
                                 int packed) {
    if (!tc_shapes_ok(d, F) || N <= 0) return ASCA_ERR_UNSUPPORTED;
    gemm_tc::Args a{};
    a.mode = ASCA_NN;
    a.A = xp; a.lda = d; a.a_rows = N; a.a_cols = d;
    a.B = w1; a.ldb = E * F; a.b_rows = d; a.b_cols = E * F; a.b_goff_inner = (int)F;
    a.C = nullptr; a.ldc = F; a.N = (int)F; a.K = (int)d;
    a.bias = b1; a.bias_gstride = F;
    a.offsets = offsets; a.n_groups = (int)E; a.group_dim = gemm_tc::GROUP_M; a.total_rows = N;
    a.epi = gemm_tc::EPI_SILU; a.C2 = hid_p; a.ldc2 = F;
    gemm_tc::Args b{};
    b.mode = ASCA_NN;
    b.A = hid_p; b.lda = F; b.a_rows = N; b.a_cols = F;
    b.B = w2; b.ldb = d; b.b_rows = E * F; b.b_cols = d; b.b_goff_outer = (int)F;
    b.C = x; b.ldc = d; b.N = (int)d; b.K = (int)F; b.c_idx = perm; b.accumulate = 1;
    b.bias = b2; b.bias_gstride = 0;
    b.offsets = offsets; b.n_groups = (int)E; b.group_dim = gemm_tc::GROUP_M; b.total_rows = N;
    b.C2 = x16; b.ldc2 = d; b.c2_mapped = 1;
    a.b_early = b.b_early = 1;   // weights and the dispatch tables predate the kernel before each product
    if (packed) {   // w1 / w2 are skinny_pack buffers of the E expert matrices
        a.b_packed = 1; a.ldb = 64; a.b_cols = 64; a.b_rows = gemm_tc::skinny_packed_rows(E, d, F); a.b_goff_inner = 0;
        b.b_packed = 1; b.ldb = 64; b.b_cols = 64; b.b_rows = gemm_tc::skinny_packed_rows(E, F, d); b.b_goff_outer = 0;
    }
    if (!gemm_tc::skinny_wanted(a) || !gemm_tc::skinny_wanted(b) || !gemm_tc::supported(a) || !gemm_tc::supported(b))
        return ASCA_ERR_UNSUPPORTED;
    if (check_only) return ASCA_OK;
    ASCA_TRY(gemm_tc::launch_skinny(ctx, a));
    return gemm_tc::launch_skinny(ctx, b);
}

extern "C" {

int asca_moe_fwd(asca_ctx* ctx, const void* xn, const void* w1, const float* b1, const void* w2, const float* b2,
                 const int32_t* perm, const int32_t* offsets, int64_t N, int64_t d, int64_t F, int64_t E, int dtype,
                 float* out, float* pre_p, void* hid_p) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, xn && w1 && b1 && w2 && b2 && perm && offsets && out && pre_p && hid_p, "moe_fwd: null pointer");
    ASCA_REQUIRE(ctx, N >= 0 && d > 0 && F > 0 && E > 0 && N < (1ll << 31) && E * F < (1ll << 31), "moe_fwd: bad shape");
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "moe_fwd: unknown dtype");
    if (N == 0) return ASCA_OK;
    const int bf = dtype == ASCA_BF16;
    if (bf && tc_shapes_ok(d, F)) {
        int rc = moe_fwd_tc(ctx, (const __nv_bfloat16*)xn, (const __nv_bfloat16*)w1, b1, (const __nv_bfloat16*)w2, b2,
                            perm, offsets, N, d, F, E, out, pre_p, (__nv_bfloat16*)hid_p);
        if (rc != ASCA_ERR_UNSUPPORTED) return rc;
    }
    // pre_p[r,:] = xn[perm[r],:] W1[:, eF:(e+1)F] + b1[e];  hid_p = silu(pre_p)
    gemm::Params p{};
    p.A = xn; p.lda = d; p.a_idx = perm;
    p.B = w1; p.ldb = E * F; p.b_gstride = F;
    p.C = pre_p; p.ldc = F;
    p.M = 0; p.N = (int)F; p.K = (int)d;
    p.bias = b1; p.bias_gstride = F;
    p.offsets = offsets; p.n_groups = (int)E; p.group_dim = gemm::GROUP_M;
    p.epi = gemm::EPI_SILU; p.C2 = hid_p; p.ldc2 = F;
    if (bf) ASCA_CUDA(ctx, gemm::launch<__nv_bfloat16>(p, ASCA_NN, 1, 1, N, ctx->stream));
    else ASCA_CUDA(ctx, gemm::launch<float>(p, ASCA_NN, 0, 0, N, ctx->stream));
    ctx->launches++;
    // out[perm[r],:] = hid_p[r,:] W2[eF:(e+1)F,:] + b2
    gemm::Params q{};
    q.A = hid_p; q.lda = F;
    q.B = w2; q.ldb = d; q.b_gstride = F * d;
    q.C = out; q.ldc = d; q.c_idx = perm;
    q.M = 0; q.N = (int)d; q.K = (int)F;
    q.bias = b2; q.bias_gstride = 0;
    q.offsets = offsets; q.n_groups = (int)E; q.group_dim = gemm::GROUP_M;
    q.epi = gemm::EPI_NONE;
    ASCA_CUDA(ctx, gemm::launch<float>(q, ASCA_NN, bf, bf, N, ctx->stream));
    ctx->launches++;
    return ASCA_OK;
}

static int moe_bwd_impl(asca_ctx* ctx, const void* xn, const void* w1, const void* w2, const float* pre_p, const void* hid_p,
                        const float* dout, const int32_t* perm, const int32_t* offsets, int64_t N, int64_t d, int64_t F,
                        int64_t E, int dtype, float* d_w1, float* d_b1, float* d_w2, float* d_b2, float* dxn, int acc) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, xn && w1 && w2 && pre_p && hid_p && dout && perm && offsets && d_w1 && d_b1 && d_w2 && d_b2 && dxn,
                 "moe_bwd: null pointer");
    ASCA_REQUIRE(ctx, N >= 0 && d > 0 && F > 0 && E > 0 && N < (1ll << 31) && E * F < (1ll << 31), "moe_bwd: bad shape");
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "moe_bwd: unknown dtype");
    const int bf = dtype == ASCA_BF16;
    cudaStream_t s = ctx->stream;
    if (N == 0 && acc) return ASCA_OK;
    if (N == 0) {
        ASCA_CUDA(ctx, cudaMemsetAsync(d_w1, 0, (size_t)(d * E * F) * 4, s));
        ASCA_CUDA(ctx, cudaMemsetAsync(d_w2, 0, (size_t)(d * E * F) * 4, s));
        ASCA_CUDA(ctx, cudaMemsetAsync(d_b1, 0, (size_t)(E * F) * 4, s));
        ASCA_CUDA(ctx, cudaMemsetAsync(d_b2, 0, (size_t)d * 4, s));
        return ASCA_OK;
    }
    if (bf && tc_shapes_ok(d, F)) {
        int rc = moe_bwd_tc(ctx, (const __nv_bfloat16*)xn, (const __nv_bfloat16*)w1, (const __nv_bfloat16*)w2, pre_p,
                            (const __nv_bfloat16*)hid_p, dout, perm, offsets, N, d, F, E, d_w1, d_b1, d_w2, d_b2, dxn, acc);
        if (rc != ASCA_ERR_UNSUPPORTED) return rc;
    }
    // scratch: dpre_p (N x F) f32, in the permuted order
    void* ws;
    ASCA_TRY(asca_workspace(ctx, (size_t)N * F * 4 + 256, &ws));
    float* dpre_p = (float*)ws;

    // d_b2[c] = sum over all tokens of dout[t,c]
    ASCA_TRY(asca_colsum(ctx, dout, d, N, d, d_b2, acc));   // row-sliced, deterministic
    // d_w2[eF+j, c] = sum_r hid_p[r,j] dout[perm[r],c]      (TN, K = rows of expert e)
    {
        gemm::Params p{};
        p.A = hid_p; p.lda = F;
        p.B = dout; p.ldb = d; p.b_idx = perm;
        p.C = d_w2; p.ldc = d; p.c_gstride = F * d; p.accumulate = acc;
        p.M = (int)F; p.N = (int)d; p.K = 0;
        p.offsets = offsets; p.n_groups = (int)E; p.group_dim = gemm::GROUP_K;
        ASCA_CUDA(ctx, gemm::launch<float>(p, ASCA_TN, bf, 0, N, s));
        ctx->launches++;
    }
    // dpre_p[r,j] = (sum_c dout[perm[r],c] W2[eF+j,c]) * silu'(pre_p[r,j])   (NT)
    {
        gemm::Params p{};
        p.A = dout; p.lda = d; p.a_idx = perm;
        p.B = w2; p.ldb = d; p.b_gstride = F * d;
        p.C = dpre_p; p.ldc = F;
        p.M = 0; p.N = (int)F; p.K = (int)d;
        p.offsets = offsets; p.n_groups = (int)E; p.group_dim = gemm::GROUP_M;
        p.epi = gemm::EPI_SILU_BWD; p.aux = pre_p; p.ldaux = F;
        ASCA_CUDA(ctx, gemm::launch<float>(p, ASCA_NT, 0, bf, N, s));
        ctx->launches++;
    }
    // d_b1[eF+j] = sum over expert e's rows of dpre_p[r,j]
    colsum_kernel<<<dim3((unsigned)ceil_div64(F, 32), (unsigned)E), 256, 0, s>>>(dpre_p, F, nullptr, offsets, N, (int)F,
                                                                               d_b1, F, acc);
    ASCA_CHECK_LAUNCH(ctx);
    // d_w1[c, eF+j] = sum_r xn[perm[r],c] dpre_p[r,j]        (TN, K = rows of expert e)
    {
        gemm::Params p{};
        p.A = xn; p.lda = d; p.a_idx = perm;
        p.B = dpre_p; p.ldb = F;
        p.C = d_w1; p.ldc = E * F; p.c_gstride = F; p.accumulate = acc;
        p.M = (int)d; p.N = (int)F; p.K = 0;
        p.offsets = offsets; p.n_groups = (int)E; p.group_dim = gemm::GROUP_K;
        ASCA_CUDA(ctx, gemm::launch<float>(p, ASCA_TN, bf, 0, N, s));
        ctx->launches++;
    }
    // dxn[perm[r], c] = sum_j dpre_p[r,j] W1[c, eF+j]          (NT)
    {
        gemm::Params p{};
        p.A = dpre_p; p.lda = F;
        p.B = w1; p.ldb = E * F; p.b_gstride = F;
        p.C = dxn; p.ldc = d; p.c_idx = perm;
        p.M = 0; p.N = (int)d; p.K = (int)F;
        p.offsets = offsets; p.n_groups = (int)E; p.group_dim = gemm::GROUP_M;
        ASCA_CUDA(ctx, gemm::launch<float>(p, ASCA_NT, 0, bf, N, s));
        ctx->launches++;
    }
    return ASCA_OK;
}

int asca_moe_bwd(asca_ctx* ctx, const void* xn, const void* w1, const void* w2, const float* pre_p, const void* hid_p,
                 const float* dout, const int32_t* perm, const int32_t* offsets, int64_t N, int64_t d, int64_t F,
                 int64_t E, int dtype, float* d_w1, float* d_b1, float* d_w2, float* d_b2, float* dxn) {
    return moe_bwd_impl(ctx, xn, w1, w2, pre_p, hid_p, dout, perm, offsets, N, d, F, E, dtype, d_w1, d_b1, d_w2, d_b2, dxn, 0);
}

int asca_moe_bwd_acc(asca_ctx* ctx, const void* xn, const void* w1, const void* w2, const float* pre_p, const void* hid_p,
                     const float* dout, const int32_t* perm, const int32_t* offsets, int64_t N, int64_t d, int64_t F,
                     int64_t E, int dtype, float* d_w1, float* d_b1, float* d_w2, float* d_b2, float* dxn) {
    return moe_bwd_impl(ctx, xn, w1, w2, pre_p, hid_p, dout, perm, offsets, N, d, F, E, dtype, d_w1, d_b1, d_w2, d_b2, dxn, 1);
}

int asca_moe_step(asca_ctx* ctx, const float* x, const uint32_t* ids, const void* w1, const float* b1, const void* w2,
                  const float* b2, int64_t n_streams, int64_t d, int64_t F, int64_t E, int dtype, float* out) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && ids && w1 && b1 && w2 && b2 && out && n_streams >= 0 && d > 0 && F > 0 && E > 0,
                 "moe_step: bad arguments");
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "moe_step: unknown dtype");
    if (n_streams == 0) return ASCA_OK;
    const size_t smem = (size_t)(d + F + 33) * 4;
    ASCA_REQUIRE(ctx, smem <= 200 * 1024, "moe_step: d + F too large for one CTA");
    if (dtype == ASCA_BF16) {
        auto kern = moe_step_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<(unsigned)n_streams, 256, smem, ctx->stream>>>(x, ids, (const __nv_bfloat16*)w1, b1,
                                                              (const __nv_bfloat16*)w2, b2, (int)d, (int)F, (int)E, out);
    } else {
        auto kern = moe_step_kernel<float>;
        if (smem > 48 * 1024) ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<(unsigned)n_streams, 256, smem, ctx->stream>>>(x, ids, (const float*)w1, b1, (const float*)w2, b2, (int)d,
                                                              (int)F, (int)E, out);
    }
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // extern "C"
