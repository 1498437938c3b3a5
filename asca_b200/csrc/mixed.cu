// bf16-mode companions of the f32 element-wise entry points: the residual stream, the norms and the
// gates stay f32; what feeds a tensor-core product is written as bf16 by the kernel that produces it.
#include "common.cuh"

#include <cuda_bf16.h>

namespace {

__device__ __forceinline__ uint2 pack4_bf16(float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

__global__ void __launch_bounds__(256) cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                        int64_t n, int vec) {
    const int64_t n4 = vec ? n >> 2 : 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 x = reinterpret_cast<const float4*>(src)[i];
        reinterpret_cast<uint2*>(dst)[i] = pack4_bf16(x.x, x.y, x.z, x.w);
    }
    for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __float2bfloat16(src[i]);
}

// Warp per row, the row held in registers (cols % 4 == 0, cols <= 128 * NV): x_mid = x (+ res), written
// when xsum is given (xsum may be x itself); xn = bf16(x_mid / sqrt(mean x_mid^2 + eps)), written to row y_row[r]
// when a row map is given (the expert-order position of the row: the MoE gather folded into the norm).
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_bf16_warp_kernel(const float* x, const float* __restrict__ res,
                                                                float* xsum, __nv_bfloat16* __restrict__ y,
                                                                int64_t rows, int cols, float eps, const int32_t* __restrict__ y_row) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    pdl_wait();
    pdl_launch_dependents();
    if (r >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + r * (int64_t)cols);
    const int n4 = cols >> 2;
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? xr[c] : make_float4(0, 0, 0, 0);
    }
    if (res) {
        const float4* rr = reinterpret_cast<const float4*>(res + r * (int64_t)cols);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            if (c < n4) {
                const float4 b = rr[c];
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
            }
        }
    }
    if (xsum) {
        float4* sr = reinterpret_cast<float4*>(xsum + r * (int64_t)cols);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            if (c < n4) sr[c] = v[i];
        }
    }
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    acc = warp_sum(acc);
    const float inv = 1.0f / sqrtf(acc / (float)cols + eps);
    uint2* yr = reinterpret_cast<uint2*>(y + (y_row ? (int64_t)y_row[r] : r) * (int64_t)cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < n4) yr[c] = pack4_bf16(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
    }
}

int residual_rmsnorm_bf16_impl(asca_ctx* ctx, const float* x, const float* yadd, float* x_mid, void* xn, int64_t rows, int64_t cols,
                               float eps, const int32_t* y_row) {
    ASCA_REQUIRE(ctx, x && xn && rows >= 0 && cols > 0, "residual_rmsnorm_bf16: bad arguments");
    ASCA_REQUIRE(ctx, (cols & 3) == 0 && cols <= 2048, "residual_rmsnorm_bf16: cols must be a multiple of 4, at most 2048");
    ASCA_REQUIRE(ctx, ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(yadd) | reinterpret_cast<uintptr_t>(x_mid)) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(xn) & 7) == 0, "residual_rmsnorm_bf16: misaligned pointer");
    if (rows == 0) return ASCA_OK;
    const unsigned grid = (unsigned)ceil_div64(rows, 8);
    __nv_bfloat16* y = (__nv_bfloat16*)xn;
    cudaError_t e;
    if (cols <= 512) e = asca_launch(ctx, rmsnorm_bf16_warp_kernel<4>, dim3(grid), dim3(256), 0, x, yadd, x_mid, y, rows, (int)cols, eps, y_row);
    else if (cols <= 1024) e = asca_launch(ctx, rmsnorm_bf16_warp_kernel<8>, dim3(grid), dim3(256), 0, x, yadd, x_mid, y, rows, (int)cols, eps, y_row);
    else e = asca_launch(ctx, rmsnorm_bf16_warp_kernel<16>, dim3(grid), dim3(256), 0, x, yadd, x_mid, y, rows, (int)cols, eps, y_row);
    ASCA_CUDA(ctx, e);
    ctx->launches++;
    return ASCA_OK;
}

// rust/src/delta.rs:134-179 with bf16 q, k, v outputs. One warp per (row, head); norms and gates f32.
// VEC: head dim 128 -- every lane holds 4 consecutive elements of q, k and v, read once.
template <bool VEC>
__global__ void __launch_bounds__(256) delta_prep_bf16_kernel(const float* __restrict__ qkv, const float* __restrict__ gate,
                                                              int64_t N, int H, int dh, __nv_bfloat16* __restrict__ q,
                                                              __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
                                                              float* __restrict__ qn, float* __restrict__ kn,
                                                              float* __restrict__ alpha, float* __restrict__ beta) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= N * H) return;
    const int64_t r = unit / H;
    const int h = (int)(unit % H);
    const int d = H * dh;
    const float* src = qkv + r * 3 * (int64_t)d + h * dh;
    const int64_t o = r * (int64_t)d + h * dh;
    float nq, nk;
    if (VEC) {
        const float4 a = reinterpret_cast<const float4*>(src)[lane], b = reinterpret_cast<const float4*>(src + d)[lane],
                     c = reinterpret_cast<const float4*>(src + 2 * d)[lane];
        const float sq = warp_sum(a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w);
        const float sk = warp_sum(b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w);
        nq = fmaxf(sqrtf(sq), 1e-8f);
        nk = fmaxf(sqrtf(sk), 1e-8f);
        reinterpret_cast<uint2*>(q + o)[lane] = pack4_bf16(a.x / nq, a.y / nq, a.z / nq, a.w / nq);
        reinterpret_cast<uint2*>(k + o)[lane] = pack4_bf16(b.x / nk, b.y / nk, b.z / nk, b.w / nk);
        reinterpret_cast<uint2*>(v + o)[lane] = pack4_bf16(c.x, c.y, c.z, c.w);
    } else {
        float sq = 0.0f, sk = 0.0f;
        for (int c = lane; c < dh; c += 32) {
            const float a = src[c], b = src[d + c];
            sq += a * a;
            sk += b * b;
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        nq = fmaxf(sqrtf(sq), 1e-8f);
        nk = fmaxf(sqrtf(sk), 1e-8f);
        for (int c = lane; c < dh; c += 32) {
            q[o + c] = __float2bfloat16(src[c] / nq);
            k[o + c] = __float2bfloat16(src[d + c] / nk);
            v[o + c] = __float2bfloat16(src[2 * d + c]);
        }
    }
    if (lane == 0) {
        qn[r * H + h] = nq;
        kn[r * H + h] = nk;
        alpha[r * H + h] = 1.0f / (1.0f + expf(-gate[r * 2 * H + h]));
        beta[r * H + h] = 1.0f / (1.0f + expf(-gate[r * 2 * H + H + h]));
    }
}

}  // namespace

// residual + RMSNorm whose bf16 rows land in expert order: row r is written to row y_row[r] of xn
int asca_residual_rmsnorm_bf16_rows(asca_ctx* ctx, const float* x, const float* yadd, float* x_mid, void* xn, int64_t rows,
                                    int64_t cols, float eps, const int32_t* y_row) {
    if (!ctx) return ASCA_ERR_ARG;
    return residual_rmsnorm_bf16_impl(ctx, x, yadd, x_mid, xn, rows, cols, eps, y_row);
}

extern "C" {

int asca_cast_bf16(asca_ctx* ctx, const float* src, void* dst, int64_t n) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, n >= 0 && (n == 0 || (src && dst)), "cast_bf16: bad arguments");
    if (n == 0) return ASCA_OK;
    const int vec = ((reinterpret_cast<uintptr_t>(src) & 15) | (reinterpret_cast<uintptr_t>(dst) & 7)) == 0;
    const int64_t blocks = std::min<int64_t>(ceil_div64((vec ? n >> 2 : n) + 1, 256), 148 * 16);
    cast_bf16_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(src, (__nv_bfloat16*)dst, n, vec);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_residual_rmsnorm_bf16(asca_ctx* ctx, const float* x, const float* yadd, float* x_mid, void* xn, int64_t rows,
                               int64_t cols, float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    return residual_rmsnorm_bf16_impl(ctx, x, yadd, x_mid, xn, rows, cols, eps, nullptr);
}

int asca_delta_prep_bf16(asca_ctx* ctx, const float* qkv, const float* gate, int64_t N, int64_t H, int64_t dh, void* q,
                         void* k, void* v, float* qnorm, float* knorm, float* alpha, float* beta) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, qkv && gate && q && k && v && qnorm && knorm && alpha && beta && N >= 0 && H > 0 && dh > 0,
                 "delta_prep_bf16: bad arguments");
    if (N == 0) return ASCA_OK;
    const bool vec = dh == 128 && (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 &&
                     ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 7) == 0;
    if (vec)
        delta_prep_bf16_kernel<true><<<(unsigned)ceil_div64(N * H, 8), 256, 0, ctx->stream>>>(
            qkv, gate, N, (int)H, (int)dh, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, qnorm, knorm, alpha, beta);
    else
        delta_prep_bf16_kernel<false><<<(unsigned)ceil_div64(N * H, 8), 256, 0, ctx->stream>>>(
            qkv, gate, N, (int)H, (int)dh, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, qnorm, knorm, alpha, beta);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // extern "C"
