// HBM-bound row / element kernels: RMSNorm forward and backward, residual+norm fusion,
// row gather / scatter, AdamW, and the q/k/v split + L2-normalise + gate prologue.
// Every reduction is a fixed tree (no float atomics), so results are run-to-run identical.
#include "common.cuh"

#include <cuda_bf16.h>

namespace {

// ------------------------------------------------------------------ RMSNorm
// TPR threads cooperate on one row; 256/TPR rows per CTA. Math: rust/src/tensor.rs:251-297.
template <int TPR>
__device__ __forceinline__ float row_group_sum(float v, float* red, int row_in_blk) {
    if (TPR == 32) return warp_sum(v);
    // TPR == 256: whole block
    (void)row_in_blk;
    return block_sum(v, red);
}

template <int TPR, bool RESIDUAL>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const float* __restrict__ x,
                                                          const float* __restrict__ res,
                                                          float* __restrict__ xsum, float* __restrict__ y,
                                                          float* __restrict__ inv_out, int64_t rows, int cols,
                                                          float eps) {
    __shared__ float red[33];
    constexpr int RPB = 256 / TPR;
    const int rib = threadIdx.x / TPR, tir = threadIdx.x % TPR;
    const int64_t r = (int64_t)blockIdx.x * RPB + rib;
    const bool live = r < rows;
    const float* xr = x + (live ? r : 0) * (int64_t)cols;
    const float* rr = RESIDUAL ? res + (live ? r : 0) * (int64_t)cols : nullptr;
    float* sr = RESIDUAL ? xsum + (live ? r : 0) * (int64_t)cols : nullptr;
    const bool vec = (cols & 3) == 0;
    float acc = 0.0f;
    if (live) {
        if (vec) {
            for (int c = tir * 4; c < cols; c += TPR * 4) {
                float4 a = *reinterpret_cast<const float4*>(xr + c);
                if (RESIDUAL) {
                    float4 b = *reinterpret_cast<const float4*>(rr + c);
                    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
                    *reinterpret_cast<float4*>(sr + c) = a;
                }
                acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        } else {
            for (int c = tir; c < cols; c += TPR) {
                float a = xr[c];
                if (RESIDUAL) { a += rr[c]; sr[c] = a; }
                acc += a * a;
            }
        }
    }
    float ss = row_group_sum<TPR>(acc, red, rib);
    if (!live || y == nullptr) return;
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    if (tir == 0 && inv_out) inv_out[r] = inv;
    const float* src = RESIDUAL ? sr : xr;  // own writes are visible to the writing thread
    float* yr = y + r * (int64_t)cols;
    if (vec) {
        for (int c = tir * 4; c < cols; c += TPR * 4) {
            float4 a = *reinterpret_cast<const float4*>(src + c);
            a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
            *reinterpret_cast<float4*>(yr + c) = a;
        }
    } else {
        for (int c = tir; c < cols; c += TPR) yr[c] = src[c] * inv;
    }
}

template <int TPR>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const float* __restrict__ x,
                                                          const float* __restrict__ dy, float* __restrict__ dx,
                                                          int64_t rows, int cols, float eps) {
    __shared__ float red[33];
    constexpr int RPB = 256 / TPR;
    const int rib = threadIdx.x / TPR, tir = threadIdx.x % TPR;
    const int64_t r = (int64_t)blockIdx.x * RPB + rib;
    const bool live = r < rows;
    const float* xr = x + (live ? r : 0) * (int64_t)cols;
    const float* dr = dy + (live ? r : 0) * (int64_t)cols;
    float a2 = 0.0f, ad = 0.0f;
    if (live)
        for (int c = tir; c < cols; c += TPR) {
            float a = xr[c];
            a2 += a * a;
            ad += dr[c] * a;
        }
    float ss = row_group_sum<TPR>(a2, red, rib);
    float sd = row_group_sum<TPR>(ad, red, rib);
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    const float mean = (sd * inv) / (float)cols;
    float* o = dx + r * (int64_t)cols;
    for (int c = tir; c < cols; c += TPR) o[c] = inv * (dr[c] - xr[c] * inv * mean);
}


// Warp-per-row variants for rows that fit in registers (cols % 4 == 0, cols <= 128 * NV): every
// load of the row is issued before the first use, the reduction is a warp shuffle tree, and the
// row is read from HBM exactly once.
template <int NV, bool RESIDUAL>
__global__ void __launch_bounds__(256) rmsnorm_fwd_warp_kernel(const float* __restrict__ x,
                                                               const float* __restrict__ res,
                                                               float* __restrict__ xsum, float* __restrict__ y,
                                                               float* __restrict__ inv_out, int64_t rows, int cols,
                                                               float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + r * (int64_t)cols);
    const int n4 = cols >> 2;
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < n4 ? xr[c] : make_float4(0, 0, 0, 0);
    }
    if (RESIDUAL) {
        const float4* rr = reinterpret_cast<const float4*>(res + r * (int64_t)cols);
        float4* sr = reinterpret_cast<float4*>(xsum + r * (int64_t)cols);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            if (c < n4) {
                const float4 b = rr[c];
                v[i].x += b.x; v[i].y += b.y; v[i].z += b.z; v[i].w += b.w;
                sr[c] = v[i];
            }
        }
    }
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    acc = warp_sum(acc);
    if (y == nullptr) return;
    const float inv = 1.0f / sqrtf(acc / (float)cols + eps);
    if (lane == 0 && inv_out) inv_out[r] = inv;
    float4* yr = reinterpret_cast<float4*>(y + r * (int64_t)cols);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < n4) yr[c] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
    }
}

// add (nullable, may be dx): a row added to the result -- the other branch of a residual; dx16 (nullable): bf16 copy
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_bwd_warp_kernel(const float* __restrict__ x,
                                                               const float* __restrict__ dy, float* dx,
                                                               int64_t rows, int cols, float eps, const float* add = nullptr,
                                                               __nv_bfloat16* __restrict__ dx16 = nullptr) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float4* xr = reinterpret_cast<const float4*>(x + r * (int64_t)cols);
    const float4* dr = reinterpret_cast<const float4*>(dy + r * (int64_t)cols);
    const int n4 = cols >> 2;
    const float4* ad = add ? reinterpret_cast<const float4*>(add + r * (int64_t)cols) : nullptr;
    float4 a[NV], g[NV], e[NV];   // every load of the row is issued before the reductions wait on any
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        a[i] = c < n4 ? xr[c] : make_float4(0, 0, 0, 0);
        g[i] = c < n4 ? dr[c] : make_float4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        e[i] = ad && c < n4 ? ad[c] : make_float4(0, 0, 0, 0);
    }
    float s2 = 0.0f, sd = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        s2 += a[i].x * a[i].x + a[i].y * a[i].y + a[i].z * a[i].z + a[i].w * a[i].w;
        sd += g[i].x * a[i].x + g[i].y * a[i].y + g[i].z * a[i].z + g[i].w * a[i].w;
    }
    s2 = warp_sum(s2);
    sd = warp_sum(sd);
    const float inv = 1.0f / sqrtf(s2 / (float)cols + eps);
    const float im = inv * ((sd * inv) / (float)cols);
    float4* o = reinterpret_cast<float4*>(dx + r * (int64_t)cols);
    uint2* o16 = dx16 ? reinterpret_cast<uint2*>(dx16 + r * (int64_t)cols) : nullptr;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < n4) {
            float4 v = make_float4(inv * (g[i].x - a[i].x * im), inv * (g[i].y - a[i].y * im), inv * (g[i].z - a[i].z * im),
                                   inv * (g[i].w - a[i].w * im));
            v.x += e[i].x; v.y += e[i].y; v.z += e[i].z; v.w += e[i].w;
            o[c] = v;
            if (o16) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                o16[c] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
            }
        }
    }
}

// ------------------------------------------------------------------ gather / scatter rows
template <bool SCATTER>
__global__ void __launch_bounds__(256) move_rows_kernel(const float* __restrict__ src,
                                                        const int32_t* __restrict__ idx, float* __restrict__ dst,
                                                        int64_t n_rows, int cols) {
    // one warp per row, 8 rows per CTA
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * 8 + w;
    if (r >= n_rows) return;
    const int64_t j = idx[r];
    const float* s = src + (SCATTER ? r : j) * (int64_t)cols;
    float* d = dst + (SCATTER ? j : r) * (int64_t)cols;
    if ((cols & 3) == 0) {
        for (int c = lane * 4; c < cols; c += 128)
            *reinterpret_cast<float4*>(d + c) = *reinterpret_cast<const float4*>(s + c);
    } else {
        for (int c = lane; c < cols; c += 32) d[c] = s[c];
    }
}

// ------------------------------------------------------------------ AdamW
// rust/src/tensor.rs:444-453 (the CPU path's decay, not the reference kernel's).
__device__ __forceinline__ void adamw_one(float& p, float g, float& m, float& v, float lr_t, float b1, float b2,
                                          float eps_t, float wd) {
    m = b1 * m + (1.0f - b1) * g;
    v = b2 * v + (1.0f - b2) * g * g;
    float upd = m / (sqrtf(v) + eps_t);
    p -= wd * p;
    p -= lr_t * upd;
}

__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                    float* __restrict__ m, float* __restrict__ v, int64_t n,
                                                    float lr_t, float b1, float b2, float eps_t, float wd) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
        if (i + 3 < n) {
            float4 P = *reinterpret_cast<float4*>(p + i), M = *reinterpret_cast<float4*>(m + i),
                   V = *reinterpret_cast<float4*>(v + i);
            const float4 G = *reinterpret_cast<const float4*>(g + i);
            adamw_one(P.x, G.x, M.x, V.x, lr_t, b1, b2, eps_t, wd);
            adamw_one(P.y, G.y, M.y, V.y, lr_t, b1, b2, eps_t, wd);
            adamw_one(P.z, G.z, M.z, V.z, lr_t, b1, b2, eps_t, wd);
            adamw_one(P.w, G.w, M.w, V.w, lr_t, b1, b2, eps_t, wd);
            *reinterpret_cast<float4*>(p + i) = P;
            *reinterpret_cast<float4*>(m + i) = M;
            *reinterpret_cast<float4*>(v + i) = V;
        } else {
            for (int64_t j = i; j < n; ++j) adamw_one(p[j], g[j], m[j], v[j], lr_t, b1, b2, eps_t, wd);
        }
    }
}

// One launch over a flat buffer of n_seg tensors with per-tensor lr_t / eps_t
// (the counter advances per tensor, rust/src/tensor.rs:393).
__device__ __forceinline__ void adamw_seg_body(float* __restrict__ p, const float* __restrict__ g,
                                               float* __restrict__ m, float* __restrict__ v,
                                               const int64_t* __restrict__ seg_off,
                                               const float* __restrict__ lr_t,
                                               const float* __restrict__ eps_t, int n_seg, float b1,
                                               float b2, float wd, __nv_bfloat16* __restrict__ p16) {
    const int64_t n = seg_off[n_seg];
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
                          reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
        int lo = 0, hi = n_seg - 1;  // last segment with seg_off[s] <= i
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (seg_off[mid] <= i) lo = mid; else hi = mid - 1;
        }
        int s = lo;
        float lr = lr_t[s], ep = eps_t[s];
        if (i + 4 <= seg_off[s + 1] && vec_ok) {   // the common case: four elements of one tensor, 16-byte accesses
            float4 P = *reinterpret_cast<float4*>(p + i), M = *reinterpret_cast<float4*>(m + i),
                   V = *reinterpret_cast<float4*>(v + i);
            const float4 G = *reinterpret_cast<const float4*>(g + i);
            adamw_one(P.x, G.x, M.x, V.x, lr, b1, b2, ep, wd);
            adamw_one(P.y, G.y, M.y, V.y, lr, b1, b2, ep, wd);
            adamw_one(P.z, G.z, M.z, V.z, lr, b1, b2, ep, wd);
            adamw_one(P.w, G.w, M.w, V.w, lr, b1, b2, ep, wd);
            *reinterpret_cast<float4*>(p + i) = P;
            *reinterpret_cast<float4*>(m + i) = M;
            *reinterpret_cast<float4*>(v + i) = V;
            if (p16) {   // bf16 copy of the updated weights for the next step's tensor-core products
                const __nv_bfloat162 lo2 = __floats2bfloat162_rn(P.x, P.y), hi2 = __floats2bfloat162_rn(P.z, P.w);
                *reinterpret_cast<uint2*>(p16 + i) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo2),
                                                                *reinterpret_cast<const uint32_t*>(&hi2));
            }
            continue;
        }
        const int64_t end = i + 4 < n ? i + 4 : n;
        for (int64_t j = i; j < end; ++j) {
            while (j >= seg_off[s + 1]) {
                ++s;
                lr = lr_t[s];
                ep = eps_t[s];
            }
            adamw_one(p[j], g[j], m[j], v[j], lr, b1, b2, ep, wd);
            if (p16) p16[j] = __float2bfloat16(p[j]);
        }
    }
}
__global__ void __launch_bounds__(256) adamw_seg_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                        float* __restrict__ m, float* __restrict__ v,
                                                        const int64_t* __restrict__ seg_off,
                                                        const float* __restrict__ lr_t,
                                                        const float* __restrict__ eps_t, int n_seg, float b1,
                                                        float b2, float wd, __nv_bfloat16* __restrict__ p16) {
    adamw_seg_body(p, g, m, v, seg_off, lr_t, eps_t, n_seg, b1, b2, wd, p16);
}
// The same with the segment table passed by value (up to 32 tensors): no host-to-device copy in front of the launch. A
// copy would queue on a copy engine, behind whatever long peer-to-peer transfers the data-parallel exchange has in flight.
struct AdamSegTab {
    int64_t off[33];
    float lr[32], eps[32];
};
__global__ void __launch_bounds__(256) adamw_seg_tab_kernel(float* __restrict__ p, const float* __restrict__ g,
                                                            float* __restrict__ m, float* __restrict__ v,
                                                            const __grid_constant__ AdamSegTab tab, int n_seg, float b1,
                                                            float b2, float wd, __nv_bfloat16* __restrict__ p16) {
    adamw_seg_body(p, g, m, v, tab.off, tab.lr, tab.eps, n_seg, b1, b2, wd, p16);
}

// ------------------------------------------------------------------ delta prologue
// rust/src/delta.rs:134-179: split, per-head L2 normalise (z / max(|z|, 1e-8)), sigmoids.
// One warp per (row, head).
__global__ void __launch_bounds__(256) delta_prep_kernel(const float* __restrict__ qkv,
                                                         const float* __restrict__ gate, int64_t N, int H, int dh,
                                                         float* __restrict__ q, float* __restrict__ k,
                                                         float* __restrict__ v, float* __restrict__ qn,
                                                         float* __restrict__ kn, float* __restrict__ alpha,
                                                         float* __restrict__ beta) {
    const int lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= N * H) return;
    const int64_t r = unit / H;
    const int h = (int)(unit % H);
    const int d = H * dh;
    const float* src = qkv + r * 3 * (int64_t)d + h * dh;
    float sq = 0.0f, sk = 0.0f;
    for (int c = lane; c < dh; c += 32) {
        float a = src[c], b = src[d + c];
        sq += a * a;
        sk += b * b;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float nq = fmaxf(sqrtf(sq), 1e-8f), nk = fmaxf(sqrtf(sk), 1e-8f);
    const int64_t o = r * (int64_t)d + h * dh;
    for (int c = lane; c < dh; c += 32) {
        q[o + c] = src[c] / nq;
        k[o + c] = src[d + c] / nk;
        v[o + c] = src[2 * d + c];
    }
    if (lane == 0) {
        qn[r * H + h] = nq;
        kn[r * H + h] = nk;
        alpha[r * H + h] = 1.0f / (1.0f + expf(-gate[r * 2 * H + h]));
        beta[r * H + h] = 1.0f / (1.0f + expf(-gate[r * 2 * H + H + h]));
    }
}

inline bool warp_rows_ok(int64_t cols, const void* a, const void* b) {
    return (cols & 3) == 0 && cols <= 2048 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
}

}  // namespace

extern "C" {

int asca_rmsnorm_fwd(asca_ctx* ctx, const float* x, float* y, float* inv, int64_t rows, int64_t cols, float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && y && rows >= 0 && cols > 0 && cols < (1 << 30), "rmsnorm_fwd: bad arguments");
    if (rows == 0) return ASCA_OK;
    if (warp_rows_ok(cols, x, y)) {
        const unsigned grid = (unsigned)ceil_div64(rows, 8);
#define ASCA_RN(NV_) rmsnorm_fwd_warp_kernel<NV_, false><<<grid, 256, 0, ctx->stream>>>(x, nullptr, nullptr, y, inv, rows, (int)cols, eps)
        if (cols <= 512) ASCA_RN(4); else if (cols <= 1024) ASCA_RN(8); else ASCA_RN(16);
#undef ASCA_RN
        ASCA_CHECK_LAUNCH(ctx);
        return ASCA_OK;
    }
    if (cols <= 512)
        rmsnorm_fwd_kernel<32, false><<<(unsigned)ceil_div64(rows, 8), 256, 0, ctx->stream>>>(x, nullptr, nullptr, y, inv, rows, (int)cols, eps);
    else
        rmsnorm_fwd_kernel<256, false><<<(unsigned)rows, 256, 0, ctx->stream>>>(x, nullptr, nullptr, y, inv, rows, (int)cols, eps);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_residual_rmsnorm(asca_ctx* ctx, const float* x, const float* yadd, float* x_mid, float* xn, int64_t rows,
                          int64_t cols, float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && yadd && x_mid && rows >= 0 && cols > 0 && cols < (1 << 30), "residual_rmsnorm: bad arguments");
    if (rows == 0) return ASCA_OK;
    if (warp_rows_ok(cols, x, yadd) && warp_rows_ok(cols, x_mid, xn ? xn : x_mid)) {
        const unsigned grid = (unsigned)ceil_div64(rows, 8);
#define ASCA_RN(NV_) rmsnorm_fwd_warp_kernel<NV_, true><<<grid, 256, 0, ctx->stream>>>(x, yadd, x_mid, xn, nullptr, rows, (int)cols, eps)
        if (cols <= 512) ASCA_RN(4); else if (cols <= 1024) ASCA_RN(8); else ASCA_RN(16);
#undef ASCA_RN
        ASCA_CHECK_LAUNCH(ctx);
        return ASCA_OK;
    }
    if (cols <= 512)
        rmsnorm_fwd_kernel<32, true><<<(unsigned)ceil_div64(rows, 8), 256, 0, ctx->stream>>>(x, yadd, x_mid, xn, nullptr, rows, (int)cols, eps);
    else
        rmsnorm_fwd_kernel<256, true><<<(unsigned)rows, 256, 0, ctx->stream>>>(x, yadd, x_mid, xn, nullptr, rows, (int)cols, eps);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_moe_combine(asca_ctx* ctx, const float* x_mid, const float* moe_out, float* x_out, float* xn_next,
                     int64_t rows, int64_t cols, float eps) {
    return asca_residual_rmsnorm(ctx, x_mid, moe_out, x_out, xn_next, rows, cols, eps);
}

}  // extern "C"

// dx = add + rmsnorm_bwd(x, dy) with a bf16 copy, one pass (the residual join of the backward: the gradient through the
// norm meets the gradient of the skip branch). ASCA_ERR_UNSUPPORTED, nothing launched, when the rows do not fit the
// warp-per-row kernel; add may be dx.
int asca_rmsnorm_bwd_add_cast(asca_ctx* ctx, const float* x, const float* dy, const float* add, float* dx, void* dx16, int64_t rows,
                              int64_t cols, float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    if (!(warp_rows_ok(cols, x, dy) && warp_rows_ok(cols, dx, add)) || (reinterpret_cast<uintptr_t>(dx16) & 7)) return ASCA_ERR_UNSUPPORTED;
    if (rows == 0) return ASCA_OK;
    const unsigned grid = (unsigned)ceil_div64(rows, 8);
#define ASCA_RN(NV_) rmsnorm_bwd_warp_kernel<NV_><<<grid, 256, 0, ctx->stream>>>(x, dy, dx, rows, (int)cols, eps, add, (__nv_bfloat16*)dx16)
    if (cols <= 512) ASCA_RN(4); else if (cols <= 1024) ASCA_RN(8); else ASCA_RN(16);
#undef ASCA_RN
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

extern "C" {

int asca_rmsnorm_bwd(asca_ctx* ctx, const float* x, const float* dy, float* dx, int64_t rows, int64_t cols, float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && dy && dx && rows >= 0 && cols > 0 && cols < (1 << 30), "rmsnorm_bwd: bad arguments");
    if (rows == 0) return ASCA_OK;
    if (warp_rows_ok(cols, x, dy) && warp_rows_ok(cols, dx, dx)) {
        const unsigned grid = (unsigned)ceil_div64(rows, 8);
#define ASCA_RN(NV_) rmsnorm_bwd_warp_kernel<NV_><<<grid, 256, 0, ctx->stream>>>(x, dy, dx, rows, (int)cols, eps)
        if (cols <= 512) ASCA_RN(4); else if (cols <= 1024) ASCA_RN(8); else ASCA_RN(16);
#undef ASCA_RN
        ASCA_CHECK_LAUNCH(ctx);
        return ASCA_OK;
    }
    if (cols <= 512)
        rmsnorm_bwd_kernel<32><<<(unsigned)ceil_div64(rows, 8), 256, 0, ctx->stream>>>(x, dy, dx, rows, (int)cols, eps);
    else
        rmsnorm_bwd_kernel<256><<<(unsigned)rows, 256, 0, ctx->stream>>>(x, dy, dx, rows, (int)cols, eps);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_gather_rows(asca_ctx* ctx, const float* src, const int32_t* idx, int64_t n_rows, int64_t cols, float* dst) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, src && idx && dst && n_rows >= 0 && cols > 0 && cols < (1 << 30), "gather_rows: bad arguments");
    if (n_rows == 0) return ASCA_OK;
    move_rows_kernel<false><<<(unsigned)ceil_div64(n_rows, 8), 256, 0, ctx->stream>>>(src, idx, dst, n_rows, (int)cols);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_scatter_rows(asca_ctx* ctx, const float* src, const int32_t* idx, int64_t n_rows, int64_t cols, float* dst) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, src && idx && dst && n_rows >= 0 && cols > 0 && cols < (1 << 30), "scatter_rows: bad arguments");
    if (n_rows == 0) return ASCA_OK;
    move_rows_kernel<true><<<(unsigned)ceil_div64(n_rows, 8), 256, 0, ctx->stream>>>(src, idx, dst, n_rows, (int)cols);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_adamw(asca_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, float lr_t, float beta1,
               float beta2, float eps_t, float wd_eff) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, p && g && m && v && n >= 0, "adamw: bad arguments");
    if (n == 0) return ASCA_OK;
    int64_t blocks = ceil_div64(n, 1024);
    int64_t cap = (int64_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    adamw_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p, g, m, v, n, lr_t, beta1, beta2, eps_t, wd_eff);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_adamw_segmented_cast(asca_ctx* ctx, float* p, const float* g, float* m, float* v, const int64_t* seg_off,
                              const float* lr_t, const float* eps_t, int n_seg, float beta1, float beta2, float wd_eff,
                              void* p_bf16);

int asca_adamw_segmented(asca_ctx* ctx, float* p, const float* g, float* m, float* v, const int64_t* seg_off,
                         const float* lr_t, const float* eps_t, int n_seg, float beta1, float beta2, float wd_eff) {
    return asca_adamw_segmented_cast(ctx, p, g, m, v, seg_off, lr_t, eps_t, n_seg, beta1, beta2, wd_eff, nullptr);
}

int asca_adamw_segmented_cast(asca_ctx* ctx, float* p, const float* g, float* m, float* v, const int64_t* seg_off,
                              const float* lr_t, const float* eps_t, int n_seg, float beta1, float beta2, float wd_eff,
                              void* p_bf16) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(p_bf16) & 7) == 0, "adamw_segmented: bf16 copy must be 8-byte aligned");
    ASCA_REQUIRE(ctx, p && g && m && v && seg_off && lr_t && eps_t && n_seg > 0, "adamw_segmented: bad arguments");
    for (int i = 0; i < n_seg; ++i)
        ASCA_REQUIRE(ctx, seg_off[i] <= seg_off[i + 1], "adamw_segmented: offsets must be non-decreasing");
    const int64_t n = seg_off[n_seg];
    if (n == 0) return ASCA_OK;
    int64_t blocks = ceil_div64(n, 1024);
    const int64_t cap = (int64_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (n_seg <= 32) {   // the table travels with the launch
        AdamSegTab tab{};
        for (int i = 0; i <= n_seg; ++i) tab.off[i] = seg_off[i];
        for (int i = 0; i < n_seg; ++i) tab.lr[i] = lr_t[i], tab.eps[i] = eps_t[i];
        asca_span sp(ctx, "adamw_seg_kernel", (double)n * (p_bf16 ? 30.0 : 28.0));   // bytes read + written
        adamw_seg_tab_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p, g, m, v, tab, n_seg, beta1, beta2, wd_eff, (__nv_bfloat16*)p_bf16);
        ASCA_CHECK_LAUNCH(ctx);
        return ASCA_OK;
    }
    // table -> device scratch: [seg_off (n_seg+1) i64][lr_t n_seg f32][eps_t n_seg f32]
    size_t off_b = (size_t)(n_seg + 1) * 8, f_b = (size_t)n_seg * 4;
    void* ws;
    ASCA_TRY(asca_workspace(ctx, off_b + 2 * f_b + 256, &ws));
    char* w = (char*)ws;
    ASCA_CUDA(ctx, cudaMemcpyAsync(w, seg_off, off_b, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_CUDA(ctx, cudaMemcpyAsync(w + off_b, lr_t, f_b, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_CUDA(ctx, cudaMemcpyAsync(w + off_b + f_b, eps_t, f_b, cudaMemcpyHostToDevice, ctx->stream));
    // pageable host arrays: the copies above have been staged by the time they return
    asca_span sp(ctx, "adamw_seg_kernel", (double)n * (p_bf16 ? 30.0 : 28.0));   // bytes read + written
    adamw_seg_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(p, g, m, v, (const int64_t*)w, (const float*)(w + off_b),
                                                                 (const float*)(w + off_b + f_b), n_seg, beta1, beta2,
                                                                 wd_eff, (__nv_bfloat16*)p_bf16);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_delta_prep(asca_ctx* ctx, const float* qkv, const float* gate, int64_t N, int64_t H, int64_t dh, float* q,
                    float* k, float* v, float* qnorm, float* knorm, float* alpha, float* beta) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, qkv && gate && q && k && v && qnorm && knorm && alpha && beta && N >= 0 && H > 0 && dh > 0,
                 "delta_prep: bad arguments");
    if (N == 0) return ASCA_OK;
    delta_prep_kernel<<<(unsigned)ceil_div64(N * H, 8), 256, 0, ctx->stream>>>(qkv, gate, N, (int)H, (int)dh, q, k, v,
                                                                               qnorm, knorm, alpha, beta);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // extern "C"
