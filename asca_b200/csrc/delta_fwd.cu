// Gated delta rule, forward direction, f32-exact kernels:
//   * delta_fwd_rec_kernel -- the per-step recurrence of rust/src/delta.rs:281-315 with the
//     dh x dh state split by VALUE column across CTAs. Column i of S evolves independently of
//     the others (u_i, S[.][i] and o_i only touch column i), so a chain (sequence, head) is
//     cut into dh/16 CTAs of 128 threads that share nothing; each thread keeps dh/8 state
//     elements in registers and the whole sequence runs without a block barrier inside a
//     16-step stage. State is written to HBM only at chunk boundaries (checkpoints for the
//     backward) and once at the end -- never per step as the reference kernel
//     (rust/kernels/asca.cu:276-312) does.
//   * delta_step_kernel -- the O(1) decode step (rust/src/delta.rs:356-406): one CTA per
//     (stream, head) streams S through registers once (read + write = the HBM floor).
#include "common.cuh"

#include <algorithm>

#include <cuda_bf16.h>

bool asca_tc_enabled();  // gemm.cu
namespace delta_tc {
bool available();
int forward(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
            int64_t B, int64_t T, int64_t H, int64_t dh, void* o, const float* s_init, float* s_final, float* ckpt);
}  // namespace delta_tc

namespace {

constexpr int FW = 16;        // value columns per CTA
constexpr int FAG = 8;        // key-row groups (lanes that share a column)
constexpr int FTHREADS = FW * FAG;
constexpr int FTS = 16;       // timesteps per staged block

template <typename T>
__device__ __forceinline__ float4 ld4(const T* p);
template <>
__device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x), b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

template <int DH, typename T>
__global__ void __launch_bounds__(FTHREADS) delta_fwd_rec_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ alpha,
    const float* __restrict__ beta, int B, int Tlen, int H, int chunk, T* __restrict__ o,
    const float* __restrict__ s_init, float* __restrict__ s_final, float* __restrict__ ckpt) {
    constexpr int RPT = DH / FAG;            // state rows per thread
    constexpr bool VEC = (RPT % 4) == 0;     // rows held as float4 groups
    constexpr int KQ4 = FTS * DH / 4;        // float4 units of k (or q) per stage
    constexpr int KQ_PT = (KQ4 + FTHREADS - 1) / FTHREADS;
    __shared__ __align__(16) float k_s[2][FTS][DH];
    __shared__ __align__(16) float q_s[2][FTS][DH];
    __shared__ float v_s[2][FTS][FW];
    __shared__ float a_s[2][FTS], b_s[2][FTS];
    __shared__ float o_s[FTS][FW];
    __shared__ float ck_s[DH][FW + 1];

    const int tid = threadIdx.x;
    const int ag = tid % FAG, col = tid / FAG;
    const int chain = blockIdx.y;              // b*H + h
    const int bi = chain / H, h = chain % H;
    const int i0 = blockIdx.x * FW;            // first value column of this CTA
    const int d = H * DH;
    const int64_t row0 = (int64_t)bi * Tlen;
    const int n_chunks = (Tlen + chunk - 1) / chunk;

    // row index of register slot r
    auto row_of = [&](int r) -> int {
        if (VEC) return ((r >> 2) * FAG + ag) * 4 + (r & 3);
        return r * FAG + ag;
    };

    float S[RPT];
    if (s_init) {
        const float* si = s_init + (int64_t)chain * DH * DH;
#pragma unroll
        for (int r = 0; r < RPT; ++r) S[r] = si[row_of(r) * DH + i0 + col];
    } else {
#pragma unroll
        for (int r = 0; r < RPT; ++r) S[r] = 0.0f;
    }

    // ---- staging: registers hold the next stage while the current one is consumed
    float4 pk[KQ_PT], pq[KQ_PT];
    float pv[(FTS * FW + FTHREADS - 1) / FTHREADS];
    float pa = 0.0f, pb = 0.0f;
    auto fetch = [&](int t0) {
#pragma unroll
        for (int u = 0; u < KQ_PT; ++u) {
            int idx = tid + u * FTHREADS;
            int t = idx / (DH / 4), c4 = idx % (DH / 4);
            if (idx < KQ4 && t0 + t < Tlen) {
                int64_t off = (row0 + t0 + t) * d + h * DH + c4 * 4;
                pk[u] = ld4<T>(k + off);
                pq[u] = ld4<T>(q + off);
            } else {
                pk[u] = make_float4(0, 0, 0, 0);
                pq[u] = make_float4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < (FTS * FW + FTHREADS - 1) / FTHREADS; ++u) {
            int idx = tid + u * FTHREADS;
            int t = idx / FW, c = idx % FW;
            pv[u] = (idx < FTS * FW && t0 + t < Tlen) ? to_f32<T>(v[(row0 + t0 + t) * d + h * DH + i0 + c]) : 0.0f;
        }
        if (tid < FTS && t0 + tid < Tlen) {
            pa = alpha[(row0 + t0 + tid) * H + h];
            pb = beta[(row0 + t0 + tid) * H + h];
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int u = 0; u < KQ_PT; ++u) {
            int idx = tid + u * FTHREADS;
            int t = idx / (DH / 4), c4 = idx % (DH / 4);
            if (idx < KQ4) {
                *reinterpret_cast<float4*>(&k_s[buf][t][c4 * 4]) = pk[u];
                *reinterpret_cast<float4*>(&q_s[buf][t][c4 * 4]) = pq[u];
            }
        }
#pragma unroll
        for (int u = 0; u < (FTS * FW + FTHREADS - 1) / FTHREADS; ++u) {
            int idx = tid + u * FTHREADS;
            if (idx < FTS * FW) v_s[buf][idx / FW][idx % FW] = pv[u];
        }
        if (tid < FTS) {
            a_s[buf][tid] = pa;
            b_s[buf][tid] = pb;
        }
    };

    auto write_state = [&](float* dst) {  // dst: dh x dh row-major, this CTA's column slice
#pragma unroll
        for (int r = 0; r < RPT; ++r) ck_s[row_of(r)][col] = S[r];
        __syncthreads();
        for (int idx = tid; idx < DH * FW; idx += FTHREADS) {
            int a = idx / FW, c = idx % FW;
            dst[a * DH + i0 + c] = ck_s[a][c];
        }
        __syncthreads();
    };

    fetch(0);
    int buf = 0;
    for (int t0 = 0; t0 < Tlen; t0 += FTS, buf ^= 1) {
        stash(buf);
        __syncthreads();
        if (t0 + FTS < Tlen) fetch(t0 + FTS);
        const int steps = Tlen - t0 < FTS ? Tlen - t0 : FTS;
        for (int ts = 0; ts < steps; ++ts) {
            const int t = t0 + ts;
            if (ckpt && (t % chunk) == 0)
                write_state(ckpt + ((int64_t)chain * n_chunks + t / chunk) * DH * DH);
            const float a = a_s[buf][ts], b = b_s[buf][ts];
            float kk[RPT];
            if (VEC) {
#pragma unroll
                for (int g = 0; g < RPT / 4; ++g) {
                    float4 t4 = *reinterpret_cast<const float4*>(&k_s[buf][ts][(g * FAG + ag) * 4]);
                    kk[g * 4] = t4.x; kk[g * 4 + 1] = t4.y; kk[g * 4 + 2] = t4.z; kk[g * 4 + 3] = t4.w;
                }
            } else {
#pragma unroll
                for (int r = 0; r < RPT; ++r) kk[r] = k_s[buf][ts][r * FAG + ag];
            }
            float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
            for (int r = 0; r < RPT; r += 2) {
                p0 = fmaf(S[r], kk[r], p0);
                if (r + 1 < RPT) p1 = fmaf(S[r + 1], kk[r + 1], p1);
            }
            float sk = p0 + p1;
#pragma unroll
            for (int off = 1; off < FAG; off <<= 1) sk += __shfl_xor_sync(0xffffffffu, sk, off);
            const float u = b * (v_s[buf][ts][col] - a * sk);
#pragma unroll
            for (int r = 0; r < RPT; ++r) S[r] = fmaf(kk[r], u, a * S[r]);
            if (VEC) {
#pragma unroll
                for (int g = 0; g < RPT / 4; ++g) {
                    float4 t4 = *reinterpret_cast<const float4*>(&q_s[buf][ts][(g * FAG + ag) * 4]);
                    kk[g * 4] = t4.x; kk[g * 4 + 1] = t4.y; kk[g * 4 + 2] = t4.z; kk[g * 4 + 3] = t4.w;
                }
            } else {
#pragma unroll
                for (int r = 0; r < RPT; ++r) kk[r] = q_s[buf][ts][r * FAG + ag];
            }
            p0 = 0.0f; p1 = 0.0f;
#pragma unroll
            for (int r = 0; r < RPT; r += 2) {
                p0 = fmaf(S[r], kk[r], p0);
                if (r + 1 < RPT) p1 = fmaf(S[r + 1], kk[r + 1], p1);
            }
            float po = p0 + p1;
#pragma unroll
            for (int off = 1; off < FAG; off <<= 1) po += __shfl_xor_sync(0xffffffffu, po, off);
            if (ag == 0) o_s[ts][col] = po;
        }
        __syncthreads();
        for (int idx = tid; idx < steps * FW; idx += FTHREADS) {
            int ts = idx / FW, c = idx % FW;
            o[(row0 + t0 + ts) * d + h * DH + i0 + c] = from_f32<T>(o_s[ts][c]);
        }
        // the next iteration's first barrier (after stash) orders these reads of o_s
        // against the next stage's writes
    }
    if (s_final) write_state(s_final + (int64_t)chain * DH * DH);
}

// ------------------------------------------------------------------ decode step
template <int DH>
struct StepCfg {
    static constexpr int THREADS = DH >= 32 ? 256 : 64;
    static constexpr int CV = DH / 4;            // float4 columns
    static constexpr int RG = THREADS / CV;      // row groups
    static constexpr int RPT = DH / RG;          // rows per thread
};

template <int DH>
__global__ void __launch_bounds__(StepCfg<DH>::THREADS) delta_step_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    const float* __restrict__ alpha, const float* __restrict__ beta, float* __restrict__ S, int H, int fused,
    float* __restrict__ o) {
    using C = StepCfg<DH>;
    __shared__ __align__(16) float qs[DH], ks[DH], vs[DH];
    __shared__ __align__(16) float red[C::RG][DH];
    __shared__ float rsum[33];
    __shared__ float ab[2];
    const int tid = threadIdx.x;
    const int unit = blockIdx.x;  // stream*H + h
    const int s = unit / H, h = unit % H;
    const int d = H * DH;
    // ---- inputs (optionally the fused prologue: L2 normalise + sigmoid)
    if (fused) {
        const float* row = q + (int64_t)s * 3 * d + h * DH;
        float qv = 0.0f, kv = 0.0f;
        if (tid < DH) {
            qv = row[tid];
            kv = row[d + tid];
            vs[tid] = row[2 * d + tid];
        }
        const float qq = block_sum(qv * qv, rsum);
        const float kk2 = block_sum(kv * kv, rsum);
        const float qi = 1.0f / fmaxf(sqrtf(qq), 1e-8f), ki = 1.0f / fmaxf(sqrtf(kk2), 1e-8f);
        if (tid < DH) {
            qs[tid] = qv * qi;
            ks[tid] = kv * ki;
        }
        if (tid == 0) {
            ab[0] = 1.0f / (1.0f + expf(-alpha[(int64_t)s * 2 * H + h]));
            ab[1] = 1.0f / (1.0f + expf(-alpha[(int64_t)s * 2 * H + H + h]));
        }
    } else {
        if (tid < DH) {
            qs[tid] = q[(int64_t)s * d + h * DH + tid];
            ks[tid] = k[(int64_t)s * d + h * DH + tid];
            vs[tid] = v[(int64_t)s * d + h * DH + tid];
        }
        if (tid == 0) {
            ab[0] = alpha[(int64_t)s * H + h];
            ab[1] = beta[(int64_t)s * H + h];
        }
    }
    const int cv = tid % C::CV, rg = tid / C::CV;
    float4* Sg = reinterpret_cast<float4*>(S + (int64_t)unit * DH * DH);
    float4 st[C::RPT];
#pragma unroll
    for (int r = 0; r < C::RPT; ++r) st[r] = Sg[(rg + C::RG * r) * C::CV + cv];  // loads in flight over the sync
    __syncthreads();
    const float a = ab[0], b = ab[1];
    float4 acc = make_float4(0, 0, 0, 0);
#pragma unroll
    for (int r = 0; r < C::RPT; ++r) {
        const float ka = ks[rg + C::RG * r];
        acc.x = fmaf(st[r].x, ka, acc.x); acc.y = fmaf(st[r].y, ka, acc.y);
        acc.z = fmaf(st[r].z, ka, acc.z); acc.w = fmaf(st[r].w, ka, acc.w);
    }
    *reinterpret_cast<float4*>(&red[rg][cv * 4]) = acc;
    __syncthreads();
    float4 sk = make_float4(0, 0, 0, 0);
#pragma unroll
    for (int g = 0; g < C::RG; ++g) {
        float4 t = *reinterpret_cast<const float4*>(&red[g][cv * 4]);
        sk.x += t.x; sk.y += t.y; sk.z += t.z; sk.w += t.w;
    }
    const float4 vv = *reinterpret_cast<const float4*>(&vs[cv * 4]);
    const float4 u = make_float4(b * (vv.x - a * sk.x), b * (vv.y - a * sk.y), b * (vv.z - a * sk.z),
                                 b * (vv.w - a * sk.w));
    acc = make_float4(0, 0, 0, 0);
#pragma unroll
    for (int r = 0; r < C::RPT; ++r) {
        const int row = rg + C::RG * r;
        const float ka = ks[row], qa = qs[row];
        st[r].x = fmaf(ka, u.x, a * st[r].x); st[r].y = fmaf(ka, u.y, a * st[r].y);
        st[r].z = fmaf(ka, u.z, a * st[r].z); st[r].w = fmaf(ka, u.w, a * st[r].w);
        Sg[row * C::CV + cv] = st[r];
        acc.x = fmaf(st[r].x, qa, acc.x); acc.y = fmaf(st[r].y, qa, acc.y);
        acc.z = fmaf(st[r].z, qa, acc.z); acc.w = fmaf(st[r].w, qa, acc.w);
    }
    __syncthreads();  // everyone has finished reading red[] for sk
    *reinterpret_cast<float4*>(&red[rg][cv * 4]) = acc;
    __syncthreads();
    if (rg == 0) {
        float4 ov = make_float4(0, 0, 0, 0);
#pragma unroll
        for (int g = 0; g < C::RG; ++g) {
            float4 t = *reinterpret_cast<const float4*>(&red[g][cv * 4]);
            ov.x += t.x; ov.y += t.y; ov.z += t.z; ov.w += t.w;
        }
        *reinterpret_cast<float4*>(o + (int64_t)s * d + h * DH + cv * 4) = ov;
    }
}

// Decode step for head dim 64, one WARP per (stream, head): lane l owns value columns 2l and 2l+1 of the 64 x 64
// state, all 64 rows (64 float2 loads issued back to back, 256 contiguous bytes per row across the warp). Every
// per-column quantity (S^T k, u, the update, S^T q) is local to the lane, so the step needs no block barrier and
// no cross-lane reduction except the two norms of the fused prologue; k and q are broadcast from the warp's slice
// of shared memory. qkv / gate may be the two parts of one wider row (row pitches ld_qkv, ld_gate); o16, when
// given, receives a bf16 copy of the output for a following tensor-core product.
constexpr int SW_WARPS = 8;
__global__ void __launch_bounds__(SW_WARPS * 32) delta_step_warp64_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ alpha,
    const float* __restrict__ beta, float* __restrict__ S, int64_t n_units, int H, int fused, int64_t ld_qkv,
    int64_t ld_gate, float* __restrict__ o, __nv_bfloat16* __restrict__ o16) {
    constexpr int DH = 64;
    __shared__ __align__(16) float kq_s[SW_WARPS][2][DH];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    bool waited = false;   // the state is this kernel's own (last written a step ago): the first unit's loads are issued
                           // before the wait for the previous kernel, whose output is only q, k, v and the gates
    // The grid is at most one block per SM and block b owns the units [b n / G, (b + 1) n / G): every SM streams the same
    // number of state bytes (within one unit), which is what it takes to reach the HBM rate -- an SM cannot pull more
    // than its share, so a grid of fixed-size blocks that leaves some SMs a block short loses that share.
    const int64_t lo = n_units * blockIdx.x / gridDim.x, hi = n_units * (blockIdx.x + 1) / gridDim.x;
    for (int64_t unit = lo + w; unit < hi; unit += SW_WARPS) {   // unit = stream * H + h
    __syncwarp();   // the previous unit's k and q have been read by every lane
    const int64_t s = unit / H;
    const int h = (int)(unit % H);
    const int d = H * DH;
    float2* Sg = reinterpret_cast<float2*>(S + unit * DH * DH);
    float2 st[DH];
#pragma unroll
    for (int a = 0; a < DH; ++a) st[a] = Sg[a * 32 + lane];   // in flight while the inputs are prepared
    if (!waited) {
        pdl_wait();
        pdl_launch_dependents();
        waited = true;
    }
    float2 q2, k2, v2;
    float al, be;
    if (fused) {
        const float* row = q + s * ld_qkv + h * DH + 2 * lane;
        q2 = *reinterpret_cast<const float2*>(row);
        k2 = *reinterpret_cast<const float2*>(row + d);
        v2 = *reinterpret_cast<const float2*>(row + 2 * d);
        const float qq = warp_sum(q2.x * q2.x + q2.y * q2.y), kk = warp_sum(k2.x * k2.x + k2.y * k2.y);
        const float qi = 1.0f / fmaxf(sqrtf(qq), 1e-8f), ki = 1.0f / fmaxf(sqrtf(kk), 1e-8f);
        q2.x *= qi; q2.y *= qi; k2.x *= ki; k2.y *= ki;
        al = 1.0f / (1.0f + expf(-alpha[s * ld_gate + h]));
        be = 1.0f / (1.0f + expf(-alpha[s * ld_gate + H + h]));
    } else {
        const int64_t off = s * d + h * DH + 2 * lane;
        q2 = *reinterpret_cast<const float2*>(q + off);
        k2 = *reinterpret_cast<const float2*>(k + off);
        v2 = *reinterpret_cast<const float2*>(v + off);
        al = alpha[s * H + h];
        be = beta[s * H + h];
    }
    *reinterpret_cast<float2*>(&kq_s[w][0][2 * lane]) = k2;
    *reinterpret_cast<float2*>(&kq_s[w][1][2 * lane]) = q2;
    __syncwarp();
    const float* ks = kq_s[w][0];
    const float* qs = kq_s[w][1];
    float2 sk = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int a4 = 0; a4 < DH; a4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + a4);
        sk.x = fmaf(st[a4].x, k4.x, sk.x);         sk.y = fmaf(st[a4].y, k4.x, sk.y);
        sk.x = fmaf(st[a4 + 1].x, k4.y, sk.x);     sk.y = fmaf(st[a4 + 1].y, k4.y, sk.y);
        sk.x = fmaf(st[a4 + 2].x, k4.z, sk.x);     sk.y = fmaf(st[a4 + 2].y, k4.z, sk.y);
        sk.x = fmaf(st[a4 + 3].x, k4.w, sk.x);     sk.y = fmaf(st[a4 + 3].y, k4.w, sk.y);
    }
    const float2 u = make_float2(be * (v2.x - al * sk.x), be * (v2.y - al * sk.y));
    float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int a4 = 0; a4 < DH; a4 += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + a4), q4 = *reinterpret_cast<const float4*>(qs + a4);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float2 t = st[a4 + e];
            t.x = fmaf(kk[e], u.x, al * t.x);
            t.y = fmaf(kk[e], u.y, al * t.y);
            Sg[(a4 + e) * 32 + lane] = t;
            acc.x = fmaf(t.x, qq[e], acc.x);
            acc.y = fmaf(t.y, qq[e], acc.y);
        }
    }
    *reinterpret_cast<float2*>(o + s * d + h * DH + 2 * lane) = acc;
    if (o16) *reinterpret_cast<__nv_bfloat162*>(o16 + s * d + h * DH + 2 * lane) = __floats2bfloat162_rn(acc.x, acc.y);
    }
    if (!waited) {   // a warp without a unit
        pdl_wait();
        pdl_launch_dependents();
    }
}

template <int DH, typename T>
cudaError_t launch_fwd(cudaStream_t st, const void* q, const void* k, const void* v, const float* alpha,
                       const float* beta, int B, int T_, int H, int chunk, void* o, const float* s_init,
                       float* s_final, float* ckpt) {
    dim3 grid(DH / FW, B * H);
    delta_fwd_rec_kernel<DH, T><<<grid, FTHREADS, 0, st>>>((const T*)q, (const T*)k, (const T*)v, alpha, beta, B, T_, H,
                                                           chunk, (T*)o, s_init, s_final, ckpt);
    return cudaGetLastError();
}

}  // namespace

extern "C" {

int64_t asca_delta_ckpt_floats(int64_t B, int64_t T, int64_t H, int64_t dh, int64_t chunk) {
    if (B <= 0 || T <= 0 || H <= 0 || dh <= 0 || chunk <= 0) return 0;
    return B * H * ((T + chunk - 1) / chunk) * dh * dh;
}

int asca_delta_fwd(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
                   int64_t B, int64_t T, int64_t H, int64_t dh, int64_t chunk, int dtype, void* o, const float* s_init,
                   float* s_final, float* ckpt) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, q && k && v && alpha && beta && o, "delta_fwd: null pointer");
    ASCA_REQUIRE(ctx, B >= 0 && T >= 0 && H > 0 && B * H < 65536 && B * T < (1ll << 31), "delta_fwd: bad shape");
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "delta_fwd: unknown dtype");
    ASCA_REQUIRE(ctx, !ckpt || chunk >= 1, "delta_fwd: chunk must be >= 1 when checkpoints are requested");
    if (dh != 16 && dh != 32 && dh != 64 && dh != 128)
        return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "delta_fwd: dh must be 16, 32, 64 or 128 (got %lld)", (long long)dh);
    const uintptr_t al = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o;
    ASCA_REQUIRE(ctx, (al & 15) == 0, "delta_fwd: q, k, v, o must be 16-byte aligned");
    if (B == 0) return ASCA_OK;
    if (T == 0) {
        if (s_final) {
            if (s_init) ASCA_CUDA(ctx, cudaMemcpyAsync(s_final, s_init, (size_t)(B * H * dh * dh) * 4, cudaMemcpyDeviceToDevice, ctx->stream));
            else ASCA_CUDA(ctx, cudaMemsetAsync(s_final, 0, (size_t)(B * H * dh * dh) * 4, ctx->stream));
        }
        return ASCA_OK;
    }
    // bf16 mode, dh = 128 (or 64, zero-padded inside): chunk-parallel WY/UT form on the tensor cores (checkpoints every 64)
    if (dtype == ASCA_BF16 && (dh == 128 || dh == 64) && (!ckpt || chunk == 64) && asca_tc_enabled() && delta_tc::available())
        return delta_tc::forward(ctx, q, k, v, alpha, beta, B, T, H, dh, o, s_init, s_final, ckpt);
    if (ckpt)
        for (auto& e : ctx->dtiles)
            if (e.ckpt == (const void*)ckpt) e.ckpt = nullptr;   // kept tiles no longer match this buffer
    const int ch = ckpt ? (int)chunk : 1;
    cudaError_t e;
    asca_span sp(ctx, "delta_fwd_rec_kernel");
#define ASCA_FWD(DH_)                                                                                              \
    e = dtype == ASCA_BF16                                                                                         \
            ? launch_fwd<DH_, __nv_bfloat16>(ctx->stream, q, k, v, alpha, beta, (int)B, (int)T, (int)H, ch, o, s_init, \
                                             s_final, ckpt)                                                        \
            : launch_fwd<DH_, float>(ctx->stream, q, k, v, alpha, beta, (int)B, (int)T, (int)H, ch, o, s_init,     \
                                     s_final, ckpt)
    switch (dh) {
        case 16: ASCA_FWD(16); break;
        case 32: ASCA_FWD(32); break;
        case 64: ASCA_FWD(64); break;
        default: ASCA_FWD(128); break;
    }
#undef ASCA_FWD
    ASCA_CUDA(ctx, e);
    ctx->launches++;
    return ASCA_OK;
}

// fused = 1 only: qkv rows of pitch ld_qkv, gate rows of pitch ld_gate (both may point into one wider buffer);
// o16 (nullable) gets a bf16 copy of o. dh = 64.
int asca_delta_step_strided(asca_ctx* ctx, const float* qkv, int64_t ld_qkv, const float* gate, int64_t ld_gate, float* S,
                            int64_t n_streams, int64_t H, float* o, void* o16) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, qkv && gate && S && o && n_streams >= 0 && H > 0, "delta_step_strided: bad arguments");
    ASCA_REQUIRE(ctx, ld_qkv >= 3 * H * 64 && ld_gate >= 2 * H && (ld_qkv & 1) == 0, "delta_step_strided: bad row pitch");
    ASCA_REQUIRE(ctx, (((uintptr_t)S | (uintptr_t)o | (uintptr_t)qkv) & 7) == 0 && ((uintptr_t)o16 & 3) == 0,
                 "delta_step_strided: misaligned pointer");
    if (n_streams == 0) return ASCA_OK;
    const int64_t units = n_streams * H;
    const int64_t n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
    asca_span sp(ctx, "delta_step_warp64_kernel", (double)units * 2.0 * 64 * 64 * 4);   // state bytes read + written
    ASCA_CUDA(ctx, asca_launch(ctx, delta_step_warp64_kernel, dim3((unsigned)std::min(n_sm, ceil_div64(units, SW_WARPS))), dim3(SW_WARPS * 32), 0,
                               qkv, nullptr, nullptr, gate, nullptr, S, units, (int)H, 1, ld_qkv, ld_gate, o, (__nv_bfloat16*)o16));
    ctx->launches++;
    return ASCA_OK;
}

int asca_delta_step(asca_ctx* ctx, const float* q, const float* k, const float* v, const float* alpha,
                    const float* beta, float* S, int64_t n_streams, int64_t H, int64_t dh, int fused, float* o) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, q && alpha && S && o && (fused || (k && v && beta)), "delta_step: null pointer");
    ASCA_REQUIRE(ctx, n_streams >= 0 && H > 0 && n_streams * H < (1ll << 31), "delta_step: bad shape");
    if (dh != 16 && dh != 32 && dh != 64 && dh != 128)
        return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "delta_step: dh must be 16, 32, 64 or 128 (got %lld)", (long long)dh);
    ASCA_REQUIRE(ctx, (((uintptr_t)S | (uintptr_t)o) & 15) == 0, "delta_step: S and o must be 16-byte aligned");
    if (n_streams == 0) return ASCA_OK;
    const unsigned grid = (unsigned)(n_streams * H);
    const bool in8 = fused ? ((uintptr_t)q & 7) == 0 : (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 7) == 0;
    if (dh == 64 && in8) {   // one warp per (stream, head), no block barrier
        const int64_t units = n_streams * H;
        const int64_t n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
        delta_step_warp64_kernel<<<(unsigned)std::min(n_sm, ceil_div64(units, SW_WARPS)), SW_WARPS * 32, 0, ctx->stream>>>(
            q, k, v, alpha, beta, S, units, (int)H, fused, 3 * H * dh, 2 * H, o, nullptr);
        ASCA_CHECK_LAUNCH(ctx);
        return ASCA_OK;
    }
    switch (dh) {
        case 16: delta_step_kernel<16><<<grid, StepCfg<16>::THREADS, 0, ctx->stream>>>(q, k, v, alpha, beta, S, (int)H, fused, o); break;
        case 32: delta_step_kernel<32><<<grid, StepCfg<32>::THREADS, 0, ctx->stream>>>(q, k, v, alpha, beta, S, (int)H, fused, o); break;
        case 64: delta_step_kernel<64><<<grid, StepCfg<64>::THREADS, 0, ctx->stream>>>(q, k, v, alpha, beta, S, (int)H, fused, o); break;
        default: delta_step_kernel<128><<<grid, StepCfg<128>::THREADS, 0, ctx->stream>>>(q, k, v, alpha, beta, S, (int)H, fused, o); break;
    }
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // extern "C"
