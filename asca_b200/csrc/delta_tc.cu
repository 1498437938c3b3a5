// Gated delta rule, bf16 mode, chunk-parallel WY/UT forward on the 5th-generation tensor cores.
//
// Chunk of C = 64 tokens, head dim 128, state S (128 x 128) kept in f32 in TMEM for the whole
// sequence. With g = cumsum(log alpha), gam = exp(g), Gam[t,i] = exp(g_t - g_i), eg = exp(g_C - g):
//
//   pre-pass (one CTA per (sequence, head, chunk) -- fully parallel, nothing depends on S):
//     KK = K K^T, QK = Q K^T                                   tcgen05, M128 N64 K128 ([K;Q] stacked)
//     L  = strictlower(beta_t Gam KK)   A = lower(Gam QK)      f32 registers
//     X  = (I + L)^-1  (T' = X - I)                            f32, 16 x 16 blocks: substitution on the
//                                                              diagonal, block products below it
//     W^ = X (beta gam K),  Uv = X (beta V)                    tcgen05, two M64 N128 K64 products sharing
//                                                              TMEM columns in the two lane halves
//     Qg = gam Q,  Kw = eg K                                   bf16 tiles for the chain kernel
//   chain (one CTA per (sequence, head), 64 dependent chunks):
//     [W^ S0 ; Qg S0]                                          tcgen05, M128 N128 K128
//     U  = Uv - W^ S0                                          TMEM -> registers -> bf16 smem operand
//     O  = Qg S0 + A U                                         tcgen05 accumulate, M128(padded) N128 K64
//     S  = gam_C S0 + Kw^T U                                   tcgen05 accumulate onto the f32 state in
//                                                              TMEM, pre-scaled by gam_C with ld/st
// The chain kernel's tiles arrive by TMA (plain 2-D tile loads, 128-byte swizzle, two stages);
// U and the bf16 copy of S are written into the same swizzled operand layouts by the compute
// threads. S reaches HBM only as chunk-boundary checkpoints (f32) and the final state.
//
// Every mbarrier wait is bounded (tc::mbar_wait): a wait that runs out sets the context's error
// word, and the CTA still frees its TMEM and exits.
//
// Head dim 64 runs on the same kernels with every head zero-padded to 128 (`dhi` = the head dim in the caller's
// tensors): the pre-pass reads 64 columns and fills the other 64 of its operand tiles with zeros, the chain kernels'
// tiles, TMEM state and products keep the 128 shapes (the padded rows and columns of S, dS and of every product are
// exact zeros), and only the accesses to the caller's tensors (q, k, v, o, dO, d_qkv, initial / final state, and the
// chunk-start states kept for the backward: the live 64 x 64 block as bf16) use the 64-wide layout.
#include "common.cuh"
#include "tc_common.cuh"

namespace delta_tc {

constexpr int C = 64;     // chunk length
constexpr int DH = 128;   // head dim handled by this file
constexpr int NB = DH / 64;

struct Tiles {            // intermediate buffers, one tile per (chain, chunk)
    __nv_bfloat16* WQ;    // [tile][128][DH]: rows 0-63 W^, rows 64-127 Qg
    __nv_bfloat16* UV;    // [tile][64][DH]
    __nv_bfloat16* KW;    // [tile][64][DH]
    __nv_bfloat16* AA;    // [tile][64][64]
    float* GC;            // [tile] gam_C (total decay of the chunk)
    // backward-only outputs (null in the forward)
    __nv_bfloat16* BK;    // [tile][64][DH]  beta gam K
    __nv_bfloat16* BV;    // [tile] beta V, 64 x DH, lane-major (see lm_off128)
    __nv_bfloat16* UVT;   // [tile] Uv, 64 x DH, lane-major copy for the backward
    __nv_bfloat16* TP;    // [tile][64][64]  T' = (I+L)^-1 - I, row-major
    __nv_bfloat16* KKo;   // [tile] K K^T, 64 x 64, lane-major (see lm_off64)
    __nv_bfloat16* QKo;   // [tile] Q K^T, 64 x 64, lane-major
    float* GV;            // [tile][64] cumulative log alpha
    float* BE;            // [tile][64] beta (0 on padded steps)
};

// Lane-major tile layouts for rows that the backward's threads read straight from global memory.
// There, thread (warp quarter wq = row / 16, lane = row % 16, column half) reads its 16-byte chunks
// j = 0.. one per instruction; storing chunk j of 16 consecutive rows side by side makes each such
// instruction touch 256 contiguous bytes. Offsets are in bf16 elements within one tile.
__device__ __forceinline__ int lm_off128(int row, int chunk16) {   // 64 x 128 tile, column halves of 8 chunks
    return ((((row >> 4) * 2 + (chunk16 >> 3)) * 8 + (chunk16 & 7)) * 16 + (row & 15)) * 8;
}
__device__ __forceinline__ int lm_off64(int row, int chunk16) {    // 64 x 64 tile, column halves of 4 chunks
    return ((((row >> 4) * 2 + (chunk16 >> 2)) * 4 + (chunk16 & 3)) * 16 + (row & 15)) * 8;
}

// ------------------------------------------------------------------ pre-pass
constexpr int PRE_THREADS = 128;
constexpr int LF_LD = 68;     // row stride (floats) of the f32 L and X matrices: float4 rows, conflict-free
constexpr int YF_LD = 16;
// Shared memory is sized for three CTAs per SM: the K/Q operand tiles are dead once KK and QK exist, so the
// f32 L and X matrices, and later the bf16 operand tile of X, live in the same region.
constexpr int PRE_R1 = 2 * 64 * LF_LD * 4;        // >= NB * 16384
constexpr size_t PRE_SMEM = 1024 + PRE_R1 + 2 * NB * 8192 /*Bop, later W^/Uv staging*/ + 3 * 16 * YF_LD * 4 + 4 * 64 * 4 + 64;
static_assert(PRE_R1 >= NB * 16384 && PRE_R1 % 1024 == 0 && (64 * LF_LD * 4) % 1024 == 0, "pre-pass shared-memory layout");

// One 1 x 4 strip of a 16 x 16 block product  acc += Lrow[0..16) * X[0..16)[c4..c4+4)  (f32, shared memory).
__device__ __forceinline__ void strip16(const float* __restrict__ lrow, const float* __restrict__ x, int ldx, float acc[4]) {
#pragma unroll
    for (int k4 = 0; k4 < 4; ++k4) {
        const float4 l4 = *reinterpret_cast<const float4*>(lrow + 4 * k4);
        const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float4 x4 = *reinterpret_cast<const float4*>(x + (4 * k4 + e) * ldx);
            acc[0] = fmaf(lv[e], x4.x, acc[0]);
            acc[1] = fmaf(lv[e], x4.y, acc[1]);
            acc[2] = fmaf(lv[e], x4.z, acc[2]);
            acc[3] = fmaf(lv[e], x4.w, acc[3]);
        }
    }
}

__global__ void __launch_bounds__(PRE_THREADS, 3) delta_prep_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ alpha, const float* __restrict__ beta, int T, int H, int dhi, int n_chunks, Tiles out,
    int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* KQ_s = base;                         // NB k-boxes x (128 rows x 128 B): rows 0-63 K, 64-127 Q
    uint8_t* Bop_s = KQ_s + PRE_R1;               // 2*NB n-boxes x (64 k-rows x 128 B): [beta gam K | beta V]
    float* Xf = reinterpret_cast<float*>(KQ_s);   // (I + L)^-1 in f32, once K and Q have been consumed
    float* Lf = Xf + 64 * LF_LD;                  // L in f32
    uint8_t* Tp_s = reinterpret_cast<uint8_t*>(Lf);   // 64 rows x 128 B: (I + L)^-1 as the K-major operand, once L is dead
    float* Yf = reinterpret_cast<float*>(Bop_s + 2 * NB * 8192);   // [3][16][YF_LD] block products in flight
    float* g_s = Yf + 3 * 16 * YF_LD;
    float* gam_s = g_s + 64;
    float* eg_s = gam_s + 64;
    float* be_s = eg_s + 64;
    uint64_t* bar = reinterpret_cast<uint64_t*>(be_s + 64);   // [0] MMA-A done, [1] MMA-B done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* wtot = reinterpret_cast<float*>(tmem_slot + 2);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x, chain = blockIdx.y;
    const int b = chain / H, h = chain % H;
    const int d = H * dhi;
    const int t0 = chunk * C;
    const int n = T - t0 < C ? T - t0 : C;
    const int64_t row0 = (int64_t)b * T + t0;
    const int64_t tix = (int64_t)chain * n_chunks + chunk;

    // K, Q, V rows of the chunk: every load is issued before anything waits on one
    const int sj = tid & 15;                      // 16-byte chunk of the row handled by this thread
    uint4 k8[8], q8[8], v8[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int t = (tid >> 4) + it * 8;
        k8[it] = q8[it] = v8[it] = make_uint4(0, 0, 0, 0);
        if (t < n && sj * 8 < dhi) {
            const int64_t off = (row0 + t) * d + h * dhi + sj * 8;
            k8[it] = *reinterpret_cast<const uint4*>(k + off);
            q8[it] = *reinterpret_cast<const uint4*>(q + off);
            v8[it] = *reinterpret_cast<const uint4*>(v + off);
        }
    }
    if (tid == 0) {
        *abort_flag = 0;
        tc::mbar_init(&bar[0], 1);
        tc::mbar_init(&bar[1], 1);
        tc::mbar_fence_init();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, 128);
    // g = cumsum(log alpha): warp scans over the 64 tokens
    float gx = 0.0f;
    if (tid < C) {
        const bool live = tid < n;
        be_s[tid] = live ? beta[(row0 + tid) * H + h] : 0.0f;
        gx = live ? logf(alpha[(row0 + tid) * H + h]) : 0.0f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, gx, o);
            if (lane >= o) gx += y;
        }
        if (tid == 31) *wtot = gx;
    }
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (tid < C) {
        if (tid >= 32) gx += *wtot;
        g_s[tid] = gx;
        gam_s[tid] = expf(gx);
    }
    __syncthreads();
    if (tid < C) eg_s[tid] = expf(g_s[C - 1] - g_s[tid]);
    __syncthreads();

    // ---- stage K, Q (K-major, swizzled), build [beta gam K | beta V], emit Qg, Kw and the backward's copies
    {
        const int box = sj >> 3, jc = sj & 7;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int t = (tid >> 4) + it * 8;
            *reinterpret_cast<uint4*>(KQ_s + box * 16384 + tc::sw128_off(t, jc)) = k8[it];
            *reinterpret_cast<uint4*>(KQ_s + box * 16384 + tc::sw128_off(64 + t, jc)) = q8[it];
            float kf[8], qf[8], vf[8], tmp[8];
            tc::unpack8_bf16(k8[it], kf);
            tc::unpack8_bf16(q8[it], qf);
            tc::unpack8_bf16(v8[it], vf);
            const float be = be_s[t], gm = gam_s[t], eg = eg_s[t];
            const int64_t o64 = (tix * 64 + t) * DH + sj * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = be * gm * kf[e];
            const uint4 bk = tc::pack8_bf16(tmp);
            *reinterpret_cast<uint4*>(Bop_s + box * 8192 + tc::sw128_off(t, jc)) = bk;
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = be * vf[e];
            *reinterpret_cast<uint4*>(Bop_s + (NB + box) * 8192 + tc::sw128_off(t, jc)) = tc::pack8_bf16(tmp);
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = gm * qf[e];
            *reinterpret_cast<uint4*>(out.WQ + (tix * 128 + 64 + t) * DH + sj * 8) = tc::pack8_bf16(tmp);
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = eg * kf[e];
            *reinterpret_cast<uint4*>(out.KW + o64) = tc::pack8_bf16(tmp);
            if (out.BK) {
                *reinterpret_cast<uint4*>(out.BK + o64) = bk;
            }
        }
    }
    if (out.GV && tid < C) {
        out.GV[tix * 64 + tid] = g_s[tid];
        out.BE[tix * 64 + tid] = be_s[tid];
    }
    tc::fence_proxy_async_smem();
    __syncthreads();

    // ---- MMA-A: [KK ; QK] = [K ; Q] K^T   (M128 N64 K128)
    if (tid == 0) {
        constexpr uint32_t IDESC = tc::idesc_bf16_f32(128, 64, 0, 0);
        const uint32_t kq = tc::smem_u32(KQ_s);
#pragma unroll
        for (int k16 = 0; k16 < DH / 16; ++k16) {
            const uint32_t off = (k16 >> 2) * 16384 + (k16 & 3) * 32;
            tc::umma_bf16(tmem, tc::smem_desc_sw128(kq + off, 16, 1024), tc::smem_desc_sw128(kq + off, 16, 1024), IDESC,
                          k16 > 0 ? 1u : 0u);
        }
        tc::umma_commit(&bar[0]);
    }
    // beta V in the lane-major layout, from the operand tile (consecutive threads, consecutive 16 bytes)
    if (out.BV) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int L = tid + it * PRE_THREADS;
            const int row = (L >> 8) * 16 + (L & 15), c16 = ((L >> 7) & 1) * 8 + ((L >> 4) & 7);
            *reinterpret_cast<uint4*>(out.BV + tix * (64 * DH) + L * 8) =
                *reinterpret_cast<const uint4*>(Bop_s + (NB + (c16 >> 3)) * 8192 + tc::sw128_off(row, c16 & 7));
        }
    }
    int got = 1;
    if (lane == 0) got = tc::mbar_wait(&bar[0], 0, abort_flag, err_word, 201) ? 1 : 0;
    bool ok = __shfl_sync(0xffffffffu, got, 0) != 0;
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    tc::tcgen05_fence_after();
    // ---- L = strictlower(beta_t Gam KK) (f32, threads 0-63); A = lower(Gam QK) (bf16, threads 64-127)
    if (ok) {
        uint32_t r[32];
        const int t = tid & 63;
        const float gt = g_s[t], bt = be_s[t];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            tc::tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + cc * 32, r);
            tc::tmem_ld_wait();
            if (tid < 64) {
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    float l[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = cc * 32 + 4 * j4 + e;
                        l[e] = i < t ? bt * __expf(gt - g_s[i]) * __uint_as_float(r[4 * j4 + e]) : 0.0f;
                    }
                    *reinterpret_cast<float4*>(&Lf[t * LF_LD + cc * 32 + 4 * j4]) = make_float4(l[0], l[1], l[2], l[3]);
                }
                if (out.KKo) {
                    float a[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) a[j] = __uint_as_float(r[j]);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(out.KKo + tix * 4096 + lm_off64(t, cc * 4 + j)) = tc::pack8_bf16(a + 8 * j);
                }
            } else {
                float a[32];
                if (out.QKo) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) a[j] = __uint_as_float(r[j]);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *reinterpret_cast<uint4*>(out.QKo + tix * 4096 + lm_off64(t, cc * 4 + j)) = tc::pack8_bf16(a + 8 * j);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int i = cc * 32 + j;
                    a[j] = i <= t ? __expf(gt - g_s[i]) * __uint_as_float(r[j]) : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(out.AA + (tix * 64 + t) * 64 + cc * 32 + j * 8) = tc::pack8_bf16(a + 8 * j);
            }
        }
    }
    tc::tcgen05_fence_before();
    __syncthreads();

    // ---- X = (I + L)^-1 in f32, by 16 x 16 blocks: the four diagonal blocks by forward substitution (one
    //      column per thread), then the blocks 1, 2 and 3 below the diagonal as X_IJ = -X_II (sum_K L_IK X_KJ)
    if (tid < 64) {
        const int I = tid >> 4, jj = tid & 15;
        const float* Lb = Lf + (I * 16) * LF_LD + I * 16;
        float x[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) x[t] = 0.0f;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            float s = 0.0f;
#pragma unroll
            for (int g4 = 0; g4 < (t + 3) / 4; ++g4) {      // entries at and right of the diagonal are zero in L
                const float4 l4 = *reinterpret_cast<const float4*>(Lb + t * LF_LD + 4 * g4);
                s = fmaf(l4.x, x[4 * g4], s);
                s = fmaf(l4.y, x[4 * g4 + 1], s);
                s = fmaf(l4.z, x[4 * g4 + 2], s);
                s = fmaf(l4.w, x[4 * g4 + 3], s);
            }
            x[t] = (t == jj ? 1.0f : 0.0f) - s;
        }
#pragma unroll
        for (int t = 0; t < 16; ++t) Xf[(I * 16 + t) * LF_LD + I * 16 + jj] = x[t];
    }
    __syncthreads();
#pragma unroll
    for (int dd = 1; dd < 4; ++dd) {
        const int pieces = (4 - dd) * 64;           // 1 x 4 strips of the (4 - dd) blocks at distance dd
        for (int p = tid; p < pieces; p += PRE_THREADS) {
            const int bI = (p >> 6) + dd, bJ = p >> 6, r = (p >> 2) & 15, c4 = (p & 3) * 4;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int kk = 0; kk < dd; ++kk)
                strip16(Lf + (bI * 16 + r) * LF_LD + (bJ + kk) * 16, Xf + ((bJ + kk) * 16) * LF_LD + bJ * 16 + c4, LF_LD, acc);
            *reinterpret_cast<float4*>(&Yf[((p >> 6) * 16 + r) * YF_LD + c4]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        __syncthreads();
        for (int p = tid; p < pieces; p += PRE_THREADS) {
            const int bI = (p >> 6) + dd, bJ = p >> 6, r = (p >> 2) & 15, c4 = (p & 3) * 4;
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            strip16(Xf + (bI * 16 + r) * LF_LD + bI * 16, Yf + ((p >> 6) * 16) * YF_LD + c4, YF_LD, acc);
            *reinterpret_cast<float4*>(&Xf[(bI * 16 + r) * LF_LD + bJ * 16 + c4]) = make_float4(-acc[0], -acc[1], -acc[2], -acc[3]);
        }
        __syncthreads();
    }
    // ---- X -> bf16 operand tile (K-major) and, for the backward, T' = X - I row-major
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = tid + it * PRE_THREADS, t = idx >> 3, jc = idx & 7;
        float x8[8];
        if ((jc >> 1) <= (t >> 4)) {
            const float4 a = *reinterpret_cast<const float4*>(&Xf[t * LF_LD + jc * 8]);
            const float4 c = *reinterpret_cast<const float4*>(&Xf[t * LF_LD + jc * 8 + 4]);
            x8[0] = a.x, x8[1] = a.y, x8[2] = a.z, x8[3] = a.w, x8[4] = c.x, x8[5] = c.y, x8[6] = c.z, x8[7] = c.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x8[e] = 0.0f;
        }
        *reinterpret_cast<uint4*>(Tp_s + tc::sw128_off(t, jc)) = tc::pack8_bf16(x8);
        if (out.TP) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (jc * 8 + e == t) x8[e] = 0.0f;
            *reinterpret_cast<uint4*>(out.TP + (tix * 64 + t) * 64 + jc * 8) = tc::pack8_bf16(x8);
        }
    }
    tc::fence_proxy_async_smem();
    __syncthreads();

    // ---- MMA-B: W^ = X (beta gam K) in lane half 0, Uv = X (beta V) in lane half 1   (2 x M64 N128 K64)
    if (tid == 0 && ok) {
        constexpr uint32_t IDESC = tc::idesc_bf16_f32(64, DH, 0, 1);
        const uint32_t ta = tc::smem_u32(Tp_s), bo = tc::smem_u32(Bop_s);
        tc::tcgen05_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < C / 16; ++k16)
            tc::umma_bf16(tmem, tc::smem_desc_sw128(ta + k16 * 32, 16, 1024), tc::smem_desc_sw128(bo + k16 * 2048, 8192, 1024),
                          IDESC, k16 > 0 ? 1u : 0u);
#pragma unroll
        for (int k16 = 0; k16 < C / 16; ++k16)
            tc::umma_bf16(tmem + (16u << 16), tc::smem_desc_sw128(ta + k16 * 32, 16, 1024),
                          tc::smem_desc_sw128(bo + NB * 8192 + k16 * 2048, 8192, 1024), IDESC, k16 > 0 ? 1u : 0u);
        tc::umma_commit(&bar[1]);
    }
    if (ok) {
        got = 1;
        if (lane == 0) got = tc::mbar_wait(&bar[1], 0, abort_flag, err_word, 202) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, got, 0) != 0;
    }
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    tc::tcgen05_fence_after();
    // rows to the staging area (the operand tiles are consumed): [W^ | Uv] 64 x 256 B each, chunks XOR-swizzled
    if (ok) {
        const int half = lane >> 4, row = 16 * warp + (lane & 15);
        uint8_t* stg = Bop_s + half * 16384 + row * 256;
#pragma unroll
        for (int cc = 0; cc < DH / 32; ++cc) {
            uint32_t r[32];
            tc::tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + cc * 32, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float o8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o8[e] = __uint_as_float(r[8 * j + e]);
                *reinterpret_cast<uint4*>(stg + (((cc * 4 + j) ^ (row & 15)) << 4)) = tc::pack8_bf16(o8);
            }
        }
    }
    __syncthreads();
    if (ok) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int idx = tid + it * PRE_THREADS, t = idx >> 4, c16 = idx & 15;
            const uint32_t so = t * 256 + ((c16 ^ (t & 15)) << 4);
            *reinterpret_cast<uint4*>(out.WQ + (tix * 128 + t) * DH + c16 * 8) = *reinterpret_cast<const uint4*>(Bop_s + so);
            *reinterpret_cast<uint4*>(out.UV + (tix * 64 + t) * DH + c16 * 8) = *reinterpret_cast<const uint4*>(Bop_s + 16384 + so);
        }
        if (out.UVT) {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int L = tid + it * PRE_THREADS;
                const int row = (L >> 8) * 16 + (L & 15), c16 = ((L >> 7) & 1) * 8 + ((L >> 4) & 7);
                *reinterpret_cast<uint4*>(out.UVT + tix * (64 * DH) + L * 8) =
                    *reinterpret_cast<const uint4*>(Bop_s + 16384 + row * 256 + ((c16 ^ (row & 15)) << 4));
            }
        }
    }
    if (tid == 0) out.GC[tix] = gam_s[C - 1];
    tc::tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, 128);
}

// ------------------------------------------------------------------ chain kernel
constexpr int CH_THREADS = 160;
constexpr int STAGE_BYTES = NB * 16384 /*WQ*/ + NB * 8192 /*UV*/ + NB * 8192 /*KW*/ + 16384 /*[0;A]*/;
constexpr int TX_BYTES = NB * 16384 + NB * 8192 + NB * 8192 + 8192;
constexpr size_t CH_SMEM = 1024 + 2 * STAGE_BYTES + NB * DH * 128 /*S bf16*/ + NB * 8192 /*U bf16*/ + 128;

template <typename TO>
__global__ void __launch_bounds__(CH_THREADS, 1) delta_fwd_tc_kernel(
    const __grid_constant__ CUtensorMap mapWQ, const __grid_constant__ CUtensorMap mapUV,
    const __grid_constant__ CUtensorMap mapKW, const __grid_constant__ CUtensorMap mapAA,
    const __grid_constant__ CUtensorMap mapS0, const float* __restrict__ GC,
    int T, int H, int dhi, int n_chunks, TO* __restrict__ o, const float* __restrict__ s_init, float* __restrict__ s_final,
    float* __restrict__ ckpt, __nv_bfloat16* __restrict__ s0b, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage0 = base;
    uint8_t* S_s = base + 2 * STAGE_BYTES;       // NB n-boxes x (DH k-rows x 128 B)
    uint8_t* U_s = S_s + NB * DH * 128;          // NB n-boxes x (64 k-rows x 128 B)
    uint64_t* bars = reinterpret_cast<uint64_t*>(U_s + NB * 8192);
    uint64_t* full = bars;            // [2]
    uint64_t* mma1_done = bars + 2;
    uint64_t* u_ready = bars + 3;
    uint64_t* mma2_done = bars + 4;
    uint64_t* s_ready = bars + 5;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chain = blockIdx.x;
    const int b = chain / H, h = chain % H;
    const int d = H * dhi;
    const int64_t row0 = (int64_t)b * T;
    const int64_t tile0 = (int64_t)chain * n_chunks;

    if (tid == 0) {
        *abort_flag = 0;
        tc::mbar_init(&full[0], 1);
        tc::mbar_init(&full[1], 1);
        tc::mbar_init(mma1_done, 1);
        tc::mbar_init(u_ready, 64);
        tc::mbar_init(mma2_done, 1);
        tc::mbar_init(s_ready, 128);
        tc::mbar_fence_init();
    }
    if (warp == 4) tc::tmem_alloc(tmem_slot, 2 * DH);
    // the zero halves of the two [0;A] operands
    for (int i = tid; i < 2 * 8192 / 16; i += CH_THREADS) {
        const int st = i / (8192 / 16), w = i % (8192 / 16);
        *reinterpret_cast<uint4*>(stage0 + st * STAGE_BYTES + NB * 32768 + w * 16) = make_uint4(0, 0, 0, 0);
    }
    tc::fence_proxy_async_smem();
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    const uint32_t tmem_S = *tmem_slot, tmem_D = tmem_S + DH;

    auto warp_wait = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        int got = 1;
        if (lane == 0) got = tc::mbar_wait(bar, parity, abort_flag, err_word, code) ? 1 : 0;
        return __shfl_sync(0xffffffffu, got, 0) != 0;
    };

    if (warp == 4) {
        // ------------------------------------------------------------ TMA + MMA issuer (one thread)
        if (lane == 0) {
            auto load = [&](int c, int s) {
                uint8_t* st = stage0 + s * STAGE_BYTES;
                const int t = (int)(tile0 + c);
                tc::mbar_expect_tx(&full[s], TX_BYTES);
#pragma unroll
                for (int kb = 0; kb < NB; ++kb) tc::tma_load_2d(st + kb * 16384, &mapWQ, kb * 64, t * 128, &full[s]);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    tc::tma_load_2d(st + NB * 16384 + nb * 8192, &mapUV, nb * 64, t * 64, &full[s]);
                    tc::tma_load_2d(st + NB * 24576 + nb * 8192, &mapKW, nb * 64, t * 64, &full[s]);
                }
                tc::tma_load_2d(st + NB * 32768 + 8192, &mapAA, 0, t * 64, &full[s]);
            };
            load(0, 0);
            if (n_chunks > 1) load(1, 1);
            constexpr uint32_t ID1 = tc::idesc_bf16_f32(128, DH, 0, 1);   // A K-major, B MN-major
            constexpr uint32_t ID3 = tc::idesc_bf16_f32(128, DH, 1, 1);   // A MN-major, B MN-major
            const uint32_t s_addr = tc::smem_u32(S_s), u_addr = tc::smem_u32(U_s);
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c & 1;
                const uint32_t st = tc::smem_u32(stage0 + s * STAGE_BYTES);
                if (!tc::mbar_wait(&full[s], (c >> 1) & 1, abort_flag, err_word, 211)) break;
                if (!tc::mbar_wait(s_ready, c & 1, abort_flag, err_word, 212)) break;
                tc::tcgen05_fence_after();
                if (s0b) {   // the state at the start of chunk c, bf16, straight from the operand tile: two 128 x 64 boxes
                             // (head dim 64: the live 64 x 64 block, the first 8 KiB of the first box)
                    tc::tma_store_2d(&mapS0, S_s, 0, (int)(tile0 + c) * dhi);
                    if (dhi == DH) tc::tma_store_2d(&mapS0, S_s + DH * 128, 64, (int)(tile0 + c) * DH);
                    tc::bulk_commit_group();
                }
                // D1 = [W^ ; Qg] S0
#pragma unroll
                for (int k16 = 0; k16 < DH / 16; ++k16)
                    tc::umma_bf16(tmem_D, tc::smem_desc_sw128(st + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024),
                                  tc::smem_desc_sw128(s_addr + k16 * 2048, DH * 128, 1024), ID1, k16 > 0 ? 1u : 0u);
                tc::umma_commit(mma1_done);
                if (!tc::mbar_wait(u_ready, c & 1, abort_flag, err_word, 213)) break;
                tc::tcgen05_fence_after();
                // D1 += [0 ; A] U      S += Kw^T U
#pragma unroll
                for (int k16 = 0; k16 < C / 16; ++k16)
                    tc::umma_bf16(tmem_D, tc::smem_desc_sw128(st + NB * 32768 + k16 * 32, 16, 1024),
                                  tc::smem_desc_sw128(u_addr + k16 * 2048, 8192, 1024), ID1, 1u);
#pragma unroll
                for (int k16 = 0; k16 < C / 16; ++k16)
                    tc::umma_bf16(tmem_S, tc::smem_desc_sw128(st + NB * 24576 + k16 * 2048, 8192, 1024),
                                  tc::smem_desc_sw128(u_addr + k16 * 2048, 8192, 1024), ID3, 1u);
                if (s0b) tc::bulk_wait_read();   // the state store has read the operand tile: it may be rewritten after this commit
                tc::umma_commit(mma2_done);
                if (c + 2 < n_chunks) {
                    if (!tc::mbar_wait(mma2_done, c & 1, abort_flag, err_word, 214)) break;
                    load(c + 2, s);
                }
            }
            if (s0b) tc::bulk_wait_all();   // stores have landed before the CTA exits
        }
    } else {
        // ------------------------------------------------------------ compute threads: TMEM lane = tid
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float* ck = ckpt ? ckpt + tile0 * DH * DH : nullptr;
        // initial state: checkpoint 0, bf16 operand copy, f32 state scaled by the first chunk's decay
        {
            const float g0 = GC[tile0];
            const float* si = s_init && tid < dhi ? s_init + (int64_t)chain * dhi * dhi + (int64_t)tid * dhi : nullptr;
#pragma unroll 1
            for (int cc = 0; cc < DH / 32; ++cc) {
                uint32_t r[32];
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = si && cc * 32 < dhi ? si[cc * 32 + j] : 0.0f;
                if (ck) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(ck + (int64_t)tid * DH + cc * 32)[j] =
                            make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int chunk16 = cc * 4 + j;   // 16-byte chunk index along the row (8 bf16 each)
                    const uint4 pk = tc::pack8_bf16(f + 8 * j);
                    *reinterpret_cast<uint4*>(S_s + (chunk16 >> 3) * (DH * 128) + tc::sw128_off(tid, chunk16 & 7)) = pk;
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(g0 * f[j]);
                tc::tmem_st_32x32(tmem_S + lane_addr + cc * 32, r);
            }
            tc::tmem_st_wait();
            tc::fence_proxy_async_smem();
            tc::tcgen05_fence_before();
            tc::mbar_arrive(s_ready);
        }
        for (int c = 0; c < n_chunks; ++c) {
            const int s = c & 1;
            uint8_t* st = stage0 + s * STAGE_BYTES;
            if (!warp_wait(mma1_done, c & 1, 221)) break;
            tc::tcgen05_fence_after();
            if (warp < 2) {
                // U = Uv - W^ S0  ->  bf16 operand (k rows = t, n cols = value index)
                if (!warp_wait(&full[s], (c >> 1) & 1, 222)) break;   // TMA-written Uv visible to this thread
                const int t = tid;
#pragma unroll 1
                for (int cc = 0; cc < DH / 32; ++cc) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(tmem_D + lane_addr + cc * 32, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk16 = cc * 4 + j;
                        const uint32_t off = (chunk16 >> 3) * 8192 + tc::sw128_off(t, chunk16 & 7);
                        float uv[8], u8[8];
                        tc::unpack8_bf16(*reinterpret_cast<const uint4*>(st + NB * 16384 + off), uv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) u8[e] = uv[e] - __uint_as_float(r[8 * j + e]);
                        *reinterpret_cast<uint4*>(U_s + off) = tc::pack8_bf16(u8);
                    }
                }
                tc::fence_proxy_async_smem();
                tc::tcgen05_fence_before();
                tc::mbar_arrive(u_ready);
            }
            if (!warp_wait(mma2_done, c & 1, 223)) break;
            tc::tcgen05_fence_after();
            if (warp >= 2) {
                // O rows (TMEM lanes 64-127 of D1)
                const int t = tid - 64;
                const bool live = c * C + t < T;
                TO* orow = o + (row0 + c * C + (live ? t : 0)) * d + h * dhi;
#pragma unroll 1
                for (int cc = 0; cc < DH / 32; ++cc) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(tmem_D + lane_addr + cc * 32, r);
                    tc::tmem_ld_wait();
                    if (live && cc * 32 < dhi) {
                        if (sizeof(TO) == 2) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float f8[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(r[8 * j + e]);
                                reinterpret_cast<uint4*>(orow + cc * 32)[j] = tc::pack8_bf16(f8);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<float4*>(orow + cc * 32)[j] =
                                    make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                        }
                    }
                }
            }
            // new state: checkpoint / final state (f32), bf16 operand copy, pre-scale for the next chunk
            const bool last = c + 1 == n_chunks;
            const float gnext = last ? 1.0f : GC[tile0 + c + 1];
            float* dst = last ? (s_final ? s_final + (int64_t)chain * dhi * dhi : nullptr)
                              : (ck ? ck + (int64_t)(c + 1) * DH * DH : nullptr);   // (f32 checkpoints: head dim 128 only)
#pragma unroll 1
            for (int cc = 0; cc < DH / 32; ++cc) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_S + lane_addr + cc * 32, r);
                tc::tmem_ld_wait();
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
                if (dst && tid < dhi && cc * 32 < dhi) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(dst + (int64_t)tid * dhi + cc * 32)[j] =
                            make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                }
                if (!last) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk16 = cc * 4 + j;
                        const uint4 pk = tc::pack8_bf16(f + 8 * j);
                        *reinterpret_cast<uint4*>(S_s + (chunk16 >> 3) * (DH * 128) + tc::sw128_off(tid, chunk16 & 7)) = pk;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(gnext * f[j]);
                    tc::tmem_st_32x32(tmem_S + lane_addr + cc * 32, r);
                }
            }
            if (!last) {
                tc::tmem_st_wait();
                tc::fence_proxy_async_smem();
                tc::tcgen05_fence_before();
                tc::mbar_arrive(s_ready);
            }
        }
    }
    tc::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(20000);
    if (warp == 4) tc::tmem_dealloc(tmem_S, 2 * DH);
}

// ------------------------------------------------------------------ backward chain kernel
// One CTA (128 threads) per (sequence, head) walks the chunks in reverse with dS (f32) resident
// in TMEM columns [0,128). Products with 64 token rows use M = 64 MMAs; two of them share a
// column range by living in the two 16-lane halves of every 32-lane TMEM quarter (lane offset 0
// and 16), so thread (warp w, lane l) sees row 16w + (l & 15) of the product in half (l >> 4).
//
//   G1  ACC_A.h0 = W^ S0               ACC_A.h1 = (beta gam K) S0  (= P2)
//   G2  ACC_B.h1 = A^T dO + Kw dS      (= dU)
//   G3  ACC_B.h1 += T'^T dU            (= dR)         G8  ACC_C.h1 = U dS^T (= dW)
//   G4  ACC_C.h0 = [dR U^T | dO U^T]   (-> dL, dA)    G5  ACC_A.h0 = dO S0^T,  ACC_A.h1 = dR S0^T
//   G6  ACC_B.h0 = (dA.Gam) K          ACC_B.h1 = M K + M^T K + (dA.Gam)^T Q
//   G9  dS = gam_C dS + Qg^T dO - (beta gam K)^T dR
// with U = Uv - W^ S0, R = beta V - P2, dV = beta dR, M = dL.Gam.beta, and
//   dq = gam X + G6.h0,  dk = G6.h1 + eg dW - beta gam Y  (X, Y = the two halves of G5),
// followed by the L2-norm backward, the gate gradients and the [dq|dk|dv] concat as in the f32
// kernel (delta_bwd.cu).
constexpr int NCQ = 4;                   // column groups per row: warp w and w + 4 k share TMEM lane quarter (w & 3)
constexpr int BW_THREADS = 128 * NCQ;
constexpr int CW = DH / NCQ;             // columns of a row handled by one thread
constexpr int NCI = CW / 32;             // 32-column TMEM loads per thread and product
constexpr int DW = C / NCQ;              // columns of the 64 x 64 dL / dA products per thread
constexpr int NWARPS = BW_THREADS / 32;
constexpr int R_WH = 0, R_BK = 16384, R_QG = 32768, R_KW = 49152, R_K = 65536, R_Q = 81920, R_DO = 98304,
              R_A = 114688, R_TP = 122880, R_S0 = 131072, R_DS = 163840, R_DR = 196608, R_END = 212992;
constexpr int R_U = R_WH, R_P = R_KW, R_DAG = R_A, R_M = R_TP, R_STG = R_S0;   // staging: S0 + dS regions (64 KiB)
constexpr int BW_NVEC = 128 + 6 * NCQ * 64 + BW_THREADS + 128 + 64 + (BW_THREADS / 64) * 64;
constexpr size_t BW_SMEM = 1024 + R_END + BW_NVEC * 4 + 256;
constexpr int BW_TX_A = 32768 + 16384 * 2;        // S0, W^, beta gam K
constexpr int BW_TX_B = 16384 * 2 + 8192;         // Kw, dO, A
constexpr int BW_TX_C = 16384 * 3 + 8192;         // Qg, K, Q, T'

// 128 * NCQ threads: warps w, w + 4, ... share TMEM lane quarter (w & 3) and split every row's 128
// columns in NCQ groups (colhalf = w >> 2), so each thread handles CW columns of one row.
__global__ void __launch_bounds__(BW_THREADS, 1) delta_bwd_tc_kernel(
    const __grid_constant__ CUtensorMap mapWQ, const __grid_constant__ CUtensorMap map64x128,  // BK tiles
    const __grid_constant__ CUtensorMap mapKW, const __grid_constant__ CUtensorMap mapKR,
    const __grid_constant__ CUtensorMap mapQR, const __grid_constant__ CUtensorMap mapDO,
    const __grid_constant__ CUtensorMap mapAA, const __grid_constant__ CUtensorMap mapTP,
    const __grid_constant__ CUtensorMap mapS0, Tiles tl,
    const float* __restrict__ alpha, const float* __restrict__ qnorm, const float* __restrict__ knorm, int T, int H, int dhi, int n_chunks,
    float* __restrict__ d_qkv, float* __restrict__ d_gate, int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float* vec = reinterpret_cast<float*>(sm + R_END);
    float* g_s = vec;              // cumulative log alpha
    float* be_s = vec + 64;        // beta
    float* v_rowp = vec + 128;                 // [NCQ][64] row sums of P per column group
    float* v_rqs = v_rowp + NCQ * 64;          // [NCQ][64]
    float* v_rkg = v_rqs + NCQ * 64;           // [NCQ][64]
    float* v_rkw = v_rkg + NCQ * 64;           // [NCQ][64]
    float* v_rdr = v_rkw + NCQ * 64;           // [NCQ][64]
    float* v_dls = v_rdr + NCQ * 64;           // [NCQ][64]
    float* v_red = v_dls + NCQ * 64;           // [BW_THREADS] partials of <S0, dS>
    float* v_nrm = v_red + BW_THREADS;         // [128] |q| rows then |k| rows of the chunk
    float* v_al = v_nrm + 128;                 // [64] alpha
    float* v_colp4 = v_al + 64;                // [BW_THREADS / 64][64] partial column sums of P
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + R_END + BW_NVEC * 4);   // [0],[7],[8] TMA groups, [1..6] MMA groups
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wq = warp & 3, colhalf = warp >> 2;
    const int half = (lane >> 4) & 1, row = 16 * wq + (lane & 15);   // M=64 accumulator mapping
    const int arow = 32 * wq + lane;                                 // M=128 accumulator (dS) mapping
    const int chain = blockIdx.x;
    const int b = chain / H, h = chain % H;
    const int d = H * dhi;
    const int64_t seq_row0 = (int64_t)b * T;
    const int64_t tile0 = (int64_t)chain * n_chunks;

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 9; ++i) tc::mbar_init(&bars[i], 1);
        tc::mbar_fence_init();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, 512);
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    const uint32_t tm = *tmem_slot;
    const uint32_t ACC_S = tm, ACC_A = tm + 128, ACC_B = tm + 256, ACC_C = tm + 384;
    const uint32_t H1 = 16u << 16;                         // lane offset of the second M=64 half
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const int c0 = colhalf * NCI;                          // first 32-column chunk of this thread

    // dS = 0 (TMEM f32 and the bf16 operand copy)
    {
        uint32_t z[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = 0u;
#pragma unroll
        for (int ci = 0; ci < NCI; ++ci) tc::tmem_st_32x32(ACC_S + lane_addr + (c0 + ci) * 32, z);
        tc::tmem_st_wait();
        for (int i = tid; i < 32768 / 16; i += BW_THREADS) *reinterpret_cast<uint4*>(sm + R_DS + i * 16) = make_uint4(0, 0, 0, 0);
    }
    // Head dim 64: a chunk-start state arrives as its live 64 x 64 block (rows 0-63 of the first column box); the rest of
    // the S0 operand must read as zeros. The region doubles as staging, so it is cleared again after every chunk.
    auto clear_s0_pad = [&] {
        for (int i = tid; i < (32768 - 8192) / 16; i += BW_THREADS) *reinterpret_cast<uint4*>(sm + R_S0 + 8192 + i * 16) = make_uint4(0, 0, 0, 0);
    };
    if (dhi != DH) clear_s0_pad();

    // Three groups in the order the chunk needs them: [0] S0, W^, beta gam K; [7] Kw, dO, A; [8] the rest.
    auto issue_tma = [&](int c) {
        const int t = (int)(tile0 + c);
        const int grow = (int)(seq_row0 + (int64_t)c * C);
        tc::mbar_expect_tx(&bars[0], dhi == DH ? BW_TX_A : BW_TX_A - 32768 + 8192);
        // caller's tensors, head dim 64: the second column box starts past the last column and arrives as TMA's zero fill
        const int xc[2] = {h * dhi, dhi == DH ? h * DH + 64 : H * dhi};
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            if (dhi == DH) tc::tma_load_2d(sm + R_S0 + kb * 16384, &mapS0, kb * 64, t * 128, &bars[0]);
            else if (kb == 0) tc::tma_load_2d(sm + R_S0, &mapS0, 0, t * 64, &bars[0]);
            tc::tma_load_2d(sm + R_WH + kb * 8192, &mapWQ, kb * 64, t * 128, &bars[0]);
            tc::tma_load_2d(sm + R_BK + kb * 8192, &map64x128, kb * 64, t * 64, &bars[0]);
        }
        tc::mbar_expect_tx(&bars[7], BW_TX_B);
        tc::tma_load_2d(sm + R_A, &mapAA, 0, t * 64, &bars[7]);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            tc::tma_load_2d(sm + R_DO + kb * 8192, &mapDO, xc[kb], grow, &bars[7]);
            tc::tma_load_2d(sm + R_KW + kb * 8192, &mapKW, kb * 64, t * 64, &bars[7]);
        }
        tc::mbar_expect_tx(&bars[8], BW_TX_C);
        tc::tma_load_2d(sm + R_TP, &mapTP, 0, t * 64, &bars[8]);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            tc::tma_load_2d(sm + R_QG + kb * 8192, &mapWQ, kb * 64, t * 128 + 64, &bars[8]);
            // K and Q straight from the caller's tensors (like dO): rows past the sequence end hold the next
            // sequence's tokens (or TMA's zero fill past the tensor); every product that reads them multiplies by an
            // exact zero there (beta = 0, U rows = 0, and dA rows masked below)
            tc::tma_load_2d(sm + R_K + kb * 8192, &mapKR, xc[kb], grow, &bars[8]);
            tc::tma_load_2d(sm + R_Q + kb * 8192, &mapQR, xc[kb], grow, &bars[8]);
        }
    };
    auto wait_bar = [&](int i, uint32_t parity) {
        if (lane == 0) tc::mbar_wait(&bars[i], parity, abort_flag, err_word, 300 + i);
        __syncwarp();
    };
    // Shared-memory matrix descriptors (128-byte swizzle, version 1). The address field is (base + offset) >> 4
    // with every offset a compile-time constant, so one add per descriptor remains at run time.
    const uint32_t sb4 = tc::smem_u32(sm) >> 4;
    auto desc = [&](uint32_t off, uint32_t lbo, uint32_t sbo) -> uint64_t {
        const uint32_t lo = sb4 + ((off >> 4) + ((lbo >> 4) << 16));
        const uint32_t hi = (sbo >> 4) | (1u << 14) | (2u << 29);
        return ((uint64_t)hi << 32) | lo;
    };
    auto kmaj = [&](int reg, int k16) {       // K-major, 64-row tile, 8 KiB per 64-wide k box
        return desc(reg + (k16 >> 2) * 8192 + (k16 & 3) * 32, 16, 1024);
    };
    auto kmaj128 = [&](int reg, int k16) {    // K-major, 128-row tile (S0 / dS), 16 KiB per k box
        return desc(reg + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024);
    };
    auto mnmaj = [&](int reg, int k16, int lbo) {   // MN-major: k rows, 64-wide mn boxes `lbo` bytes apart
        return desc(reg + k16 * 2048, lbo, 1024);
    };
    // 64-row operand tile written by the threads: 16-byte chunk `chunk16` (0..15) of row r
    auto tile64 = [&](int reg, int r, int chunk16) -> uint4* {
        return reinterpret_cast<uint4*>(sm + reg + (chunk16 >> 3) * 8192 + tc::sw128_off(r, chunk16 & 7));
    };
    auto tile128 = [&](int reg, int r, int chunk16) -> uint4* {
        return reinterpret_cast<uint4*>(sm + reg + (chunk16 >> 3) * 16384 + tc::sw128_off(r, chunk16 & 7));
    };
    constexpr uint32_t I64_KM = tc::idesc_bf16_f32(64, 128, 0, 1);
    constexpr uint32_t I64_MM = tc::idesc_bf16_f32(64, 128, 1, 1);
    constexpr uint32_t I64_KK = tc::idesc_bf16_f32(64, 128, 0, 0);
    constexpr uint32_t I64_KK64 = tc::idesc_bf16_f32(64, 64, 0, 0);
    constexpr uint32_t I128_MM = tc::idesc_bf16_f32(128, 128, 1, 1);
    constexpr uint32_t I128_MM_NEG = I128_MM | (1u << 13);

    // Small per-chunk inputs are fetched one chunk ahead, before that chunk's TMA traffic is queued:
    // rows of Uv (half 0) / beta V (half 1), 64 columns each, and the per-token scalars.
    uint4 pre[CW / 8];
    float nx0 = 0.0f, nx1 = 0.0f;
    auto fetch_small = [&](int c) {
        const int64_t tix = tile0 + c;
        const int t0 = c * C;
        const int n = T - t0 < C ? T - t0 : C;
        const int64_t grow = seq_row0 + t0;
        const __nv_bfloat16* src = (half == 0 ? tl.UVT : tl.BV) + tix * (64 * DH) + lm_off128(row, colhalf * (CW / 8));
#pragma unroll
        for (int j = 0; j < CW / 8; ++j) pre[j] = *reinterpret_cast<const uint4*>(src + j * 128);
        if (tid < 64) {
            nx0 = tl.GV[tix * 64 + tid];
            nx1 = tl.BE[tix * 64 + tid];
        } else if (tid < 128) {
            const int t = min(tid - 64, n - 1);          // unconditional loads: nothing waits on them here
            nx0 = alpha[(grow + t) * H + h];
        } else if (tid < 256) {
            const int t = min(tid & 63, n - 1);
            nx0 = (tid < 192 ? qnorm : knorm)[(grow + t) * H + h];
        }
    };
    fetch_small(n_chunks - 1);
    if (tid == 0) issue_tma(n_chunks - 1);
    // A wait that gives up raises *abort_flag; later waits then return at once, the iteration runs to its
    // end on whatever data it has (every block barrier is still reached by every thread) and the loop
    // exits at the block-uniform check below. The host sees the error word.
    for (int c = n_chunks - 1, it = 0; c >= 0; --c, ++it) {
        const uint32_t par = it & 1;
        const int t0 = c * C;
        const int n = T - t0 < C ? T - t0 : C;
        const int64_t tix = tile0 + c;
        const int64_t grow = seq_row0 + t0;
        // ---- A. per-token scalars of the chunk (fetched during the previous chunk)
        if (tid < 64) {
            g_s[tid] = nx0;
            be_s[tid] = nx1;
        } else if (tid < 128) {
            v_al[tid - 64] = nx0;
        } else if (tid < 256) {
            v_nrm[tid - 128] = nx0;
        }
        tc::fence_proxy_async_smem();   // the dS operand copy written at the end of the previous chunk
        tc::tcgen05_fence_before();
        __syncthreads();
        wait_bar(0, par);
        if (tid == 0) {
            tc::tcgen05_fence_after();
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_A, kmaj(R_WH, k16), mnmaj(R_S0, k16, 16384), I64_KM, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_A + H1, kmaj(R_BK, k16), mnmaj(R_S0, k16, 16384), I64_KM, k16 > 0);
            tc::umma_commit(&bars[1]);
        }
        wait_bar(7, par);
        if (tid == 0) {
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16) tc::umma_bf16(ACC_B + H1, mnmaj(R_A, k16, 8192), mnmaj(R_DO, k16, 8192), I64_MM, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_B + H1, kmaj(R_KW, k16), mnmaj(R_DS, k16, 16384), I64_KM, 1u);
            tc::umma_commit(&bars[2]);
        }
        const float g_row = g_s[row], g_last = g_s[C - 1];
        const float gam_row = __expf(g_row), eg_row = __expf(g_last - g_row), be_row = be_s[row];
        const bool live = row < n;
        // ---- B. U = Uv - W^ S0 (half 0);  dU -> bf16 (half 1)
        wait_bar(1, par);
        tc::tcgen05_fence_after();
#pragma unroll
        for (int ci = 0; ci < NCI; ++ci) {
            uint32_t r[32];
            tc::tmem_ld_32x32(ACC_A + lane_addr + (c0 + ci) * 32, r);
            tc::tmem_ld_wait();
            if (half == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x8[8], u8[8];
                    tc::unpack8_bf16(pre[ci * 4 + j], x8);
#pragma unroll
                    for (int e = 0; e < 8; ++e) u8[e] = x8[e] - __uint_as_float(r[8 * j + e]);
                    *tile64(R_U, row, (c0 + ci) * 4 + j) = tc::pack8_bf16(u8);
                }
            }
        }
        wait_bar(2, par);
        tc::tcgen05_fence_after();
#pragma unroll
        for (int ci = 0; ci < NCI; ++ci) {
            uint32_t r[32];
            tc::tmem_ld_32x32(ACC_B + lane_addr + (c0 + ci) * 32, r);
            tc::tmem_ld_wait();
            if (half == 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float f8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(r[8 * j + e]);
                    *tile64(R_DR, row, (c0 + ci) * 4 + j) = tc::pack8_bf16(f8);
                }
            }
        }
        tc::fence_proxy_async_smem();
        tc::tcgen05_fence_before();
        wait_bar(8, par);
        __syncthreads();
        if (tid == 0) {
            tc::tcgen05_fence_after();
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16) tc::umma_bf16(ACC_B + H1, mnmaj(R_TP, k16, 8192), mnmaj(R_DR, k16, 8192), I64_MM, 1u);
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_C + H1, kmaj(R_U, k16), kmaj128(R_DS, k16), I64_KK, k16 > 0);
            tc::umma_commit(&bars[3]);
        }
        // rows of K K^T and Q K^T (32 columns each) for the dL / dA phase, fetched ahead
        uint4 pkk[DW / 8], pqk[DW / 8];
        if (half == 0) {
            const __nv_bfloat16* kk = tl.KKo + tix * 4096 + lm_off64(row, colhalf * (DW / 8));
            const __nv_bfloat16* qk = tl.QKo + tix * 4096 + lm_off64(row, colhalf * (DW / 8));
#pragma unroll
            for (int j = 0; j < DW / 8; ++j) {
                pkk[j] = *reinterpret_cast<const uint4*>(kk + j * 128);
                pqk[j] = *reinterpret_cast<const uint4*>(qk + j * 128);
            }
        }
        // ---- C. dR: dV out, R = beta V - P2, r_dr, r_kg, bf16 dR tile (half 1)
        wait_bar(3, par);
        tc::tcgen05_fence_after();
        {
            float r_dr = 0.0f, r_kg = 0.0f;
#pragma unroll
            for (int ci = 0; ci < NCI; ++ci) {
                uint32_t r[32], p2[32];
                tc::tmem_ld_32x32(ACC_B + lane_addr + (c0 + ci) * 32, r);
                tc::tmem_ld_32x32(ACC_A + lane_addr + (c0 + ci) * 32, p2);
                tc::tmem_ld_wait();
                if (half == 1) {
                    float4* dvs = reinterpret_cast<float4*>(sm + R_DS) + row * 32;   // dV rows staged in the free dS region
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float x8[8], f8[8];
                        tc::unpack8_bf16(pre[ci * 4 + j], x8);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float dr = __uint_as_float(r[8 * j + e]), pp = __uint_as_float(p2[8 * j + e]);
                            f8[e] = dr;
                            r_dr = fmaf(dr, x8[e] - pp, r_dr);
                            r_kg = fmaf(-dr, pp, r_kg);
                        }
                        {
                            const int f4 = ((c0 + ci) * 4 + j) * 2, swz = row & 31;
                            dvs[f4 ^ swz] = make_float4(be_row * f8[0], be_row * f8[1], be_row * f8[2], be_row * f8[3]);
                            dvs[(f4 + 1) ^ swz] = make_float4(be_row * f8[4], be_row * f8[5], be_row * f8[6], be_row * f8[7]);
                        }
                        *tile64(R_DR, row, (c0 + ci) * 4 + j) = tc::pack8_bf16(f8);
                    }
                }
            }
            if (half == 1) {
                v_rdr[colhalf * 64 + row] = r_dr;
                v_rkg[colhalf * 64 + row] = r_kg;
            }
        }
        tc::fence_proxy_async_smem();
        tc::tcgen05_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc::tcgen05_fence_after();
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_C, kmaj(R_DR, k16), kmaj(R_U, k16), I64_KK64, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_C + 64, kmaj(R_DO, k16), kmaj(R_U, k16), I64_KK64, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_A, kmaj(R_DO, k16), kmaj128(R_S0, k16), I64_KK, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 8; ++k16) tc::umma_bf16(ACC_A + H1, kmaj(R_DR, k16), kmaj128(R_S0, k16), I64_KK, k16 > 0);
            tc::umma_commit(&bars[4]);
        }
        // ---- D. while G4/G5 run: dV rows out (8 lanes per row, coalesced), scale dS by gam_C, <S0, dS>
#pragma unroll
        for (int itv = 0; itv < 64 / (BW_THREADS / 8); ++itv) {
            const int r_ = itv * (BW_THREADS / 8) + (tid >> 3), l8 = tid & 7;
            if (r_ < n) {
                float* dv = d_qkv + (grow + r_) * 3 * d + 2 * d + h * dhi;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if ((l8 + 8 * i) * 4 < dhi)
                        reinterpret_cast<float4*>(dv)[l8 + 8 * i] = reinterpret_cast<const float4*>(sm + R_DS)[r_ * 32 + ((l8 + 8 * i) ^ (r_ & 31))];
            }
        }
        {
            const float gC = __expf(g_last);
            float part = 0.0f;
#pragma unroll
            for (int ci = 0; ci < NCI; ++ci) {
                uint32_t r[32];
                tc::tmem_ld_32x32(ACC_S + lane_addr + (c0 + ci) * 32, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float s8[8];
                    tc::unpack8_bf16(*tile128(R_S0, arow, (c0 + ci) * 4 + j), s8);
#pragma unroll
                    for (int e = 0; e < 8; ++e) part = fmaf(s8[e], __uint_as_float(r[8 * j + e]), part);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(gC * __uint_as_float(r[j]));
                tc::tmem_st_32x32(ACC_S + lane_addr + (c0 + ci) * 32, r);
            }
            tc::tmem_st_wait();
            v_red[tid] = part;
        }
        wait_bar(4, par);
        tc::tcgen05_fence_after();
        // dL / dA rows (half 0; this thread's DW columns): M tile, dA.Gam tile, P row, dbeta
        {
            float rowp = 0.0f, dls = 0.0f;
            uint32_t rl[DW], ra[DW];
            tc::tmem_ld_cols<DW>(ACC_C + lane_addr + colhalf * DW, rl);
            tc::tmem_ld_cols<DW>(ACC_C + lane_addr + 64 + colhalf * DW, ra);
            tc::tmem_ld_wait();
            if (half == 0) {
#pragma unroll
                for (int j = 0; j < DW / 8; ++j) {
                    float kk8[8], qk8[8], m8[8], a8[8];
                    tc::unpack8_bf16(pkk[j], kk8);
                    tc::unpack8_bf16(pqk[j], qk8);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int i = colhalf * DW + 8 * j + e;
                        const float gm = i <= row ? __expf(g_row - g_s[i]) : 0.0f;
                        const float dlg = i < row ? -__uint_as_float(rl[8 * j + e]) * gm : 0.0f;   // dL.Gam
                        const float dag = live ? __uint_as_float(ra[8 * j + e]) * gm : 0.0f;       // dA.Gam (dO rows past the end are not ours)
                        dls = fmaf(dlg, kk8[e], dls);
                        m8[e] = dlg * be_row;
                        a8[e] = dag;
                        const float pv = dag * qk8[e] + m8[e] * kk8[e];
                        rowp += pv;
                        reinterpret_cast<float*>(sm + R_P)[row * 64 + ((i + row) & 63)] = pv;
                    }
                    const int chunk16 = colhalf * (DW / 8) + j;
                    *reinterpret_cast<uint4*>(sm + R_M + tc::sw128_off(row, chunk16)) = tc::pack8_bf16(m8);
                    *reinterpret_cast<uint4*>(sm + R_DAG + tc::sw128_off(row, chunk16)) = tc::pack8_bf16(a8);
                }
                v_rowp[colhalf * 64 + row] = rowp;
                v_dls[colhalf * 64 + row] = dls;
            }
        }
        tc::fence_proxy_async_smem();
        tc::tcgen05_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc::tcgen05_fence_after();
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16)
                tc::umma_bf16(ACC_B, desc(R_DAG + k16 * 32, 16, 1024), mnmaj(R_K, k16, 8192), I64_KM, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16)
                tc::umma_bf16(ACC_B + H1, desc(R_M + k16 * 32, 16, 1024), mnmaj(R_K, k16, 8192), I64_KM, k16 > 0);
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16) tc::umma_bf16(ACC_B + H1, mnmaj(R_M, k16, 8192), mnmaj(R_K, k16, 8192), I64_MM, 1u);
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16) tc::umma_bf16(ACC_B + H1, mnmaj(R_DAG, k16, 8192), mnmaj(R_Q, k16, 8192), I64_MM, 1u);
            tc::umma_commit(&bars[5]);
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16) tc::umma_bf16(ACC_S, mnmaj(R_QG, k16, 8192), mnmaj(R_DO, k16, 8192), I128_MM, 1u);
            _Pragma("unroll") for (int k16 = 0; k16 < 4; ++k16) tc::umma_bf16(ACC_S, mnmaj(R_BK, k16, 8192), mnmaj(R_DR, k16, 8192), I128_MM_NEG, 1u);
            tc::umma_commit(&bars[6]);
        }
        // column sums of P while G6 runs: BW_THREADS / 64 threads per column
        {
            constexpr int RPP = 64 / (BW_THREADS / 64);   // rows per partial sum
            const int col = tid & 63, part = tid >> 6;
            float cs = 0.0f;
            const float* P = reinterpret_cast<const float*>(sm + R_P);
#pragma unroll
            for (int t = part * RPP; t < part * RPP + RPP; ++t) cs += P[t * 64 + ((col + t) & 63)];
            v_colp4[part * 64 + col] = cs;
        }
        // ---- E. dq rows (half 0) and dk rows (half 1) into the f32 staging area (S0 + dS regions are free)
        wait_bar(5, par);
        tc::tcgen05_fence_after();
        {
            const int srow = half * 64 + row;
            float4* stg = reinterpret_cast<float4*>(sm + R_STG) + srow * 32;
            const int swz = (row + 16 * half) & 31;
            float rr = 0.0f;
#pragma unroll
            for (int pc = 0; pc < CW / 16; ++pc) {   // 16 columns at a time keeps the three accumulators in 48 registers
                uint32_t xa[16], xb[16], xc[16];
                const uint32_t col = (uint32_t)(colhalf * CW + pc * 16);
                tc::tmem_ld_cols<16>(ACC_A + lane_addr + col, xa);    // X (h0) | Y (h1)
                tc::tmem_ld_cols<16>(ACC_B + lane_addr + col, xb);    // G6
                tc::tmem_ld_cols<16>(ACC_C + lane_addr + col, xc);    // (h0: dL|dA) | dW (h1)
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int chunk16 = colhalf * (CW / 8) + pc * 2 + j;
                    float z8[8], g8[8];
                    tc::unpack8_bf16(*tile64(half == 0 ? R_QG : R_K, row, chunk16), z8);   // Qg_t | k_t
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float A_ = __uint_as_float(xa[8 * j + e]), B_ = __uint_as_float(xb[8 * j + e]),
                                    C_ = __uint_as_float(xc[8 * j + e]);
                        if (half == 0) {
                            g8[e] = fmaf(gam_row, A_, B_);
                            rr = fmaf(z8[e], A_, rr);                    // Qg_t . X_t
                        } else {
                            g8[e] = B_ + eg_row * C_ - be_row * gam_row * A_;
                            rr = fmaf(eg_row * z8[e], C_, rr);           // eg k_t . dW_t
                        }
                    }
                    stg[(2 * chunk16) ^ swz] = make_float4(g8[0], g8[1], g8[2], g8[3]);
                    stg[(2 * chunk16 + 1) ^ swz] = make_float4(g8[4], g8[5], g8[6], g8[7]);
                }
            }
            (half == 0 ? v_rqs : v_rkw)[colhalf * 64 + row] = rr;
        }
        __syncthreads();
        if (c > 0) fetch_small(c - 1);
        // L2-norm backward and store: 8 lanes per staged row (4 float4 each), 4 rows per warp at a time
        {
            constexpr int RPW = 128 / NWARPS;            // staged rows per warp (64 dq rows, then 64 dk rows)
            const int l8 = lane & 7, hh = (warp * RPW) >> 6;
            const int ytile = hh == 0 ? R_Q : R_K;
#pragma unroll
            for (int itn = 0; itn < RPW / 4; ++itn) {
                const int srow = warp * RPW + itn * 4 + (lane >> 3), r_ = srow & 63;
                const int swz = (r_ + 16 * hh) & 31;
                float4 g4[4];
                float y[4][4];
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int f4 = l8 + 8 * i;
                    g4[i] = reinterpret_cast<const float4*>(sm + R_STG)[srow * 32 + (f4 ^ swz)];
                    const uint2 yraw = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(tile64(ytile, r_, f4 >> 1)) + (f4 & 1) * 8);
                    const __nv_bfloat162 y01 = *reinterpret_cast<const __nv_bfloat162*>(&yraw.x), y23 = *reinterpret_cast<const __nv_bfloat162*>(&yraw.y);
                    y[i][0] = __low2float(y01), y[i][1] = __high2float(y01), y[i][2] = __low2float(y23), y[i][3] = __high2float(y23);
                    dot += y[i][0] * g4[i].x + y[i][1] * g4[i].y + y[i][2] * g4[i].z + y[i][3] * g4[i].w;
                }
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                dot += __shfl_xor_sync(0xffffffffu, dot, 4);
                if (r_ < n) {
                    const float inv = 1.0f / v_nrm[srow];
                    float* dst = d_qkv + (grow + r_) * 3 * d + (hh == 0 ? 0 : d) + h * dhi;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if ((l8 + 8 * i) * 4 < dhi)
                            reinterpret_cast<float4*>(dst)[l8 + 8 * i] = make_float4((g4[i].x - y[i][0] * dot) * inv, (g4[i].y - y[i][1] * dot) * inv,
                                                                                  (g4[i].z - y[i][2] * dot) * inv, (g4[i].w - y[i][3] * dot) * inv);
                }
            }
        }
        // gates (warp 0): dg, reverse cumulative sum, sigmoid backward
        if (warp == 0) {
            float sds = 0.0f;
            for (int i = lane; i < BW_THREADS; i += 32) sds += v_red[i];
            sds = warp_sum(sds);
            auto sumq = [&](const float* v, int t) {   // the NCQ column-group partials of one token
                float a = 0.0f;
#pragma unroll
                for (int qd = 0; qd < NCQ; ++qd) a += v[qd * 64 + t];
                return a;
            };
            auto colp = [&](int t) {
                float a = 0.0f;
#pragma unroll
                for (int qd = 0; qd < BW_THREADS / 64; ++qd) a += v_colp4[qd * 64 + t];
                return a;
            };
            const int tA = lane, tB = lane + 32;
            const float kwA = sumq(v_rkw, tA), kwB = sumq(v_rkw, tB);
            const float extra = __expf(g_last) * sds + warp_sum(kwA + kwB);
            float dgA = sumq(v_rowp, tA) - colp(tA) + sumq(v_rqs, tA) + sumq(v_rkg, tA) - kwA;
            float dgB = sumq(v_rowp, tB) - colp(tB) + sumq(v_rqs, tB) + sumq(v_rkg, tB) - kwB;
            if (lane == 31) dgB += extra;
            // suffix sums over t = 0..63 (A holds 0..31, B holds 32..63)
            float sB = dgB, sA = dgA;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float nb = __shfl_down_sync(0xffffffffu, sB, o), na = __shfl_down_sync(0xffffffffu, sA, o);
                if (lane + o < 32) {
                    sB += nb;
                    sA += na;
                }
            }
            const float totB = __shfl_sync(0xffffffffu, sB, 0);
            sA += totB;
            if (tA < n) {
                const int64_t r = grow + tA;
                const float be = be_s[tA];
                d_gate[r * 2 * H + h] = sA * (1.0f - v_al[tA]);
                d_gate[r * 2 * H + H + h] = (sumq(v_rdr, tA) + be * sumq(v_dls, tA)) * (1.0f - be);
            }
            if (tB < n) {
                const int64_t r = grow + tB;
                const float be = be_s[tB];
                d_gate[r * 2 * H + h] = sB * (1.0f - v_al[tB]);
                d_gate[r * 2 * H + H + h] = (sumq(v_rdr, tB) + be * sumq(v_dls, tB)) * (1.0f - be);
            }
        }
        // ---- F. new dS -> bf16 operand copy for the next chunk; next chunk's tiles
        wait_bar(6, par);
        tc::tcgen05_fence_after();
        __syncthreads();   // staging reads are finished before the dS region is rewritten
        if (c > 0) {
            if (dhi != DH) clear_s0_pad();
            if (tid == 0) {
                tc::fence_proxy_async_smem();
                issue_tma(c - 1);
            }
#pragma unroll
            for (int ci = 0; ci < NCI; ++ci) {
                uint32_t r[32];
                tc::tmem_ld_32x32(ACC_S + lane_addr + (c0 + ci) * 32, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float f8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(r[8 * j + e]);
                    *tile128(R_DS, arow, (c0 + ci) * 4 + j) = tc::pack8_bf16(f8);
                }
            }
        }
        if (__syncthreads_or(*abort_flag ? 1 : 0)) break;
    }
    tc::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) __nanosleep(20000);
    if (warp == 0) tc::tmem_dealloc(tm, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}
static bool make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static inline size_t al(size_t x) { return (x + 1023) & ~(size_t)1023; }

bool available() { return encode_fn() != nullptr; }

// Carves the per-(chain, chunk) tile buffers out of `w` (1024-byte aligned). With `full` the
// backward-only tiles are included.
static size_t carve_tiles(char* w, int64_t n_tiles, bool full, Tiles* t) {
    const size_t b128 = al((size_t)n_tiles * 128 * DH * 2), b64 = al((size_t)n_tiles * 64 * DH * 2),
                 bcc = al((size_t)n_tiles * 64 * 64 * 2), bv = al((size_t)n_tiles * 64 * 4), bg = al((size_t)n_tiles * 4);
    char* p = w;
    auto take = [&](size_t n) {
        char* r = p;
        p += n;
        return r;
    };
    Tiles z{};
    z.WQ = (__nv_bfloat16*)take(b128);
    z.UV = (__nv_bfloat16*)take(b64);
    z.KW = (__nv_bfloat16*)take(b64);
    z.AA = (__nv_bfloat16*)take(bcc);
    z.GC = (float*)take(bg);
    if (full) {
        z.BK = (__nv_bfloat16*)take(b64);
        z.BV = (__nv_bfloat16*)take(b64);
        z.UVT = (__nv_bfloat16*)take(b64);
        z.TP = (__nv_bfloat16*)take(bcc);
        z.KKo = (__nv_bfloat16*)take(bcc);
        z.QKo = (__nv_bfloat16*)take(bcc);
        z.GV = (float*)take(bv);
        z.BE = (float*)take(bv);
    }
    if (t) *t = z;
    return (size_t)(p - w);
}

static int run_prepass(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha,
                       const float* beta, int64_t T, int64_t H, int64_t dh, int64_t n_chunks, int64_t chains, const Tiles& t) {
    ASCA_CUDA(ctx, cudaFuncSetAttribute(delta_prep_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PRE_SMEM));
    {
        asca_span sp(ctx, "delta_prep_tc_kernel");
        delta_prep_tc_kernel<<<dim3((unsigned)n_chunks, (unsigned)chains), PRE_THREADS, PRE_SMEM, ctx->stream>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, alpha, beta, (int)T, (int)H, (int)dh,
            (int)n_chunks, t, ctx->err_word);
    }
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

// Forward for bf16 q,k,v (dh = 128, or 64 zero-padded to 128 inside). o is bf16. When checkpoints are requested (a
// backward will follow) the pre-pass also writes the backward-only tiles into a context-owned buffer keyed by
// the checkpoint pointer, so that the backward does not repeat the pre-pass. In this mode the
// checkpoint buffer holds the chunk-start states rounded to bf16, (B, H, n_chunks, dh, dh) row-major
// in its first half: the backward loads them by TMA as tensor-core operands.
int forward(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
            int64_t B, int64_t T, int64_t H, int64_t dh, void* o, const float* s_init, float* s_final, float* ckpt) {
    const int64_t n_chunks = (T + C - 1) / C, chains = B * H, n_tiles = chains * n_chunks;
    Tiles t{};
    const bool keep = ckpt != nullptr;
    const size_t need = carve_tiles(nullptr, n_tiles, keep, nullptr) + 1024;
    char* w;
    int slot = -1;
    if (keep) {
        auto& dt = ctx->dtiles;
        for (size_t i = 0; i < dt.size(); ++i)
            if (dt[i].buf && dt[i].ckpt == (const void*)ckpt) slot = (int)i;
        if (slot < 0) {   // a free entry, a new one, or the least recently used one
            for (size_t i = 0; i < dt.size() && slot < 0; ++i)
                if (!dt[i].ckpt) slot = (int)i;
            size_t total = 0;
            for (auto& e : dt) total += e.bytes;
            if (slot < 0 && dt.size() < 32 && total + need <= ctx->dtiles_cap) {
                dt.emplace_back();
                slot = (int)dt.size() - 1;
            }
            if (slot < 0) {
                slot = 0;
                for (size_t i = 1; i < dt.size(); ++i)
                    if (dt[i].stamp < dt[slot].stamp) slot = (int)i;
            }
        }
        auto& e = dt[slot];
        e.ckpt = nullptr;   // invalid until this forward has been queued
        if (need > e.bytes) {
            ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            if (e.buf) cudaFree(e.buf);
            e.buf = nullptr;
            e.bytes = 0;
            ASCA_CUDA(ctx, cudaMalloc(&e.buf, need));
            e.bytes = need;
        }
        w = (char*)e.buf;
    } else {
        void* ws;
        ASCA_TRY(asca_workspace(ctx, need, &ws));
        w = (char*)ws;
    }
    w = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(w) + 1023) & ~(uintptr_t)1023);
    carve_tiles(w, n_tiles, keep, &t);
    ASCA_TRY(run_prepass(ctx, q, k, v, alpha, beta, T, H, dh, n_chunks, chains, t));
    CUtensorMap mWQ, mUV, mKW, mAA, mS0;
    if (!make_map(&mWQ, t.WQ, n_tiles * 128, DH, 64, 128) || !make_map(&mUV, t.UV, n_tiles * 64, DH, 64, 64) ||
        !make_map(&mKW, t.KW, n_tiles * 64, DH, 64, 64) || !make_map(&mAA, t.AA, n_tiles * 64, 64, 64, 64) ||
        !(keep ? make_map(&mS0, ckpt, n_tiles * dh, dh, 64, (int)dh)   // bf16 states in the checkpoint buffer
               : make_map(&mS0, t.WQ, n_tiles * DH, DH, 64, 128)))    // (unused)
        return asca_fail(ctx, ASCA_ERR_CUDA, "delta_tc: cuTensorMapEncodeTiled failed");
    auto kern = delta_fwd_tc_kernel<__nv_bfloat16>;
    ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CH_SMEM));
    {
        asca_span sp(ctx, "delta_fwd_tc_kernel");
        kern<<<(unsigned)chains, CH_THREADS, CH_SMEM, ctx->stream>>>(mWQ, mUV, mKW, mAA, mS0, t.GC, (int)T, (int)H, (int)dh,
                                                                    (int)n_chunks, (__nv_bfloat16*)o, s_init, s_final,
                                                                    nullptr, reinterpret_cast<__nv_bfloat16*>(ckpt), ctx->err_word);
    }
    ASCA_CHECK_LAUNCH(ctx);
    if (keep) {
        auto& e = ctx->dtiles[slot];
        e.ckpt = ckpt;
        e.q = q; e.k = k; e.v = v; e.alpha = alpha; e.beta = beta;
        e.B = B;
        e.T = T;
        e.H = H * 1024 + dh;   // heads and head dim in one key field
        e.stamp = ++ctx->dtiles_clock;
    }
    return ASCA_OK;
}

// Backward for bf16 q,k,v,d_o (dh = 128 or 64, checkpoints every 64 tokens from the forward).
int backward(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
             const float* qnorm, const float* knorm, const void* d_o, const float* ckpt, int64_t B, int64_t T, int64_t H,
             int64_t dh, float* d_qkv, float* d_gate) {
    const int64_t n_chunks = (T + C - 1) / C, chains = B * H, n_tiles = chains * n_chunks;
    Tiles t{};
    int slot = -1;
    for (size_t i = 0; i < ctx->dtiles.size(); ++i) {
        const auto& e = ctx->dtiles[i];
        // the tiles are functions of q, k, v, alpha, beta: the same buffers must come back (their contents are the
        // caller's contract, see the header); anything else rebuilds the tiles
        if (e.buf && e.ckpt == (const void*)ckpt && e.q == q && e.k == k && e.v == v && e.alpha == (const void*)alpha &&
            e.beta == (const void*)beta && e.B == B && e.T == T && e.H == H * 1024 + dh)
            slot = (int)i;
    }
    if (slot >= 0) {
        // the forward that wrote `ckpt` left its tiles (functions of the same q,k,v,alpha,beta) here
        ctx->dtiles[slot].stamp = ++ctx->dtiles_clock;
        char* w = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ctx->dtiles[slot].buf) + 1023) & ~(uintptr_t)1023);
        carve_tiles(w, n_tiles, true, &t);
    } else {
        void* ws;
        ASCA_TRY(asca_workspace(ctx, carve_tiles(nullptr, n_tiles, true, nullptr) + 1024, &ws));
        char* w = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 1023) & ~(uintptr_t)1023);
        carve_tiles(w, n_tiles, true, &t);
        ASCA_TRY(run_prepass(ctx, q, k, v, alpha, beta, T, H, dh, n_chunks, chains, t));
    }
    CUtensorMap mWQ, mBK, mKW, mKR, mQR, mDO, mAA, mTP, mS0;
    bool ok = make_map(&mWQ, t.WQ, n_tiles * 128, DH, 64, 64) && make_map(&mBK, t.BK, n_tiles * 64, DH, 64, 64) &&
              make_map(&mKW, t.KW, n_tiles * 64, DH, 64, 64) && make_map(&mKR, k, B * T, H * dh, 64, 64) &&
              make_map(&mQR, q, B * T, H * dh, 64, 64) && make_map(&mDO, d_o, B * T, H * dh, 64, 64) &&
              make_map(&mAA, t.AA, n_tiles * 64, 64, 64, 64) && make_map(&mTP, t.TP, n_tiles * 64, 64, 64, 64) &&
              make_map(&mS0, ckpt, n_tiles * dh, dh, 64, (int)dh);
    if (!ok) return asca_fail(ctx, ASCA_ERR_CUDA, "delta_tc: cuTensorMapEncodeTiled failed");
    ASCA_CUDA(ctx, cudaFuncSetAttribute(delta_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BW_SMEM));
    {
        asca_span sp(ctx, "delta_bwd_tc_kernel");
        delta_bwd_tc_kernel<<<(unsigned)chains, BW_THREADS, BW_SMEM, ctx->stream>>>(
            mWQ, mBK, mKW, mKR, mQR, mDO, mAA, mTP, mS0, t, alpha, qnorm, knorm, (int)T, (int)H, (int)dh, (int)n_chunks, d_qkv,
            d_gate, ctx->err_word);
    }
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // namespace delta_tc
