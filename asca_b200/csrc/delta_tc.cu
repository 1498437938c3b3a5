// Gated delta rule, bf16 mode, chunk-parallel WY/UT forward on the 5th-generation tensor cores.
//
// Chunk of C = 64 tokens, head dim 128, state S (128 x 128) kept in f32 in TMEM for the whole
// sequence. With g = cumsum(log alpha), gam = exp(g), Gam[t,i] = exp(g_t - g_i), eg = exp(g_C - g):
//
//   pre-pass (one CTA per (sequence, head, chunk) -- fully parallel, nothing depends on S):
//     KK = K K^T, QK = Q K^T                                   tcgen05, M128 N64 K128 ([K;Q] stacked)
//     L  = strictlower(beta_t Gam KK)   A = lower(Gam QK)      f32 registers
//     T' = (I + L)^-1 - I                                      f32 forward substitution per column
//     [W^ | Uv] = (I + T') [beta gam K | beta V]               tcgen05, M128(padded) N256 K64; the
//                                                              identity part is added exactly in f32
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
};

// ------------------------------------------------------------------ pre-pass
constexpr int PRE_THREADS = 128;
constexpr int LF_LD = 68;
constexpr size_t PRE_SMEM = 1024 + NB * 16384 /*KQ*/ + 2 * NB * 8192 /*Bop*/ + 16384 /*Tp*/ + 64 * LF_LD * 4 + 4 * 64 * 4 + 64;

__global__ void __launch_bounds__(PRE_THREADS) delta_prep_tc_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const float* __restrict__ alpha, const float* __restrict__ beta, int T, int H, int n_chunks, Tiles out,
    int* err_word) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* KQ_s = base;                         // NB k-boxes x (128 rows x 128 B): rows 0-63 K, 64-127 Q
    uint8_t* Bop_s = KQ_s + NB * 16384;           // 2*NB n-boxes x (64 k-rows x 128 B): [beta gam K | beta V]
    uint8_t* Tp_s = Bop_s + 2 * NB * 8192;        // 128 rows x 128 B: T' (rows 64-127 zero)
    float* Lf = reinterpret_cast<float*>(Tp_s + 16384);
    float* g_s = Lf + 64 * LF_LD;
    float* gam_s = g_s + 64;
    float* eg_s = gam_s + 64;
    float* be_s = eg_s + 64;
    uint64_t* bar = reinterpret_cast<uint64_t*>(be_s + 64);   // [0] MMA-A done, [1] MMA-B done
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int chunk = blockIdx.x, chain = blockIdx.y;
    const int b = chain / H, h = chain % H;
    const int d = H * DH;
    const int t0 = chunk * C;
    const int n = T - t0 < C ? T - t0 : C;
    const int64_t row0 = (int64_t)b * T + t0;
    const int64_t tix = (int64_t)chain * n_chunks + chunk;

    if (tid == 0) {
        *abort_flag = 0;
        tc::mbar_init(&bar[0], 1);
        tc::mbar_init(&bar[1], 1);
        tc::mbar_fence_init();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, 256);
    if (tid < C) {
        const bool live = tid < n;
        const float a = live ? alpha[(row0 + tid) * H + h] : 1.0f;
        be_s[tid] = live ? beta[(row0 + tid) * H + h] : 0.0f;
        g_s[tid] = logf(a);
    }
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) {
        float run = 0.0f;
        for (int t = 0; t < C; ++t) {
            run += g_s[t];
            g_s[t] = run;
        }
    }
    __syncthreads();
    if (tid < C) {
        gam_s[tid] = expf(g_s[tid]);
        eg_s[tid] = expf(g_s[C - 1] - g_s[tid]);
    }
    __syncthreads();

    // ---- stage K, Q (K-major, swizzled), build [beta gam K | beta V], emit Qg and Kw
    for (int idx = tid; idx < C * (DH / 8); idx += PRE_THREADS) {
        const int t = idx / (DH / 8), j = idx % (DH / 8);
        uint4 k8 = make_uint4(0, 0, 0, 0), q8 = k8, v8 = k8;
        if (t < n) {
            const int64_t off = (row0 + t) * d + h * DH + j * 8;
            k8 = *reinterpret_cast<const uint4*>(k + off);
            q8 = *reinterpret_cast<const uint4*>(q + off);
            v8 = *reinterpret_cast<const uint4*>(v + off);
        }
        const int box = j >> 3, jc = j & 7;
        *reinterpret_cast<uint4*>(KQ_s + box * 16384 + tc::sw128_off(t, jc)) = k8;
        *reinterpret_cast<uint4*>(KQ_s + box * 16384 + tc::sw128_off(64 + t, jc)) = q8;
        float kf[8], qf[8], vf[8], tmp[8];
        tc::unpack8_bf16(k8, kf);
        tc::unpack8_bf16(q8, qf);
        tc::unpack8_bf16(v8, vf);
        const float be = be_s[t], gm = gam_s[t], eg = eg_s[t];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = be * gm * kf[e];
        *reinterpret_cast<uint4*>(Bop_s + box * 8192 + tc::sw128_off(t, jc)) = tc::pack8_bf16(tmp);
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = be * vf[e];
        *reinterpret_cast<uint4*>(Bop_s + (NB + box) * 8192 + tc::sw128_off(t, jc)) = tc::pack8_bf16(tmp);
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = gm * qf[e];
        *reinterpret_cast<uint4*>(out.WQ + (tix * 128 + 64 + t) * DH + j * 8) = tc::pack8_bf16(tmp);
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = eg * kf[e];
        *reinterpret_cast<uint4*>(out.KW + (tix * 64 + t) * DH + j * 8) = tc::pack8_bf16(tmp);
    }
    // rows 64-127 of the T' operand stay zero
    for (int i = tid; i < 8192 / 16; i += PRE_THREADS) *reinterpret_cast<uint4*>(Tp_s + 8192 + i * 16) = make_uint4(0, 0, 0, 0);
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
    int got = 1;
    if (lane == 0) got = tc::mbar_wait(&bar[0], 0, abort_flag, err_word, 201) ? 1 : 0;
    bool ok = __shfl_sync(0xffffffffu, got, 0) != 0;
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    tc::tcgen05_fence_after();
    if (ok) {
        uint32_t r[32];
        const int t = tid & 63;
        const float gt = g_s[t], bt = be_s[t];
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
            tc::tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + cc * 32, r);
            tc::tmem_ld_wait();
            if (tid < 64) {   // L = strictlower(beta_t Gam KK), f32
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int i = cc * 32 + j;
                    Lf[t * LF_LD + i] = i < t ? bt * __expf(gt - g_s[i]) * __uint_as_float(r[j]) : 0.0f;
                }
            } else {          // A = lower(Gam QK), bf16 tile for the chain kernel
                float a[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int i = cc * 32 + j;
                    a[j] = i <= t ? __expf(gt - g_s[i]) * __uint_as_float(r[j]) : 0.0f;
                }
                uint4* dst = reinterpret_cast<uint4*>(out.AA + (tix * 64 + t) * 64 + cc * 32);
#pragma unroll
                for (int j = 0; j < 4; ++j) dst[j] = tc::pack8_bf16(a + 8 * j);
            }
        }
    }
    tc::tcgen05_fence_before();
    __syncthreads();

    // ---- T' = (I + L)^-1 - I, one column per thread (f32 forward substitution)
    if (tid < 64 && ok) {
        const int j = tid;
        float x[C];
#pragma unroll
        for (int t = 0; t < C; ++t) {
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i + 3 < t; i += 4) {
                const float4 l4 = *reinterpret_cast<const float4*>(&Lf[t * LF_LD + i]);
                s0 = fmaf(l4.x, x[i], s0);
                s1 = fmaf(l4.y, x[i + 1], s1);
                s2 = fmaf(l4.z, x[i + 2], s2);
                s3 = fmaf(l4.w, x[i + 3], s3);
            }
#pragma unroll
            for (int i = t & ~3; i < t; ++i) s0 = fmaf(Lf[t * LF_LD + i], x[i], s0);
            x[t] = (t == j ? 1.0f : 0.0f) - ((s0 + s1) + (s2 + s3));
            const float tp = t == j ? 0.0f : x[t];
            *reinterpret_cast<__nv_bfloat16*>(Tp_s + tc::sw128_off(t, j >> 3) + (j & 7) * 2) = __float2bfloat16(tp);
        }
    }
    tc::fence_proxy_async_smem();
    __syncthreads();

    // ---- MMA-B: [T'(beta gam K) | T'(beta V)]   (M128 N256 K64)
    if (tid == 0 && ok) {
        constexpr uint32_t IDESC = tc::idesc_bf16_f32(128, 2 * DH, 0, 1);
        const uint32_t ta = tc::smem_u32(Tp_s), bo = tc::smem_u32(Bop_s);
        tc::tcgen05_fence_after();
#pragma unroll
        for (int k16 = 0; k16 < C / 16; ++k16)
            tc::umma_bf16(tmem, tc::smem_desc_sw128(ta + k16 * 32, 16, 1024),
                          tc::smem_desc_sw128(bo + k16 * 2048, 8192, 1024), IDESC, k16 > 0 ? 1u : 0u);
        tc::umma_commit(&bar[1]);
    }
    if (warp < 2 && ok) {
        got = 1;
        if (lane == 0) got = tc::mbar_wait(&bar[1], 0, abort_flag, err_word, 202) ? 1 : 0;
        const bool ok2 = __shfl_sync(0xffffffffu, got, 0) != 0;
        tc::tcgen05_fence_after();
        if (ok2) {
            const int t = tid;
            const float be = be_s[t], bg = be_s[t] * gam_s[t];
            const bool live = t < n;
            const int64_t in_off = (row0 + (live ? t : 0)) * d + h * DH;
            uint32_t r[32];
#pragma unroll 1
            for (int cc = 0; cc < 2 * DH / 32; ++cc) {
                tc::tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + cc * 32, r);
                tc::tmem_ld_wait();
                const bool is_w = cc < DH / 32;
                const int c0 = (is_w ? cc : cc - DH / 32) * 32;
                const __nv_bfloat16* src = (is_w ? k : v) + in_off + c0;
                const float sc = is_w ? bg : be;
                __nv_bfloat16* dst = is_w ? out.WQ + (tix * 128 + t) * DH + c0 : out.UV + (tix * 64 + t) * DH + c0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float x8[8], o8[8];
                    if (live) tc::unpack8_bf16(*reinterpret_cast<const uint4*>(src + 8 * j), x8);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o8[e] = __uint_as_float(r[8 * j + e]) + (live ? sc * x8[e] : 0.0f);
                    *reinterpret_cast<uint4*>(dst + 8 * j) = tc::pack8_bf16(o8);
                }
            }
        }
    }
    if (tid == 0) out.GC[tix] = gam_s[C - 1];
    tc::tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------ chain kernel
constexpr int CH_THREADS = 160;
constexpr int STAGE_BYTES = NB * 16384 /*WQ*/ + NB * 8192 /*UV*/ + NB * 8192 /*KW*/ + 16384 /*[0;A]*/;
constexpr int TX_BYTES = NB * 16384 + NB * 8192 + NB * 8192 + 8192;
constexpr size_t CH_SMEM = 1024 + 2 * STAGE_BYTES + NB * DH * 128 /*S bf16*/ + NB * 8192 /*U bf16*/ + 128;

template <typename TO>
__global__ void __launch_bounds__(CH_THREADS, 1) delta_fwd_tc_kernel(
    const __grid_constant__ CUtensorMap mapWQ, const __grid_constant__ CUtensorMap mapUV,
    const __grid_constant__ CUtensorMap mapKW, const __grid_constant__ CUtensorMap mapAA, const float* __restrict__ GC,
    int T, int H, int n_chunks, TO* __restrict__ o, const float* __restrict__ s_init, float* __restrict__ s_final,
    float* __restrict__ ckpt, int* err_word) {
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
    const int d = H * DH;
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
                tc::umma_commit(mma2_done);
                if (c + 2 < n_chunks) {
                    if (!tc::mbar_wait(mma2_done, c & 1, abort_flag, err_word, 214)) break;
                    load(c + 2, s);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ compute threads: TMEM lane = tid
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float* ck = ckpt ? ckpt + tile0 * DH * DH : nullptr;
        // initial state: checkpoint 0, bf16 operand copy, f32 state scaled by the first chunk's decay
        {
            const float g0 = GC[tile0];
            const float* si = s_init ? s_init + (int64_t)chain * DH * DH + (int64_t)tid * DH : nullptr;
#pragma unroll 1
            for (int cc = 0; cc < DH / 32; ++cc) {
                uint32_t r[32];
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = si ? si[cc * 32 + j] : 0.0f;
                if (ck) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(ck + (int64_t)tid * DH + cc * 32)[j] =
                            make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int chunk16 = cc * 4 + j;   // 16-byte chunk index along the row (8 bf16 each)
                    *reinterpret_cast<uint4*>(S_s + (chunk16 >> 3) * (DH * 128) + tc::sw128_off(tid, chunk16 & 7)) =
                        tc::pack8_bf16(f + 8 * j);
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
                TO* orow = o + (row0 + c * C + (live ? t : 0)) * d + h * DH;
#pragma unroll 1
                for (int cc = 0; cc < DH / 32; ++cc) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(tmem_D + lane_addr + cc * 32, r);
                    tc::tmem_ld_wait();
                    if (live) {
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
            float* dst = last ? (s_final ? s_final + (int64_t)chain * DH * DH : nullptr)
                              : (ck ? ck + (int64_t)(c + 1) * DH * DH : nullptr);
#pragma unroll 1
            for (int cc = 0; cc < DH / 32; ++cc) {
                uint32_t r[32];
                tc::tmem_ld_32x32(tmem_S + lane_addr + cc * 32, r);
                tc::tmem_ld_wait();
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
                if (dst) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<float4*>(dst + (int64_t)tid * DH + cc * 32)[j] =
                            make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
                }
                if (!last) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int chunk16 = cc * 4 + j;
                        *reinterpret_cast<uint4*>(S_s + (chunk16 >> 3) * (DH * 128) + tc::sw128_off(tid, chunk16 & 7)) =
                            tc::pack8_bf16(f + 8 * j);
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

// Forward for bf16 q,k,v (dh = 128). o may be bf16 (same dtype as the inputs).
int forward(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
            int64_t B, int64_t T, int64_t H, void* o, const float* s_init, float* s_final, float* ckpt) {
    const int64_t n_chunks = (T + C - 1) / C, chains = B * H, n_tiles = chains * n_chunks;
    const size_t b_wq = al((size_t)n_tiles * 128 * DH * 2), b_uv = al((size_t)n_tiles * 64 * DH * 2),
                 b_aa = al((size_t)n_tiles * 64 * 64 * 2), b_gc = al((size_t)n_tiles * 4);
    void* ws;
    ASCA_TRY(asca_workspace(ctx, b_wq + 2 * b_uv + b_aa + b_gc + 1024, &ws));
    char* w = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 1023) & ~(uintptr_t)1023);
    Tiles t;
    t.WQ = (__nv_bfloat16*)w;
    t.UV = (__nv_bfloat16*)(w + b_wq);
    t.KW = (__nv_bfloat16*)(w + b_wq + b_uv);
    t.AA = (__nv_bfloat16*)(w + b_wq + 2 * b_uv);
    t.GC = (float*)(w + b_wq + 2 * b_uv + b_aa);
    ASCA_CUDA(ctx, cudaFuncSetAttribute(delta_prep_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PRE_SMEM));
    delta_prep_tc_kernel<<<dim3((unsigned)n_chunks, (unsigned)chains), PRE_THREADS, PRE_SMEM, ctx->stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, alpha, beta, (int)T, (int)H,
        (int)n_chunks, t, ctx->err_word);
    ASCA_CHECK_LAUNCH(ctx);
    CUtensorMap mWQ, mUV, mKW, mAA;
    if (!make_map(&mWQ, t.WQ, n_tiles * 128, DH, 64, 128) || !make_map(&mUV, t.UV, n_tiles * 64, DH, 64, 64) ||
        !make_map(&mKW, t.KW, n_tiles * 64, DH, 64, 64) || !make_map(&mAA, t.AA, n_tiles * 64, 64, 64, 64))
        return asca_fail(ctx, ASCA_ERR_CUDA, "delta_tc: cuTensorMapEncodeTiled failed");
    auto kern = delta_fwd_tc_kernel<__nv_bfloat16>;
    ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CH_SMEM));
    kern<<<(unsigned)chains, CH_THREADS, CH_SMEM, ctx->stream>>>(mWQ, mUV, mKW, mAA, t.GC, (int)T, (int)H, (int)n_chunks,
                                                                (__nv_bfloat16*)o, s_init, s_final, ckpt, ctx->err_word);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // namespace delta_tc
