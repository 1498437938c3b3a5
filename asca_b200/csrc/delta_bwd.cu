// Gated delta rule, BPTT backward, f32-exact, as a reverse CHUNKED scan.
//
// The reference walks time backwards one step at a time and reads two full dh x dh states per
// step from a (T+1)*dh*dh history (rust/src/delta.rs:485-572, rust/kernels/asca.cu:340-485).
// Here no per-step state exists. The forward leaves one state per `chunk` tokens; one CTA per
// (sequence, head) walks those checkpoints in reverse, and inside a checkpoint interval works
// on sub-chunks of C tokens in the WY/UT form:
//
//   g_t = sum_{j<=t} log(alpha_j), gam = exp(g), Gam[t,i] = exp(g_t - g_i) (i <= t, always <= 1)
//   L = strictlower(beta_t Gam (K K^T)),  A = lower(Gam (Q K^T)),  eg_t = exp(g_last - g_t)
//   Z = V - diag(gam) K S0,  U = (I+L)^-1 diag(beta) Z            (forward recompute)
//   dU  = A^T dO + diag(eg) K dS          dR = (I+L)^-T dU        dV = diag(beta) dR = dZ
//   dL  = -strictlower(dR U^T)            dA = lower(dO U^T)
//   dbeta_t = dR_t.Z_t + sum_i dL[t,i] Gam[t,i] (k_t.k_i)
//   dQ  = diag(gam) dO S0^T + (dA.Gam) K
//   dK  = (dA.Gam)^T Q + (M + M^T) K + diag(eg) U dS^T - diag(gam) dZ S0^T,  M = dL.beta_t.Gam
//   dg_t = rowsum_t(P) - colsum_t(P) + gam_t q_t.(S0 dO_t) + gam_t k_t.dKg_t - eg_t k_t.dW_t,
//          P = (dA.Gam).(Q K^T) + M.(K K^T);  dg_last += sum_t eg_t k_t.dW_t + gam_last <S0,dS>
//   dlogalpha_j = sum_{t>=j} dg_t;   d_gate_alpha = dlogalpha (1 - alpha)
//   dS0 = gam_last dS + (diag(gam) Q)^T dO - (diag(gam) K)^T dZ    -> dS of the previous sub-chunk
//
// followed in the same kernel by the per-head L2-norm backward (rust/src/delta.rs:678-698), the
// sigmoid backward and the [dq|dk|dv] concat (rust/src/delta.rs:594-611). When a checkpoint
// interval spans several sub-chunks, the states at the inner boundaries are first recomputed
// forward (S_C = gam_last S0 + (diag(eg) K)^T U) into a small per-CTA scratch that stays in L2.
//
// All products are FFMA with f32 accumulation from shared memory; row strides are padded by 4
// floats so float4 reads along a row are aligned and rows fall in different banks.
#include "common.cuh"

bool asca_tc_enabled();  // gemm.cu
namespace delta_tc {
bool available();
int backward(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
             const float* qnorm, const float* knorm, const void* d_o, const float* ckpt, int64_t B, int64_t T, int64_t H,
             int64_t dh, float* d_qkv, float* d_gate);
}  // namespace delta_tc

namespace {

constexpr int BT = 256;  // threads per CTA

enum { L_MK = 0, L_KM = 1 };  // A operand layout: [m][k] or [k][m]
enum { L_KN = 0, L_NK = 1 };  // B operand layout: [k][n] or [n][k]

// C[m][n] = sum_k A(m,k) B(k,n) for an M x N output with N % 4 == 0 and operands in shared
// memory (lda/ldb multiples of 4, 16-byte aligned). Threads tile the output TM x 4; `epi(m, n,
// acc)` receives each finished element. K % 4 == 0 where an operand is contiguous along k.
template <int M, int N, int K, int ALAY, int BLAY, class Epi>
__device__ __forceinline__ void cta_gemm(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb,
                                         Epi epi) {
    constexpr int TN = 4;
    constexpr int THR_N = N / TN;
    constexpr int THR_M_MAX = BT / THR_N > 0 ? BT / THR_N : 1;
    constexpr int THR_M = THR_M_MAX < M ? THR_M_MAX : M;
    constexpr int TM = M / THR_M;
    constexpr bool KM_VEC = ALAY == L_KM && BLAY == L_KN && TM % 4 == 0 && THR_N % 32 == 0;
    static_assert(N % TN == 0 && THR_N <= BT && M % THR_M == 0, "tile shape");
    const int tid = threadIdx.x;
    if (tid >= THR_N * THR_M) return;
    const int tn = tid % THR_N, tm = tid / THR_N;
    const int n0 = tn * TN;
    // rows of this thread: m = tm + THR_M * i  (interleaved so KM loads stay scalar-broadcast)
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    constexpr int UNR = TM <= 2 ? 4 : 2;   // small register tiles: more k-steps of loads in flight per warp
    if (ALAY == L_MK && BLAY == L_KN) {
#pragma unroll UNR
        for (int k = 0; k < K; k += 4) {
            float4 a[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = *reinterpret_cast<const float4*>(A + (tm + THR_M * i) * lda + k);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float4 b = *reinterpret_cast<const float4*>(B + (k + kk) * ldb + n0);
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float av = kk == 0 ? a[i].x : kk == 1 ? a[i].y : kk == 2 ? a[i].z : a[i].w;
                    acc[i][0] = fmaf(av, b.x, acc[i][0]);
                    acc[i][1] = fmaf(av, b.y, acc[i][1]);
                    acc[i][2] = fmaf(av, b.z, acc[i][2]);
                    acc[i][3] = fmaf(av, b.w, acc[i][3]);
                }
            }
        }
    } else if (ALAY == L_KM && BLAY == L_KN) {
        if (KM_VEC) {   // rows tm * TM + i: the lanes of a warp share tm, so A arrives as broadcast float4 loads
#pragma unroll 2
            for (int k = 0; k < K; ++k) {
                const float4 b = *reinterpret_cast<const float4*>(B + k * ldb + n0);
#pragma unroll
                for (int i4 = 0; i4 < TM / 4; ++i4) {
                    const float4 a4 = *reinterpret_cast<const float4*>(A + k * lda + tm * TM + 4 * i4);
                    const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[4 * i4 + e][0] = fmaf(av[e], b.x, acc[4 * i4 + e][0]);
                        acc[4 * i4 + e][1] = fmaf(av[e], b.y, acc[4 * i4 + e][1]);
                        acc[4 * i4 + e][2] = fmaf(av[e], b.z, acc[4 * i4 + e][2]);
                        acc[4 * i4 + e][3] = fmaf(av[e], b.w, acc[4 * i4 + e][3]);
                    }
                }
            }
        } else {
#pragma unroll 4
            for (int k = 0; k < K; ++k) {
                const float4 b = *reinterpret_cast<const float4*>(B + k * ldb + n0);
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float av = A[k * lda + tm + THR_M * i];
                    acc[i][0] = fmaf(av, b.x, acc[i][0]);
                    acc[i][1] = fmaf(av, b.y, acc[i][1]);
                    acc[i][2] = fmaf(av, b.z, acc[i][2]);
                    acc[i][3] = fmaf(av, b.w, acc[i][3]);
                }
            }
        }
    } else {  // L_MK x L_NK: both contiguous along k; this thread's columns are tn + THR_N * j, so that the lanes of a
              // quarter warp read 8 consecutive rows of B (row stride = 4 banks: all 32 banks, no conflict)
#pragma unroll UNR
        for (int k = 0; k < K; k += 4) {
            float4 b[TN];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = *reinterpret_cast<const float4*>(B + (tn + THR_N * j) * ldb + k);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
                const float4 a = *reinterpret_cast<const float4*>(A + (tm + THR_M * i) * lda + k);
#pragma unroll
                for (int j = 0; j < TN; ++j) {
                    acc[i][j] = fmaf(a.x, b[j].x, acc[i][j]);
                    acc[i][j] = fmaf(a.y, b[j].y, acc[i][j]);
                    acc[i][j] = fmaf(a.z, b[j].z, acc[i][j]);
                    acc[i][j] = fmaf(a.w, b[j].w, acc[i][j]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j)
            epi(KM_VEC ? tm * TM + i : tm + THR_M * i, (ALAY == L_MK && BLAY == L_NK) ? tn + THR_N * j : n0 + j, acc[i][j]);
}

template <typename T>
__device__ __forceinline__ void load_rows(const T* __restrict__ src, int64_t row0, int64_t ld, int col0, int n, int C,
                                          int W, float* __restrict__ dst, int ldd) {
    // dst[t][c] = src[(row0+t)*ld + col0 + c] for t < n, zero for n <= t < C.  W % 4 == 0.
    const int w4 = W / 4;
    for (int idx = threadIdx.x; idx < C * w4; idx += BT) {
        const int t = idx / w4, c = (idx % w4) * 4;
        float4 val = make_float4(0, 0, 0, 0);
        if (t < n) {
            const T* p = src + (row0 + t) * ld + col0 + c;
            if (sizeof(T) == 4) {
                val = *reinterpret_cast<const float4*>(p);
            } else {
                uint2 raw = *reinterpret_cast<const uint2*>(p);
                __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&raw.x),
                               b = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
                val = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
            }
        }
        *reinterpret_cast<float4*>(dst + t * ldd + c) = val;
    }
}

template <int DH, int C>
struct BwdSmem {
    static constexpr int LDK = DH + 4;   // K, Q, bufA, bufB rows
    static constexpr int LDV = DH + 4;   // value-width rows (Z, U, dO, dR, S0, dS)
    static constexpr int LDC = C + 4;    // C x C rows
    static constexpr int N_CC = 7;       // KK, QK, Gam, L, A, dL/M, dA
    static constexpr int floats = 2 * C * LDK      /* K, Q */
                                  + 4 * C * LDV    /* Z, U, dO, dR */
                                  + 2 * DH * LDV   /* S0, dS */
                                  + 2 * C * LDK    /* bufA, bufB */
                                  + N_CC * C * LDC + 16 * C + 64;
    static constexpr size_t bytes = (size_t)floats * 4;
};

template <int DH, int C, typename T>
__global__ void __launch_bounds__(BT, 1) delta_bwd_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ alpha,
    const float* __restrict__ beta, const float* __restrict__ qnorm, const float* __restrict__ knorm,
    const T* __restrict__ d_o, const float* __restrict__ ckpt, float* __restrict__ sub_ckpt, int B, int Tlen, int H,
    int chunk, float* __restrict__ d_qkv, float* __restrict__ d_gate) {
    using SM = BwdSmem<DH, C>;
    constexpr int LDK = SM::LDK, LDV = SM::LDV, LDC = SM::LDC;
    static_assert(C <= 32, "the gate scans run in one warp");
    extern __shared__ __align__(16) float smem[];
    float* Ks = smem;
    float* Qs = Ks + C * LDK;
    float* Zs = Qs + C * LDK;     // V, then Z = V - gam K S0
    float* Us = Zs + C * LDV;     // R = beta Z, then U
    float* dOs = Us + C * LDV;
    float* dRs = dOs + C * LDV;   // dU -> dR -> dZ
    float* S0 = dRs + C * LDV;
    float* dS = S0 + DH * LDV;
    float* bufA = dS + DH * LDV;
    float* bufB = bufA + C * LDK;
    float* KK = bufB + C * LDK;
    float* QK = KK + C * LDC;
    float* Gm = QK + C * LDC;
    float* Lm = Gm + C * LDC;
    float* Am = Lm + C * LDC;
    float* dLm = Am + C * LDC;
    float* dAm = dLm + C * LDC;
    float* vec = dAm + C * LDC;
    float* g_s = vec;             // cumulative log alpha
    float* gam_s = vec + C;       // exp(g)
    float* eg_s = vec + 2 * C;    // exp(g_last - g)
    float* be_s = vec + 3 * C;    // beta (0 on padded steps)
    float* al_s = vec + 4 * C;    // alpha (1 on padded steps)
    float* r_qs = vec + 5 * C;    // gam_t q_t.(S0 dO_t)
    float* r_kg = vec + 6 * C;    // gam_t k_t.dKg_t
    float* r_kw = vec + 7 * C;    // eg_t k_t.dW_t
    float* dbe_s = vec + 8 * C;   // dbeta
    float* dg_s = vec + 9 * C;    // dg
    float* red = vec + 16 * C;    // 33 floats

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chain = blockIdx.x;
    const int bi = chain / H, h = chain % H;
    const int d = H * DH;
    const int64_t row0 = (int64_t)bi * Tlen;
    const int n_ck = (Tlen + chunk - 1) / chunk;
    const int sub_per_ck = (chunk + C - 1) / C;
    float* my_sub = sub_ckpt + (int64_t)chain * sub_per_ck * DH * DH;

    for (int i = tid; i < DH * LDV; i += BT) dS[i] = 0.0f;

    auto load_state = [&](const float* src) {
        for (int idx = tid; idx < DH * (DH / 4); idx += BT) {
            const int a = idx / (DH / 4), c = (idx % (DH / 4)) * 4;
            *reinterpret_cast<float4*>(S0 + a * LDV + c) = *reinterpret_cast<const float4*>(src + a * DH + c);
        }
    };
    auto store_state = [&](float* dst) {
        for (int idx = tid; idx < DH * (DH / 4); idx += BT) {
            const int a = idx / (DH / 4), c = (idx % (DH / 4)) * 4;
            *reinterpret_cast<float4*>(dst + a * DH + c) = *reinterpret_cast<const float4*>(S0 + a * LDV + c);
        }
    };

    // Shared front part of a sub-chunk starting at token t0 with n live steps: loads K (and Q,
    // dO when `full`), V, gates; builds g, gam, eg, Gam, KK, L (and QK, A); Z, R; solves U.
    auto chunk_front = [&](int t0, int n, bool full) {
        load_rows<T>(k, row0 + t0, d, h * DH, n, C, DH, Ks, LDK);
        load_rows<T>(v, row0 + t0, d, h * DH, n, C, DH, Zs, LDV);
        if (full) {
            load_rows<T>(q, row0 + t0, d, h * DH, n, C, DH, Qs, LDK);
            load_rows<T>(d_o, row0 + t0, d, h * DH, n, C, DH, dOs, LDV);
        }
        if (tid < C) {
            const bool live = tid < n;
            const float a = live ? alpha[(row0 + t0 + tid) * H + h] : 1.0f;
            al_s[tid] = a;
            be_s[tid] = live ? beta[(row0 + t0 + tid) * H + h] : 0.0f;
            g_s[tid] = logf(a);
        }
        __syncthreads();
        if (warp == 0) {   // inclusive scan of the C (<= 32) log alphas, left to right
            float gx = lane < C ? g_s[lane] : 0.0f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float y = __shfl_up_sync(0xffffffffu, gx, o);
                if (lane >= o) gx += y;
            }
            if (lane < C) g_s[lane] = gx;
        }
        __syncthreads();
        if (tid < C) {
            gam_s[tid] = expf(g_s[tid]);
            eg_s[tid] = expf(g_s[C - 1] - g_s[tid]);
        }
        for (int idx = tid; idx < C * C; idx += BT) {
            const int t = idx / C, i = idx % C;
            Gm[t * LDC + i] = i <= t ? expf(g_s[t] - g_s[i]) : 0.0f;
        }
        __syncthreads();
        // KK = K K^T (and QK = Q K^T): one output element per thread pass
        for (int idx = tid; idx < C * C; idx += BT) {
            const int t = idx / C, i = idx % C;
            float s1 = 0.0f, s2 = 0.0f;
            const float* kt = Ks + t * LDK;
            const float* ki = Ks + i * LDK;
            const float* qt = Qs + t * LDK;
#pragma unroll 4
            for (int a = 0; a < DH; a += 4) {
                const float4 x = *reinterpret_cast<const float4*>(kt + a), y = *reinterpret_cast<const float4*>(ki + a);
                s1 = fmaf(x.x, y.x, s1); s1 = fmaf(x.y, y.y, s1); s1 = fmaf(x.z, y.z, s1); s1 = fmaf(x.w, y.w, s1);
                if (full) {
                    const float4 z = *reinterpret_cast<const float4*>(qt + a);
                    s2 = fmaf(z.x, y.x, s2); s2 = fmaf(z.y, y.y, s2); s2 = fmaf(z.z, y.z, s2); s2 = fmaf(z.w, y.w, s2);
                }
            }
            const float gm = Gm[t * LDC + i];
            KK[t * LDC + i] = s1;
            Lm[t * LDC + i] = i < t ? be_s[t] * gm * s1 : 0.0f;
            if (full) {
                QK[t * LDC + i] = s2;
                Am[t * LDC + i] = gm * s2;  // gm is 0 above the diagonal
            }
        }
        // Z = V - gam K S0 ; R = beta Z
        cta_gemm<C, DH, DH, L_MK, L_KN>(Ks, LDK, S0, LDV, [&](int t, int c, float acc) {
            const float z = Zs[t * LDV + c] - gam_s[t] * acc;
            Zs[t * LDV + c] = z;
            Us[t * LDV + c] = be_s[t] * z;
        });
        __syncthreads();
        // U = (I + L)^-1 R : one thread per value column, forward substitution in registers
        if (tid < DH) {
            float x[C];
#pragma unroll
            for (int t = 0; t < C; ++t) {
                float s = Us[t * LDV + tid];
#pragma unroll
                for (int i = 0; i < t; ++i) s = fmaf(-Lm[t * LDC + i], x[i], s);
                x[t] = s;
                Us[t * LDV + tid] = s;
            }
        }
        __syncthreads();
    };

    for (int ck = n_ck - 1; ck >= 0; --ck) {
        const int t_lo = ck * chunk;
        const int t_hi = t_lo + chunk < Tlen ? t_lo + chunk : Tlen;
        const int nsub = (t_hi - t_lo + C - 1) / C;
        const float* ck_state = ckpt + ((int64_t)chain * n_ck + ck) * DH * DH;

        // ---- phase F: states at the inner sub-chunk boundaries
        if (nsub > 1) {
            __syncthreads();
            load_state(ck_state);
            __syncthreads();
            for (int j = 0; j + 1 < nsub; ++j) {
                chunk_front(t_lo + j * C, C, false);
                // S0 <- gam_last S0 + (diag(eg) K)^T U
                for (int idx = tid; idx < C * DH; idx += BT) {
                    const int t = idx / DH, a = idx % DH;
                    bufA[t * LDK + a] = eg_s[t] * Ks[t * LDK + a];
                }
                __syncthreads();
                const float gl = gam_s[C - 1];
                cta_gemm<DH, DH, C, L_KM, L_KN>(bufA, LDK, Us, LDV, [&](int a, int c, float acc) {
                    S0[a * LDV + c] = fmaf(gl, S0[a * LDV + c], acc);
                });
                __syncthreads();
                store_state(my_sub + (int64_t)(j + 1) * DH * DH);
                __syncthreads();
            }
        }

        // the interval processed next (the one before this): its k, v rows and its checkpoint are requested into L2 now,
        // so that its phase F does not start on DRAM latency (q and dO of an interval are re-read shortly after phase F)
        if (ck > 0) {
            const int p_lo = (ck - 1) * chunk;
            constexpr int LPR = DH * (int)sizeof(T) / 128 > 0 ? DH * (int)sizeof(T) / 128 : 1;   // 128-byte lines per row
            for (int idx = tid; idx < chunk * LPR * 2; idx += BT) {
                const int which = idx / (chunk * LPR), rem = idx % (chunk * LPR);
                const T* base = which == 0 ? k : v;
                const char* ptr = reinterpret_cast<const char*>(base + (row0 + p_lo + rem / LPR) * d + h * DH) + (rem % LPR) * 128;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
            }
            const char* st = reinterpret_cast<const char*>(ckpt + ((int64_t)chain * n_ck + ck - 1) * DH * DH);
            for (int idx = tid; idx < DH * DH * 4 / 128; idx += BT) asm volatile("prefetch.global.L2 [%0];" ::"l"(st + idx * 128));
        }
        // ---- phase B: sub-chunks in reverse
        for (int j = nsub - 1; j >= 0; --j) {
            const int t0 = t_lo + j * C;
            const int n = t_hi - t0 < C ? t_hi - t0 : C;
            __syncthreads();
            load_state(j == 0 ? ck_state : my_sub + (int64_t)j * DH * DH);
            __syncthreads();
            chunk_front(t0, n, true);

            // dU = A^T dO + diag(eg) K dS
            cta_gemm<C, DH, C, L_KM, L_KN>(Am, LDC, dOs, LDV, [&](int i, int c, float acc) { dRs[i * LDV + c] = acc; });
            __syncthreads();
            cta_gemm<C, DH, DH, L_MK, L_KN>(Ks, LDK, dS, LDV,
                                            [&](int i, int c, float acc) { dRs[i * LDV + c] += eg_s[i] * acc; });
            __syncthreads();
            // dR = (I + L)^-T dU : back substitution, one thread per value column
            if (tid < DH) {
                float y[C];
#pragma unroll
                for (int t = C - 1; t >= 0; --t) {
                    float s = dRs[t * LDV + tid];
#pragma unroll
                    for (int jj = C - 1; jj > t; --jj) s = fmaf(-Lm[jj * LDC + t], y[jj], s);
                    y[t] = s;
                    dRs[t * LDV + tid] = s;
                }
            }
            __syncthreads();
            // dL = -strictlower(dR U^T), dA = lower(dO U^T); then M = dL beta Gam, dAG = dA Gam
            for (int idx = tid; idx < C * C; idx += BT) {
                const int t = idx / C, i = idx % C;
                float s1 = 0.0f, s2 = 0.0f;
                if (i <= t) {
                    const float* rt = dRs + t * LDV;
                    const float* ot = dOs + t * LDV;
                    const float* ui = Us + i * LDV;
#pragma unroll 4
                    for (int c = 0; c < DH; c += 4) {
                        const float4 u4 = *reinterpret_cast<const float4*>(ui + c);
                        const float4 r4 = *reinterpret_cast<const float4*>(rt + c);
                        const float4 o4 = *reinterpret_cast<const float4*>(ot + c);
                        s1 = fmaf(r4.x, u4.x, s1); s1 = fmaf(r4.y, u4.y, s1); s1 = fmaf(r4.z, u4.z, s1); s1 = fmaf(r4.w, u4.w, s1);
                        s2 = fmaf(o4.x, u4.x, s2); s2 = fmaf(o4.y, u4.y, s2); s2 = fmaf(o4.z, u4.z, s2); s2 = fmaf(o4.w, u4.w, s2);
                    }
                }
                const float gm = Gm[t * LDC + i];
                const float dl = i < t ? -s1 : 0.0f;
                dLm[t * LDC + i] = dl * gm;               // dL Gam  (times beta_t below -> M)
                dAm[t * LDC + i] = s2 * gm;               // dA Gam  (gm = 0 above the diagonal)
            }
            __syncthreads();
            // dbeta_t = dR_t.Z_t + sum_i (dL Gam)[t,i] KK[t,i]; then M = (dL Gam) beta_t.
            // per-row P sums: rowP[t] = sum_i dAG[t,i] QK[t,i] + M[t,i] KK[t,i]
            for (int t = warp; t < C; t += BT / 32) {
                float s = 0.0f;
                for (int c = lane; c < DH; c += 32) s = fmaf(dRs[t * LDV + c], Zs[t * LDV + c], s);
                float s2 = 0.0f;
                for (int i = lane; i < C; i += 32) s2 = fmaf(dLm[t * LDC + i], KK[t * LDC + i], s2);
                s = warp_sum(s);
                s2 = warp_sum(s2);
                if (lane == 0) dbe_s[t] = s + s2;
            }
            __syncthreads();
            for (int idx = tid; idx < C * C; idx += BT) {
                const int t = idx / C, i = idx % C;
                dLm[t * LDC + i] *= be_s[t];
            }
            // dV = beta dR (written out), dZ = dV kept in dRs
            for (int idx = tid; idx < C * DH; idx += BT) {
                const int t = idx / DH, c = idx % DH;
                const float dz = be_s[t] * dRs[t * LDV + c];
                dRs[t * LDV + c] = dz;
                if (t < n) d_qkv[(row0 + t0 + t) * 3 * d + 2 * d + h * DH + c] = dz;
            }
            __syncthreads();
            // bufA = dO S0^T (dQ inter, unscaled) ; bufB = -dZ S0^T (dKg)
            cta_gemm<C, DH, DH, L_MK, L_NK>(dOs, LDV, S0, LDV, [&](int t, int a, float acc) { bufA[t * LDK + a] = acc; });
            cta_gemm<C, DH, DH, L_MK, L_NK>(dRs, LDV, S0, LDV, [&](int t, int a, float acc) { bufB[t * LDK + a] = -acc; });
            __syncthreads();
            for (int t = warp; t < C; t += BT / 32) {
                float s1 = 0.0f, s2 = 0.0f;
                for (int a = lane; a < DH; a += 32) {
                    s1 = fmaf(Qs[t * LDK + a], bufA[t * LDK + a], s1);
                    s2 = fmaf(Ks[t * LDK + a], bufB[t * LDK + a], s2);
                }
                s1 = warp_sum(s1);
                s2 = warp_sum(s2);
                if (lane == 0) {
                    r_qs[t] = gam_s[t] * s1;
                    r_kg[t] = gam_s[t] * s2;
                }
            }
            __syncthreads();
            // dQ = gam bufA + dAG K  (in bufA)
            cta_gemm<C, DH, C, L_MK, L_KN>(dAm, LDC, Ks, LDK, [&](int t, int a, float acc) {
                bufA[t * LDK + a] = fmaf(gam_s[t], bufA[t * LDK + a], acc);
            });
            __syncthreads();
            // L2-norm backward of dq rows and store: (g - y (y.g)) / norm   (y = normalised q)
            for (int t = warp; t < n; t += BT / 32) {
                float s = 0.0f;
                for (int a = lane; a < DH; a += 32) s = fmaf(Qs[t * LDK + a], bufA[t * LDK + a], s);
                s = warp_sum(s);
                const float nq = qnorm[(row0 + t0 + t) * H + h];
                float* dst = d_qkv + (row0 + t0 + t) * 3 * d + h * DH;
                for (int a = lane; a < DH; a += 32) dst[a] = (bufA[t * LDK + a] - Qs[t * LDK + a] * s) / nq;
            }
            __syncthreads();
            // bufA = dW = U dS^T ; r_kw[t] = eg_t k_t.dW_t
            cta_gemm<C, DH, DH, L_MK, L_NK>(Us, LDV, dS, LDV, [&](int t, int a, float acc) { bufA[t * LDK + a] = acc; });
            __syncthreads();
            for (int t = warp; t < C; t += BT / 32) {
                float s = 0.0f;
                for (int a = lane; a < DH; a += 32) s = fmaf(Ks[t * LDK + a], bufA[t * LDK + a], s);
                s = warp_sum(s);
                if (lane == 0) r_kw[t] = eg_s[t] * s;
            }
            // dK = gam dKg + eg dW  (into bufB), then += dAG^T Q + (M + M^T) K
            for (int idx = tid; idx < C * DH; idx += BT) {
                const int t = idx / DH, a = idx % DH;
                bufB[t * LDK + a] = fmaf(gam_s[t], bufB[t * LDK + a], eg_s[t] * bufA[t * LDK + a]);
            }
            __syncthreads();
            cta_gemm<C, DH, C, L_KM, L_KN>(dAm, LDC, Qs, LDK, [&](int i, int a, float acc) { bufB[i * LDK + a] += acc; });
            __syncthreads();
            // P row/col sums before M is symmetrised: rowP, colP over P = dAG.QK + M.KK
            if (tid < C) {
                const int t = tid;
                float rs = 0.0f, cs = 0.0f;
                for (int i = 0; i < C; ++i) {
                    rs = fmaf(dAm[t * LDC + i], QK[t * LDC + i], rs);
                    rs = fmaf(dLm[t * LDC + i], KK[t * LDC + i], rs);
                    cs = fmaf(dAm[i * LDC + t], QK[i * LDC + t], cs);
                    cs = fmaf(dLm[i * LDC + t], KK[i * LDC + t], cs);
                }
                dg_s[t] = rs - cs + r_qs[t] + r_kg[t] - r_kw[t];
            }
            __syncthreads();
            // Msym = M + M^T into Am (A is no longer needed)
            for (int idx = tid; idx < C * C; idx += BT) {
                const int t = idx / C, i = idx % C;
                Am[t * LDC + i] = dLm[t * LDC + i] + dLm[i * LDC + t];
            }
            __syncthreads();
            cta_gemm<C, DH, C, L_MK, L_KN>(Am, LDC, Ks, LDK, [&](int i, int a, float acc) { bufB[i * LDK + a] += acc; });
            // <S0, dS> for dg_last (all threads), meanwhile nothing else writes S0/dS
            float part = 0.0f;
            for (int idx = tid; idx < DH * DH; idx += BT) {
                const int a = idx / DH, c = idx % DH;
                part = fmaf(S0[a * LDV + c], dS[a * LDV + c], part);
            }
            const float sds = block_sum(part, red);  // contains __syncthreads
            // gates: dg_last += sum_t r_kw[t] + gam_last <S0,dS>; reverse cumsum; sigmoid backward
            if (warp == 0) {
                float kw = lane < C ? r_kw[lane] : 0.0f;
                kw = warp_sum(kw);
                float gx = lane < C ? dg_s[lane] : 0.0f;
                if (lane == C - 1) gx += gam_s[C - 1] * sds + kw;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {   // suffix sums: dlogalpha_t = sum_{j >= t} dg_j
                    const float y = __shfl_down_sync(0xffffffffu, gx, o);
                    if (lane + o < 32) gx += y;
                }
                if (lane < C) dg_s[lane] = gx;
            }
            __syncthreads();
            if (tid < n) {
                const int64_t r = row0 + t0 + tid;
                const float al = al_s[tid], be = be_s[tid];
                d_gate[r * 2 * H + h] = dg_s[tid] * (1.0f - al);            // (dlogalpha/alpha) alpha (1-alpha)
                d_gate[r * 2 * H + H + h] = dbe_s[tid] * be * (1.0f - be);
            }
            // L2-norm backward of dk rows and store
            for (int t = warp; t < n; t += BT / 32) {
                float s = 0.0f;
                for (int a = lane; a < DH; a += 32) s = fmaf(Ks[t * LDK + a], bufB[t * LDK + a], s);
                s = warp_sum(s);
                const float nk = knorm[(row0 + t0 + t) * H + h];
                float* dst = d_qkv + (row0 + t0 + t) * 3 * d + d + h * DH;
                for (int a = lane; a < DH; a += 32) dst[a] = (bufB[t * LDK + a] - Ks[t * LDK + a] * s) / nk;
            }
            __syncthreads();
            // dS <- gam_last dS + (gam Q)^T dO - (gam K)^T dZ
            for (int idx = tid; idx < C * DH; idx += BT) {
                const int t = idx / DH, a = idx % DH;
                bufA[t * LDK + a] = gam_s[t] * Qs[t * LDK + a];
                bufB[t * LDK + a] = -gam_s[t] * Ks[t * LDK + a];
            }
            __syncthreads();
            const float gl = gam_s[C - 1];
            cta_gemm<DH, DH, C, L_KM, L_KN>(bufA, LDK, dOs, LDV, [&](int a, int c, float acc) {
                dS[a * LDV + c] = fmaf(gl, dS[a * LDV + c], acc);
            });
            __syncthreads();
            cta_gemm<DH, DH, C, L_KM, L_KN>(bufB, LDK, dRs, LDV, [&](int a, int c, float acc) { dS[a * LDV + c] += acc; });
            __syncthreads();
        }
    }
}

template <int DH, int C, typename T>
int launch_bwd(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha, const float* beta,
               const float* qnorm, const float* knorm, const void* d_o, const float* ckpt, int B, int Tlen, int H,
               int chunk, float* d_qkv, float* d_gate) {
    using SM = BwdSmem<DH, C>;
    static_assert(SM::bytes <= 227 * 1024, "shared memory budget");
    const int sub_per_ck = (chunk + C - 1) / C;
    void* ws;
    ASCA_TRY(asca_workspace(ctx, (size_t)B * H * sub_per_ck * DH * DH * 4 + 256, &ws));
    auto kern = delta_bwd_kernel<DH, C, T>;
    ASCA_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::bytes));
    asca_span sp(ctx, "delta_bwd_kernel");
    kern<<<B * H, BT, SM::bytes, ctx->stream>>>((const T*)q, (const T*)k, (const T*)v, alpha, beta, qnorm, knorm,
                                                (const T*)d_o, ckpt, (float*)ws, B, Tlen, H, chunk, d_qkv, d_gate);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

}  // namespace

extern "C" int asca_delta_bwd(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha,
                              const float* beta, const float* qnorm, const float* knorm, const void* d_o,
                              const float* ckpt, int64_t B, int64_t T, int64_t H, int64_t dh, int64_t chunk, int dtype,
                              float* d_qkv, float* d_gate) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, q && k && v && alpha && beta && qnorm && knorm && d_o && ckpt && d_qkv && d_gate,
                 "delta_bwd: null pointer");
    ASCA_REQUIRE(ctx, B >= 0 && T >= 0 && H > 0 && chunk >= 1 && B * T < (1ll << 31), "delta_bwd: bad shape");
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "delta_bwd: unknown dtype");
    if (dh != 16 && dh != 32 && dh != 64 && dh != 128)
        return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "delta_bwd: dh must be 16, 32, 64 or 128 (got %lld)", (long long)dh);
    const uintptr_t al = (uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)d_o | (uintptr_t)ckpt;
    ASCA_REQUIRE(ctx, (al & 15) == 0, "delta_bwd: q, k, v, d_o, ckpt must be 16-byte aligned");
    if (B == 0 || T == 0) return ASCA_OK;
    // bf16 mode, dh = 128, checkpoints every 64 tokens: reverse chunked scan on the tensor cores
    if (dtype == ASCA_BF16 && (dh == 128 || dh == 64) && chunk == 64 && asca_tc_enabled() && delta_tc::available())
        return delta_tc::backward(ctx, q, k, v, alpha, beta, qnorm, knorm, d_o, ckpt, B, T, H, dh, d_qkv, d_gate);
#define ASCA_BWD(DH_, C_)                                                                                             \
    return dtype == ASCA_BF16                                                                                         \
               ? launch_bwd<DH_, C_, __nv_bfloat16>(ctx, q, k, v, alpha, beta, qnorm, knorm, d_o, ckpt, (int)B, (int)T, \
                                                    (int)H, (int)chunk, d_qkv, d_gate)                                \
               : launch_bwd<DH_, C_, float>(ctx, q, k, v, alpha, beta, qnorm, knorm, d_o, ckpt, (int)B, (int)T, (int)H, \
                                            (int)chunk, d_qkv, d_gate)
    switch (dh) {
        case 16: ASCA_BWD(16, 32);
        case 32: ASCA_BWD(32, 32);
        case 64: ASCA_BWD(64, 32);
        default: ASCA_BWD(128, 16);
    }
#undef ASCA_BWD
}
