// bf16 GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
// Persistent: two CTAs per SM work through the 128 x 128 f32 output tiles, each claiming the next unclaimed tile when it
// starts one (KP::dyn_ctr below; a fixed walk t, t + grid, ... with ASCA_GEMM_DYNAMIC=0). Warp roles (192 threads):
//   warp 0      TMA producer: one thread streams 128x64 A and 64x128 B bf16 tiles (128-byte
//               swizzle, plain non-multicast cp.async.bulk.tensor) through a 3-stage ring of
//               mbarriers, running ahead across tile boundaries;
//   warp 1      allocates 256 TMEM columns = two accumulator buffers, and one thread issues
//               tcgen05.mma (M128 N128 K16, 4 per k-tile) into the buffer of the current tile;
//               tcgen05.commit releases ring slots and hands the finished buffer to the epilogue;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp its 32-lane quarter), 32 columns at a
//               time, through the warp's shared-memory staging rows so that global memory sees
//               whole 64-byte row segments; bias / SiLU / SiLU' / accumulate are applied there;
//               f32 output (and an optional bf16 second output), optionally through a row map (the
//               un-permute scatter of the MoE combine). The buffer is released after the last
//               tcgen05.ld, and the main loop of the next tile runs meanwhile in the other buffer.
//
// Operand majorness covers the three modes without any transposed copy: NN = A K-major, B
// MN-major; TN = A MN-major, B MN-major; NT = A K-major, B K-major. Expert grouping: GROUP_M
// tiles the rows of each expert's segment (rows past the segment end are computed and not
// stored); GROUP_K runs the k-loop over an expert's rows and zeroes the ragged last k-tile in
// shared memory before it is multiplied.
//
// Every mbarrier wait is bounded; a wait that runs out raises an error word that the host reads
// back as ASCA_ERR_DEVICE, and the CTA still frees its TMEM and exits.
#include "gemm_tc.cuh"

#include <algorithm>
#include <cstdlib>
#include "tc_common.cuh"

namespace gemm_tc {
namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
// Two tile shapes. 128 x 128: 3-stage ring, 256 TMEM columns, two CTAs per SM (two independent MMA streams keep the
// tensor pipe fed). 128 x 256: one M128 N256 K16 instruction does twice the work of an N128 one for the same issue
// latency, so a single stream per SM suffices: 4-stage ring of 48 KiB, all 512 TMEM columns, one CTA per SM. It is
// used when the problem has at least two waves of such tiles.
// DEEP: a problem of at most one 128 x 128 tile per SM (a decode step's products) runs one CTA per SM with a
// 6-stage ring: its k-loop streams weights that are cold in L2, and three stages do not cover the HBM latency.
// PAIR: a cluster of two CTAs computes 256 x 256 tiles with cta_group::2 instructions (M = 256, N = 256). Each CTA
// loads its own 128 rows of A and its own 128 of the tile's 256 B columns (32 KiB per k-tile for 4.2 MFLOP on this SM
// against 48 KiB for the 128 x 256 tile and 32 KiB per 2.1 MFLOP for the 128 x 128 one): shared-memory traffic per
// FLOP, which is what bounds the single-CTA shapes, halves. 6-stage ring, all 512 TMEM columns, one CTA per SM.
template <int BN, bool DEEP = false, bool PAIR = false, bool EW8 = false> struct Shape {
    static constexpr int STAGES = PAIR ? 6 : BN == 128 ? (DEEP ? 6 : 3) : 4;
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = 2 * BN;      // two accumulator buffers
    static constexpr int CTAS_PER_SM = (BN == 128 && !DEEP) ? 2 : 1;
    // epilogue warps: one per TMEM lane quarter. EW8 (pair shape): two warps share each quarter and split the 256 columns
    // -- for the row-grouped expert products, whose epilogues (activation, two outputs, row scatter) would otherwise
    // outlast the main loop (837 against 603 TFLOP/s inside the training step), and for the fused qkv epilogue (a warp's
    // 128 columns are one head). Plain dense and k-grouped products are faster with four (1181 / 878 against 1056 / 781).
    static constexpr int EPI_WARPS = (PAIR && EW8) ? 8 : 4;
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr size_t SMEM_FIXED = (size_t)STAGES * STAGE_BYTES + EPI_WARPS * 2048 /*epilogue staging*/ + 1024 /*alignment slack*/ +
                                         256 /*barriers*/;   // + (groups + 2) * 4 for the tile table
};
constexpr int MAX_GROUPS = 2048;

struct KP {
    float* C;
    int64_t ldc;
    int M, N, K;
    const float* bias;
    int accumulate;
    const int32_t* c_idx;
    const int32_t* offsets;
    int n_groups, group_dim;
    int b_goff_inner, b_goff_outer;
    int64_t c_gstride, bias_gstride;
    int epi;
    const float* aux;
    int64_t ldaux;
    __nv_bfloat16* C2;
    int64_t ldc2;
    int c2_only;
    __nv_bfloat16 *qkv_q, *qkv_k, *qkv_v;
    float *qkv_qn, *qkv_kn;
    int qkv_d;
    const uint32_t* ce_targets;
    float* ce_loss;
    float ce_scale;
    // Dynamic tile claims (null: every walker takes tiles walker, walker + n_walkers, ...). With them a walker -- a CTA,
    // or a CTA pair -- takes the next unclaimed tile whenever it starts one, so CTAs that find their SM occupied by
    // another stream's kernels (a collective running beside the step) simply claim fewer tiles instead of holding the
    // launch up with a fixed share. The producer thread of the walker's first CTA claims (atomicAdd) and publishes the
    // claim in a small ring in global memory, tagged with launch and claim number; every other role of the walker, and
    // the pair's second CTA, read it from there.
    int* dyn_ctr;                      // this launch's counter (zero at launch)
    int* dyn_reset;                    // the next launch's counter, zeroed by this launch
    unsigned long long* dyn_ring;      // [walkers][DYN_Q] (tag << 32 | tile)
    uint32_t dyn_seq;                  // launch number
    int dyn_batch;                     // consecutive tiles per claim (short tiles: one claim's latency per several tiles)
    int* err_word;
};
// 32-column accumulator loads issued per wait in the epilogue. 4 (128 registers) was measured on the four-warp shapes:
// no gain (expert weight-gradient products at 512 rows per expert 1.09 against 1.05 ms, train step 335.6 against 334.4 ms).
#ifndef ASCA_EPI_LG
#define ASCA_EPI_LG 1
#endif
constexpr int DYN_Q = 16;              // claims a walker's producer can be ahead of its slowest role, with room to spare

// bf16 mode only (2e-2 tolerance; the results are rounded to bf16 or multiply bf16 products): fast exp and divide.
// A 128 x 128 tile applies these 16 k times, which with the accurate forms costs more than the tile's main loop.
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float p) {
    const float sg = __fdividef(1.0f, 1.0f + __expf(-p));
    return sg * (1.0f + p * (1.0f - sg));
}

template <int MODE, int BN, bool DEEP, bool PAIR, bool EW8>
__global__ void __launch_bounds__(Shape<BN, DEEP, PAIR, EW8>::THREADS, Shape<BN, DEEP, PAIR, EW8>::CTAS_PER_SM) gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA,
                                                             const __grid_constant__ CUtensorMap mapB, const KP p) {
    constexpr bool A_MN = (MODE == ASCA_TN);   // A operand MN-major
    constexpr bool B_MN = (MODE != ASCA_NT);   // B operand MN-major
    using SH = Shape<BN, DEEP, PAIR, EW8>;
    constexpr int STAGES = SH::STAGES, STAGE_BYTES = SH::STAGE_BYTES, TMEM_COLS = SH::TMEM_COLS;
    constexpr int TM = PAIR ? 2 * BM : BM;       // rows of an output tile (both CTAs of a pair)
    constexpr int BNL = PAIR ? BN / 2 : BN;      // B columns this CTA loads per tile
    const int rank = PAIR ? (int)tc::cluster_ctarank() : 0;   // 0 = the CTA that issues the pair's instructions
    const int n_walkers = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x, walker = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* staging = tiles + STAGES * STAGE_BYTES;                 // 4 epilogue warps x 2 KiB
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + SH::EPI_WARPS * 2048);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;     // [2] accumulator buffer written (MMA -> epilogue)
    uint64_t* acc_empty = acc_full + 2;      // [2] accumulator buffer read out (epilogue -> MMA)
    uint64_t* peer_full = acc_empty + 2;     // [STAGES] PAIR, even CTA: the odd CTA's stage has landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(peer_full + STAGES);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* prefix = const_cast<int*>(abort_flag) + 1;                  // [n_groups + 1] first tile of every group

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int n_groups = p.group_dim == GROUP_NONE ? 1 : p.n_groups;

    // ---- tile table: group g owns tiles [prefix[g], prefix[g+1]), tile = tile_m * tiles_n + tile_n within it
    if (warp == 1) {
        if (PAIR) tc::tmem_alloc_pair(tmem_slot, TMEM_COLS);
        else tc::tmem_alloc(tmem_slot, TMEM_COLS);
    }
    pdl_wait();   // the group offsets below may be the previous kernel's output
    if (warp == 0) {
        int base = 0;
        for (int g0 = 0; g0 < n_groups; g0 += 32) {
            const int g = g0 + lane;
            int cnt = 0;
            if (g < n_groups) {
                if (p.group_dim == GROUP_M) cnt = ((p.offsets[g + 1] - p.offsets[g] + TM - 1) / TM) * tiles_n;
                else cnt = ((p.M + TM - 1) / TM) * tiles_n;
            }
            int inc = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int nb = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += nb;
            }
            if (g < n_groups) prefix[g] = base + inc - cnt;
            base += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (p.group_dim != GROUP_NONE)   // the group offsets once more in shared memory: locate() runs per tile and role
            for (int g = lane; g <= n_groups; g += 32) prefix[n_groups + 1 + g] = p.offsets[g];
        if (lane == 0) {
            prefix[n_groups] = base;
            *abort_flag = 0;
            for (int s = 0; s < STAGES; ++s) {
                tc::mbar_init(&full[s], 1);
                tc::mbar_init(&empty[s], 1);
                tc::mbar_init(&peer_full[s], 1);
            }
            for (int b = 0; b < 2; ++b) {
                tc::mbar_init(&acc_full[b], 1);
                tc::mbar_init(&acc_empty[b], PAIR ? 2 * SH::EPI_WARPS : SH::EPI_WARPS);   // epilogue warps (of both CTAs)
            }
            tc::mbar_fence_init();
            tc::prefetch_tensormap(&mapA);
            tc::prefetch_tensormap(&mapB);
        }
    }
    tc::tcgen05_fence_before();
    __syncthreads();
    if (PAIR) tc::cluster_sync_all();   // the peer's barriers exist before anything is signalled across
    tc::tcgen05_fence_after();
    pdl_launch_dependents();   // after this CTA holds its TMEM: a dependent that becomes resident early cannot take it
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = prefix[n_groups];

    // Geometry of one tile; every role walks the same tile sequence blockIdx.x, + gridDim.x, ...
    struct Tile {
        int g, m0, n0, M, num_k, K, row_base_m, row_base_k, b_in, b_out;
    };
    auto locate = [&](int t) {
        int lo = 0, hi = n_groups - 1;   // last group with prefix[g] <= t
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= t) lo = mid; else hi = mid - 1;
        }
        Tile x;
        x.g = lo;
        const int in = t - prefix[lo];
        x.m0 = (in / tiles_n) * TM + rank * BM;   // this CTA's 128 rows of the tile
        x.n0 = (in % tiles_n) * BN;
        int seg_lo = 0;
        x.M = p.M;
        x.K = p.K;
        if (p.group_dim != GROUP_NONE) {
            seg_lo = prefix[n_groups + 1 + lo];
            const int n_g = prefix[n_groups + 2 + lo] - seg_lo;
            if (p.group_dim == GROUP_M) x.M = n_g; else x.K = n_g;
        }
        x.num_k = (x.K + BK - 1) / BK;
        x.row_base_m = p.group_dim == GROUP_M ? seg_lo : 0;   // added to A/C row coordinates
        x.row_base_k = p.group_dim == GROUP_K ? seg_lo : 0;   // added to k-row coordinates (TN)
        x.b_in = lo * p.b_goff_inner;
        x.b_out = lo * p.b_goff_outer;
        return x;
    };

    // The i-th tile of this walker (-1: none left). claim_tile is for the walker's claiming thread only.
    const bool dyn = p.dyn_ctr != nullptr;
    unsigned long long* dyn_slot0 = dyn ? p.dyn_ring + (size_t)walker * DYN_Q : nullptr;
    auto dyn_tag = [&](int i) { return p.dyn_seq * 4096u + (uint32_t)(i & 4095); };
    const int batch = dyn ? p.dyn_batch : 1;
    auto publish_claim = [&](int i, int t) {   // claim i = tiles [t, t + batch) (-1: none left)
        if (t >= total_tiles) t = -1;
        const unsigned long long v = ((unsigned long long)dyn_tag(i) << 32) | (uint32_t)t;
        asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(dyn_slot0 + (i % DYN_Q)), "l"(v) : "memory");
    };
    auto read_tile = [&](int i) -> int {   // one thread polls; bounded like every other wait of the kernel
        if (!dyn) {
            const int t = walker + i * n_walkers;
            return t < total_tiles ? t : -1;
        }
        const unsigned long long* e = dyn_slot0 + (i % DYN_Q);
        const uint32_t want = dyn_tag(i);
        const long long t0 = clock64();
        while (true) {
            unsigned long long v;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(e) : "memory");
            if ((uint32_t)(v >> 32) == want) return (int)(uint32_t)v;
            if (*abort_flag) return -1;
            if (clock64() - t0 > tc::WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                if (p.err_word) atomicExch(p.err_word, 107);
                return -1;
            }
        }
    };
    if (dyn && blockIdx.x == 0 && threadIdx.x == 0) *p.dyn_reset = 0;   // the launch after this one starts from zero

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            uint32_t it = 0;   // k-tiles issued so far, across tiles: ring slot it % STAGES
            bool ok = true;
            // The claiming thread asks for claim ci + 1 before it loads claim ci's tiles and publishes it after them: the
            // atomic's round trip hides behind the loads, and no other role needs the next claim before this one is used up.
            const bool claimer = dyn && rank == 0;
            int cur = 0;
            if (claimer) {
                cur = atomicAdd(p.dyn_ctr, batch);
                publish_claim(0, cur);
            }
            for (int ci = 0; ok; ++ci) {
                const int t0 = claimer ? (cur < total_tiles ? cur : -1) : read_tile(ci);
                if (t0 < 0) break;
                int nxt = 0;
                if (claimer) nxt = atomicAdd(p.dyn_ctr, batch);
              for (int t = t0; t < t0 + batch && t < total_tiles && ok; ++t) {
                const Tile x = locate(t);
                const int nl0 = x.n0 + rank * BNL;   // first B column this CTA loads
                for (int kt = 0; kt < x.num_k; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !tc::mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag, p.err_word, 101)) {
                        ok = false;
                        break;
                    }
                    uint8_t* a_s = tiles + s * STAGE_BYTES;
                    uint8_t* b_s = a_s + A_BYTES;
                    tc::mbar_expect_tx(&full[s], STAGE_BYTES);
                    const int k0 = kt * BK;
                    if (A_MN) {   // memory (k rows x M): two boxes of 64 columns
                        tc::tma_load_2d(a_s, &mapA, x.m0, x.row_base_k + k0, &full[s]);
                        tc::tma_load_2d(a_s + 8192, &mapA, x.m0 + 64, x.row_base_k + k0, &full[s]);
                    } else {      // memory (rows x K): one box 64 k x 128 rows
                        tc::tma_load_2d(a_s, &mapA, k0, x.row_base_m + x.m0, &full[s]);
                    }
                    if (B_MN) {   // memory (k rows x N)
                        const int kr = (MODE == ASCA_TN ? x.row_base_k : 0) + k0 + x.b_out;
#pragma unroll
                        for (int nb = 0; nb < BNL / 64; ++nb)   // boxes of 64 columns
                            tc::tma_load_2d(b_s + nb * 8192, &mapB, nl0 + nb * 64 + x.b_in, kr, &full[s]);
                    } else {      // memory (N rows x K)
                        tc::tma_load_2d(b_s, &mapB, k0 + x.b_in, nl0 + x.b_out, &full[s]);
                    }
                }
              }
                if (claimer) {   // (after a wait that gave up: "none left", so that the walker's other roles stop too)
                    cur = ok ? nxt : total_tiles;
                    publish_claim(ci + 1, cur);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // One thread runs the loop (the rest of the warp joins only to zero a ragged k-tile): wait for the
        // stage, four tcgen05.mma whose descriptors are the stage's base descriptor plus a constant, commit.
        // The loop's own dependent instructions are what bounds a single MMA stream, so it is kept short.
        constexpr uint32_t IDESC = tc::idesc_bf16_f32(TM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);          // SBO 1024, version 1, 128-byte swizzle
        constexpr uint32_t A_LBO = (A_MN ? 8192u : 16u) >> 4, B_LBO = (B_MN ? 8192u : 16u) >> 4;
        constexpr uint32_t A_K16 = (A_MN ? 2048u : 32u) >> 4, B_K16 = (B_MN ? 2048u : 32u) >> 4;   // per k16 step, in 16-byte units
        const uint32_t a_lo0 = ((tc::smem_u32(tiles) >> 4) & 0x3FFF) | (A_LBO << 16);
        const uint32_t b_lo0 = (((tc::smem_u32(tiles) + A_BYTES) >> 4) & 0x3FFF) | (B_LBO << 16);
        bool ok = true;
        uint32_t it = 0;
        int tl = 0;   // tiles done by this CTA: accumulator buffer tl & 1
        for (int ci = 0;; ++ci) {
            int t0 = lane == 0 && ok ? read_tile(ci) : -1;
            t0 = __shfl_sync(0xffffffffu, t0, 0);
            if (t0 < 0) break;
          for (int t = t0; t < t0 + batch && t < total_tiles && ok; ++t, ++tl) {
            const Tile x = locate(t);
            const int buf = tl & 1;
            const uint32_t tmem_acc = tmem_base + buf * BN;
            const bool ragged = p.group_dim == GROUP_K && (x.K % BK) != 0;   // warp-uniform
            const int n_plain = ragged ? x.num_k - 1 : x.num_k;
            if (PAIR && rank == 1) {
                // the odd CTA issues nothing: it tells the even CTA when each of its stages has landed
                if (lane == 0) {
                    for (int kt = 0; kt < n_plain && ok; ++kt, ++it) {
                        const uint32_t s = it % STAGES;
                        ok = tc::mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, p.err_word, 105);
                        if (ok) tc::mbar_arrive_cluster(tc::mapa_u32(tc::smem_u32(&peer_full[s]), 0));
                    }
                }
            } else if (lane == 0) {
                if (tl >= 2) {   // the epilogue (of both CTAs) has read this buffer's previous tile out
                    ok = PAIR ? tc::mbar_wait_cluster(&acc_empty[buf], ((tl >> 1) - 1) & 1, abort_flag, p.err_word, 104)
                              : tc::mbar_wait(&acc_empty[buf], ((tl >> 1) - 1) & 1, abort_flag, p.err_word, 104);
                }
                tc::tcgen05_fence_after();
                for (int kt = 0; kt < n_plain && ok; ++kt, ++it) {
                    const uint32_t s = it % STAGES;
                    ok = tc::mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, p.err_word, 102);
                    if (ok && PAIR) ok = tc::mbar_wait_cluster(&peer_full[s], (it / STAGES) & 1, abort_flag, p.err_word, 106);
                    if (!ok) break;
                    tc::tcgen05_fence_after();
                    const uint32_t a_lo = a_lo0 + s * (STAGE_BYTES >> 4), b_lo = b_lo0 + s * (STAGE_BYTES >> 4);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        const uint64_t da = ((uint64_t)DESC_HI << 32) | (a_lo + k16 * A_K16), db = ((uint64_t)DESC_HI << 32) | (b_lo + k16 * B_K16);
                        if (PAIR) tc::umma_bf16_pair(tmem_acc, da, db, IDESC, (kt > 0 || k16 > 0) ? 1u : 0u);
                        else tc::umma_bf16(tmem_acc, da, db, IDESC, (kt > 0 || k16 > 0) ? 1u : 0u);
                    }
                    if (PAIR) {
                        tc::umma_commit_pair(&empty[s]);              // the slot is free in both CTAs once these MMAs retire
                        if (kt == x.num_k - 1) tc::umma_commit_pair(&acc_full[buf]);
                    } else {
                        tc::umma_commit(&empty[s]);                   // slot free once these MMAs retire
                        if (kt == x.num_k - 1) tc::umma_commit(&acc_full[buf]);
                    }
                }
            }
            if (ragged) {
                // last k-tile of this expert: rows >= K - kt*BK belong to the next expert and are zeroed by the whole warp
                const int kt = x.num_k - 1;
                int got = 0;
                if (lane == 0) {
                    got = ok && tc::mbar_wait(&full[(it) % STAGES], ((it) / STAGES) & 1, abort_flag, p.err_word, 102) ? 1 : 0;
                    if (got && PAIR && rank == 0)   // the odd CTA zeroes its own tile before it reports the stage
                        got = tc::mbar_wait_cluster(&peer_full[(it) % STAGES], ((it) / STAGES) & 1, abort_flag, p.err_word, 106) ? 1 : 0;
                }
                got = __shfl_sync(0xffffffffu, got, 0);
                const uint32_t it_r = __shfl_sync(0xffffffffu, it, 0);
                ok = got != 0;
                if (ok) {
                    tc::tcgen05_fence_after();
                    const uint32_t s = it_r % STAGES;
                    uint8_t* a_s = tiles + s * STAGE_BYTES;
                    const int valid = x.K - kt * BK;
                    const int lines = (BK - valid) * 2;  // 128-byte lines in the two A boxes
                    for (int i = lane; i < lines * 8; i += 32) {
                        const int line = i >> 3, chunk = i & 7;
                        const int h = line / (BK - valid), kr = valid + line % (BK - valid);
                        *reinterpret_cast<uint4*>(a_s + h * 8192 + kr * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                    }
                    tc::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR && rank == 1) {
                            tc::mbar_arrive_cluster(tc::mapa_u32(tc::smem_u32(&peer_full[s]), 0));
                        } else {
                            const uint32_t a_lo = a_lo0 + s * (STAGE_BYTES >> 4), b_lo = b_lo0 + s * (STAGE_BYTES >> 4);
#pragma unroll
                            for (int k16 = 0; k16 < BK / 16; ++k16) {
                                const uint64_t da = ((uint64_t)DESC_HI << 32) | (a_lo + k16 * A_K16), db = ((uint64_t)DESC_HI << 32) | (b_lo + k16 * B_K16);
                                if (PAIR) tc::umma_bf16_pair(tmem_acc, da, db, IDESC, (kt > 0 || k16 > 0) ? 1u : 0u);
                                else tc::umma_bf16(tmem_acc, da, db, IDESC, (kt > 0 || k16 > 0) ? 1u : 0u);
                            }
                            if (PAIR) {
                                tc::umma_commit_pair(&empty[s]);
                                tc::umma_commit_pair(&acc_full[buf]);
                            } else {
                                tc::umma_commit(&empty[s]);
                                tc::umma_commit(&acc_full[buf]);
                            }
                        }
                        ++it;
                    }
                }
            }
            if (lane == 0 && ok && x.num_k == 0 && rank == 0) {   // empty expert: the epilogue stores zeros
                tc::mbar_arrive(&acc_full[buf]);
                if (PAIR) tc::mbar_arrive_cluster(tc::mapa_u32(tc::smem_u32(&acc_full[buf]), 1));
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;   // lane 0's verdict; keeps the warp's tile loops in step
          }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        // Each warp owns the 32 accumulator rows of its TMEM lane quarter and moves them 32 columns at a time:
        // tcgen05.ld (one row per lane) -> the warp's 2 KiB of shared memory, 16 columns per pass -> global
        // memory with 4 lanes on each row's 64 bytes, where bias, activation and accumulation are applied. The TMEM buffer is
        // released after the last tcgen05.ld; the next tile's main loop runs meanwhile in the other buffer.
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int ew = warp - 2;                // epilogue warp index; warps ew and ew + 4 share lane quarter q
        constexpr int C_PER_WARP = (BN / 32) / (SH::EPI_WARPS / 4);   // 32-column passes of a row per warp
        const int c_lo = (ew >> 2) * C_PER_WARP;
        float4* stg = reinterpret_cast<float4*>(staging + ew * 2048);   // [32 rows][4 float4], index XOR ((row >> 1) & 3)
        const bool c_vec = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && ((p.c_gstride & 3) == 0);
        const bool c2_vec = p.C2 && ((p.ldc2 & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C2) & 7) == 0);
        const bool aux_vec = p.aux && ((p.ldaux & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.aux) & 15) == 0);
        const int l4 = lane & 3, rsub = lane >> 2;   // store phase: 4 lanes per row (64 bytes), 8 rows per instruction
        bool ok = true;
        int tl = 0;
        for (int ci = 0; ok; ++ci) {
            int t0 = lane == 0 ? read_tile(ci) : -1;
            t0 = __shfl_sync(0xffffffffu, t0, 0);
            if (t0 < 0) break;
          for (int t = t0; t < t0 + batch && t < total_tiles; ++t, ++tl) {
            const Tile x = locate(t);
            const int buf = tl & 1;
            const uint32_t tmem_acc = tmem_base + buf * BN;
            int got = 0;
            if (lane == 0)
                got = (PAIR ? tc::mbar_wait_cluster(&acc_full[buf], (tl >> 1) & 1, abort_flag, p.err_word, 103)
                            : tc::mbar_wait(&acc_full[buf], (tl >> 1) & 1, abort_flag, p.err_word, 103)) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, got, 0) != 0;  // uniform: tcgen05.ld below is warp-aligned
            if (!ok) break;
            tc::tcgen05_fence_after();
            float* cbase = p.C + (p.group_dim == GROUP_K ? (int64_t)x.g * p.c_gstride : 0);
            const int rows_here = x.M - (x.m0 + q * 32);   // live rows of this warp's quarter (may be <= 0 or > 32)
            // the common case gets straight-line code: full tile, plain f32 output (bias and accumulate allowed)
            // fused qkv epilogue (pair shape, whole tiles: the launcher checks): this warp's 128 columns are one head of q, k or v
            const bool qkv = PAIR && EW8 && p.epi == EPI_QKV;
            float qkv_scale = 1.0f;                 // 1 / max(|z|, 1e-8) of this lane's row (q, k), 1 for v
            __nv_bfloat16* c2p = p.C2;
            int64_t ldc2 = p.ldc2;
            if (qkv) {
                const int hc0 = x.n0 + c_lo * 32;   // first column of the head
                const int sec = hc0 / p.qkv_d;      // 0 q, 1 k, 2 v
                c2p = (sec == 0 ? p.qkv_q : sec == 1 ? p.qkv_k : p.qkv_v) - sec * p.qkv_d;   // column = global column - sec d
                ldc2 = p.qkv_d;
                if (sec < 2) {
                    float ss = 0.0f;
#pragma unroll 1
                    for (int c = c_lo; c < c_lo + C_PER_WARP; ++c) {
                        uint32_t r[32];
                        tc::tmem_ld_32x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
                        tc::tmem_ld_wait();
                        const float4* bb = reinterpret_cast<const float4*>(p.bias + x.n0 + c * 32);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 b4 = bb[j];
                            const float v0 = __uint_as_float(r[4 * j]) + b4.x, v1 = __uint_as_float(r[4 * j + 1]) + b4.y,
                                        v2 = __uint_as_float(r[4 * j + 2]) + b4.z, v3 = __uint_as_float(r[4 * j + 3]) + b4.w;
                            ss += (v0 * v0 + v1 * v1) + (v2 * v2 + v3 * v3);
                        }
                    }
                    const float nrm = fmaxf(sqrtf(ss), 1e-8f);
                    qkv_scale = 1.0f / nrm;
                    const int heads = p.qkv_d / 128, head = (hc0 - sec * p.qkv_d) / 128;
                    (sec == 0 ? p.qkv_qn : p.qkv_kn)[((int64_t)x.m0 + q * 32 + lane) * heads + head] = nrm;
                }
            }
            // fused cross-entropy (pair shape, four epilogue warps: a warp's lanes hold whole rows of 256 logits)
            const bool ce = PAIR && !EW8 && p.epi == EPI_CE;
            float ce_max = 0.0f, ce_inv = 0.0f;
            int ce_t = 0;
            if (ce) {
                const int64_t row = (int64_t)x.m0 + q * 32 + lane;
                ce_t = (int)p.ce_targets[row];
                float mx = -INFINITY, sum = 0.0f, zt = 0.0f;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {   // online max / sum of exponentials over the row
                    uint32_t r[32];
                    tc::tmem_ld_32x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
                    tc::tmem_ld_wait();
                    float cm = mx;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float z = __uint_as_float(r[j]);
                        cm = fmaxf(cm, z);
                        if (c * 32 + j == ce_t) zt = z;
                    }
                    float part = 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) part += expf(__uint_as_float(r[j]) - cm);
                    sum = sum * expf(mx - cm) + part;
                    mx = cm;
                }
                p.ce_loss[row] = (mx + logf(sum)) - zt;
                ce_max = mx;
                ce_inv = 1.0f / sum;
            }
            const bool fast = qkv || ce || (c_vec && !p.c_idx && (!p.C2 || (p.c2_only && c2_vec)) && p.epi == EPI_NONE && rows_here >= 32 && x.n0 + BN <= p.N &&
                              (!p.bias || (((reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) && (p.bias_gstride & 3) == 0)));
            float* frow = cbase + ((int64_t)x.row_base_m + x.m0 + q * 32 + rsub) * p.ldc + x.n0 + 4 * l4;   // row rsub, this lane's columns
            const float* fbias = (p.bias && !qkv) ? p.bias + (int64_t)x.g * p.bias_gstride + x.n0 + 4 * l4 : nullptr;
            // row bookkeeping of the 4 store iterations: row = 8 * i + rsub
            int64_t lrs[4], crs[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int rr = 8 * i + rsub;
                lrs[i] = (int64_t)x.row_base_m + x.m0 + (rr < rows_here ? q * 32 + rr : 0);
                crs[i] = p.c_idx && rr < rows_here ? (int64_t)p.c_idx[lrs[i]] : lrs[i];
            }
            // LG 32-column loads are issued together and waited for once: a tcgen05.ld queues behind the MMAs the issuer
            // has in flight for the next tile, and one wait per load pays that queue once per 32 columns.
            constexpr int LG = (SH::CTAS_PER_SM == 2 || EW8) ? 1 : ASCA_EPI_LG;   // (two CTAs per SM, or 320 threads: no room for 128 more registers)
            static_assert(C_PER_WARP % LG == 0, "epilogue load groups");
#pragma unroll 1
            for (int cg = c_lo; cg < c_lo + C_PER_WARP; cg += LG) {
                uint32_t rr[LG][32];
                if (x.num_k > 0) {
#pragma unroll
                    for (int g = 0; g < LG; ++g)
                        tc::tmem_ld_32x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)((cg + g) * 32), rr[g]);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int g = 0; g < LG; ++g)
#pragma unroll
                        for (int j = 0; j < 32; ++j) rr[g][j] = 0u;
                }
                if (cg + LG == c_lo + C_PER_WARP) {   // this warp's share of the buffer is free for the tile after next
                    tc::tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) tc::mbar_arrive_cluster(tc::mapa_u32(tc::smem_u32(&acc_empty[buf]), 0));   // counted by the even CTA
                        else tc::mbar_arrive(&acc_empty[buf]);
                    }
                }
#pragma unroll
              for (int g = 0; g < LG; ++g) {
                const int c = cg + g;
                uint32_t(&r)[32] = rr[g];
                if (ce) {    // dlogits = (softmax - onehot) * scale
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float pr = expf(__uint_as_float(r[j]) - ce_max) * ce_inv;
                        if (c * 32 + j == ce_t) pr -= 1.0f;
                        r[j] = __float_as_uint(pr * p.ce_scale);
                    }
                }
                if (qkv) {   // bias, then the row's scale, on the f32 accumulators (lane = row)
                    const float4* bb = reinterpret_cast<const float4*>(p.bias + x.n0 + c * 32);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 b4 = bb[j];
                        r[4 * j] = __float_as_uint((__uint_as_float(r[4 * j]) + b4.x) * qkv_scale);
                        r[4 * j + 1] = __float_as_uint((__uint_as_float(r[4 * j + 1]) + b4.y) * qkv_scale);
                        r[4 * j + 2] = __float_as_uint((__uint_as_float(r[4 * j + 2]) + b4.z) * qkv_scale);
                        r[4 * j + 3] = __float_as_uint((__uint_as_float(r[4 * j + 3]) + b4.w) * qkv_scale);
                    }
                }
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        stg[lane * 4 + (j ^ ((lane >> 1) & 3))] =
                            make_float4(__uint_as_float(r[16 * hlf + 4 * j]), __uint_as_float(r[16 * hlf + 4 * j + 1]),
                                        __uint_as_float(r[16 * hlf + 4 * j + 2]), __uint_as_float(r[16 * hlf + 4 * j + 3]));
                    __syncwarp();
                    if (fast) {
                        const int co = c * 32 + hlf * 16;
                        float4 b4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), acc4[4], old4[4];
                        if (fbias) b4 = *reinterpret_cast<const float4*>(fbias + co);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            acc4[i] = stg[(8 * i + rsub) * 4 + (l4 ^ (((8 * i + rsub) >> 1) & 3))];
                            old4[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            if (p.accumulate) old4[i] = *reinterpret_cast<const float4*>(frow + (int64_t)(8 * i) * p.ldc + co);
                        }
                        if (p.c2_only || qkv || ce) {   // bf16 is all the consumer reads
                            __nv_bfloat16* hrow = c2p + ((int64_t)x.row_base_m + x.m0 + q * 32 + rsub) * ldc2 + x.n0 + 4 * l4 + co;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc4[i].x + b4.x, acc4[i].y + b4.y),
                                                     hi2 = __floats2bfloat162_rn(acc4[i].z + b4.z, acc4[i].w + b4.w);
                                *reinterpret_cast<uint2*>(hrow + (int64_t)(8 * i) * ldc2) =
                                    make_uint2(*reinterpret_cast<const uint32_t*>(&lo2), *reinterpret_cast<const uint32_t*>(&hi2));
                            }
                            __syncwarp();
                            continue;
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *reinterpret_cast<float4*>(frow + (int64_t)(8 * i) * p.ldc + co) =
                                make_float4(acc4[i].x + b4.x + old4[i].x, acc4[i].y + b4.y + old4[i].y,
                                            acc4[i].z + b4.z + old4[i].z, acc4[i].w + b4.w + old4[i].w);
                        __syncwarp();
                        continue;
                    }
                    const int nb = x.n0 + c * 32 + hlf * 16 + 4 * l4;   // this lane's 4 columns in the store phase
                    if (nb < p.N) {
                        const bool full4 = nb + 4 <= p.N;
                        float bias4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (p.bias) {
                            const float* bias = p.bias + (int64_t)x.g * p.bias_gstride;
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (nb + j < p.N) bias4[j] = bias[nb + j];
                        }
                        float4 aux4[4], old4[4];   // every global load of the pass is issued before any is used
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            aux4[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                            old4[i] = aux4[i];
                            if (8 * i + rsub >= rows_here) continue;
                            if (p.epi == EPI_SILU_BWD) {
                                const float* ax = p.aux + lrs[i] * p.ldaux + nb;
                                if (full4 && aux_vec) aux4[i] = *reinterpret_cast<const float4*>(ax);
                                else {
                                    aux4[i].x = ax[0];
                                    if (nb + 1 < p.N) aux4[i].y = ax[1];
                                    if (nb + 2 < p.N) aux4[i].z = ax[2];
                                    if (nb + 3 < p.N) aux4[i].w = ax[3];
                                }
                            }
                            if (p.accumulate) {
                                const float* crow = cbase + crs[i] * p.ldc + nb;
                                if (full4 && c_vec) old4[i] = *reinterpret_cast<const float4*>(crow);
                                else {
                                    old4[i].x = crow[0];
                                    if (nb + 1 < p.N) old4[i].y = crow[1];
                                    if (nb + 2 < p.N) old4[i].z = crow[2];
                                    if (nb + 3 < p.N) old4[i].w = crow[3];
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = 8 * i + rsub;
                            if (rr >= rows_here) continue;
                            const float4 acc4 = stg[rr * 4 + (l4 ^ ((rr >> 1) & 3))];
                            float v[4] = {acc4.x + bias4[0], acc4.y + bias4[1], acc4.z + bias4[2], acc4.w + bias4[3]};
                            if (p.epi == EPI_SILU_BWD) {
                                v[0] *= silu_grad_f(aux4[i].x); v[1] *= silu_grad_f(aux4[i].y);
                                v[2] *= silu_grad_f(aux4[i].z); v[3] *= silu_grad_f(aux4[i].w);
                            }
                            v[0] += old4[i].x; v[1] += old4[i].y; v[2] += old4[i].z; v[3] += old4[i].w;
                            float* crow = cbase + crs[i] * p.ldc + nb;
                            if (p.c2_only) {
                                // bf16 output only
                            } else if (full4 && c_vec) {
                                *reinterpret_cast<float4*>(crow) = make_float4(v[0], v[1], v[2], v[3]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    if (nb + j < p.N) crow[j] = v[j];
                            }
                            if (p.C2) {
                                __nv_bfloat16* c2 = p.C2 + lrs[i] * p.ldc2 + nb;
                                float y[4] = {v[0], v[1], v[2], v[3]};
                                if (p.epi == EPI_SILU) {
#pragma unroll
                                    for (int j = 0; j < 4; ++j) y[j] = silu_f(y[j]);
                                }
                                if (full4 && c2_vec) {
                                    const __nv_bfloat162 lo2 = __floats2bfloat162_rn(y[0], y[1]), hi2 = __floats2bfloat162_rn(y[2], y[3]);
                                    *reinterpret_cast<uint2*>(c2) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo2),
                                                                               *reinterpret_cast<const uint32_t*>(&hi2));
                                } else {
#pragma unroll
                                    for (int j = 0; j < 4; ++j)
                                        if (nb + j < p.N) c2[j] = __float2bfloat16(y[j]);
                                }
                            }
                        }
                    }
                    __syncwarp();   // every lane is done with the staging rows before the next pass overwrites them
                }
              }
            }
          }
        }
    }
    // ---- teardown: everyone meets, then the allocating warp frees TMEM
    tc::tcgen05_fence_before();
    __syncthreads();
    if (PAIR) tc::cluster_sync_all();     // neither CTA leaves (or frees TMEM) while its peer may still signal it
    if (*abort_flag) __nanosleep(20000);  // let copies already in flight land before the CTA exits
    if (warp == 1) {
        if (PAIR) tc::tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D bf16 tensor map: `cols` contiguous elements per row, `rows` rows, row pitch `ld` elements.
bool make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool supported(const Args& a) {
    if (!encode_fn()) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15)) return false;
    if ((a.lda & 7) || (a.ldb & 7)) return false;                       // row pitch multiple of 16 bytes
    if ((a.b_goff_inner & 7)) return false;                             // TMA inner coordinate: 16-byte aligned
    if (a.a_rows <= 0 || a.b_rows <= 0 || a.a_cols <= 0 || a.b_cols <= 0) return false;
    // grouped coordinate offsets must not let a ragged tile read a neighbouring expert's k range
    if (a.group_dim == GROUP_M && a.mode == ASCA_NT && a.b_goff_inner != 0 && (a.K % BK) != 0) return false;
    if (a.group_dim == GROUP_M && a.mode == ASCA_NN && a.b_goff_outer != 0 && (a.K % BK) != 0) return false;
    if (a.group_dim != GROUP_NONE && a.n_groups > MAX_GROUPS) return false;
    if (a.group_dim == GROUP_K && a.mode != ASCA_TN) return false;
    if (a.group_dim == GROUP_M && a.mode == ASCA_TN) return false;
    if (a.c2_only && (!a.C2 || a.accumulate || (a.epi != EPI_NONE && a.epi != EPI_SILU_BWD) || a.c_idx || skinny_wanted(a))) return false;
    if ((a.c2_mapped || a.b_packed) && !skinny_wanted(a)) return false;
    return true;
}

template <int BN, bool DEEP, bool PAIR = false, bool EW8 = false>
static int launch_shape(asca_ctx* ctx, const Args& a, int64_t grid, int64_t tiles_est) {
    CUtensorMap mapA, mapB;
    bool ok;
    if (a.mode == ASCA_TN) ok = make_map(&mapA, a.A, a.a_rows, a.a_cols, a.lda, 64, 64);
    else ok = make_map(&mapA, a.A, a.a_rows, a.a_cols, a.lda, 64, 128);
    if (a.mode == ASCA_NT) ok = ok && make_map(&mapB, a.B, a.b_rows, a.b_cols, a.ldb, 64, PAIR ? BN / 2 : BN);
    else ok = ok && make_map(&mapB, a.B, a.b_rows, a.b_cols, a.ldb, 64, 64);
    if (!ok) return asca_fail(ctx, ASCA_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled failed");
    KP p{};
    p.C = a.C; p.ldc = a.ldc; p.M = a.M; p.N = a.N; p.K = a.K;
    p.bias = a.bias; p.accumulate = a.accumulate; p.c_idx = a.c_idx;
    p.offsets = a.offsets; p.n_groups = a.n_groups; p.group_dim = a.group_dim;
    p.b_goff_inner = a.b_goff_inner; p.b_goff_outer = a.b_goff_outer;
    p.c_gstride = a.c_gstride; p.bias_gstride = a.bias_gstride;
    p.epi = a.epi; p.aux = a.aux; p.ldaux = a.ldaux; p.C2 = a.C2; p.ldc2 = a.ldc2; p.c2_only = a.c2_only;
    p.ce_targets = a.ce_targets; p.ce_loss = a.ce_loss; p.ce_scale = a.ce_scale;
    p.qkv_q = a.qkv_q; p.qkv_k = a.qkv_k; p.qkv_v = a.qkv_v; p.qkv_qn = a.qkv_qn; p.qkv_kn = a.qkv_kn; p.qkv_d = a.qkv_d;
    p.err_word = ctx->err_word;
    {   // dynamic tile claims: not under programmatic dependent launch (the counter hand-over relies on stream order)
        static const int dyn_env = [] { const char* e = getenv("ASCA_GEMM_DYNAMIC"); return e ? atoi(e) : 1; }();
        const bool want = dyn_env != 0;   // on unless ASCA_GEMM_DYNAMIC=0
        if (want && !ctx->pdl) {
            constexpr size_t RING_OFF = 256, BYTES = RING_OFF + 1024 * DYN_Q * 8;   // up to 1024 walkers
            if (!ctx->dyn_buf) {
                if (cudaMalloc(&ctx->dyn_buf, BYTES) != cudaSuccess) return asca_fail(ctx, ASCA_ERR_OOM, "gemm_tc: cannot allocate the tile-claim buffer");
                ASCA_CUDA(ctx, cudaMemsetAsync(ctx->dyn_buf, 0, BYTES, ctx->stream));
                ctx->dyn_seq = 0;
            }
            if (grid <= 1024) {
                const uint32_t seq = ++ctx->dyn_seq;
                int* ctrs = static_cast<int*>(ctx->dyn_buf);
                p.dyn_ctr = ctrs + (seq & 1) * 32;          // the two counters sit in different 128-byte lines
                p.dyn_reset = ctrs + ((seq + 1) & 1) * 32;
                p.dyn_ring = reinterpret_cast<unsigned long long*>(static_cast<char*>(ctx->dyn_buf) + RING_OFF);
                p.dyn_seq = seq;
                // One tile per claim. Several consecutive tiles per claim were measured (8 where a walker has > 128 tiles):
                // the train step went from 335.9 to 355.4 ms -- neighbouring walkers no longer work on neighbouring tiles
                // at the same time, which is what lets them share operand tiles in L2.
                (void)tiles_est;
                p.dyn_batch = 1;
            }
        }
    }
    using SH = Shape<BN, DEEP, PAIR, EW8>;
    const size_t smem = SH::SMEM_FIXED + (size_t)(2 * (a.group_dim == GROUP_NONE ? 1 : a.n_groups) + 4) * 4;   // tile table + group offsets
    auto go = [&](auto kern) -> cudaError_t {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SH::SMEM_FIXED + (2 * MAX_GROUPS + 4) * 4));
        if (e != cudaSuccess) return e;
        if (!PAIR) return asca_launch(ctx, kern, dim3((unsigned)grid), dim3(SH::THREADS), smem, mapA, mapB, p);
        // pairs of CTAs: a cluster of two per walker (grid = 2 x walkers)
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(SH::THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = ctx->pdl ? 2 : 1;
        return cudaLaunchKernelEx(&cfg, kern, mapA, mapB, p);
    };
    cudaError_t e = a.mode == ASCA_NN ? go(gemm_tc_kernel<ASCA_NN, BN, DEEP, PAIR, EW8>)
                    : a.mode == ASCA_TN ? go(gemm_tc_kernel<ASCA_TN, BN, DEEP, PAIR, EW8>) : go(gemm_tc_kernel<ASCA_NT, BN, DEEP, PAIR, EW8>);
    ASCA_CUDA(ctx, e);
    ctx->launches++;
    return ASCA_OK;
}

// upper bound on the number of bm x bn tiles (exact unless rows are grouped by expert)
static int64_t tile_bound(const Args& a, int bn, int bm = BM) {
    const int64_t tn = (a.N + bn - 1) / bn;
    if (a.group_dim == GROUP_NONE) return ((int64_t)(a.M + bm - 1) / bm) * tn;
    if (a.group_dim == GROUP_M) return (a.total_rows / bm + a.n_groups) * tn;
    return (int64_t)a.n_groups * ((a.M + bm - 1) / bm) * tn;
}

// ASCA_GEMM_PAIR=0 switches the CTA-pair shape off (A/B measurements); read once.
static bool pair_enabled() {
    static const bool on = [] {
        const char* e = getenv("ASCA_GEMM_PAIR");
        return !(e && e[0] == '0');
    }();
    return on;
}

static bool pair_wanted(asca_ctx* ctx, const Args& a);

bool qkv_fusable(asca_ctx* ctx, const Args& a) {
    return supported(a) && !skinny_wanted(a) && a.group_dim == GROUP_NONE && a.mode == ASCA_NN && pair_wanted(ctx, a) && a.qkv_d > 0 &&
           a.qkv_d % 256 == 0 && a.N == 3 * a.qkv_d && a.M % 256 == 0 && a.bias && (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0 &&
           a.qkv_q && a.qkv_k && a.qkv_v && a.qkv_qn && a.qkv_kn && !a.accumulate && !a.c_idx &&
           ((reinterpret_cast<uintptr_t>(a.qkv_q) | reinterpret_cast<uintptr_t>(a.qkv_k) | reinterpret_cast<uintptr_t>(a.qkv_v)) & 7) == 0;
}

bool ce_fusable(asca_ctx* ctx, const Args& a) {
    return supported(a) && !skinny_wanted(a) && a.group_dim == GROUP_NONE && a.mode == ASCA_NN && pair_wanted(ctx, a) && a.N == 256 &&
           a.M % 256 == 0 && !a.bias && !a.accumulate && !a.c_idx && a.C2 && a.ldc2 == 256 && (reinterpret_cast<uintptr_t>(a.C2) & 7) == 0 &&
           a.ce_targets && a.ce_loss;
}

int launch(asca_ctx* ctx, const Args& a) {
    if (a.epi == EPI_CE && !ce_fusable(ctx, a)) return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "gemm_tc: this product cannot take the fused cross-entropy epilogue");
    if (a.epi == EPI_QKV && !qkv_fusable(ctx, a)) return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "gemm_tc: this product cannot take the fused qkv epilogue");
    if (skinny_wanted(a)) return launch_skinny(ctx, a);
    // measurement harnesses: the product's algorithmic FLOPs go with the timed span
    const double rows_m = a.group_dim == GROUP_M ? (double)a.total_rows : (double)a.M;
    const double rows_k = a.group_dim == GROUP_K ? (double)a.total_rows : (double)a.K;
    asca_span sp(ctx, a.group_dim == GROUP_NONE ? "gemm_tc_kernel (dense)"
                      : a.group_dim == GROUP_M  ? "gemm_tc_kernel (expert-grouped rows)"
                                                : "gemm_tc_kernel (expert-grouped k)",
                 2.0 * rows_m * (double)a.N * rows_k);
    const int n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
    // persistent: the CTAs claim tile after tile. Wide tiles for dense problems with a long k-loop and at least
    // two waves of tiles (measured: +10-15 % there; with k <= 2048 or expert-grouped rows the 128 KiB epilogue per
    // tile and the single stream per SM cost more than the wider instruction gains).
    // CTA pairs on 256 x 256 tiles: dense and expert-grouped products with at least one tile per pair of SMs
    const int64_t pairs = tile_bound(a, 256, 256);
    const int64_t wide = tile_bound(a, 256);
    const bool wide_ok = a.group_dim == GROUP_NONE && a.K >= 4096 && a.N >= 256 && wide >= 2 * n_sm;
    // measured at 32768 x 2048 x 6144: A B^T with a long k runs 1389 TFLOP/s on 128 x 256 single-CTA tiles against 1320 on
    // pairs (both operands K-major: the widest TMA boxes); every other dense form is faster on pairs
    if (pair_wanted(ctx, a) && !(wide_ok && a.mode == ASCA_NT && a.epi != EPI_QKV)) {
        const int64_t g2 = 2 * std::min<int64_t>(pairs, n_sm / 2);
        if (a.group_dim == GROUP_M || a.epi == EPI_QKV) return launch_shape<256, false, true, true>(ctx, a, g2, pairs);
        return launch_shape<256, false, true, false>(ctx, a, g2, pairs);
    }
    if (wide_ok)
        return launch_shape<256, false>(ctx, a, std::min<int64_t>(wide, n_sm), wide);
    const int64_t grid = tile_bound(a, 128);
    if (grid <= 0) return ASCA_OK;
    if (grid <= n_sm) return launch_shape<128, true>(ctx, a, grid, grid);
    return launch_shape<128, false>(ctx, a, std::min<int64_t>(grid, 2 * n_sm), grid);
}

static bool pair_wanted(asca_ctx* ctx, const Args& a) {
    const int n_sm = ctx->sm_count > 0 ? ctx->sm_count : 148;
    const int64_t pairs = tile_bound(a, 256, 256);
    static const bool pair_rows = [] { const char* e = getenv("ASCA_GEMM_PAIR"); return !(e && e[0] == '1'); }();
    const bool pair_shape = a.group_dim == GROUP_M ? (pair_rows && a.total_rows >= 512 * (int64_t)a.n_groups) : a.M >= 256;
    return pair_enabled() && pair_shape && a.N >= 256 && pairs >= n_sm / 2;
}

}  // namespace gemm_tc
