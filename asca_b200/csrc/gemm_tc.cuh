// bf16 tensor-core GEMM for sm_100a: TMA-fed, tcgen05.mma with the f32 accumulator in TMEM.
// Interface shared by gemm.cu (dense) and moe.cu (grouped expert products).
#pragma once
#include "common.cuh"

namespace gemm_tc {

// EPI_QKV: the product is the qkv projection of a Delta block (N = 3 d, head dim 128): instead of C, the epilogue writes
// q and k L2-normalised per head (z / max(|z|, 1e-8), rust/src/delta.rs:146-165) and v, all as bf16 (rows x d each), and
// the norms of q and k (rows x H, f32). Bias is added first. CTA-pair shape only; see qkv_fusable().
// EPI_CE: the product is the output head (N = 256 = the byte vocabulary, one tile wide): the epilogue holds a row's 256
// logits in TMEM, so it takes the softmax cross-entropy there (cpu_cross_entropy, rust/src/model.rs:821-837): per-row loss
// log-sum-exp - z[target] to ce_loss (f32, one per row) and dlogits = (softmax - onehot) * ce_scale as bf16 to C2; the
// logits never reach HBM. CTA-pair shape only; see ce_fusable().
enum { EPI_NONE = 0, EPI_SILU = 1, EPI_SILU_BWD = 2, EPI_QKV = 3, EPI_CE = 4 };
enum { GROUP_NONE = 0, GROUP_M = 1, GROUP_K = 2 };

struct Args {
    int mode;                 // ASCA_NN / ASCA_TN / ASCA_NT
    const void* A;            // bf16; NN/NT: (rowsA x K) row-major, TN: (rowsK x M) row-major
    const void* B;            // bf16; NN/TN: (rowsK x colsB) row-major, NT: (rowsN x K) row-major
    int64_t lda, ldb;         // elements
    int64_t a_rows, b_rows;   // memory rows of A and B (tensor-map bounds)
    int64_t a_cols, b_cols;   // memory columns of A and B
    float* C;
    int64_t ldc;
    int M, N, K;              // per-group problem (GROUP_M: M ignored, GROUP_K: K ignored)
    const float* bias;        // per output column, nullable
    int accumulate;
    const int32_t* c_idx;     // optional logical-row -> memory-row map for C
    // grouping
    const int32_t* offsets;   // device, n_groups + 1
    int n_groups;
    int group_dim;
    int64_t total_rows;       // sum of group sizes (host upper bound for the GROUP_M grid)
    int b_goff_inner, b_goff_outer;  // B tensor-map coordinate offsets per group (elements / rows)
    int64_t c_gstride, bias_gstride; // C / bias element offsets per group
    // epilogue
    int epi;
    const float* aux;         // EPI_SILU_BWD: pre-activation, rows follow the logical row
    int64_t ldaux;
    __nv_bfloat16* C2;        // EPI_SILU: silu(C); EPI_SILU_BWD: bf16 copy of C; nullable
    int64_t ldc2;
    int c2_only;              // row-tiled kernel, EPI_NONE or EPI_SILU_BWD, no accumulate: the result is wanted as bf16 only (C is
                              // not written and may be null)
    int c2_mapped;            // few-row kernel only: C2's rows go through c_idx like C's
    int b_packed;             // few-row kernel only: B is a buffer made by skinny_pack (b_rows = its rows of 64)
    __nv_bfloat16 *qkv_q, *qkv_k, *qkv_v;   // EPI_QKV outputs (rows x qkv_d, bf16)
    float *qkv_qn, *qkv_kn;                 // EPI_QKV: norms (rows x qkv_d / 128)
    int qkv_d;
    const uint32_t* ce_targets;             // EPI_CE: target id per row
    float* ce_loss;                         // EPI_CE: per-row loss
    float ce_scale;                         // EPI_CE: multiplies (softmax - onehot): grad scale / rows
    int b_early;              // few-row kernel only: B and the group offsets were written before the PREVIOUS kernel on
                              // the stream started, so under programmatic dependent launch they may be read while it runs.
                              // Rule for every call site that sets it: whatever the kernel reads before its wait (B, the
                              // offsets) must have been written before the nearest preceding kernel on the stream that
                              // waits before it triggers its dependents -- never by the kernel directly ahead.
};

// True when the tensor-core kernel can take this problem (alignment and divisibility rules of
// TMA and of the grouped coordinate offsets); otherwise the caller uses the SIMT kernel.
bool supported(const Args& a);
// Enqueues the kernel on ctx->stream. Returns ASCA_OK or an error code.
int launch(asca_ctx* ctx, const Args& a);
// True when launch() would run this dense product on CTA pairs AND its shape suits the fused qkv epilogue (EPI_QKV):
// whole 256-row tiles, N = 3 d with d a multiple of 256, bias present and 16-byte aligned.
bool qkv_fusable(asca_ctx* ctx, const Args& a);
// Likewise for the fused cross-entropy epilogue (EPI_CE): N = 256, whole 256-row tiles, no bias, bf16 dlogits in C2.
bool ce_fusable(asca_ctx* ctx, const Args& a);
// Few rows (per expert): the weight-streaming kernel of gemm_skinny.cu; launch() routes to it by itself.
bool skinny_wanted(const Args& a);
int launch_skinny(asca_ctx* ctx, const Args& a);
// Weights in the order the few-row kernel streams them: for every (group, 128-feature tile, 64-row k-tile) the 16 KiB
// of its shared-memory stage are contiguous (two halves of 64 k-rows x 64 features; zero beyond K and N), so a CTA
// reads one sequential run of memory instead of 128-byte pieces a weight-matrix row apart.
int64_t skinny_packed_rows(int64_t groups, int64_t K, int64_t N);   // rows of 64 bf16
int skinny_pack(asca_ctx* ctx, const __nv_bfloat16* src, int64_t ld, int64_t groups, int64_t goff_inner, int64_t goff_outer,
                int64_t K, int64_t N, __nv_bfloat16* dst);

}  // namespace gemm_tc
