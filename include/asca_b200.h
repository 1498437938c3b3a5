/* asca_b200 -- C ABI of the B200 (sm_100a) backend for ASCA's Delta Memory / hash-MoE path.
 *
 * This header is the drop-in boundary: each entry point replaces one method of the
 * reference's `impl Gpu` (rust/src/cuda/mod.rs) or one kernel of rust/kernels/asca.cu, and is
 * what a Rust `extern "C"` block (or any FFI) binds. Plain pointers and sizes only.
 *
 * Conventions
 *  - Every function returns 0 (ASCA_OK) or a negative ASCA_ERR_* code; the message is kept
 *    per context and read with asca_last_error(). Nothing throws across the boundary and
 *    nothing falls back to the CPU: if the device path cannot run, the call fails.
 *  - One asca_ctx per GPU. A context is not thread-safe; different contexts may be used from
 *    different threads. All work is enqueued on the context's stream (asca_ctx_set_stream).
 *  - Functions without the `_host` suffix take DEVICE pointers and are asynchronous with
 *    respect to the host. `_host` variants take HOST pointers, copy in, run the same
 *    kernels, copy out and synchronise -- the semantics of today's `Gpu::*` methods.
 *  - Matrices are row-major. f32 unless a `dtype` argument says otherwise; ASCA_BF16 means
 *    the activation/weight operands are bfloat16 while recurrent state, gates, accumulators
 *    and gradients of parameters stay f32.
 *  - Token rows are B sequences of T tokens stacked: row = b*T + t (rust/src/delta.rs:118-127).
 *    Head h owns columns [h*dh, (h+1)*dh). State S[a][i] is row-major a*dh + i (a = key
 *    index, i = value index), one dh x dh f32 matrix per (sequence, head).
 */
#ifndef ASCA_B200_H
#define ASCA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct asca_ctx asca_ctx;

enum {
    ASCA_OK = 0,
    ASCA_ERR_ARG = -1,         /* bad shape / null pointer / unsupported combination */
    ASCA_ERR_CUDA = -2,        /* a CUDA runtime or driver call failed */
    ASCA_ERR_OOM = -3,         /* device allocation failed */
    ASCA_ERR_UNSUPPORTED = -4, /* valid request the build does not cover (e.g. dh) */
    ASCA_ERR_DEVICE = -5       /* a kernel reported an error word (bounded wait ran out) */
};
enum { ASCA_F32 = 0, ASCA_BF16 = 1 };
enum { ASCA_NN = 0, ASCA_TN = 1, ASCA_NT = 2 };

/* ------------------------------------------------------------------ context
 * Replaces the lazily created singleton `Gpu` (rust/src/cuda/mod.rs:177-237, :1488-1496). */
int asca_ctx_create(int device, asca_ctx** out);
int asca_ctx_destroy(asca_ctx* ctx);
/* Use an existing cudaStream_t (e.g. the caller framework's current stream); NULL = the
 * context's own non-blocking stream. To run on CUDA's legacy default stream pass its explicit
 * handle cudaStreamLegacy ((cudaStream_t)0x1), not 0. The new stream is made to wait for what the
 * old one still holds (the context's scratch and counters pass from launch to launch in stream order). */
int asca_ctx_set_stream(asca_ctx* ctx, void* cuda_stream);
int asca_ctx_sync(asca_ctx* ctx);
const char* asca_last_error(const asca_ctx* ctx);
/* One-line description: device name, SM count, memory (rust/src/cuda/mod.rs:1566-1579). */
const char* asca_describe(asca_ctx* ctx);
/* Kernel launches issued through this context since creation (rust/src/cuda/mod.rs:25-33). */
int64_t asca_launch_count(const asca_ctx* ctx);
/* Per-kernel timing for measurement harnesses (the role of the reference's ASCA_PROF scopes,
 * rust/src/prof.rs): while on, the delta-rule kernels and the tensor-core products are bracketed by CUDA events on the
 * context's stream. asca_ctx_profile(ctx, on) clears the record and switches it;
 * asca_ctx_profile_read returns entry `index` (kernel name, milliseconds), or 1 past the end. */
int asca_ctx_profile(asca_ctx* ctx, int on);
int asca_ctx_profile_read(asca_ctx* ctx, int index, const char** name, float* ms);
/* Algorithmic work of entry `index` where the launcher states it (FLOPs of a tensor-core product), else 0. */
int asca_ctx_profile_work(asca_ctx* ctx, int index, double* work);
/* Self-test of the kernels' give-up path: launches one CTA that holds TMEM and waits, with the same bounded wait
 * the tensor-core kernels use but a limit of `limit_cycles` (at most 1e8), on an mbarrier nothing will complete. The
 * wait runs out, the kernel raises the context's error word, frees its TMEM and returns; the call reports
 * ASCA_ERR_DEVICE (the expected answer), *gave_up = 1 and *abort_seen = 1, and the context stays usable. Nothing
 * hangs and nothing faults: this is how the error path is tested. */
int asca_selftest_wait_timeout(asca_ctx* ctx, int64_t limit_cycles, int* gave_up, int* abort_seen);
/* Library version string and the arch it was compiled for ("sm_100a"). */
const char* asca_version(void);

/* Memory the context holds beyond what the caller sees: freed asca_malloc blocks (cached per size class),
 * the grow-only scratch of the kernels, and the tiles the tensor-core delta forward keeps for its backward
 * (at most `bytes` of them, default 32 GiB, least recently used set reused beyond that).
 * asca_ctx_trim synchronises the stream and gives all three back to the driver. */
int asca_ctx_trim(asca_ctx* ctx);
int asca_ctx_set_tile_cache_bytes(asca_ctx* ctx, size_t bytes);

/* Device memory for callers that have no allocator of their own (the reference's DevBuf,
 * rust/src/cuda/mod.rs:104-174). Freed blocks are cached per size class. */
int asca_malloc(asca_ctx* ctx, size_t bytes, void** dptr);
int asca_free(asca_ctx* ctx, void* dptr);
int asca_memcpy_h2d(asca_ctx* ctx, void* dst, const void* src, size_t bytes);
int asca_memcpy_d2h(asca_ctx* ctx, void* dst, const void* src, size_t bytes);
int asca_memset(asca_ctx* ctx, void* dst, int byte, size_t bytes);

/* ------------------------------------------------------------------ GEMM (G1)
 * Gpu::matmul (rust/src/cuda/mod.rs:286-313), Gpu::matmul_ta (:316-344) and the NT form the
 * CPU engine has as Mat::matmul_t (rust/src/tensor.rs:180-201).
 *   ASCA_NN: C[M,N] = A[M,K] B[K,N];  ASCA_TN: C[M,N] = A[K,M]^T B[K,N];
 *   ASCA_NT: C[M,N] = A[M,K] B[N,K]^T.
 * asca_gemm adds leading dimensions, an optional per-column bias (C += bias[n]) and
 * accumulate (C += result) -- the fused forms of add_row_bias and of `grad.axpy(1, dW)`. */
int asca_matmul(asca_ctx* ctx, const void* A, const void* B, void* C, int64_t M, int64_t K,
                int64_t N, int mode, int dtype);
int asca_gemm(asca_ctx* ctx, int mode, int64_t M, int64_t N, int64_t K, const void* A,
              int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, const float* bias,
              int accumulate, int dtype);
int asca_matmul_host(asca_ctx* ctx, const float* A, const float* B, float* C, int64_t M,
                     int64_t K, int64_t N, int mode);

/* ------------------------------------------------------------------ RMSNorm (N1)
 * Gpu::rmsnorm (rust/src/cuda/mod.rs:911-939) / Gpu::rmsnorm_bwd (:1122-1153); math of
 * rust/src/tensor.rs:251-297 (no gain). inv (rows) may be NULL. */
int asca_rmsnorm_fwd(asca_ctx* ctx, const float* x, float* y, float* inv, int64_t rows,
                     int64_t cols, float eps);
int asca_rmsnorm_bwd(asca_ctx* ctx, const float* x, const float* dy, float* dx, int64_t rows,
                     int64_t cols, float eps);
int asca_rmsnorm_fwd_host(asca_ctx* ctx, const float* x, float* y, float* inv, int64_t rows,
                          int64_t cols, float eps);
int asca_rmsnorm_bwd_host(asca_ctx* ctx, const float* x, const float* dy, float* dx,
                          int64_t rows, int64_t cols, float eps);
/* Fused residual + norm: x_mid = x + y (written to x_mid) and xn = rmsnorm(x_mid); the pair
 * rust/src/model.rs:666-667 + :200 computes. xn may be NULL (residual only). */
int asca_residual_rmsnorm(asca_ctx* ctx, const float* x, const float* y, float* x_mid, float* xn,
                          int64_t rows, int64_t cols, float eps);

/* ------------------------------------------------------------------ gather / scatter
 * Gpu::gather_rows (rust/src/cuda/mod.rs:1156-1187): dst[r,:] = src[idx[r],:];
 * Gpu::scatter_rows (:1190-1221): dst[idx[r],:] = src[r,:] (overwrite). idx is int32. */
int asca_gather_rows(asca_ctx* ctx, const float* src, const int32_t* idx, int64_t n_rows,
                     int64_t cols, float* dst);
int asca_scatter_rows(asca_ctx* ctx, const float* src, const int32_t* idx, int64_t n_rows,
                      int64_t cols, float* dst);
int asca_gather_rows_host(asca_ctx* ctx, const float* src, int64_t src_rows, const int32_t* idx,
                          int64_t n_rows, int64_t cols, float* dst);
int asca_scatter_rows_host(asca_ctx* ctx, const float* src, const int32_t* idx, int64_t n_rows,
                           int64_t cols, float* dst, int64_t dst_rows);

/* ------------------------------------------------------------------ AdamW (A1)
 * Gpu::adamw_update (rust/src/cuda/mod.rs:1057-1120) with the CPU path's decay
 * (rust/src/tensor.rs:444-453): m=b1 m+(1-b1)g; v=b2 v+(1-b2)g^2; p-=wd_eff p;
 * p-=lr_t m/(sqrt(v)+eps_t). The caller derives lr_t, eps_t, wd_eff per tensor
 * (rust/src/tensor.rs:393-402). */
int asca_adamw(asca_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, float lr_t,
               float beta1, float beta2, float eps_t, float wd_eff);
/* Same update over a flat buffer holding n_seg tensors; seg_off[n_seg+1] (element offsets,
 * host array) and per-tensor lr_t / eps_t (host arrays). One launch for the whole model. */
int asca_adamw_segmented(asca_ctx* ctx, float* p, const float* g, float* m, float* v,
                         const int64_t* seg_off, const float* lr_t, const float* eps_t,
                         int n_seg, float beta1, float beta2, float wd_eff);
/* Same update; when p_bf16 is not NULL the updated parameters are also written there as bf16 (same
 * offsets), which saves the separate cast pass of the bf16 compute mode. */
int asca_adamw_segmented_cast(asca_ctx* ctx, float* p, const float* g, float* m, float* v,
                              const int64_t* seg_off, const float* lr_t, const float* eps_t, int n_seg,
                              float beta1, float beta2, float wd_eff, void* p_bf16);
int asca_adamw_host(asca_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n,
                    float lr_t, float beta1, float beta2, float eps_t, float wd_eff);

/* ------------------------------------------------------------------ delta rule (D1, D2, D4)
 * Forward scan: Gpu::delta_scan (rust/src/cuda/mod.rs:1253-1321), recurrence of
 * rust/src/delta.rs:281-315. q,k already L2-normalised per head; q,k,v,o are (B*T, H*dh) in
 * `dtype`; alpha,beta (B*T, H) f32.
 *   s_final : nullable, (B, H, dh, dh) f32 -- the state after the last token (prefill).
 *   ckpt    : nullable, asca_delta_ckpt_floats() f32 -- the state at every `chunk`-token
 *             boundary, layout (B, H, ceil(T/chunk), dh, dh); entry c is S before token
 *             c*chunk. This replaces the reference's per-step state history
 *             ((T+1)*dh*dh per chain) and is what asca_delta_bwd recomputes from.
 *             With dtype ASCA_BF16, dh = 128 or 64 and chunk = 64 (the tensor-core kernels; heads of 64 are
 *             zero-padded to 128 inside them) the same
 *             states are stored rounded to bf16, same layout, in the first half of the buffer;
 *             either way the buffer is meant to be handed back to asca_delta_bwd unchanged.
 *             Contract of the tensor-core mode: that forward also keeps, inside the context, tiles it derived
 *             from q, k, v, alpha, beta, filed under the addresses of ckpt and of those five inputs. A backward
 *             that presents the same six addresses (and B, T, H) reuses the tiles instead of rebuilding them, so
 *             between the two calls the CONTENTS of q, k, v, alpha, beta and ckpt must not change (a caller that
 *             offloads and restores them may restore them anywhere but into the same addresses with other
 *             contents). Any other address combination rebuilds the tiles from the arguments. The kept tiles
 *             count against asca_ctx_set_tile_cache_bytes and are released by asca_ctx_trim.
 *   s_init  : nullable, (B, H, dh, dh) f32 initial state (continuing a prefix); NULL = 0. */
int64_t asca_delta_ckpt_floats(int64_t B, int64_t T, int64_t H, int64_t dh, int64_t chunk);
int asca_delta_fwd(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha,
                   const float* beta, int64_t B, int64_t T, int64_t H, int64_t dh, int64_t chunk,
                   int dtype, void* o, const float* s_init, float* s_final, float* ckpt);
/* BPTT: Gpu::delta_bwd_dev (rust/src/cuda/mod.rs:1328-1382), math of
 * rust/src/delta.rs:485-611. Outputs d_qkv (B*T, 3*H*dh) = [dq|dk|dv] after the per-head
 * L2-norm backward and d_gate (B*T, 2H) after the sigmoid backward, both f32. qnorm, knorm
 * (B*T, H) are the pre-normalisation norms from the forward. ckpt comes from asca_delta_fwd
 * with the same `chunk`. */
int asca_delta_bwd(asca_ctx* ctx, const void* q, const void* k, const void* v, const float* alpha,
                   const float* beta, const float* qnorm, const float* knorm, const void* d_o,
                   const float* ckpt, int64_t B, int64_t T, int64_t H, int64_t dh, int64_t chunk,
                   int dtype, float* d_qkv, float* d_gate);
/* Decode step for n_streams independent streams (DeltaBlock::step, rust/src/delta.rs:356-406):
 * S (n_streams, H, dh, dh) f32 updated in place, o (n_streams, H*dh) f32.
 *   fused = 0: q,k,v are separate (n_streams, H*dh) arrays, q,k already normalised; alpha,
 *              beta (n_streams, H) are the gate values.
 *   fused = 1: q points at the raw qkv projection (n_streams, 3*H*dh), alpha at the raw gate
 *              logits (n_streams, 2H); k, v, beta are ignored. The kernel applies
 *              z/max(|z|,1e-8) and the sigmoids itself (rust/src/delta.rs:358-376). */
int asca_delta_step(asca_ctx* ctx, const float* q, const float* k, const float* v,
                    const float* alpha, const float* beta, float* S, int64_t n_streams, int64_t H,
                    int64_t dh, int fused, float* o);
/* The fused form for head dim 64 with explicit row pitches: qkv rows (3*H*64 used) ld_qkv floats apart,
 * gate-logit rows (2H used) ld_gate apart -- the two may be column ranges of one projection output.
 * o16 (nullable): bf16 copy of o for a following tensor-core product. No counterpart in the reference. */
int asca_delta_step_strided(asca_ctx* ctx, const float* qkv, int64_t ld_qkv, const float* gate,
                            int64_t ld_gate, float* S, int64_t n_streams, int64_t H, float* o, void* o16);
/* Fused prologue of DeltaBlock::forward (rust/src/delta.rs:134-179): split qkv (N, 3d) into
 * q,k,v (N, d), L2-normalise q,k per head keeping the norms, and alpha/beta = sigmoid of the
 * gate logits (N, 2H). */
int asca_delta_prep(asca_ctx* ctx, const float* qkv, const float* gate, int64_t N, int64_t H,
                    int64_t dh, float* q, float* k, float* v, float* qnorm, float* knorm,
                    float* alpha, float* beta);
/* bf16-mode companions (no counterpart in the reference, whose backend is f32 only): the same
 * math with the operands of the next tensor-core product written as bf16.
 *   asca_cast_bf16             dst[i] = bf16(src[i])
 *   asca_residual_rmsnorm_bf16 x_mid = x + yadd (yadd, x_mid nullable: plain norm), xn = bf16(rmsnorm(x_mid))
 *   asca_delta_prep_bf16       asca_delta_prep with bf16 q, k, v */
int asca_cast_bf16(asca_ctx* ctx, const float* src, void* dst, int64_t n);
int asca_residual_rmsnorm_bf16(asca_ctx* ctx, const float* x, const float* yadd, float* x_mid, void* xn,
                               int64_t rows, int64_t cols, float eps);
int asca_delta_prep_bf16(asca_ctx* ctx, const float* qkv, const float* gate, int64_t N, int64_t H,
                         int64_t dh, void* q, void* k, void* v, float* qnorm, float* knorm,
                         float* alpha, float* beta);

/* Host-pointer forms with the reference's ownership model: the forward returns an opaque
 * device-resident handle (DeltaDev, rust/src/cuda/mod.rs:1386-1397) that the backward
 * consumes. */
typedef struct asca_delta_dev asca_delta_dev;
int asca_delta_scan_host(asca_ctx* ctx, const float* q, const float* k, const float* v,
                         const float* alpha, const float* beta, int64_t B, int64_t T, int64_t H,
                         int64_t dh, float* o, asca_delta_dev** dev);
int asca_delta_bwd_dev_host(asca_ctx* ctx, const asca_delta_dev* dev, const float* d_o,
                            const float* qnorm, const float* knorm, float* d_qkv, float* d_gate);
/* DeltaDev::download_states (rust/src/cuda/mod.rs:1473-1480): the per-step history
 * ((H*B) chains of (T+1)*dh*dh floats, chain index h*B+b) recomputed on the device from the
 * checkpoints. Refused with ASCA_ERR_ARG above 2^28 floats. */
int asca_delta_dev_download_states(asca_ctx* ctx, const asca_delta_dev* dev, float* states);
int asca_delta_dev_free(asca_ctx* ctx, asca_delta_dev* dev);

/* ------------------------------------------------------------------ hash MoE (M0-M5)
 * Dispatch: expert(t) = hash_route(ids[t], E) (rust/src/model.rs:69-77) and the stable
 * bucket order of rust/src/model.rs:190-193 as one permutation:
 *   perm[offsets[e] .. offsets[e+1]) = tokens of expert e in ascending token order.
 * perm (N) and offsets (E+1) are int32 device arrays; route (N, nullable) gets the expert of
 * each token. Integer only; bit-exact with the reference. */
int asca_moe_dispatch(asca_ctx* ctx, const uint32_t* ids, int64_t N, int64_t E, int32_t* perm,
                      int32_t* offsets, int32_t* route);
int asca_moe_dispatch_host(asca_ctx* ctx, const uint32_t* ids, int64_t N, int64_t E,
                           int32_t* perm, int32_t* offsets, int32_t* route);
/* The same dispatch for callers that must not allocate device memory while they run: a
 * serving loop that has handed all of HBM to its own arena at start-up (so a later cudaMalloc
 * fails or stalls the device), or a host whose policy forbids cudaMalloc / cudaFree once
 * requests are flowing because both synchronise the GPU. asca_moe_dispatch may grow the
 * context's scratch with cudaMalloc; this variant keeps its scratch (the per-segment expert
 * histogram) in a fixed 256 KiB array inside the library's device image instead, and calls no
 * cudaMalloc, cudaFree or other allocating routine. It has no counterpart in the reference.
 *   - Limit: ceil(N/1024), rounded up to a multiple of 4, times E must be <= 65536 (e.g.
 *     N <= 1,048,576 tokens at E = 64); larger requests return ASCA_ERR_ARG with a message.
 *   - The first call on each device looks the array's device address up (a host-side set-up
 *     step); make that first call before starting any stream capture.
 *   - Every call on a device shares the one array, and it keeps the previous call's contents
 *     (each call overwrites all entries it later reads, so nothing needs clearing). Two calls
 *     that overlap on the same GPU -- different streams or contexts -- race on it; serialise
 *     them.
 * Inputs, outputs and results are exactly those of asca_moe_dispatch. */
int asca_moe_dispatch_noalloc(asca_ctx* ctx, const uint32_t* ids, int64_t N, int64_t E,
                              int32_t* perm, int32_t* offsets, int32_t* route);
/* Expert FFN forward: Gpu::moe_forward_dev (rust/src/cuda/mod.rs:523-607), math of
 * rust/src/model.rs:237-293. xn (N,d) normalised rows; w1 (d, E*F), b1 (E*F) f32, w2 (E*F, d),
 * b2 (d) f32; out (N,d) f32 in token order. pre_p / hid_p (N,F): pre-activation and SiLU
 * output in PERMUTED (expert-contiguous) row order, kept for the backward. xn,w1,w2,hid_p
 * are `dtype`; pre_p is f32. */
int asca_moe_fwd(asca_ctx* ctx, const void* xn, const void* w1, const float* b1, const void* w2,
                 const float* b2, const int32_t* perm, const int32_t* offsets, int64_t N, int64_t d,
                 int64_t F, int64_t E, int dtype, float* out, float* pre_p, void* hid_p);
/* Expert FFN backward: Gpu::moe_bwd_dev (rust/src/cuda/mod.rs:745-824), math of
 * rust/src/model.rs:417-495. Writes (overwrites) d_w1 (d,E*F), d_b1 (E*F), d_w2 (E*F,d),
 * d_b2 (d), dxn (N,d), all f32. */
int asca_moe_bwd(asca_ctx* ctx, const void* xn, const void* w1, const void* w2,
                 const float* pre_p, const void* hid_p, const float* dout, const int32_t* perm,
                 const int32_t* offsets, int64_t N, int64_t d, int64_t F, int64_t E, int dtype,
                 float* d_w1, float* d_b1, float* d_w2, float* d_b2, float* dxn);
/* Same, but d_w1, d_b1, d_w2, d_b2 are accumulated into (+=) instead of overwritten: the form
 * `grad.axpy(1.0, &dW)` of HashMoe::backward (rust/src/model.rs:483-493) without a temporary. */
int asca_moe_bwd_acc(asca_ctx* ctx, const void* xn, const void* w1, const void* w2,
                     const float* pre_p, const void* hid_p, const float* dout, const int32_t* perm,
                     const int32_t* offsets, int64_t N, int64_t d, int64_t F, int64_t E, int dtype,
                     float* d_w1, float* d_b1, float* d_w2, float* d_b2, float* dxn);
/* Fused combine: x_out = x_mid + moe_out (rust/src/model.rs:669-671); when xn_next is not
 * NULL also xn_next = rmsnorm(x_out) (the final norm, rust/src/model.rs:680). Alias of
 * asca_residual_rmsnorm kept under the name the MoE path uses. */
int asca_moe_combine(asca_ctx* ctx, const float* x_mid, const float* moe_out, float* x_out,
                     float* xn_next, int64_t rows, int64_t cols, float eps);
/* Decode step for n_streams tokens (HashMoe::step, rust/src/model.rs:309-337): rmsnorm, one
 * expert per token, two GEMVs. x (n,d) f32 -> out (n,d) f32. */
int asca_moe_step(asca_ctx* ctx, const float* x, const uint32_t* ids, const void* w1,
                  const float* b1, const void* w2, const float* b2, int64_t n_streams, int64_t d,
                  int64_t F, int64_t E, int dtype, float* out);

typedef struct asca_moe_dev asca_moe_dev;
/* Host forms. `ids` replaces the reference's host-built `buckets` argument (the library
 * builds the same buckets on the device). */
int asca_moe_forward_dev_host(asca_ctx* ctx, const float* xn, const float* w1, const float* b1,
                              const float* w2, const float* b2, const uint32_t* ids, int64_t N,
                              int64_t d, int64_t F, int64_t E, float* out, asca_moe_dev** dev);
int asca_moe_bwd_dev_host(asca_ctx* ctx, const asca_moe_dev* dev, const float* dout, float* d_w1,
                          float* d_b1, float* d_w2, float* d_b2, float* dxn);
/* Gpu::moe_forward_dev with its own argument list (rust/src/cuda/mod.rs:523-532): the caller passes the
 * host-built `buckets` (rust/src/model.rs:190-193), flattened -- bucket_idx holds the buckets back to back (N token
 * indices), bucket_off[E + 1] their bounds. They are used as the dispatch permutation as they are; no sort runs on
 * the device, and `Model::forward` needs no edit. The handle is consumed by asca_moe_bwd_dev_host. */
int asca_moe_forward_dev_buckets_host(asca_ctx* ctx, const float* xn, const float* w1, const float* b1,
                                      const float* w2, const float* b2, const int32_t* bucket_idx,
                                      const int32_t* bucket_off, int64_t N, int64_t d, int64_t F, int64_t E,
                                      float* out, asca_moe_dev** dev);
/* MoeDev::download_pre_hidden (rust/src/cuda/mod.rs:1445-1470): pre and hidden as (N,F) in
 * token order. */
int asca_moe_dev_download_pre_hidden(asca_ctx* ctx, const asca_moe_dev* dev, float* pre,
                                     float* hidden);
int asca_moe_dev_free(asca_ctx* ctx, asca_moe_dev* dev);


/* ------------------------------------------------------------------ column sums, cross-entropy, embedding
 * Helpers of the model glue (bias gradients, loss, embedding table), all deterministic.
 * asca_colsum: out[c] (+)= sum_r src[r, c] over `rows` rows of pitch `ld` -- the bias-gradient
 * loops of rust/src/delta.rs:623-666 and the reference kernel colsum_f32
 * (rust/kernels/asca.cu:166-178). */
int asca_colsum(asca_ctx* ctx, const float* src, int64_t ld, int64_t rows, int64_t cols, float* out,
                int accumulate);
/* Cross-entropy over N rows of V logits (cpu_cross_entropy, rust/src/model.rs:804-844; reference
 * kernel cross_entropy_bwd_f32, rust/kernels/asca.cu:490-548): writes dlogits = (softmax -
 * onehot) / N (nullable) and the mean loss to *loss (device float). targets are uint32. */
int asca_cross_entropy(asca_ctx* ctx, const float* logits, const uint32_t* targets, int64_t N,
                       int64_t V, float* dlogits, float* loss);
/* Embedding lookup x[t,:] = table[ids[t],:] (rust/src/model.rs:654-660) and its gradient
 * d_table[v,:] += sum over tokens with ids[t] == v, in token order, of dx[t,:]
 * (rust/src/model.rs:785-791). */
int asca_embed_fwd(asca_ctx* ctx, const float* table, const uint32_t* ids, int64_t N, int64_t d,
                   float* x);
int asca_embed_bwd(asca_ctx* ctx, const float* dx, const uint32_t* ids, int64_t N, int64_t d,
                   int64_t vocab, float* d_table);

/* Host forms of the head / loss / optimizer methods of `impl Gpu`:
 *   asca_head_forward_dev_host   Gpu::head_forward_dev (rust/src/cuda/mod.rs:828-846): logits = h_final (T,d) x head
 *                                (d,V), kept on the device with h_final behind a LogitsDev handle (:1400-1413)
 *   asca_logits_dev_download     LogitsDev::download
 *   asca_head_bwd_dev_host       Gpu::head_bwd_dev (:851-908): *loss = mean token loss, d_head (d,V) = h_final^T dlogits,
 *                                dh (T,d) = dlogits x head_t, head_t (V,d) the transposed head the caller passes
 *   asca_cross_entropy_bwd_host  Gpu::cross_entropy_bwd (:945-1000): *loss and dlogits = (softmax - onehot) / T
 *   asca_adamw_resident_host     Gpu::adamw_resident (:1003-1055): Adam moments stay on the device between calls,
 *                                keyed by (key_addr = host address of the caller's m buffer, n); the first call for a
 *                                key uploads m0 / v0; val is updated in place. CPU-path decay, scalars as asca_adamw.
 *   asca_param_moments_host      param_moments (:57-73): the device-resident moments of a key; returns 1 if the key
 *                                has none
 *   asca_reset_param_cache       reset_param_cache (:50-54): drop every resident moment (call when a new model is built)
 *   asca_silu_inplace_host       Gpu::silu_inplace (:1224-1250) */
typedef struct asca_logits_dev asca_logits_dev;
int asca_head_forward_dev_host(asca_ctx* ctx, const float* h_final, const float* head, int64_t T, int64_t d,
                               int64_t V, asca_logits_dev** dev);
int asca_logits_dev_download(asca_ctx* ctx, const asca_logits_dev* dev, float* logits);
int asca_head_bwd_dev_host(asca_ctx* ctx, const asca_logits_dev* dev, const uint32_t* targets,
                           const float* head_t, float* loss, float* d_head, float* dh);
int asca_logits_dev_free(asca_ctx* ctx, asca_logits_dev* dev);
int asca_cross_entropy_bwd_host(asca_ctx* ctx, const float* logits, const uint32_t* targets, int64_t T, int64_t V,
                                float* loss, float* dlogits);
int asca_adamw_resident_host(asca_ctx* ctx, const void* key_addr, float* val, const float* grad, const float* m0,
                             const float* v0, int64_t n, float lr_t, float beta1, float beta2, float eps_t,
                             float wd_eff);
int asca_param_moments_host(asca_ctx* ctx, const void* key_addr, int64_t n, float* m, float* v);
int asca_reset_param_cache(asca_ctx* ctx);
int asca_silu_inplace_host(asca_ctx* ctx, float* x, int64_t n);

/* ------------------------------------------------------------------ model glue (X1)
 * Model::forward / backward / step and the AdamW loop (rust/src/model.rs:631-802) on one flat
 * f32 parameter buffer in the reference's parameter order (rust/src/model.rs:593-609: embed,
 * head, then per layer w_qkv, b_qkv, w_gate, b_gate, w_o, b_o, w1, b1, w2, b2). Everything
 * stays on the device between calls; the Delta block takes the un-normalised residual stream
 * as the reference code does (rust/src/model.rs:664-667). f32 arithmetic by default;
 * asca_model_set_compute(ASCA_BF16) moves every product of the training step to the tensor cores
 * (bf16 operands from a bf16 copy of the weights, f32 accumulation; residual stream, norms,
 * gates, recurrent state, loss, gradients, master weights and AdamW stay f32). */
typedef struct asca_model asca_model;
int asca_model_create(asca_ctx* ctx, int64_t vocab, int64_t d, int64_t H, int64_t L, int64_t E,
                      int64_t F, asca_model** out);
int asca_model_destroy(asca_ctx* ctx, asca_model* m);
int64_t asca_model_num_params(const asca_model* m);
/* Device pointers of the flat buffers (params, grads, Adam m, Adam v), each num_params floats. */
int asca_model_buffers(asca_model* m, float** params, float** grads, float** adam_m, float** adam_v);
int asca_model_set_compute(asca_ctx* ctx, asca_model* m, int dtype);
/* Gradient-ready hook: `fn(user, offset, count)` is called on the host, from inside
 * asca_model_forward_backward_host, each time every kernel that writes grads[offset, offset+count) has been
 * enqueued on the context's stream. Per block, last block first, there are two calls: the block's expert tensors
 * (w1, b1, w2, b2 -- final as soon as the expert backward is queued, before the rest of the block's backward), then
 * the block's projections; a last call covers embedding + head. Together they cover the buffer exactly once.
 * The library's own exchange (asca_model_dp_attach below) is driven from the same points; the hook is for callers
 * that bring their own collective. NULL removes the hook. */
/* bf16 compute mode, head dim 128: with on != 0 (the default) the qkv projection's own epilogue adds the bias, L2-normalises q and k
 * per head and writes q, k, v as bf16 (with the norms) wherever that product runs on CTA pairs (whole 256-row tiles,
 * d a multiple of 256); the f32 qkv matrix and the separate prologue pass then do not exist. Same results to bf16
 * rounding (the scale is a multiply by 1/norm where the prologue divides). Elsewhere, and with on = 0, the product
 * writes f32 qkv and asca_delta_prep_bf16 follows. No counterpart in the reference. */
int asca_model_set_fused_qkv(asca_model* m, int on);
/* bf16 compute mode, vocabulary 256: with on != 0 (the default) the output head's product takes the cross-entropy in its own
 * epilogue wherever it runs on CTA pairs and the caller asks for no logits: a CTA holds each of its rows' 256 logits in
 * TMEM, so the per-row loss and dlogits = (softmax - onehot) / N (bf16, what the two head gradients read) are produced
 * there and the (N x 256) logits and f32 dlogits never reach HBM -- the fusion of final norm's successor steps
 * Model::forward + cpu_cross_entropy (rust/src/model.rs:680-690, :821-837). Elsewhere the product writes the logits and
 * asca_cross_entropy's kernel follows. */
int asca_model_set_fused_head(asca_model* m, int on);
/* Gradient accumulation over k micro-batches: with scale = 1/k every backward adds its share of the
 * mean over all k micro-batches (the loss returned stays the mean over the micro-batch's own tokens). */
int asca_model_set_grad_scale(asca_model* m, float scale);
typedef void (*asca_grad_ready_fn)(void* user, int64_t offset, int64_t count);
int asca_model_set_grad_hook(asca_model* m, asca_grad_ready_fn fn, void* user);
/* Call after writing the parameter buffer directly (asca_model_buffers): derived copies are rebuilt. */
int asca_model_params_changed(asca_model* m);
int asca_model_set_params_host(asca_ctx* ctx, asca_model* m, const float* params);
/* AdamW's step counter (`AdamW::step`, rust/src/tensor.rs:393: it advances once per parameter tensor).
 * set / get may be NULL. A resume checkpoint restores it with the training step number, as
 * load_resume does (rust/src/train.rs:454-455). asca_model_set_params_host resets it to 0. */
int asca_model_adam_counter(asca_model* m, const uint32_t* set, uint32_t* get);
int asca_model_get_host(asca_ctx* ctx, asca_model* m, float* params, float* grads);
int asca_model_zero_grads(asca_ctx* ctx, asca_model* m);
/* Forward + backward over B sequences of T tokens (ids, targets: host uint32 arrays of B*T).
 * Gradients are accumulated into the flat grad buffer; *loss gets the mean token loss; logits
 * (host, B*T x vocab, nullable) receives the forward's logits. */
int asca_model_forward_backward_host(asca_ctx* ctx, asca_model* m, const uint32_t* ids,
                                     const uint32_t* targets, int64_t B, int64_t T, float* loss,
                                     float* logits);
/* One optimizer step = AdamW::update per tensor in parameter order; the step counter advances
 * once per TENSOR (rust/src/tensor.rs:393), bias corrections and decay as in
 * rust/src/tensor.rs:396-402. One segmented launch. */
int asca_model_adamw_step(asca_ctx* ctx, asca_model* m, float lr, float beta1, float beta2, float eps,
                          float wd);
/* Sharded optimizer support (bf16 compute mode, unpadded bf16 copy). asca_model_adamw_slices is one optimizer step
 * restricted to n sorted, disjoint slices [lo[i], hi[i]) of the flat buffer -- a rank's parts of the large tensors
 * plus the small tensors every rank updates; every tensor gets the step number asca_model_adamw_step would give
 * it; the counter advances as for a full step when `advance` is non-zero (an optimizer step may be issued as several
 * calls so that the exchange of finished tensors can start, the last call advancing); the bf16 copy is written for
 * the slices only.
 * asca_model_params16 returns the device address of the bf16 copy so that the caller can all-gather the other
 * ranks' slices into it. The f32 master weights and moments outside a rank's slices are then stale on that rank
 * by design. No reference counterpart (the reference's trainer is single-process). */
int asca_model_adamw_slices(asca_ctx* ctx, asca_model* m, float lr, float beta1, float beta2, float eps,
                            float wd, const int64_t* lo, const int64_t* hi, int n, int advance);
int asca_model_params16(asca_ctx* ctx, asca_model* m, void** out, int64_t* n16);
/* ------------------------------------------------------------------ data-parallel training (the gradient exchange)
 * The path shards by sequence with heads and experts local, so the only exchange is the mean of the flat
 * gradient buffer over the ranks, once per step (one process per GPU; the property rust/tests/batch_parity.rs
 * pins: batch = B equals the mean of B x batch = 1). The reference's trainer is single-process
 * (rust/src/train.rs:201-288) and has no counterpart; these entry points keep its FFI as thin as
 * rust/src/cuda/sys.rs:33-65: the Rust side binds five functions and never sees NCCL. NCCL is loaded with dlopen
 * on the first call (ASCA_NCCL_LIB overrides the path); a single-GPU user needs none.
 *
 * asca_comm_unique_id fills 128 bytes on one rank; the caller hands them to every rank (a file, a socket, an
 * environment variable) and all ranks call asca_comm_init together. A communicator owns a side stream on which
 * all its collectives run; it is tied to the context's device. */
typedef struct asca_comm asca_comm;
int asca_comm_unique_id(asca_ctx* ctx, void* id128);
int asca_comm_init(asca_ctx* ctx, int nranks, int rank, const void* id128, asca_comm** out);
int asca_comm_destroy(asca_ctx* ctx, asca_comm* comm);
int asca_comm_info(const asca_comm* comm, int* nranks, int* rank);
/* flat_grad[0, n) <- mean over ranks, in stream order with the context's stream (work queued before the call is
 * waited for; work queued after the call sees the result). bucket_off[n_buckets + 1] cuts the buffer into
 * buckets exchanged last bucket first (the backward finishes the end of the buffer first); NULL = one bucket. */
int asca_allreduce_grads(asca_ctx* ctx, asca_comm* comm, float* flat_grad, int64_t n, const int64_t* bucket_off,
                         int n_buckets);
/* The exchange overlapped with the backward. After asca_model_dp_attach, a backward that runs while the model is
 * armed (asca_model_dp_arm(m, 1); with gradient accumulation arm the last micro-batch only) queues the exchange of
 * every finished gradient range on the communicator's side stream from inside asca_model_forward_backward_host.
 * asca_model_dp_step then waits for the exchanges and applies the optimizer step (it replaces
 * asca_model_adamw_step and disarms the model):
 *   sharded = 0  every range is all-reduced; every rank applies the same full update.
 *   sharded = 1  (bf16 compute mode) W1 / W2 of every block are reduce-scattered instead, this rank updates its
 *                1/nranks chunk of them and all small tensors, and the updated bf16 chunks are all-gathered into
 *                the bf16 weight copy block by block; the next forward waits for a block's gathered weights only when
 *                it reaches that block's expert products. The f32 master weights and moments of other ranks' chunks
 *                are then stale on this rank: asca_model_get_host refuses to read them until
 *                asca_model_dp_gather_master has collected them (do that before writing a checkpoint).
 * comm = NULL detaches. asca_model_dp_timeline reads, for the last step, in milliseconds: [0] how long the end of
 * the backward waited for the gradient exchange, [1] the optimizer update, [2] how long the weight all-gather ran
 * past the update, [3] how long the forward of that step waited for gathered weights of the step before.
 * asca_dp_shard_plan is the host-side arithmetic alone (no GPU needed): the sorted, disjoint [lo, hi) ranges of
 * the flat buffer that `rank` updates under the sharded optimizer, and the sharded tensors (offset, length). */
int asca_model_dp_attach(asca_ctx* ctx, asca_model* m, asca_comm* comm, int sharded);
int asca_model_dp_arm(asca_model* m, int on);
int asca_model_dp_step(asca_ctx* ctx, asca_model* m, float lr, float beta1, float beta2, float eps, float wd);
int asca_model_dp_gather_master(asca_ctx* ctx, asca_model* m);
int asca_model_dp_timeline(asca_ctx* ctx, asca_model* m, float* ms4);
int asca_dp_shard_plan(int64_t vocab, int64_t d, int64_t H, int64_t L, int64_t E, int64_t F, int nranks, int rank,
                       int64_t* lo, int64_t* hi, int capacity, int* n_slices, int64_t* big_off, int64_t* big_len,
                       int big_capacity, int* n_big);
/* Copy-engine transport for the sharded tensors (ranks of one node, one process per GPU; no counterpart in the
 * reference). After asca_model_dp_attach(..., sharded = 1) every rank calls asca_model_dp_peer_export, which allocates
 * a staging area for incoming gradient chunks ((nranks - 1) / nranks of the sharded tensors' bytes) and fills 256 bytes
 * (CUDA IPC handles of the staging area, a flag array and the bf16 weight copy); the caller carries the ranks' blobs to
 * every rank (rank order) and each calls asca_model_dp_peer_open. From then on a sharded tensor's gradient chunks move
 * as one cudaMemcpyAsync per peer into that peer's staging slot, each followed by a step-numbered flag in the peer's
 * flag array; the chunk's owner polls the flags of all peers (bounded: about 20 s, then ASCA_ERR_DEVICE) and sums the
 * slots in rank order. The updated bf16 chunks go straight into the peers' weight copies the same way. No SM is held
 * while bytes move (NCCL's collectives keep 24 - 32 CTAs resident); the small tensors stay on NCCL. The mean then differs
 * from NCCL's in summation order only. Every rank must keep stepping in lock-step and detach together. */
int asca_model_dp_peer_export(asca_ctx* ctx, asca_model* m, void* blob256);
int asca_model_dp_peer_open(asca_ctx* ctx, asca_model* m, const void* blobs, int nranks);

/* Decode: n_streams independent streams advance one token each (Model::step,
 * rust/src/model.rs:631-649). state: device f32 (L, n_streams, H, dh, dh), updated in place;
 * ids: host uint32 (n_streams); logits: host (n_streams x vocab), nullable; next_ids: host
 * uint32 (n_streams), nullable -- the greedy argmax (lowest index on ties). */
int asca_model_decode_step_host(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids,
                                int64_t n_streams, float* logits, uint32_t* next_ids);
/* Chunked prefill (no counterpart in the reference, whose decoder prefills by stepping, rust/src/main.rs:367-371):
 * the forward of Model::forward (rust/src/model.rs:651-690) over n_streams prompts of T tokens each (ids: host
 * uint32, n_streams x T, one prompt per row), keeping the recurrent state after the last token of every block, head
 * and stream in `state` (same layout as the decode step; its incoming contents are the initial state, zeros for a
 * fresh stream, so a prompt may be fed in several calls) and returning the logits of each stream's LAST token
 * (host, n_streams x vocab, nullable) and their argmax (next_ids, nullable). Stepping the same tokens through
 * asca_model_decode_step_host gives the same state and logits (the property rust/tests/decode_parity.rs pins). */
int asca_model_prefill_host(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids, int64_t n_streams,
                            int64_t T, float* logits, uint32_t* next_ids);
/* Greedy decode of n_steps tokens per stream (the loop of the reference's `asca gen` with argmax sampling,
 * rust/src/main.rs: step, pick the largest logit, feed it back): step 0 consumes ids (host, n_streams), every later
 * step the argmax of the step before, which stays on the device; tokens (host, n_steps x n_streams, one row per
 * step) receives every chosen id after the last step. One synchronisation per call instead of one per token. */
int asca_model_decode_greedy_host(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids,
                                  int64_t n_streams, int64_t n_steps, uint32_t* tokens);

#ifdef __cplusplus
}
#endif
#endif /* ASCA_B200_H */
