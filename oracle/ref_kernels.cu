// Host launchers around the REFERENCE's own CUDA kernels (rust/kernels/asca.cu), so that the
// oracle can be pinned against outputs of the reference itself on a GPU.
//
// TEST INFRASTRUCTURE ONLY. The reference source is not copied: it is #included from where it
// lies (macro ASCA_REF_CU, set by oracle/build_ref.py) and compiled unmodified; the built library
// goes to oracle/_ref/ (git-ignored). Each launcher uses the grid / block / shared-memory shape of
// the reference's host call site (rust/src/cuda/mod.rs, lines cited per function), host pointers
// in and out, NULL stream, synchronise -- i.e. what `Gpu::*` does around the same kernel.
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include ASCA_REF_CU

namespace {
struct Dev {
    std::vector<void*> p;
    ~Dev() {
        for (void* x : p) cudaFree(x);
    }
    template <typename T>
    T* up(const T* h, size_t n) {
        void* d = nullptr;
        if (cudaMalloc(&d, n * sizeof(T) + 16) != cudaSuccess) return nullptr;
        p.push_back(d);
        if (h) cudaMemcpy(d, h, n * sizeof(T), cudaMemcpyHostToDevice);
        else cudaMemset(d, 0, n * sizeof(T));
        return (T*)d;
    }
};
template <typename T>
void down(T* h, const T* d, size_t n) { cudaMemcpy(h, d, n * sizeof(T), cudaMemcpyDeviceToHost); }
int finish() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}
}  // namespace

extern "C" {

// Gpu::matmul, rust/src/cuda/mod.rs:286-313 (grid (ceil(N/32), ceil(M/32)), block 32x32)
int ref_matmul(const float* A, const float* B, float* C, int M, int K, int N) {
    Dev d;
    float *a = d.up(A, (size_t)M * K), *b = d.up(B, (size_t)K * N), *c = d.up<float>(nullptr, (size_t)M * N);
    matmul_f32<<<dim3((N + 31) / 32, (M + 31) / 32), dim3(32, 32)>>>(a, b, c, M, K, N);
    int rc = finish();
    down(C, c, (size_t)M * N);
    return rc;
}
// Gpu::matmul_ta, rust/src/cuda/mod.rs:316-344: A is (K x M)
int ref_matmul_ta(const float* A, const float* B, float* C, int M, int K, int N) {
    Dev d;
    float *a = d.up(A, (size_t)K * M), *b = d.up(B, (size_t)K * N), *c = d.up<float>(nullptr, (size_t)M * N);
    matmul_ta_f32<<<dim3((N + 31) / 32, (M + 31) / 32), dim3(32, 32)>>>(a, b, c, M, K, N);
    int rc = finish();
    down(C, c, (size_t)M * N);
    return rc;
}
// Gpu::rmsnorm, rust/src/cuda/mod.rs:911-939 (grid rows, block 256)
int ref_rmsnorm(const float* X, float* Y, float* inv, int rows, int cols, float eps) {
    Dev d;
    float *x = d.up(X, (size_t)rows * cols), *y = d.up<float>(nullptr, (size_t)rows * cols),
          *iv = d.up<float>(nullptr, rows);
    rmsnorm_f32<<<rows, 256>>>(x, y, iv, rows, cols, eps);
    int rc = finish();
    down(Y, y, (size_t)rows * cols);
    down(inv, iv, rows);
    return rc;
}
// Gpu::rmsnorm_bwd, rust/src/cuda/mod.rs:1122-1153
int ref_rmsnorm_bwd(const float* X, const float* DY, float* DX, int rows, int cols, float eps) {
    Dev d;
    float *x = d.up(X, (size_t)rows * cols), *dy = d.up(DY, (size_t)rows * cols),
          *dx = d.up<float>(nullptr, (size_t)rows * cols);
    rmsnorm_bwd_f32<<<rows, 256>>>(x, dy, dx, rows, cols, eps);
    int rc = finish();
    down(DX, dx, (size_t)rows * cols);
    return rc;
}
// Gpu::delta_scan, rust/src/cuda/mod.rs:1253-1321 (grid (H, B), block 128,
// smem (dh*dh + 3*dh)*4, opt-in above 48 KiB as in `launch`, :254-275).
// states: (H*B) chains of (seq+1)*dh*dh floats.
int ref_delta_scan(const float* q, const float* k, const float* v, const float* alpha, const float* beta, int B,
                   int seq, int H, int dh, float* out, float* states) {
    Dev d;
    const size_t nd = (size_t)B * seq * H * dh, nh = (size_t)B * seq * H;
    const size_t ns = (size_t)H * B * (seq + 1) * dh * dh;
    float *dq = d.up(q, nd), *dk = d.up(k, nd), *dv = d.up(v, nd), *da = d.up(alpha, nh), *db = d.up(beta, nh);
    float *dout = d.up<float>(nullptr, nd), *dst = d.up<float>(nullptr, ns);
    const int shared = (dh * dh + 3 * dh) * 4;
    if (shared > 48 * 1024)
        cudaFuncSetAttribute(delta_fwd_batch_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    delta_fwd_batch_f32<<<dim3(H, B), 128, shared>>>(dq, dk, dv, da, db, dout, dst, H, dh, B, seq);
    int rc = finish();
    down(out, dout, nd);
    if (states) down(states, dst, ns);
    return rc;
}
// Gpu::delta_scan + Gpu::delta_bwd_dev, rust/src/cuda/mod.rs:1328-1382 (grid (H, B), block 128,
// smem (2*dh*dh + 9*dh + 128)*4). The backward consumes the state history the forward kernel
// wrote, exactly as the reference chains the two.
int ref_delta_fwd_bwd(const float* q, const float* k, const float* v, const float* alpha, const float* beta,
                      const float* qnorm, const float* knorm, const float* d_o, int B, int seq, int H, int dh,
                      float* out, float* d_qkv, float* d_gate) {
    Dev d;
    const size_t nd = (size_t)B * seq * H * dh, nh = (size_t)B * seq * H;
    const size_t ns = (size_t)H * B * (seq + 1) * dh * dh;
    float *dq = d.up(q, nd), *dk = d.up(k, nd), *dv = d.up(v, nd), *da = d.up(alpha, nh), *db = d.up(beta, nh);
    float *dqn = d.up(qnorm, nh), *dkn = d.up(knorm, nh), *ddo = d.up(d_o, nd);
    float *dout = d.up<float>(nullptr, nd), *dst = d.up<float>(nullptr, ns);
    float *dqkv = d.up<float>(nullptr, 3 * nd), *dgate = d.up<float>(nullptr, 2 * nh);
    int shared = (dh * dh + 3 * dh) * 4;
    if (shared > 48 * 1024)
        cudaFuncSetAttribute(delta_fwd_batch_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    delta_fwd_batch_f32<<<dim3(H, B), 128, shared>>>(dq, dk, dv, da, db, dout, dst, H, dh, B, seq);
    shared = (2 * dh * dh + 9 * dh + 128) * 4;
    if (shared > 48 * 1024) cudaFuncSetAttribute(delta_bwd_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    delta_bwd_f32<<<dim3(H, B), 128, shared>>>(dst, dq, dk, dv, da, db, dqn, dkn, ddo, dqkv, dgate, H, dh, B, seq);
    int rc = finish();
    down(out, dout, nd);
    down(d_qkv, dqkv, 3 * nd);
    down(d_gate, dgate, 2 * nh);
    return rc;
}
// silu_out_f32 / silu_bwd_f32 as Gpu::moe_forward_dev / moe_bwd_dev launch them
// (rust/src/cuda/mod.rs:610-639: grid ceil(n/256), block 256)
int ref_silu(const float* pre, float* hid, int n) {
    Dev d;
    float *p = d.up(pre, n), *h = d.up<float>(nullptr, n);
    silu_out_f32<<<(n + 255) / 256, 256>>>(h, p, n);
    int rc = finish();
    down(hid, h, n);
    return rc;
}
int ref_silu_bwd(float* dpre, const float* pre, int n) {
    Dev d;
    float *g = d.up(dpre, n), *p = d.up(pre, n);
    silu_bwd_f32<<<(n + 255) / 256, 256>>>(g, p, n);
    int rc = finish();
    down(dpre, g, n);
    return rc;
}
// cross_entropy_bwd_f32 as Gpu::cross_entropy_bwd launches it (rust/src/cuda/mod.rs:945-1000:
// grid T, block 256): per-token losses and dlogits = (p - onehot) * inv_T.
int ref_cross_entropy(const float* logits, const unsigned int* targets, float* dlogits, float* losses, int T, int V) {
    Dev d;
    float *lg = d.up(logits, (size_t)T * V), *dl = d.up<float>(nullptr, (size_t)T * V), *ls = d.up<float>(nullptr, T);
    unsigned int* tg = d.up(targets, T);
    cross_entropy_bwd_f32<<<T, 256>>>(lg, tg, dl, ls, T, V, 1.0f / (float)T);
    int rc = finish();
    down(dlogits, dl, (size_t)T * V);
    down(losses, ls, T);
    return rc;
}

// Gpu::moe_forward_dev followed by Gpu::moe_bwd_dev (rust/src/cuda/mod.rs:523-607, :745-824): the reference's own
// per-expert sequence of its own kernels -- forward gather_rows_f32, matmul_ld_f32, add_bias_f32, silu_out_f32,
// matmul_ld_f32, add_bias_f32, scatter_rows_f32 (:575-584); backward gather, matmul_ta_ld_f32, colsum_f32,
// matmul_tb_f32, silu_bwd_f32, colsum_f32, gather, matmul_ta_ld_f32, matmul_tb_f32, scatter (:768-804) -- with the
// launch shapes of its raw helpers (:401-520, :626-745). bucket_idx holds the host-built buckets back to back,
// bucket_off[E+1] their bounds (the `buckets: &[Vec<usize>]` argument flattened). pre / hid come back in token order.
int ref_moe_fwd_bwd(const float* xn, const float* w1, const float* b1, const float* w2, const float* b2,
                    const int* bucket_idx, const int* bucket_off, const float* dout_h, int T, int d, int F, int E,
                    float* out, float* pre_tok, float* hid_tok, float* d_w1, float* d_b1, float* d_w2, float* d_b2,
                    float* dxn_h) {
    Dev dv;
    const int w1_cols = E * F;
    float *dxn = dv.up(xn, (size_t)T * d), *dw1 = dv.up(w1, (size_t)d * w1_cols), *dw2 = dv.up(w2, (size_t)w1_cols * d);
    float *db1 = dv.up(b1, (size_t)w1_cols), *db2 = dv.up(b2, (size_t)d);
    float* dout = dv.up<float>(nullptr, (size_t)T * d);
    float* ddout = dv.up(dout_h, (size_t)T * d);
    float *ddw1 = dv.up<float>(nullptr, (size_t)d * w1_cols), *ddw2 = dv.up<float>(nullptr, (size_t)w1_cols * d);
    float *ddb1 = dv.up<float>(nullptr, (size_t)w1_cols), *ddb2 = dv.up<float>(nullptr, (size_t)d);
    float* ddxn = dv.up<float>(nullptr, (size_t)T * d);
    float *dpre_tok = dv.up<float>(nullptr, (size_t)T * F), *dhid_tok = dv.up<float>(nullptr, (size_t)T * F);
    struct Ex { int* idx; float *pre, *hid; int n; };
    std::vector<Ex> ex(E);
    auto g32 = [](int n, int m) { return dim3((n + 31) / 32, (m + 31) / 32); };
    for (int e = 0; e < E; ++e) {
        const int n = bucket_off[e + 1] - bucket_off[e];
        ex[e] = {nullptr, nullptr, nullptr, n};
        if (n == 0) continue;
        int* didx = dv.up(bucket_idx + bucket_off[e], (size_t)n);
        float *dxe = dv.up<float>(nullptr, (size_t)n * d), *dpe = dv.up<float>(nullptr, (size_t)n * F),
              *dhe = dv.up<float>(nullptr, (size_t)n * F), *doe = dv.up<float>(nullptr, (size_t)n * d);
        gather_rows_f32<<<n, 256>>>(dxn, didx, dxe, n, d);
        matmul_ld_f32<<<g32(F, n), dim3(32, 32)>>>(dxe, dw1, dpe, n, d, F, w1_cols, e * F);
        add_bias_f32<<<(n * F + 255) / 256, 256>>>(dpe, db1 + (size_t)e * F, n, F);
        silu_out_f32<<<(n * F + 255) / 256, 256>>>(dhe, dpe, n * F);
        matmul_ld_f32<<<g32(d, n), dim3(32, 32)>>>(dhe, dw2 + (size_t)e * F * d, doe, n, F, d, d, 0);
        add_bias_f32<<<(n * d + 255) / 256, 256>>>(doe, db2, n, d);
        scatter_rows_f32<<<n, 256>>>(doe, didx, dout, n, d);
        // MoeDev::download_pre_hidden (:1445-1470) returns per-expert matrices; here scattered to token order
        scatter_rows_f32<<<n, 256>>>(dpe, didx, dpre_tok, n, F);
        scatter_rows_f32<<<n, 256>>>(dhe, didx, dhid_tok, n, F);
        ex[e] = {didx, dpe, dhe, n};
    }
    int rc = finish();
    if (rc) return rc;
    for (int e = 0; e < E; ++e) {
        const int n = ex[e].n;
        if (n == 0) continue;
        float* ddhe = dv.up<float>(nullptr, (size_t)n * d);
        gather_rows_f32<<<n, 256>>>(ddout, ex[e].idx, ddhe, n, d);
        matmul_ta_ld_f32<<<g32(d, F), dim3(32, 32)>>>(ex[e].hid, ddhe, ddw2 + (size_t)e * F * d, F, n, d, d, 0);
        colsum_f32<<<(d + 127) / 128, 128>>>(ddhe, ddb2, n, d, 1);
        float* ddpre = dv.up<float>(nullptr, (size_t)n * F);
        matmul_tb_f32<<<g32(F, n), dim3(32, 32)>>>(ddhe, dw2 + (size_t)e * F * d, ddpre, n, d, F, d, 0);
        silu_bwd_f32<<<(n * F + 255) / 256, 256>>>(ddpre, ex[e].pre, n * F);
        colsum_f32<<<(F + 127) / 128, 128>>>(ddpre, ddb1 + (size_t)e * F, n, F, 1);
        float* dxe = dv.up<float>(nullptr, (size_t)n * d);
        gather_rows_f32<<<n, 256>>>(dxn, ex[e].idx, dxe, n, d);
        matmul_ta_ld_f32<<<g32(F, d), dim3(32, 32)>>>(dxe, ddpre, ddw1, d, n, F, w1_cols, e * F);
        float* ddxn_e = dv.up<float>(nullptr, (size_t)n * d);
        matmul_tb_f32<<<g32(d, n), dim3(32, 32)>>>(ddpre, dw1, ddxn_e, n, F, d, w1_cols, e * F);
        scatter_rows_f32<<<n, 256>>>(ddxn_e, ex[e].idx, ddxn, n, d);
    }
    rc = finish();
    down(out, dout, (size_t)T * d);
    down(pre_tok, dpre_tok, (size_t)T * F);
    down(hid_tok, dhid_tok, (size_t)T * F);
    down(d_w1, ddw1, (size_t)d * w1_cols);
    down(d_b1, ddb1, (size_t)w1_cols);
    down(d_w2, ddw2, (size_t)w1_cols * d);
    down(d_b2, ddb2, (size_t)d);
    down(dxn_h, ddxn, (size_t)T * d);
    return rc;
}

// Gpu::gather_rows / Gpu::scatter_rows (rust/src/cuda/mod.rs:1156-1221: grid n_rows, block 256)
int ref_gather_rows(const float* src, int src_rows, const int* idx, int n, int cols, float* dst) {
    Dev dv;
    float *s = dv.up(src, (size_t)src_rows * cols), *o = dv.up<float>(nullptr, (size_t)n * cols);
    int* i = dv.up(idx, (size_t)n);
    gather_rows_f32<<<n, 256>>>(s, i, o, n, cols);
    int rc = finish();
    down(dst, o, (size_t)n * cols);
    return rc;
}
int ref_scatter_rows(const float* src, const int* idx, int n, int cols, float* dst, int dst_rows) {
    Dev dv;
    float *s = dv.up(src, (size_t)n * cols), *o = dv.up(dst, (size_t)dst_rows * cols);
    int* i = dv.up(idx, (size_t)n);
    scatter_rows_f32<<<n, 256>>>(s, i, o, n, cols);
    int rc = finish();
    down(dst, o, (size_t)dst_rows * cols);
    return rc;
}

// Gpu::adamw_update (rust/src/cuda/mod.rs:1057-1120: grid ceil(n/256), block 256). With wd > 0 this kernel decays by
// lr*wd*p where its caller has already folded lr into wd (rust/src/tensor.rs:402, rust/kernels/asca.cu:561-563), which
// the CPU path does not do; the pin therefore runs it at wd = 0, where the two paths state the same update.
int ref_adamw(float* val, const float* grad, float* m, float* v, int n, float lr_t, float beta1, float beta2, float eps_t,
              float wd) {
    Dev dv;
    float *p = dv.up(val, (size_t)n), *g = dv.up(grad, (size_t)n), *dm = dv.up(m, (size_t)n), *dvv = dv.up(v, (size_t)n);
    adamw_f32<<<(n + 255) / 256, 256>>>(p, g, dm, dvv, lr_t, beta1, beta2, eps_t, wd, n);
    int rc = finish();
    down(val, p, (size_t)n);
    down(m, dm, (size_t)n);
    down(v, dvv, (size_t)n);
    return rc;
}

}  // extern "C"
