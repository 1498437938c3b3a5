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

}  // extern "C"
