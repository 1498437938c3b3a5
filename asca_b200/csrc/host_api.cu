// Host-pointer entry points: the call shapes of today's `impl Gpu` methods
// (rust/src/cuda/mod.rs) -- borrow host slices, upload, run the device path, download,
// synchronise -- plus the two device-resident handles the reference keeps between a forward
// and its backward (DeltaDev :1386-1397, MoeDev :1416-1431).
#include "common.cuh"

namespace {

// Scoped device buffers from the context's cache; released on every exit path.
struct Scope {
    asca_ctx* ctx;
    std::vector<void*> bufs;
    explicit Scope(asca_ctx* c) : ctx(c) {}
    ~Scope() {
        for (void* b : bufs) asca_free(ctx, b);
    }
    int alloc(size_t bytes, void** out) {
        int rc = asca_malloc(ctx, bytes, out);
        if (rc == ASCA_OK) bufs.push_back(*out);
        return rc;
    }
    int upload(const void* host, size_t bytes, void** out) {
        int rc = alloc(bytes, out);
        if (rc != ASCA_OK) return rc;
        cudaError_t e = cudaMemcpyAsync(*out, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
        return e == cudaSuccess ? ASCA_OK : asca_fail(ctx, ASCA_ERR_CUDA, "H2D copy failed: %s", cudaGetErrorString(e));
    }
    void keep(void* p) {  // ownership moves to a handle
        for (auto& b : bufs)
            if (b == p) {
                b = bufs.back();
                bufs.pop_back();
                return;
            }
    }
};

int download(asca_ctx* ctx, void* host, const void* dev, size_t bytes) {
    ASCA_CUDA(ctx, cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return ASCA_OK;
}

constexpr int64_t HOST_CHUNK = 64;  // checkpoint interval used by the host-form delta scan

}  // namespace

struct asca_delta_dev {
    float *q, *k, *v, *alpha, *beta, *ckpt;
    int64_t B, T, H, dh, chunk;
};
struct asca_moe_dev {
    float *xn, *w1, *w2, *pre_p, *hid_p;
    int32_t *perm, *offsets;
    int64_t N, d, F, E;
};
struct asca_logits_dev {   // LogitsDev, rust/src/cuda/mod.rs:1400-1413: logits and h_final stay on the device
    float *logits, *h_final;
    int64_t T, d, V;
};

namespace {
__global__ void silu_inplace_kernel(float* __restrict__ x, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float v = x[i];
        x[i] = v / (1.0f + expf(-v));   // rust/src/model.rs:79-85
    }
}
}  // namespace

extern "C" {

int asca_matmul_host(asca_ctx* ctx, const float* A, const float* B, float* C, int64_t M, int64_t K, int64_t N,
                     int mode) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, A && B && C && M >= 0 && K >= 0 && N >= 0, "matmul_host: bad arguments");
    if (M == 0 || N == 0) return ASCA_OK;
    Scope s(ctx);
    void *dA, *dB, *dC;
    ASCA_TRY(s.upload(A, (size_t)(M * K) * 4, &dA));
    ASCA_TRY(s.upload(B, (size_t)(K * N) * 4, &dB));
    ASCA_TRY(s.alloc((size_t)(M * N) * 4, &dC));
    ASCA_TRY(asca_matmul(ctx, dA, dB, dC, M, K, N, mode, ASCA_F32));
    ASCA_TRY(download(ctx, C, dC, (size_t)(M * N) * 4));
    return asca_ctx_sync(ctx);
}

int asca_rmsnorm_fwd_host(asca_ctx* ctx, const float* x, float* y, float* inv, int64_t rows, int64_t cols, float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && y && rows >= 0 && cols > 0, "rmsnorm_fwd_host: bad arguments");
    if (rows == 0) return ASCA_OK;
    Scope s(ctx);
    void *dx, *dy, *di;
    ASCA_TRY(s.upload(x, (size_t)(rows * cols) * 4, &dx));
    ASCA_TRY(s.alloc((size_t)(rows * cols) * 4, &dy));
    ASCA_TRY(s.alloc((size_t)rows * 4, &di));
    ASCA_TRY(asca_rmsnorm_fwd(ctx, (float*)dx, (float*)dy, (float*)di, rows, cols, eps));
    ASCA_TRY(download(ctx, y, dy, (size_t)(rows * cols) * 4));
    if (inv) ASCA_TRY(download(ctx, inv, di, (size_t)rows * 4));
    return asca_ctx_sync(ctx);
}

int asca_rmsnorm_bwd_host(asca_ctx* ctx, const float* x, const float* dy, float* dx, int64_t rows, int64_t cols,
                          float eps) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && dy && dx && rows >= 0 && cols > 0, "rmsnorm_bwd_host: bad arguments");
    if (rows == 0) return ASCA_OK;
    Scope s(ctx);
    void *a, *b, *c;
    ASCA_TRY(s.upload(x, (size_t)(rows * cols) * 4, &a));
    ASCA_TRY(s.upload(dy, (size_t)(rows * cols) * 4, &b));
    ASCA_TRY(s.alloc((size_t)(rows * cols) * 4, &c));
    ASCA_TRY(asca_rmsnorm_bwd(ctx, (float*)a, (float*)b, (float*)c, rows, cols, eps));
    ASCA_TRY(download(ctx, dx, c, (size_t)(rows * cols) * 4));
    return asca_ctx_sync(ctx);
}

int asca_gather_rows_host(asca_ctx* ctx, const float* src, int64_t src_rows, const int32_t* idx, int64_t n_rows,
                          int64_t cols, float* dst) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, src && idx && dst && n_rows >= 0 && cols > 0 && src_rows >= 0, "gather_rows_host: bad arguments");
    for (int64_t i = 0; i < n_rows; ++i)
        ASCA_REQUIRE(ctx, idx[i] >= 0 && idx[i] < src_rows, "gather_rows_host: index %d out of range at %lld", idx[i], (long long)i);
    if (n_rows == 0) return ASCA_OK;
    Scope s(ctx);
    void *a, *b, *c;
    ASCA_TRY(s.upload(src, (size_t)(src_rows * cols) * 4, &a));
    ASCA_TRY(s.upload(idx, (size_t)n_rows * 4, &b));
    ASCA_TRY(s.alloc((size_t)(n_rows * cols) * 4, &c));
    ASCA_TRY(asca_gather_rows(ctx, (float*)a, (int32_t*)b, n_rows, cols, (float*)c));
    ASCA_TRY(download(ctx, dst, c, (size_t)(n_rows * cols) * 4));
    return asca_ctx_sync(ctx);
}

int asca_scatter_rows_host(asca_ctx* ctx, const float* src, const int32_t* idx, int64_t n_rows, int64_t cols,
                           float* dst, int64_t dst_rows) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, src && idx && dst && n_rows >= 0 && cols > 0 && dst_rows >= 0, "scatter_rows_host: bad arguments");
    for (int64_t i = 0; i < n_rows; ++i)
        ASCA_REQUIRE(ctx, idx[i] >= 0 && idx[i] < dst_rows, "scatter_rows_host: index %d out of range at %lld", idx[i], (long long)i);
    if (n_rows == 0) return ASCA_OK;
    Scope s(ctx);
    void *a, *b, *c;
    ASCA_TRY(s.upload(src, (size_t)(n_rows * cols) * 4, &a));
    ASCA_TRY(s.upload(idx, (size_t)n_rows * 4, &b));
    ASCA_TRY(s.upload(dst, (size_t)(dst_rows * cols) * 4, &c));  // rows not named keep their content
    ASCA_TRY(asca_scatter_rows(ctx, (float*)a, (int32_t*)b, n_rows, cols, (float*)c));
    ASCA_TRY(download(ctx, dst, c, (size_t)(dst_rows * cols) * 4));
    return asca_ctx_sync(ctx);
}

int asca_adamw_host(asca_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, float lr_t, float beta1,
                    float beta2, float eps_t, float wd_eff) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, p && g && m && v && n >= 0, "adamw_host: bad arguments");
    if (n == 0) return ASCA_OK;
    Scope s(ctx);
    void *dp, *dg, *dm, *dv;
    ASCA_TRY(s.upload(p, (size_t)n * 4, &dp));
    ASCA_TRY(s.upload(g, (size_t)n * 4, &dg));
    ASCA_TRY(s.upload(m, (size_t)n * 4, &dm));
    ASCA_TRY(s.upload(v, (size_t)n * 4, &dv));
    ASCA_TRY(asca_adamw(ctx, (float*)dp, (float*)dg, (float*)dm, (float*)dv, n, lr_t, beta1, beta2, eps_t, wd_eff));
    ASCA_TRY(download(ctx, p, dp, (size_t)n * 4));
    ASCA_TRY(download(ctx, m, dm, (size_t)n * 4));
    ASCA_TRY(download(ctx, v, dv, (size_t)n * 4));
    return asca_ctx_sync(ctx);
}

int asca_moe_dispatch_host(asca_ctx* ctx, const uint32_t* ids, int64_t N, int64_t E, int32_t* perm, int32_t* offsets,
                           int32_t* route) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, ids && perm && offsets && N >= 0 && E >= 1, "moe_dispatch_host: bad arguments");
    Scope s(ctx);
    void *di, *dp, *dof, *dr = nullptr;
    ASCA_TRY(s.upload(ids, (size_t)(N ? N : 1) * 4, &di));
    ASCA_TRY(s.alloc((size_t)(N ? N : 1) * 4, &dp));
    ASCA_TRY(s.alloc((size_t)(E + 1) * 4, &dof));
    if (route) ASCA_TRY(s.alloc((size_t)(N ? N : 1) * 4, &dr));
    ASCA_TRY(asca_moe_dispatch(ctx, (uint32_t*)di, N, E, (int32_t*)dp, (int32_t*)dof, (int32_t*)dr));
    if (N) ASCA_TRY(download(ctx, perm, dp, (size_t)N * 4));
    ASCA_TRY(download(ctx, offsets, dof, (size_t)(E + 1) * 4));
    if (route && N) ASCA_TRY(download(ctx, route, dr, (size_t)N * 4));
    return asca_ctx_sync(ctx);
}

// ------------------------------------------------------------------ delta: host forms
int asca_delta_scan_host(asca_ctx* ctx, const float* q, const float* k, const float* v, const float* alpha,
                         const float* beta, int64_t B, int64_t T, int64_t H, int64_t dh, float* o,
                         asca_delta_dev** dev) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, q && k && v && alpha && beta && o && B > 0 && T > 0 && H > 0 && dh > 0, "delta_scan_host: bad arguments");
    if (dev) *dev = nullptr;
    const size_t nd = (size_t)(B * T * H * dh) * 4, nh = (size_t)(B * T * H) * 4;
    Scope s(ctx);
    void *dq, *dk, *dv, *da, *db, *dO, *dck;
    ASCA_TRY(s.upload(q, nd, &dq));
    ASCA_TRY(s.upload(k, nd, &dk));
    ASCA_TRY(s.upload(v, nd, &dv));
    ASCA_TRY(s.upload(alpha, nh, &da));
    ASCA_TRY(s.upload(beta, nh, &db));
    ASCA_TRY(s.alloc(nd, &dO));
    ASCA_TRY(s.alloc((size_t)asca_delta_ckpt_floats(B, T, H, dh, HOST_CHUNK) * 4, &dck));
    ASCA_TRY(asca_delta_fwd(ctx, dq, dk, dv, (float*)da, (float*)db, B, T, H, dh, HOST_CHUNK, ASCA_F32, dO, nullptr,
                            nullptr, dev ? (float*)dck : nullptr));
    ASCA_TRY(download(ctx, o, dO, nd));
    ASCA_TRY(asca_ctx_sync(ctx));
    if (dev) {
        asca_delta_dev* h = new asca_delta_dev{(float*)dq, (float*)dk, (float*)dv, (float*)da, (float*)db,
                                               (float*)dck, B, T, H, dh, HOST_CHUNK};
        for (void* p : {dq, dk, dv, da, db, dck}) s.keep(p);
        *dev = h;
    }
    return ASCA_OK;
}

int asca_delta_bwd_dev_host(asca_ctx* ctx, const asca_delta_dev* dev, const float* d_o, const float* qnorm,
                            const float* knorm, float* d_qkv, float* d_gate) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dev && d_o && qnorm && knorm && d_qkv && d_gate, "delta_bwd_dev_host: null pointer");
    const int64_t N = dev->B * dev->T, d = dev->H * dev->dh;
    Scope s(ctx);
    void *ddo, *dqn, *dkn, *dqkv, *dgate;
    ASCA_TRY(s.upload(d_o, (size_t)(N * d) * 4, &ddo));
    ASCA_TRY(s.upload(qnorm, (size_t)(N * dev->H) * 4, &dqn));
    ASCA_TRY(s.upload(knorm, (size_t)(N * dev->H) * 4, &dkn));
    ASCA_TRY(s.alloc((size_t)(N * 3 * d) * 4, &dqkv));
    ASCA_TRY(s.alloc((size_t)(N * 2 * dev->H) * 4, &dgate));
    ASCA_TRY(asca_delta_bwd(ctx, dev->q, dev->k, dev->v, dev->alpha, dev->beta, (float*)dqn, (float*)dkn, ddo,
                            dev->ckpt, dev->B, dev->T, dev->H, dev->dh, dev->chunk, ASCA_F32, (float*)dqkv,
                            (float*)dgate));
    ASCA_TRY(download(ctx, d_qkv, dqkv, (size_t)(N * 3 * d) * 4));
    ASCA_TRY(download(ctx, d_gate, dgate, (size_t)(N * 2 * dev->H) * 4));
    return asca_ctx_sync(ctx);
}

int asca_delta_dev_download_states(asca_ctx* ctx, const asca_delta_dev* dev, float* states) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dev && states, "download_states: null pointer");
    const int64_t dd = dev->dh * dev->dh, per_chain = (dev->T + 1) * dd, total = dev->B * dev->H * per_chain;
    ASCA_REQUIRE(ctx, total <= (1ll << 28),
                 "download_states: %lld floats of per-step history refused (limit 2^28); the backward recomputes "
                 "from chunk checkpoints and never needs it", (long long)total);
    // Re-run the scan with a checkpoint at EVERY step: entry t is the state before token t,
    // and s_final is the state after the last one -- the reference's (T+1) history.
    Scope s(ctx);
    void *dO, *dck, *dfin;
    ASCA_TRY(s.alloc((size_t)(dev->B * dev->T * dev->H * dev->dh) * 4, &dO));
    ASCA_TRY(s.alloc((size_t)(dev->B * dev->H * dev->T * dd) * 4, &dck));
    ASCA_TRY(s.alloc((size_t)(dev->B * dev->H * dd) * 4, &dfin));
    ASCA_TRY(asca_delta_fwd(ctx, dev->q, dev->k, dev->v, dev->alpha, dev->beta, dev->B, dev->T, dev->H, dev->dh, 1,
                            ASCA_F32, dO, nullptr, (float*)dfin, (float*)dck));
    // device layouts are (B, H, T, dd) and (B, H, dd); the reference's chain index is h*B + b
    for (int64_t b = 0; b < dev->B; ++b)
        for (int64_t h = 0; h < dev->H; ++h) {
            float* dst = states + (h * dev->B + b) * per_chain;
            ASCA_TRY(download(ctx, dst, (float*)dck + (b * dev->H + h) * dev->T * dd, (size_t)(dev->T * dd) * 4));
            ASCA_TRY(download(ctx, dst + dev->T * dd, (float*)dfin + (b * dev->H + h) * dd, (size_t)dd * 4));
        }
    return asca_ctx_sync(ctx);
}

int asca_delta_dev_free(asca_ctx* ctx, asca_delta_dev* dev) {
    if (!ctx) return ASCA_ERR_ARG;
    if (!dev) return ASCA_OK;
    cudaStreamSynchronize(ctx->stream);
    for (void* p : {(void*)dev->q, (void*)dev->k, (void*)dev->v, (void*)dev->alpha, (void*)dev->beta, (void*)dev->ckpt})
        asca_free(ctx, p);
    delete dev;
    return ASCA_OK;
}

// ------------------------------------------------------------------ MoE: host forms
int asca_moe_forward_dev_host(asca_ctx* ctx, const float* xn, const float* w1, const float* b1, const float* w2,
                              const float* b2, const uint32_t* ids, int64_t N, int64_t d, int64_t F, int64_t E,
                              float* out, asca_moe_dev** dev) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, xn && w1 && b1 && w2 && b2 && ids && out && N > 0 && d > 0 && F > 0 && E > 0,
                 "moe_forward_dev_host: bad arguments");
    if (dev) *dev = nullptr;
    Scope s(ctx);
    void *dxn, *dw1, *db1, *dw2, *db2, *dids, *dperm, *doff, *dout, *dpre, *dhid;
    ASCA_TRY(s.upload(xn, (size_t)(N * d) * 4, &dxn));
    ASCA_TRY(s.upload(w1, (size_t)(d * E * F) * 4, &dw1));
    ASCA_TRY(s.upload(b1, (size_t)(E * F) * 4, &db1));
    ASCA_TRY(s.upload(w2, (size_t)(E * F * d) * 4, &dw2));
    ASCA_TRY(s.upload(b2, (size_t)d * 4, &db2));
    ASCA_TRY(s.upload(ids, (size_t)N * 4, &dids));
    ASCA_TRY(s.alloc((size_t)N * 4, &dperm));
    ASCA_TRY(s.alloc((size_t)(E + 1) * 4, &doff));
    ASCA_TRY(s.alloc((size_t)(N * d) * 4, &dout));
    ASCA_TRY(s.alloc((size_t)(N * F) * 4, &dpre));
    ASCA_TRY(s.alloc((size_t)(N * F) * 4, &dhid));
    ASCA_TRY(asca_moe_dispatch(ctx, (uint32_t*)dids, N, E, (int32_t*)dperm, (int32_t*)doff, nullptr));
    ASCA_TRY(asca_moe_fwd(ctx, dxn, dw1, (float*)db1, dw2, (float*)db2, (int32_t*)dperm, (int32_t*)doff, N, d, F, E,
                          ASCA_F32, (float*)dout, (float*)dpre, dhid));
    ASCA_TRY(download(ctx, out, dout, (size_t)(N * d) * 4));
    ASCA_TRY(asca_ctx_sync(ctx));
    if (dev) {
        *dev = new asca_moe_dev{(float*)dxn, (float*)dw1, (float*)dw2, (float*)dpre, (float*)dhid,
                                (int32_t*)dperm, (int32_t*)doff, N, d, F, E};
        for (void* p : {dxn, dw1, dw2, dpre, dhid, dperm, doff}) s.keep(p);
    }
    return ASCA_OK;
}

int asca_moe_bwd_dev_host(asca_ctx* ctx, const asca_moe_dev* dev, const float* dout, float* d_w1, float* d_b1,
                          float* d_w2, float* d_b2, float* dxn) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dev && dout && d_w1 && d_b1 && d_w2 && d_b2 && dxn, "moe_bwd_dev_host: null pointer");
    const int64_t N = dev->N, d = dev->d, F = dev->F, E = dev->E;
    Scope s(ctx);
    void *ddout, *g1, *gb1, *g2, *gb2, *gx;
    ASCA_TRY(s.upload(dout, (size_t)(N * d) * 4, &ddout));
    ASCA_TRY(s.alloc((size_t)(d * E * F) * 4, &g1));
    ASCA_TRY(s.alloc((size_t)(E * F) * 4, &gb1));
    ASCA_TRY(s.alloc((size_t)(E * F * d) * 4, &g2));
    ASCA_TRY(s.alloc((size_t)d * 4, &gb2));
    ASCA_TRY(s.alloc((size_t)(N * d) * 4, &gx));
    ASCA_TRY(asca_moe_bwd(ctx, dev->xn, dev->w1, dev->w2, dev->pre_p, dev->hid_p, (float*)ddout, dev->perm,
                          dev->offsets, N, d, F, E, ASCA_F32, (float*)g1, (float*)gb1, (float*)g2, (float*)gb2,
                          (float*)gx));
    ASCA_TRY(download(ctx, d_w1, g1, (size_t)(d * E * F) * 4));
    ASCA_TRY(download(ctx, d_b1, gb1, (size_t)(E * F) * 4));
    ASCA_TRY(download(ctx, d_w2, g2, (size_t)(E * F * d) * 4));
    ASCA_TRY(download(ctx, d_b2, gb2, (size_t)d * 4));
    ASCA_TRY(download(ctx, dxn, gx, (size_t)(N * d) * 4));
    return asca_ctx_sync(ctx);
}

int asca_moe_dev_download_pre_hidden(asca_ctx* ctx, const asca_moe_dev* dev, float* pre, float* hidden) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dev && pre && hidden, "download_pre_hidden: null pointer");
    // un-permute on the device (scatter rows by perm), then copy out in token order
    Scope s(ctx);
    void* tmp;
    ASCA_TRY(s.alloc((size_t)(dev->N * dev->F) * 4, &tmp));
    ASCA_TRY(asca_scatter_rows(ctx, dev->pre_p, dev->perm, dev->N, dev->F, (float*)tmp));
    ASCA_TRY(download(ctx, pre, tmp, (size_t)(dev->N * dev->F) * 4));
    ASCA_TRY(asca_ctx_sync(ctx));
    ASCA_TRY(asca_scatter_rows(ctx, dev->hid_p, dev->perm, dev->N, dev->F, (float*)tmp));
    ASCA_TRY(download(ctx, hidden, tmp, (size_t)(dev->N * dev->F) * 4));
    return asca_ctx_sync(ctx);
}

int asca_moe_dev_free(asca_ctx* ctx, asca_moe_dev* dev) {
    if (!ctx) return ASCA_ERR_ARG;
    if (!dev) return ASCA_OK;
    cudaStreamSynchronize(ctx->stream);
    for (void* p : {(void*)dev->xn, (void*)dev->w1, (void*)dev->w2, (void*)dev->pre_p, (void*)dev->hid_p,
                    (void*)dev->perm, (void*)dev->offsets})
        asca_free(ctx, p);
    delete dev;
    return ASCA_OK;
}

// The reference's own call shape for the expert FFN: the caller has already built `buckets` on the host
// (rust/src/model.rs:190-193) and passes them (Gpu::moe_forward_dev, rust/src/cuda/mod.rs:523-532). Flattened for
// the C ABI: bucket_idx holds the buckets back to back (N token indices), bucket_off[E + 1] their bounds. They ARE the
// dispatch permutation and its offsets, so nothing is sorted on the device.
int asca_moe_forward_dev_buckets_host(asca_ctx* ctx, const float* xn, const float* w1, const float* b1, const float* w2,
                                      const float* b2, const int32_t* bucket_idx, const int32_t* bucket_off, int64_t N,
                                      int64_t d, int64_t F, int64_t E, float* out, asca_moe_dev** dev) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, xn && w1 && b1 && w2 && b2 && bucket_idx && bucket_off && out && N > 0 && d > 0 && F > 0 && E > 0,
                 "moe_forward_dev_buckets_host: bad arguments");
    ASCA_REQUIRE(ctx, bucket_off[0] == 0 && bucket_off[E] == N, "moe_forward_dev_buckets_host: the buckets must hold every token once");
    for (int64_t e = 0; e < E; ++e)
        ASCA_REQUIRE(ctx, bucket_off[e + 1] >= bucket_off[e], "moe_forward_dev_buckets_host: bucket bounds must ascend");
    for (int64_t i = 0; i < N; ++i)
        ASCA_REQUIRE(ctx, bucket_idx[i] >= 0 && bucket_idx[i] < N, "moe_forward_dev_buckets_host: token index out of range");
    if (dev) *dev = nullptr;
    Scope s(ctx);
    void *dxn, *dw1, *db1, *dw2, *db2, *dperm, *doff, *dout, *dpre, *dhid;
    ASCA_TRY(s.upload(xn, (size_t)(N * d) * 4, &dxn));
    ASCA_TRY(s.upload(w1, (size_t)(d * E * F) * 4, &dw1));
    ASCA_TRY(s.upload(b1, (size_t)(E * F) * 4, &db1));
    ASCA_TRY(s.upload(w2, (size_t)(E * F * d) * 4, &dw2));
    ASCA_TRY(s.upload(b2, (size_t)d * 4, &db2));
    ASCA_TRY(s.upload(bucket_idx, (size_t)N * 4, &dperm));
    ASCA_TRY(s.upload(bucket_off, (size_t)(E + 1) * 4, &doff));
    ASCA_TRY(s.alloc((size_t)(N * d) * 4, &dout));
    ASCA_TRY(s.alloc((size_t)(N * F) * 4, &dpre));
    ASCA_TRY(s.alloc((size_t)(N * F) * 4, &dhid));
    ASCA_TRY(asca_moe_fwd(ctx, dxn, dw1, (float*)db1, dw2, (float*)db2, (int32_t*)dperm, (int32_t*)doff, N, d, F, E,
                          ASCA_F32, (float*)dout, (float*)dpre, dhid));
    ASCA_TRY(download(ctx, out, dout, (size_t)(N * d) * 4));
    ASCA_TRY(asca_ctx_sync(ctx));
    if (dev) {
        *dev = new asca_moe_dev{(float*)dxn, (float*)dw1, (float*)dw2, (float*)dpre, (float*)dhid,
                                (int32_t*)dperm, (int32_t*)doff, N, d, F, E};
        for (void* p : {dxn, dw1, dw2, dpre, dhid, dperm, doff}) s.keep(p);
    }
    return ASCA_OK;
}

// ------------------------------------------------------------------ head, cross-entropy, resident AdamW, SiLU
// Gpu::head_forward_dev (rust/src/cuda/mod.rs:828-846): logits = h_final head, kept on the device with h_final.
int asca_head_forward_dev_host(asca_ctx* ctx, const float* h_final, const float* head, int64_t T, int64_t d, int64_t V,
                               asca_logits_dev** dev) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, h_final && head && dev && T > 0 && d > 0 && V > 0, "head_forward_dev_host: bad arguments");
    *dev = nullptr;
    Scope s(ctx);
    void *dh, *dw, *dl;
    ASCA_TRY(s.upload(h_final, (size_t)(T * d) * 4, &dh));
    ASCA_TRY(s.upload(head, (size_t)(d * V) * 4, &dw));
    ASCA_TRY(s.alloc((size_t)(T * V) * 4, &dl));
    ASCA_TRY(asca_matmul(ctx, dh, dw, dl, T, d, V, ASCA_NN, ASCA_F32));
    ASCA_TRY(asca_ctx_sync(ctx));
    *dev = new asca_logits_dev{(float*)dl, (float*)dh, T, d, V};
    s.keep(dl);
    s.keep(dh);
    return ASCA_OK;
}

// LogitsDev::download (rust/src/cuda/mod.rs:1400-1413)
int asca_logits_dev_download(asca_ctx* ctx, const asca_logits_dev* dev, float* logits) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dev && logits, "logits_dev_download: null pointer");
    ASCA_TRY(download(ctx, logits, dev->logits, (size_t)(dev->T * dev->V) * 4));
    return asca_ctx_sync(ctx);
}

// Gpu::head_bwd_dev (rust/src/cuda/mod.rs:851-908): cross-entropy backward on the resident logits, then
// d_head = h_final^T dlogits (d x V) and dh = dlogits head_t (T x d), head_t being the head transposed (V x d).
int asca_head_bwd_dev_host(asca_ctx* ctx, const asca_logits_dev* dev, const uint32_t* targets, const float* head_t, float* loss,
                           float* d_head, float* dh) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dev && targets && head_t && loss && d_head && dh, "head_bwd_dev_host: null pointer");
    const int64_t T = dev->T, d = dev->d, V = dev->V;
    for (int64_t i = 0; i < T; ++i) ASCA_REQUIRE(ctx, targets[i] < (uint32_t)V, "head_bwd_dev_host: target out of range");
    Scope s(ctx);
    void *dt, *dht, *ddl, *dloss, *ddh, *ddx;
    ASCA_TRY(s.upload(targets, (size_t)T * 4, &dt));
    ASCA_TRY(s.upload(head_t, (size_t)(V * d) * 4, &dht));
    ASCA_TRY(s.alloc((size_t)(T * V) * 4, &ddl));
    ASCA_TRY(s.alloc(256, &dloss));
    ASCA_TRY(s.alloc((size_t)(d * V) * 4, &ddh));
    ASCA_TRY(s.alloc((size_t)(T * d) * 4, &ddx));
    ASCA_TRY(asca_cross_entropy(ctx, dev->logits, (const uint32_t*)dt, T, V, (float*)ddl, (float*)dloss));
    ASCA_TRY(asca_matmul(ctx, dev->h_final, ddl, ddh, d, T, V, ASCA_TN, ASCA_F32));
    ASCA_TRY(asca_matmul(ctx, ddl, dht, ddx, T, V, d, ASCA_NN, ASCA_F32));
    ASCA_TRY(download(ctx, loss, dloss, 4));
    ASCA_TRY(download(ctx, d_head, ddh, (size_t)(d * V) * 4));
    ASCA_TRY(download(ctx, dh, ddx, (size_t)(T * d) * 4));
    return asca_ctx_sync(ctx);
}

int asca_logits_dev_free(asca_ctx* ctx, asca_logits_dev* dev) {
    if (!ctx) return ASCA_ERR_ARG;
    if (!dev) return ASCA_OK;
    cudaStreamSynchronize(ctx->stream);
    asca_free(ctx, dev->logits);
    asca_free(ctx, dev->h_final);
    delete dev;
    return ASCA_OK;
}

// Gpu::cross_entropy_bwd (rust/src/cuda/mod.rs:945-1000): mean loss and dlogits = (softmax - onehot) / T.
int asca_cross_entropy_bwd_host(asca_ctx* ctx, const float* logits, const uint32_t* targets, int64_t T, int64_t V, float* loss,
                                float* dlogits) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, logits && targets && loss && dlogits && T > 0 && V > 0, "cross_entropy_bwd_host: bad arguments");
    for (int64_t i = 0; i < T; ++i) ASCA_REQUIRE(ctx, targets[i] < (uint32_t)V, "cross_entropy_bwd_host: target out of range");
    Scope s(ctx);
    void *dl, *dt, *ddl, *dloss;
    ASCA_TRY(s.upload(logits, (size_t)(T * V) * 4, &dl));
    ASCA_TRY(s.upload(targets, (size_t)T * 4, &dt));
    ASCA_TRY(s.alloc((size_t)(T * V) * 4, &ddl));
    ASCA_TRY(s.alloc(256, &dloss));
    ASCA_TRY(asca_cross_entropy(ctx, (const float*)dl, (const uint32_t*)dt, T, V, (float*)ddl, (float*)dloss));
    ASCA_TRY(download(ctx, loss, dloss, 4));
    ASCA_TRY(download(ctx, dlogits, ddl, (size_t)(T * V) * 4));
    return asca_ctx_sync(ctx);
}

// Gpu::adamw_resident (rust/src/cuda/mod.rs:1003-1055): the moments live on the device between calls, keyed by the
// caller's (host address of its m buffer, length); the first call for a key uploads m0 / v0. val and grad cross per
// call. CPU-path decay, as asca_adamw. asca_param_moments_host = param_moments (:57-73); asca_reset_param_cache =
// reset_param_cache (:50-54), to be called whenever a new model is created.
int asca_adamw_resident_host(asca_ctx* ctx, const void* key_addr, float* val, const float* grad, const float* m0,
                             const float* v0, int64_t n, float lr_t, float beta1, float beta2, float eps_t, float wd_eff) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, key_addr && val && grad && m0 && v0 && n > 0, "adamw_resident_host: bad arguments");
    const auto key = std::make_pair((uintptr_t)key_addr, (size_t)n);
    auto it = ctx->resident.find(key);
    if (it == ctx->resident.end()) {
        float *dm = nullptr, *dv = nullptr;
        if (cudaMalloc((void**)&dm, (size_t)n * 4) != cudaSuccess || cudaMalloc((void**)&dv, (size_t)n * 4) != cudaSuccess) {
            if (dm) cudaFree(dm);
            return asca_fail(ctx, ASCA_ERR_OOM, "adamw_resident_host: cannot allocate the moments");
        }
        ASCA_CUDA(ctx, cudaMemcpyAsync(dm, m0, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
        ASCA_CUDA(ctx, cudaMemcpyAsync(dv, v0, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
        it = ctx->resident.emplace(key, std::make_pair(dm, dv)).first;
    }
    Scope s(ctx);
    void *dp, *dg;
    ASCA_TRY(s.upload(val, (size_t)n * 4, &dp));
    ASCA_TRY(s.upload(grad, (size_t)n * 4, &dg));
    ASCA_TRY(asca_adamw(ctx, (float*)dp, (const float*)dg, it->second.first, it->second.second, n, lr_t, beta1, beta2, eps_t, wd_eff));
    ASCA_TRY(download(ctx, val, dp, (size_t)n * 4));
    return asca_ctx_sync(ctx);
}

int asca_param_moments_host(asca_ctx* ctx, const void* key_addr, int64_t n, float* m, float* v) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, key_addr && m && v && n > 0, "param_moments_host: bad arguments");
    auto it = ctx->resident.find(std::make_pair((uintptr_t)key_addr, (size_t)n));
    if (it == ctx->resident.end()) return 1;   // this parameter has no state on the device
    ASCA_TRY(download(ctx, m, it->second.first, (size_t)n * 4));
    ASCA_TRY(download(ctx, v, it->second.second, (size_t)n * 4));
    return asca_ctx_sync(ctx);
}

int asca_reset_param_cache(asca_ctx* ctx) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (auto& kv : ctx->resident) {
        cudaFree(kv.second.first);
        cudaFree(kv.second.second);
    }
    ctx->resident.clear();
    return ASCA_OK;
}

// Gpu::silu_inplace (rust/src/cuda/mod.rs:1224-1250)
int asca_silu_inplace_host(asca_ctx* ctx, float* x, int64_t n) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, x && n >= 0, "silu_inplace_host: bad arguments");
    if (n == 0) return ASCA_OK;
    Scope s(ctx);
    void* dx;
    ASCA_TRY(s.upload(x, (size_t)n * 4, &dx));
    silu_inplace_kernel<<<(unsigned)ceil_div64(n, 256), 256, 0, ctx->stream>>>((float*)dx, n);
    ASCA_CHECK_LAUNCH(ctx);
    ASCA_TRY(download(ctx, x, dx, (size_t)n * 4));
    return asca_ctx_sync(ctx);
}

}  // extern "C"
