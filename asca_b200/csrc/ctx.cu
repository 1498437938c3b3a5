// Context, device-memory cache and copies. Replaces the reference's lazily created `Gpu`
// singleton and its DevBuf pool (rust/src/cuda/mod.rs:104-237).
#include "common.cuh"

int asca_fail(asca_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf;
    return code;
}

int asca_workspace(asca_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->ws_bytes) {
        // growing the scratch must not race with kernels still reading the old one
        ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        if (ctx->ws) cudaFree(ctx->ws);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
        size_t want = (bytes + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
        ASCA_CUDA(ctx, cudaMalloc(&ctx->ws, want));
        ctx->ws_bytes = want;
    }
    *out = ctx->ws;
    return ASCA_OK;
}

extern "C" {

const char* asca_version(void) { return "asca_b200 0.1 (sm_100a)"; }

int asca_ctx_create(int device, asca_ctx** out) {
    if (!out) return ASCA_ERR_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || device < 0 || device >= n) return ASCA_ERR_CUDA;
    asca_ctx* c = new asca_ctx();
    c->device = device;
    if (cudaSetDevice(device) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete c;
        return ASCA_ERR_CUDA;
    }
    c->stream = c->own_stream;
    cudaDeviceProp p;
    cudaGetDeviceProperties(&p, device);
    c->sm_count = p.multiProcessorCount;
    c->smem_optin = p.sharedMemPerBlockOptin;
    char buf[256];
    snprintf(buf, sizeof buf, "asca_b200: device %d %s, sm_%d%d, %d SMs, %.1f GiB, %zu KiB smem/CTA", device,
             p.name, p.major, p.minor, p.multiProcessorCount, (double)p.totalGlobalMem / (1 << 30),
             p.sharedMemPerBlockOptin >> 10);
    c->desc = buf;
    if (cudaMalloc((void**)&c->err_word, 256) != cudaSuccess || cudaMemset(c->err_word, 0, 256) != cudaSuccess) {
        cudaStreamDestroy(c->own_stream);
        delete c;
        return ASCA_ERR_OOM;
    }
    *out = c;
    return ASCA_OK;
}

int asca_ctx_destroy(asca_ctx* ctx) {
    if (!ctx) return ASCA_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& kv : ctx->pool) cudaFree(kv.second);
    for (auto& kv : ctx->live) cudaFree(kv.first);
    if (ctx->ws) cudaFree(ctx->ws);
    for (auto& e : ctx->dtiles)
        if (e.buf) cudaFree(e.buf);
    for (auto& kv : ctx->resident) {
        cudaFree(kv.second.first);
        cudaFree(kv.second.second);
    }
    if (ctx->err_word) cudaFree(ctx->err_word);
    if (ctx->dyn_buf) cudaFree(ctx->dyn_buf);
    cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return ASCA_OK;
}

int asca_ctx_set_stream(asca_ctx* ctx, void* s) {
    if (!ctx) return ASCA_ERR_ARG;
    cudaStream_t next = s ? (cudaStream_t)s : ctx->own_stream;
    if (next != ctx->stream && ctx->stream) {
        // the context's scratch, caches and tile-claim counters are handed from launch to launch in stream order: what
        // the old stream still holds runs before anything the new one gets
        cudaSetDevice(ctx->device);
        cudaEvent_t e;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess) {
            // (an old stream its owner has destroyed meanwhile has nothing left to wait for)
            if (cudaEventRecord(e, ctx->stream) == cudaSuccess) cudaStreamWaitEvent(next, e, 0);
            cudaEventDestroy(e);
        }
        cudaGetLastError();
    }
    ctx->stream = next;
    return ASCA_OK;
}

int asca_ctx_sync(asca_ctx* ctx) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // kernels with bounded waits report a give-up through this word
    int word = 0;
    ASCA_CUDA(ctx, cudaMemcpy(&word, ctx->err_word, sizeof(int), cudaMemcpyDeviceToHost));
    if (word != 0) {
        cudaMemset(ctx->err_word, 0, sizeof(int));
        return asca_fail(ctx, ASCA_ERR_DEVICE, "a kernel gave up on a bounded wait (code %d)", word);
    }
    return ASCA_OK;
}

int asca_ctx_trim(asca_ctx* ctx) {
    if (!ctx) return ASCA_ERR_ARG;
    cudaSetDevice(ctx->device);
    ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (auto& e : ctx->dtiles)
        if (e.buf) cudaFree(e.buf);
    ctx->dtiles.clear();
    for (auto& kv : ctx->pool) cudaFree(kv.second);
    ctx->pool.clear();
    if (ctx->ws) cudaFree(ctx->ws);
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    return ASCA_OK;
}

int asca_ctx_set_tile_cache_bytes(asca_ctx* ctx, size_t bytes) {
    if (!ctx) return ASCA_ERR_ARG;
    ctx->dtiles_cap = bytes;
    return ASCA_OK;
}

int asca_ctx_profile(asca_ctx* ctx, int on) {
    if (!ctx) return ASCA_ERR_ARG;
    for (auto& sp : ctx->spans) {
        cudaEventDestroy(sp.e0);
        cudaEventDestroy(sp.e1);
    }
    ctx->spans.clear();
    ctx->profiling = on != 0;
    return ASCA_OK;
}

int asca_ctx_profile_read(asca_ctx* ctx, int index, const char** name, float* ms) {
    if (!ctx || !name || !ms) return ASCA_ERR_ARG;
    if (index < 0 || index >= (int)ctx->spans.size()) return 1;  // past the end
    ASCA_CUDA(ctx, cudaEventSynchronize(ctx->spans[index].e1));
    ASCA_CUDA(ctx, cudaEventElapsedTime(ms, ctx->spans[index].e0, ctx->spans[index].e1));
    *name = ctx->spans[index].name;
    return ASCA_OK;
}

int asca_ctx_profile_work(asca_ctx* ctx, int index, double* work) {
    if (!ctx || !work) return ASCA_ERR_ARG;
    if (index < 0 || index >= (int)ctx->spans.size()) return 1;
    *work = ctx->spans[index].work;
    return ASCA_OK;
}

const char* asca_last_error(const asca_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }
const char* asca_describe(asca_ctx* ctx) { return ctx ? ctx->desc.c_str() : "null context"; }
int64_t asca_launch_count(const asca_ctx* ctx) { return ctx ? ctx->launches : 0; }

static size_t size_class(size_t bytes) {
    size_t c = 256;
    while (c < bytes) c <<= 1;  // power-of-two classes like the reference's DevBuf
    // above 64 MiB round to 2 MiB instead so 180 GB is not wasted on rounding
    if (bytes > ((size_t)64 << 20)) c = (bytes + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);
    return c;
}

int asca_malloc(asca_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx || !dptr) return ASCA_ERR_ARG;
    size_t c = size_class(bytes ? bytes : 1);
    auto it = ctx->pool.find(c);
    if (it != ctx->pool.end()) {
        *dptr = it->second;
        ctx->pool.erase(it);
    } else {
        cudaError_t e = cudaMalloc(dptr, c);
        if (e != cudaSuccess) {
            // give cached blocks back and retry once
            ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            for (auto& kv : ctx->pool) cudaFree(kv.second);
            ctx->pool.clear();
            cudaGetLastError();
            ASCA_CUDA(ctx, cudaMalloc(dptr, c));
        }
    }
    ctx->live[*dptr] = c;
    return ASCA_OK;
}

int asca_free(asca_ctx* ctx, void* dptr) {
    if (!ctx) return ASCA_ERR_ARG;
    if (!dptr) return ASCA_OK;
    auto it = ctx->live.find(dptr);
    if (it == ctx->live.end()) return asca_fail(ctx, ASCA_ERR_ARG, "asca_free: pointer not from asca_malloc");
    ctx->pool.insert({it->second, dptr});
    ctx->live.erase(it);
    // tiles kept for a backward of this checkpoint buffer can no longer be claimed: their storage becomes reusable
    for (auto& e : ctx->dtiles)
        if (e.ckpt == dptr) e.ckpt = nullptr;
    return ASCA_OK;
}

int asca_memcpy_h2d(asca_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ASCA_OK;
}
int asca_memcpy_d2h(asca_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return ASCA_OK;
}
int asca_memset(asca_ctx* ctx, void* dst, int byte, size_t bytes) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_CUDA(ctx, cudaMemsetAsync(dst, byte, bytes, ctx->stream));
    return ASCA_OK;
}

}  // extern "C"
