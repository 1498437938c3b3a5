// Model glue: embedding, N x [x += Delta(x); x += HashMoE(RMSNorm(x))], final RMSNorm, head,
// cross-entropy, backward, AdamW, and the per-token decode step -- the dataflow of
// rust/src/model.rs:631-802 and rust/src/delta.rs:121-207 / :615-674, composed from the
// library's own entry points with every activation resident in HBM. f32 arithmetic.
#include "common.cuh"

#include <algorithm>
#include "gemm_tc.cuh"
#include "model.cuh"

namespace {

// ------------------------------------------------------------------ small kernels
// out[c] (+)= sum_r src[r, c], deterministic. Pass 1: CTA (x, y) owns 32 columns of row slice y, its 8 warps
// stride the slice's rows, fixed-order tree -> part[y][c]. Pass 2 adds the slices in order.
__global__ void __launch_bounds__(256) colsum_slices_kernel(const float* __restrict__ src, int64_t ld, int64_t rows,
                                                            int cols, int64_t rows_per_slice, float* __restrict__ part) {
    __shared__ float red[8][33];
    const int c = blockIdx.x * 32 + (threadIdx.x & 31), w = threadIdx.x >> 5;
    const int64_t lo = blockIdx.y * rows_per_slice, hi = lo + rows_per_slice < rows ? lo + rows_per_slice : rows;
    float acc = 0.0f;
    if (c < cols) {
        int64_t r = lo + w;
        for (; r + 24 < hi; r += 32) {   // four independent loads in flight
            const float a0 = src[r * ld + c], a1 = src[(r + 8) * ld + c], a2 = src[(r + 16) * ld + c], a3 = src[(r + 24) * ld + c];
            acc += (a0 + a1) + (a2 + a3);
        }
        for (; r < hi; r += 8) acc += src[r * ld + c];
    }
    red[w][threadIdx.x & 31] = acc;
    __syncthreads();
    if (w == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][threadIdx.x];
        part[(int64_t)blockIdx.y * cols + c] = t;
    }
}
__global__ void __launch_bounds__(256) colsum_finish_kernel(const float* __restrict__ part, int n_slices, int cols,
                                                            float* __restrict__ out, int accumulate) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= cols) return;
    float t = 0.0f;
    for (int s = 0; s < n_slices; ++s) t += part[(int64_t)s * cols + c];
    out[c] = accumulate ? out[c] + t : t;
}

// One warp per row: log-sum-exp, loss_t, dlogits = (p - onehot) * inv_n. rust/src/model.rs:821-837.
__global__ void __launch_bounds__(256) cross_entropy_kernel(const float* __restrict__ logits,
                                                            const uint32_t* __restrict__ targets, int64_t N, int V,
                                                            float* __restrict__ dlogits, float* __restrict__ losses,
                                                            float inv_n) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= N) return;
    const float* row = logits + t * V;
    float mx = -INFINITY;
    for (int c = lane; c < V; c += 32) mx = fmaxf(mx, row[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (int c = lane; c < V; c += 32) sum += expf(row[c] - mx);
    sum = warp_sum(sum);
    const float lse = mx + logf(sum);
    const uint32_t tg = targets[t];
    if (lane == 0) losses[t] = lse - row[tg];
    if (dlogits) {
        float* drow = dlogits + t * V;
        for (int c = lane; c < V; c += 32) drow[c] = expf(row[c] - lse) * inv_n - ((uint32_t)c == tg ? inv_n : 0.0f);
    }
}
// Deterministic mean of n values (one CTA, fixed tree).
__global__ void __launch_bounds__(1024) mean_kernel(const float* __restrict__ v, int64_t n, float scale,
                                                    float* __restrict__ out) {
    __shared__ float red[33];
    float acc = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += 1024) acc += v[i];
    const float s = block_sum(acc, red);
    if (threadIdx.x == 0) *out = s * scale;
}

__global__ void __launch_bounds__(256) embed_fwd_kernel(const float* __restrict__ table,
                                                        const uint32_t* __restrict__ ids, int64_t N, int d,
                                                        float* __restrict__ x) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (t >= N) return;
    const float* src = table + (int64_t)ids[t] * d;
    for (int c = lane; c < d; c += 32) x[t * d + c] = src[c];
}
// d_table[v, c] += sum over tokens t with ids[t] == v of dx[t, c]. grid (vocab, ceil(d/128)): the fallback for
// row lengths that are not a multiple of 4.
__global__ void __launch_bounds__(128) embed_bwd_kernel(const float* __restrict__ dx, const uint32_t* __restrict__ ids,
                                                        int64_t N, int d, float* __restrict__ d_table) {
    const uint32_t v = blockIdx.x;
    const int c = blockIdx.y * 128 + threadIdx.x;
    float acc = 0.0f;
    bool any = false;
    for (int64_t t = 0; t < N; ++t)
        if (ids[t] == v) {
            any = true;
            if (c < d) acc += dx[t * d + c];
        }
    if (any && c < d) d_table[(int64_t)v * d + c] += acc;
}
// Same sum, deterministic, for d % 4 == 0: CTA (v, y) owns 256 columns of table row v; each of its 8 warps scans
// a fixed stride of the ids 32 at a time (ballot), adds the matching rows with every lane holding 8 columns,
// and the 8 partial rows are added in warp order.
__global__ void __launch_bounds__(256) embed_bwd_ballot_kernel(const float* __restrict__ dx, const uint32_t* __restrict__ ids,
                                                               int64_t N, int d, float* __restrict__ d_table) {
    __shared__ float red[8][256];
    const uint32_t v = blockIdx.x;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = blockIdx.y * 256 + lane * 8;
    const bool lo_ok = c0 + 4 <= d, hi_ok = c0 + 8 <= d;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t base = (int64_t)w * 32; base < N; base += 256) {
        const int64_t t = base + lane;
        unsigned mask = __ballot_sync(0xffffffffu, t < N && ids[t] == v);
        while (mask) {
            const int b = __ffs(mask) - 1;
            mask &= mask - 1;
            const float* row = dx + (base + b) * d + c0;
            if (lo_ok) {
                const float4 x = *reinterpret_cast<const float4*>(row);
                acc[0] += x.x; acc[1] += x.y; acc[2] += x.z; acc[3] += x.w;
            }
            if (hi_ok) {
                const float4 x = *reinterpret_cast<const float4*>(row + 4);
                acc[4] += x.x; acc[5] += x.y; acc[6] += x.z; acc[7] += x.w;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) red[w][lane * 8 + j] = acc[j];
    __syncthreads();
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c < d) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][threadIdx.x];
        d_table[(int64_t)v * d + c] += t;
    }
}
__global__ void __launch_bounds__(256) add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                  float* __restrict__ out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < n) out[i] = a[i] + 1.0f * b[i];
}
// out = a + b with a bf16 copy, four elements per thread (n % 4 == 0, 16-byte aligned; out may be a)
__global__ void __launch_bounds__(256) add_cast4_kernel(const float* a, const float* __restrict__ b, float* out,
                                                        __nv_bfloat16* __restrict__ out16, int64_t n4) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
        const float4 x = reinterpret_cast<const float4*>(a)[i], y = reinterpret_cast<const float4*>(b)[i];
        const float4 v = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
        reinterpret_cast<float4*>(out)[i] = v;
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        reinterpret_cast<uint2*>(out16)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}
// A decode step's token prologue in one launch (at most 1024 streams and 1024 experts, d % 4 == 0): every block
// embeds 8 rows (f32 + bf16 copy); block 0 also builds the dispatch tables -- expert = hash(id) % E
// (rust/src/model.rs:69-77), stable counting sort by expert: perm (tokens grouped by expert, ascending inside an
// expert), offsets, and the inverse permutation. Integer work, the same permutation as asca_moe_dispatch.
__global__ void __launch_bounds__(256) decode_prologue_kernel(const float* __restrict__ table, const uint32_t* __restrict__ ids, int ns,
                                                              int d, int E, float* __restrict__ x, __nv_bfloat16* __restrict__ x16,
                                                              int32_t* __restrict__ perm, int32_t* __restrict__ offs,
                                                              int32_t* __restrict__ inv_perm) {
    __shared__ int32_t cnt[1024 + 1];
    __shared__ uint16_t ex[1024];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int t = blockIdx.x * 8 + w;
    pdl_wait();   // the ids may be the previous kernel's argmax
    pdl_launch_dependents();
    if (t < ns) {
        const float4* src = reinterpret_cast<const float4*>(table + (int64_t)ids[t] * d);
        float4* dst = reinterpret_cast<float4*>(x + (int64_t)t * d);
        uint2* dst16 = reinterpret_cast<uint2*>(x16 + (int64_t)t * d);
        for (int c = lane; c < d / 4; c += 32) {
            const float4 v = src[c];
            dst[c] = v;
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
            dst16[c] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
        }
    }
    if (blockIdx.x != 0) return;
    for (int e = threadIdx.x; e <= E; e += 256) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < ns; i += 256) {
        uint32_t h = ids[i] * 0x9E3779B1u;
        h ^= h >> 15;
        h *= 0x85EBCA6Bu;
        h ^= h >> 13;
        const uint32_t e = h % (uint32_t)E;
        ex[i] = (uint16_t)e;
        atomicAdd(&cnt[e + 1], 1);   // integer counts: the order of the additions does not matter
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int e = 0; e < E; ++e) cnt[e + 1] += cnt[e];   // cnt[e] = first position of expert e
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += 256) offs[e] = cnt[e];
    for (int i = threadIdx.x; i < ns; i += 256) {
        const uint16_t e = ex[i];
        int rank = 0;
        for (int j = 0; j < i; ++j) rank += ex[j] == e;   // tokens of the same expert before this one
        const int pos = cnt[e] + rank;
        perm[pos] = i;
        inv_perm[i] = pos;
    }
}
// dst[r, 0:cols] (bf16, row pitch ld_dst) = src[r, 0:cols] (f32, contiguous rows); cols % 4 == 0
__global__ void __launch_bounds__(256) cast_cols_kernel(const float* __restrict__ src, int cols4, int64_t n4, __nv_bfloat16* __restrict__ dst,
                                                        int64_t ld_dst) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
        const int64_t r = i / cols4;
        const int c = (int)(i % cols4);
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(dst + r * ld_dst + 4 * c) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}
// The same cast with the column sums of src taken in the same pass (a bias gradient): CTA (x, y) owns 1024 columns (a
// thread 4 consecutive ones: every row is read in runs of 4 KiB) of row slab y; a thread adds its slab's rows in order
// -> part[y][c], and the slabs are added in order by colsum_finish_kernel. cols % 4 == 0.
__global__ void __launch_bounds__(256) cast_colsum_kernel(const float* __restrict__ src, int cols, int64_t rows, int64_t rows_per_slab,
                                                          __nv_bfloat16* __restrict__ dst, int64_t ld_dst, float* __restrict__ part) {
    const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
    if (c >= cols) return;
    const int64_t lo = blockIdx.y * rows_per_slab, hi = lo + rows_per_slab < rows ? lo + rows_per_slab : rows;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const auto put = [&](int64_t r, const float4& v) {
        const __nv_bfloat162 l2 = __floats2bfloat162_rn(v.x, v.y), h2 = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(dst + r * ld_dst + c) = make_uint2(*reinterpret_cast<const uint32_t*>(&l2), *reinterpret_cast<const uint32_t*>(&h2));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    };
    int64_t r = lo;
    for (; r + 4 <= hi; r += 4) {   // four rows in flight per thread
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const float4*>(src + (r + i) * cols + c);
#pragma unroll
        for (int i = 0; i < 4; ++i) put(r + i, v[i]);
    }
    for (; r < hi; ++r) put(r, *reinterpret_cast<const float4*>(src + r * cols + c));
    *reinterpret_cast<float4*>(part + (int64_t)blockIdx.y * cols + c) = acc;
}
// inv[perm[i]] = i
__global__ void __launch_bounds__(256) invert_perm_kernel(const int32_t* __restrict__ perm, int32_t* __restrict__ inv, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < n) inv[perm[i]] = (int32_t)i;
}
// out = a + b, with a bf16 copy (the next block's product reads the copy)
__global__ void __launch_bounds__(256) add_cast_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                       float* __restrict__ out, __nv_bfloat16* __restrict__ out16, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    if (i < n) {
        const float v = a[i] + b[i];
        out[i] = v;
        out16[i] = __float2bfloat16(v);
    }
}
// dst (rows x ld, bf16) = [a (rows x ca) | b (rows x cb) | 0]; bias likewise (f32)
__global__ void __launch_bounds__(256) concat_cols_kernel(const float* __restrict__ a, int ca, const float* __restrict__ b, int cb,
                                                          int64_t rows, int ld, __nv_bfloat16* __restrict__ dst) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= rows * ld) return;
    const int64_t r = i / ld;
    const int c = (int)(i % ld);
    const float v = c < ca ? a[r * ca + c] : (c < ca + cb ? b[r * cb + (c - ca)] : 0.0f);
    dst[i] = __float2bfloat16(v);
}
__global__ void __launch_bounds__(256) concat_bias_kernel(const float* __restrict__ a, int ca, const float* __restrict__ b, int cb,
                                                          int ld, float* __restrict__ dst) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < ld) dst[c] = c < ca ? a[c] : (c < ca + cb ? b[c - ca] : 0.0f);
}
// greedy argmax per row, lowest index on ties
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int64_t N, int V,
                                                     uint32_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    pdl_wait();
    pdl_launch_dependents();
    if (t >= N) return;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < V; c += 32) {
        const float x = logits[t * V + c];
        if (x > best) {
            best = x;
            bi = c;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) {
            best = ob;
            bi = oi;
        }
    }
    if (lane == 0) out[t] = (uint32_t)bi;
}

// alpha, beta = sigmoid of the gate logits (rust/src/delta.rs:167-179): logits (N, 2H), one thread per (row, head).
__global__ void __launch_bounds__(256) gate_sigmoid_kernel(const float* __restrict__ gate, int64_t units, int H,
                                                           float* __restrict__ alpha, float* __restrict__ beta) {
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = u / H;
        const int h = (int)(u % H);
        alpha[u] = 1.0f / (1.0f + expf(-gate[r * 2 * H + h]));
        beta[u] = 1.0f / (1.0f + expf(-gate[r * 2 * H + H + h]));
    }
}

struct Bufs {   // device buffers from the context cache, released together
    asca_ctx* ctx;
    std::vector<void*> p;
    explicit Bufs(asca_ctx* c) : ctx(c) {}
    ~Bufs() {
        for (void* x : p) asca_free(ctx, x);
    }
    float* f(int64_t n) {
        void* d = nullptr;
        if (asca_malloc(ctx, (size_t)(n > 0 ? n : 1) * 4, &d) != ASCA_OK) return nullptr;
        p.push_back(d);
        return (float*)d;
    }
};

}  // namespace


// A contiguous range of the gradient buffer has had all its kernels enqueued: tell the caller's hook and the
// data-parallel exchange. Per block, in backward order: the expert tensors (w1, b1, w2, b2 -- final right after the
// expert backward, the first thing a block's backward does), then the block's projections; last embedding + head.
static int grad_ready(asca_ctx* ctx, asca_model* m, int64_t off, int64_t cnt) {
    if (m->grad_hook) m->grad_hook(m->grad_hook_user, off, cnt);
    return m->dp ? asca_dp_grad_ready(ctx, m, off, cnt) : ASCA_OK;
}

// The bf16 copy of the weights that the tensor-core products read: allocated on first use, rebuilt whenever the
// f32 master copy changed behind it (set_params, an AdamW step that did not write it itself, params_changed).
static int refresh_params16(asca_ctx* ctx, asca_model* m) {
    if (!m->params16) {
        if (cudaMalloc((void**)&m->params16, (size_t)m->n16 * 2) != cudaSuccess)
            return asca_fail(ctx, ASCA_ERR_OOM, "model: cannot allocate the bf16 weight copy");
        m->params16_stale = true;
    }
    if (!m->params16_stale) return ASCA_OK;
    ASCA_REQUIRE(ctx, !m->master_stale,
                 "model: the bf16 weight copy would be rebuilt from master weights that are stale on this rank (sharded "
                 "optimizer); call asca_model_dp_gather_master first");
    if (m->n16 == m->n_params) {   // no padding anywhere: one pass over the flat buffer
        ASCA_TRY(asca_cast_bf16(ctx, m->params, m->params16, m->n_params));
    } else {
        for (size_t i = 0; i + 1 < m->seg_off.size(); ++i)
            ASCA_TRY(asca_cast_bf16(ctx, m->params + m->seg_off[i], m->params16 + m->seg16[i], m->seg_off[i + 1] - m->seg_off[i]));
    }
    m->params16_stale = false;
    return ASCA_OK;
}

// Decode step in bf16 compute mode: same dataflow as Model::step (rust/src/model.rs:703-720) for ns streams at
// once, products on the tensor cores from the bf16 weight copy, the expert FFN through the dispatch + grouped
// GEMM path (every expert's weights are read once per step, not once per stream); state, residual stream and
// logits stay f32.
bool asca_tc_enabled();  // gemm.cu
// elementwise.cu
int asca_rmsnorm_bwd_add_cast(asca_ctx* ctx, const float* x, const float* dy, const float* add, float* dx, void* dx16, int64_t rows,
                              int64_t cols, float eps);
// moe.cu / mixed.cu: the decode-step forms on rows in expert order
int asca_moe_fwd_sorted_residual(asca_ctx* ctx, const __nv_bfloat16* xp, const __nv_bfloat16* w1, const float* b1,
                                 const __nv_bfloat16* w2, const float* b2, const int32_t* perm, const int32_t* offsets, int64_t N,
                                 int64_t d, int64_t F, int64_t E, float* x, __nv_bfloat16* x16, __nv_bfloat16* hid_p, int check_only,
                                 int packed);
int asca_residual_rmsnorm_bf16_rows(asca_ctx* ctx, const float* x, const float* yadd, float* x_mid, void* xn, int64_t rows,
                                    int64_t cols, float eps, const int32_t* y_row);

// The qkv and gate projections of every block as one (d, 3d + 2H rounded up to 8) bf16 matrix, and their biases:
// one product instead of two wherever both read the same rows (the decode step; the input gradient of the block).
static int refresh_dec_w(asca_ctx* ctx, asca_model* m) {
    const int64_t d = m->d, H = m->H, ldq = (3 * d + 2 * H + 7) & ~(int64_t)7;
    const float* P = m->params;
    if (!m->dec_w) {
        if (cudaMalloc((void**)&m->dec_w, (size_t)m->L * d * ldq * 2) != cudaSuccess ||
            cudaMalloc((void**)&m->dec_b, (size_t)m->L * ldq * 4) != cudaSuccess)
            return asca_fail(ctx, ASCA_ERR_OOM, "model: cannot allocate the fused qkv + gate projection");
        m->dec_stale = true;
        m->dec_pk_stale = true;
    }
    if (m->dec_stale) {
        for (int64_t li = 0; li < m->L; ++li) {
            const Lyr& w = m->lay[li];
            concat_cols_kernel<<<(unsigned)ceil_div64(d * ldq, 256), 256, 0, ctx->stream>>>(
                P + w.w_qkv, (int)(3 * d), P + w.w_gate, (int)(2 * H), d, (int)ldq, m->dec_w + li * d * ldq);
            concat_bias_kernel<<<(unsigned)ceil_div64(ldq, 256), 256, 0, ctx->stream>>>(P + w.b_qkv, (int)(3 * d), P + w.b_gate,
                                                                                     (int)(2 * H), (int)ldq, m->dec_b + li * ldq);
            ctx->launches += 2;
        }
        ASCA_CUDA(ctx, cudaGetLastError());
        m->dec_stale = false;
    }
    return ASCA_OK;
}

// n_steps steps in bf16 mode. Step 0 consumes ids_h; a later step consumes the previous step's argmax, which never
// leaves the device (tokens_h, n_steps x ns, receives all of them after the last step). One synchronisation at the end.
static int decode_step_bf16(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids_h, int64_t ns, float* logits_h,
                            uint32_t* next_h, int64_t n_steps = 1, uint32_t* tokens_h = nullptr) {
    typedef __nv_bfloat16 bf16;
    const int64_t d = m->d, H = m->H, dh = d / H, E = m->E, F = m->F, V = m->vocab;
    const int BF = ASCA_BF16;
    ASCA_TRY(refresh_params16(ctx, m));
    ASCA_TRY(asca_dp_wait_all(ctx, m));
    const float* P = m->params;
    const bf16* W = m->params16;
    Bufs bf(ctx);
    auto h16 = [&](int64_t n) { return (bf16*)bf.f((n + 1) / 2); };
    uint32_t* ids = (uint32_t*)bf.f(ns);
    uint32_t* toks = (uint32_t*)bf.f(ns * n_steps);   // every step's chosen ids
    int32_t* perm = (int32_t*)bf.f(ns);
    int32_t* offs = (int32_t*)bf.f(E + 1);
    float *x = bf.f(ns * d), *qkv = bf.f(ns * 3 * d), *gate = bf.f(ns * 2 * H), *o = bf.f(ns * d), *y = bf.f(ns * d),
          *x_mid = bf.f(ns * d), *mo = bf.f(ns * d), *logits = bf.f(ns * V), *pre_p = bf.f(ns * F);
    bf16 *x16 = h16(ns * d), *o16 = h16(ns * d), *xn16 = h16(ns * d), *hid16 = h16(ns * F), *hf16 = h16(ns * d);
    ASCA_REQUIRE(ctx, ids && toks && perm && offs && x && qkv && gate && o && y && x_mid && mo && logits && pre_p && x16 && o16 &&
                          xn16 && hid16 && hf16, "model_decode_step: out of memory");
    ASCA_CUDA(ctx, cudaMemcpyAsync(ids, ids_h, (size_t)ns * 4, cudaMemcpyHostToDevice, ctx->stream));
    const bool fused64 = dh == 64;   // one projection for qkv + gate, the warp-per-head state update, casts folded in
    const int64_t ldq = (3 * d + 2 * H + 7) & ~(int64_t)7;
    if (fused64) ASCA_TRY(refresh_dec_w(ctx, m));
    float* qg = fused64 ? bf.f(ns * ldq) : nullptr;
    ASCA_REQUIRE(ctx, !fused64 || qg, "model_decode_step: out of memory");
    // With a handful of tokens per expert the MoE runs on rows in expert order end to end: the norm writes its bf16
    // rows at their expert-order position (the gather), and the second expert product adds into the residual rows
    // through the permutation and writes the next block's bf16 input (the combine, the residual add and the cast).
    const bool sorted_moe = asca_moe_fwd_sorted_residual(ctx, xn16, W + m->lay16[0].w1, P + m->lay[0].b1, W + m->lay16[0].w2,
                                                         P + m->lay[0].b2, perm, offs, ns, d, F, E, x, x16, hid16, 1, 0) == ASCA_OK;
    // ... and then every product of the step is a few-row product whose weights are read once: they are kept a second
    // time in the order that kernel streams them (per layer: qkv+gate, out, experts' W1, experts' W2; then the head)
    const bool packed = fused64 && sorted_moe && ns <= 256;
    const int64_t r_qg = gemm_tc::skinny_packed_rows(1, d, ldq), r_o = gemm_tc::skinny_packed_rows(1, d, d),
                  r_w1 = gemm_tc::skinny_packed_rows(E, d, F), r_w2 = gemm_tc::skinny_packed_rows(E, F, d),
                  r_layer = r_qg + r_o + r_w1 + r_w2, r_head = gemm_tc::skinny_packed_rows(1, d, V);
    if (packed && !m->dec_pk) {
        if (cudaMalloc((void**)&m->dec_pk, (size_t)(m->L * r_layer + r_head) * 128) != cudaSuccess)
            return asca_fail(ctx, ASCA_ERR_OOM, "model: cannot allocate the decode weight copy");
        m->dec_pk_stale = true;
    }
    if (packed && m->dec_pk_stale) {
        for (int64_t li = 0; li < m->L; ++li) {
            const Lyr& w16 = m->lay16[li];
            bf16* pk = m->dec_pk + li * r_layer * 64;
            ASCA_TRY(gemm_tc::skinny_pack(ctx, m->dec_w + li * d * ldq, ldq, 1, 0, 0, d, ldq, pk));
            ASCA_TRY(gemm_tc::skinny_pack(ctx, W + w16.w_o, d, 1, 0, 0, d, d, pk + r_qg * 64));
            ASCA_TRY(gemm_tc::skinny_pack(ctx, W + w16.w1, E * F, E, F, 0, d, F, pk + (r_qg + r_o) * 64));
            ASCA_TRY(gemm_tc::skinny_pack(ctx, W + w16.w2, d, E, 0, F, F, d, pk + (r_qg + r_o + r_w1) * 64));
        }
        ASCA_TRY(gemm_tc::skinny_pack(ctx, W + m->head16, V, 1, 0, 0, d, V, m->dec_pk + m->L * r_layer * 64));
        m->dec_pk_stale = false;
    }
    auto few_rows = [&](const bf16* X, int64_t K, const bf16* Wpk, int64_t N, float* C, int64_t ldc, const float* bias) -> int {
        gemm_tc::Args t{};
        t.mode = ASCA_NN;
        t.A = X; t.lda = K; t.a_rows = ns; t.a_cols = K;
        t.B = Wpk; t.ldb = 64; t.b_rows = gemm_tc::skinny_packed_rows(1, K, N); t.b_cols = 64; t.b_packed = 1;
        t.C = C; t.ldc = ldc; t.M = (int)ns; t.N = (int)N; t.K = (int)K; t.bias = bias;
        t.group_dim = gemm_tc::GROUP_NONE; t.epi = gemm_tc::EPI_NONE;
        t.b_early = 1;   // weights: written long before the previous kernel
        if (!gemm_tc::supported(t)) return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "model_decode_step: product not supported");
        return gemm_tc::launch_skinny(ctx, t);
    };
    int32_t* inv_perm = sorted_moe ? (int32_t*)bf.f(ns) : nullptr;
    ASCA_REQUIRE(ctx, !sorted_moe || inv_perm, "model_decode_step: out of memory");
    struct PdlScope {
        asca_ctx* c;
        explicit PdlScope(asca_ctx* c_) : c(c_) {}
        ~PdlScope() { c->pdl = false; }
    } pdl_scope(ctx);
    for (int64_t step = 0; step < n_steps; ++step) {
    const uint32_t* cur = step == 0 ? ids : toks + (step - 1) * ns;
    uint32_t* nxt = toks + step * ns;
    ctx->pdl = false;
    if (sorted_moe && ns <= 1024 && E <= 1024 && (d & 3) == 0) {   // dispatch, embedding and its bf16 copy: one launch
        ctx->pdl = step > 0;   // after the previous step's argmax
        ASCA_CUDA(ctx, asca_launch(ctx, decode_prologue_kernel, dim3((unsigned)ceil_div64(ns, 8)), dim3(256), 0, P + m->embed, cur, (int)ns,
                                   (int)d, (int)E, x, x16, perm, offs, inv_perm));
        ctx->launches++;
    } else {
        ASCA_TRY(asca_moe_dispatch(ctx, cur, ns, E, perm, offs, nullptr));
        ASCA_TRY(asca_embed_fwd(ctx, P + m->embed, cur, ns, d, x));
        if (sorted_moe) {
            invert_perm_kernel<<<(unsigned)ceil_div64(ns, 256), 256, 0, ctx->stream>>>(perm, inv_perm, ns);
            ASCA_CHECK_LAUNCH(ctx);
        }
        ASCA_TRY(asca_cast_bf16(ctx, x, x16, ns * d));
    }
    // the block chain is short kernels back to back: each may become resident while its predecessor drains
    ctx->pdl = true;
    for (int64_t li = 0; li < m->L; ++li) {
        const Lyr& w = m->lay[li];
        const Lyr& w16 = m->lay16[li];
        if (fused64) {
            if (packed) ASCA_TRY(few_rows(x16, d, m->dec_pk + li * r_layer * 64, ldq, qg, ldq, m->dec_b + li * ldq));
            else ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, ldq, d, x16, d, m->dec_w + li * d * ldq, ldq, qg, ldq, m->dec_b + li * ldq, 0, BF));
            ASCA_TRY(asca_delta_step_strided(ctx, qg, ldq, qg + 3 * d, ldq, state + li * ns * H * dh * dh, ns, H, o, o16));
        } else {
            ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, 3 * d, d, x16, d, W + w16.w_qkv, 3 * d, qkv, 3 * d, P + w.b_qkv, 0, BF));
            ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, 2 * H, d, x16, d, W + w16.w_gate, 2 * H, gate, 2 * H, P + w.b_gate, 0, BF));
            ASCA_TRY(asca_delta_step(ctx, qkv, nullptr, nullptr, gate, nullptr, state + li * ns * H * dh * dh, ns, H, dh, 1, o));
            ASCA_TRY(asca_cast_bf16(ctx, o, o16, ns * d));
        }
        if (packed) ASCA_TRY(few_rows(o16, d, m->dec_pk + (li * r_layer + r_qg) * 64, d, y, d, P + w.b_o));
        else ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, d, d, o16, d, W + w16.w_o, d, y, d, P + w.b_o, 0, BF));
        if (sorted_moe) {
            ASCA_TRY(asca_residual_rmsnorm_bf16_rows(ctx, x, y, x, xn16, ns, d, 1e-6f, inv_perm));   // x += y in place
            const bf16* pk = m->dec_pk + (li * r_layer + r_qg + r_o) * 64;
            ASCA_TRY(asca_moe_fwd_sorted_residual(ctx, xn16, packed ? pk : W + w16.w1, P + w.b1, packed ? pk + r_w1 * 64 : W + w16.w2,
                                                  P + w.b2, perm, offs, ns, d, F, E, x, x16, hid16, 0, packed ? 1 : 0));
            continue;
        }
        ASCA_TRY(asca_residual_rmsnorm_bf16(ctx, x, y, x_mid, xn16, ns, d, 1e-6f));
        ASCA_TRY(asca_moe_fwd(ctx, xn16, W + w16.w1, P + w.b1, W + w16.w2, P + w.b2, perm, offs, ns, d, F, E, BF, mo, pre_p, hid16));
        ASCA_CUDA(ctx, asca_launch(ctx, add_cast_kernel, dim3((unsigned)ceil_div64(ns * d, 256)), dim3(256), 0, x_mid, mo, x, x16,
                                   ns * d));   // x_out (+ bf16)
        ctx->launches++;
    }
    ASCA_TRY(asca_residual_rmsnorm_bf16(ctx, x, nullptr, nullptr, hf16, ns, d, 1e-6f));
    if (packed) ASCA_TRY(few_rows(hf16, d, m->dec_pk + m->L * r_layer * 64, V, logits, V, nullptr));
    else ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, V, d, hf16, d, W + m->head16, V, logits, V, nullptr, 0, BF));
    if (logits_h && step == n_steps - 1) {
        ctx->pdl = false;   // a copy sits between the head product and the argmax
        ASCA_CUDA(ctx, cudaMemcpyAsync(logits_h, logits, (size_t)ns * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    if (next_h || tokens_h || step + 1 < n_steps) {
        ASCA_CUDA(ctx, asca_launch(ctx, argmax_kernel, dim3((unsigned)ceil_div64(ns, 8)), dim3(256), 0, (const float*)logits, ns, (int)V, nxt));
        ctx->launches++;
    }
    ctx->pdl = false;
    }   // steps
    if (next_h) ASCA_CUDA(ctx, cudaMemcpyAsync(next_h, toks + (n_steps - 1) * ns, (size_t)ns * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (tokens_h) ASCA_CUDA(ctx, cudaMemcpyAsync(tokens_h, toks, (size_t)ns * n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return asca_ctx_sync(ctx);
}

extern "C" {
static int cross_entropy_scaled(asca_ctx* ctx, const float* logits, const uint32_t* targets, int64_t N, int64_t V,
                                float* dlogits, float* loss, float grad_scale);
}

static int materialize_zero_grads(asca_ctx* ctx, asca_model* m) {
    if (!m->grads_zero_pending) return ASCA_OK;
    m->grads_zero_pending = false;
    if (ctx) {
        ASCA_CUDA(ctx, cudaMemsetAsync(m->grads, 0, (size_t)m->n_params * 4, ctx->stream));
        return ASCA_OK;
    }
    return cudaMemset(m->grads, 0, (size_t)m->n_params * 4) == cudaSuccess ? ASCA_OK : ASCA_ERR_CUDA;
}

// ---------------------------------------------------------------------------------------------
// bf16 compute mode: the dataflow of Model::forward / Model::backward (rust/src/model.rs:631-700,
// :744-794) with every product on the tensor cores. The residual stream, norms, gates, the
// recurrent state, the loss, the gradients and the master weights stay f32; what a product reads
// is bf16 (weights from a bf16 copy of the master buffer, activations written as bf16 by the
// kernel that produces them or by a cast pass).
static int forward_backward_bf16(asca_ctx* ctx, asca_model* m, const uint32_t* ids_h, const uint32_t* tg_h, int64_t B,
                                 int64_t T, float* loss_h, float* logits_h) {
    typedef __nv_bfloat16 bf16;
    const int64_t N = B * T, d = m->d, H = m->H, dh = d / H, E = m->E, F = m->F, V = m->vocab, L = m->L;
    const int64_t CH = 64;
    const int BF = ASCA_BF16;
    ASCA_TRY(refresh_params16(ctx, m));
    const float* P = m->params;
    const bf16* W = m->params16;
    float* G = m->grads;
    const int acc = m->grads_zero_pending ? 0 : 1;   // first backward after zero_grads: overwrite
    m->grads_zero_pending = false;
    Bufs bf(ctx);
    auto h16 = [&](int64_t n) { return (bf16*)bf.f((n + 1) / 2); };
    uint32_t* ids = (uint32_t*)bf.f(N);
    uint32_t* tg = (uint32_t*)bf.f(N);
    int32_t* perm = (int32_t*)bf.f(N);
    int32_t* offs = (int32_t*)bf.f(E + 1);
    ASCA_REQUIRE(ctx, ids && tg && perm && offs, "model_forward_backward: out of memory");
    ASCA_CUDA(ctx, cudaMemcpyAsync(ids, ids_h, (size_t)N * 4, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_CUDA(ctx, cudaMemcpyAsync(tg, tg_h, (size_t)N * 4, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_TRY(asca_moe_dispatch(ctx, ids, N, E, perm, offs, nullptr));

    struct Act {
        bf16 *x_in, *q, *k, *v, *o, *xn, *hid_p;
        float *qn, *kn, *al, *be, *ckpt, *x_mid, *pre_p;
    };
    std::vector<Act> acts(L);
    const int64_t nck = asca_delta_ckpt_floats(B, T, H, dh, CH);
    float* x = bf.f(N * d);
    float* qkv = bf.f(N * 3 * d);
    float* gate = bf.f(N * 2 * H);
    float* y = bf.f(N * d);
    float* mo = bf.f(N * d);
    ASCA_REQUIRE(ctx, x && qkv && gate && y && mo, "model_forward_backward: out of memory");
    ASCA_TRY(asca_embed_fwd(ctx, P + m->embed, ids, N, d, x));
    const bool vec4 = (d & 3) == 0;
    const unsigned add_grid = (unsigned)std::min<int64_t>(ceil_div64(N * d / 4, 256), 148 * 16);
    bf16* next_x_in = nullptr;
    for (int64_t li = 0; li < L; ++li) {
        const Lyr& w = m->lay[li];
        const Lyr& w16 = m->lay16[li];
        Act& a = acts[li];
        a.x_in = li == 0 ? h16(N * d) : next_x_in; a.q = h16(N * d); a.k = h16(N * d); a.v = h16(N * d); a.o = h16(N * d); a.xn = h16(N * d);
        a.hid_p = h16(N * F);
        a.qn = bf.f(N * H); a.kn = bf.f(N * H); a.al = bf.f(N * H); a.be = bf.f(N * H);
        a.ckpt = bf.f(nck); a.x_mid = bf.f(N * d); a.pre_p = bf.f(N * F);
        ASCA_REQUIRE(ctx, a.x_in && a.q && a.k && a.v && a.o && a.xn && a.hid_p && a.qn && a.kn && a.al && a.be && a.ckpt &&
                              a.x_mid && a.pre_p, "model_forward_backward: out of memory");
        if (li == 0) ASCA_TRY(asca_cast_bf16(ctx, x, a.x_in, N * d));   // later blocks: written with the residual add below
        // qkv projection: where the CTA-pair product can take it, its epilogue adds the bias, L2-normalises q and k per
        // head and writes q, k, v as bf16 with the norms (the f32 qkv matrix and the prologue pass over it disappear)
        gemm_tc::Args tq{};
        tq.mode = ASCA_NN; tq.A = a.x_in; tq.lda = d; tq.a_rows = N; tq.a_cols = d;
        tq.B = W + w16.w_qkv; tq.ldb = 3 * d; tq.b_rows = d; tq.b_cols = 3 * d;
        tq.C = qkv; tq.ldc = 3 * d; tq.M = (int)N; tq.N = (int)(3 * d); tq.K = (int)d;
        tq.bias = P + w.b_qkv; tq.group_dim = gemm_tc::GROUP_NONE; tq.epi = gemm_tc::EPI_QKV;
        tq.qkv_q = a.q; tq.qkv_k = a.k; tq.qkv_v = a.v; tq.qkv_qn = a.qn; tq.qkv_kn = a.kn; tq.qkv_d = (int)d;
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, 2 * H, d, a.x_in, d, W + w16.w_gate, 2 * H, gate, 2 * H, P + w.b_gate, 0, BF));
        if (m->fused_qkv && dh == 128 && asca_tc_enabled() && gemm_tc::qkv_fusable(ctx, tq)) {
            ASCA_TRY(gemm_tc::launch(ctx, tq));
            gate_sigmoid_kernel<<<(unsigned)std::min<int64_t>(ceil_div64(N * H, 256), 148 * 8), 256, 0, ctx->stream>>>(gate, N * H, (int)H, a.al, a.be);
            ASCA_CHECK_LAUNCH(ctx);
        } else {
            ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, 3 * d, d, a.x_in, d, W + w16.w_qkv, 3 * d, qkv, 3 * d, P + w.b_qkv, 0, BF));
            ASCA_TRY(asca_delta_prep_bf16(ctx, qkv, gate, N, H, dh, a.q, a.k, a.v, a.qn, a.kn, a.al, a.be));
        }
        ASCA_TRY(asca_delta_fwd(ctx, a.q, a.k, a.v, a.al, a.be, B, T, H, dh, CH, BF, a.o, nullptr, nullptr, a.ckpt));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, d, d, a.o, d, W + w16.w_o, d, y, d, P + w.b_o, 0, BF));
        ASCA_TRY(asca_residual_rmsnorm_bf16(ctx, x, y, a.x_mid, a.xn, N, d, 1e-6f));
        ASCA_TRY(asca_dp_before_expert_weights(ctx, m, li));
        ASCA_TRY(asca_moe_fwd(ctx, a.xn, W + w16.w1, P + w.b1, W + w16.w2, P + w.b2, perm, offs, N, d, F, E, BF, mo, a.pre_p,
                              a.hid_p));
        if (li + 1 < L && vec4) {   // x_out = x_mid + moe, with the bf16 copy the next block's products read
            next_x_in = h16(N * d);
            ASCA_REQUIRE(ctx, next_x_in, "model_forward_backward: out of memory");
            add_cast4_kernel<<<add_grid, 256, 0, ctx->stream>>>(a.x_mid, mo, x, next_x_in, N * d / 4);
            ASCA_CHECK_LAUNCH(ctx);
        } else {
            ASCA_TRY(asca_residual_rmsnorm(ctx, a.x_mid, mo, x, nullptr, N, d, 1e-6f));
            if (li + 1 < L) {
                next_x_in = h16(N * d);
                ASCA_REQUIRE(ctx, next_x_in, "model_forward_backward: out of memory");
                ASCA_TRY(asca_cast_bf16(ctx, x, next_x_in, N * d));
            }
        }
    }
    bf16* h_final = h16(N * d);
    float* logits = bf.f(N * V);
    float* dlogits = bf.f(N * V);
    bf16* dl16 = h16(N * V);
    float* loss_d = bf.f(1);
    ASCA_REQUIRE(ctx, h_final && logits && dlogits && dl16 && loss_d, "model_forward_backward: out of memory");
    ASCA_TRY(asca_residual_rmsnorm_bf16(ctx, x, nullptr, nullptr, h_final, N, d, 1e-6f));
    // head + cross-entropy: fused into the head product's epilogue where it can be (the logits then never reach HBM)
    gemm_tc::Args th{};
    th.mode = ASCA_NN; th.A = h_final; th.lda = d; th.a_rows = N; th.a_cols = d;
    th.B = W + m->head16; th.ldb = V; th.b_rows = d; th.b_cols = V;
    th.C = logits; th.ldc = V; th.M = (int)N; th.N = (int)V; th.K = (int)d;
    th.group_dim = gemm_tc::GROUP_NONE; th.epi = gemm_tc::EPI_CE;
    th.C2 = dl16; th.ldc2 = V; th.ce_targets = tg; th.ce_loss = dlogits /* N floats of it hold the per-row losses */;
    th.ce_scale = m->grad_scale / (float)N;
    if (m->fused_head && !logits_h && asca_tc_enabled() && gemm_tc::ce_fusable(ctx, th)) {
        ASCA_TRY(gemm_tc::launch(ctx, th));
        mean_kernel<<<1, 1024, 0, ctx->stream>>>(dlogits, N, 1.0f / (float)N, loss_d);
        ASCA_CHECK_LAUNCH(ctx);
        ASCA_CUDA(ctx, cudaMemcpyAsync(loss_h, loss_d, 4, cudaMemcpyDeviceToHost, ctx->stream));
    } else {
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, V, d, h_final, d, W + m->head16, V, logits, V, nullptr, 0, BF));
        if (logits_h) ASCA_CUDA(ctx, cudaMemcpyAsync(logits_h, logits, (size_t)N * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
        ASCA_TRY(cross_entropy_scaled(ctx, logits, tg, N, V, dlogits, loss_d, m->grad_scale));
        ASCA_CUDA(ctx, cudaMemcpyAsync(loss_h, loss_d, 4, cudaMemcpyDeviceToHost, ctx->stream));
        ASCA_TRY(asca_cast_bf16(ctx, dlogits, dl16, N * V));
    }
    ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, V, N, h_final, d, dl16, V, G + m->head, V, nullptr, acc, BF));
    float* dh_ = bf.f(N * d);
    float* dx = bf.f(N * d);
    float* dxn = bf.f(N * d);
    float* d_moe = bf.f(N * d);
    float* d_o = bf.f(N * d);
    float* d_qkv = bf.f(N * 3 * d);
    float* d_gate = bf.f(N * 2 * H);
    bf16* dx16 = h16(N * d);
    bf16* do16 = h16(N * d);
    // d_qkv and d_gate side by side as bf16 (row pitch ldq) when that needs no padding: their input gradient is then one
    // product with the concatenated projection instead of two passes over dx
    const int64_t ldq = 3 * d + 2 * H;
    const bool cat = (ldq & 7) == 0 && (d & 3) == 0 && ((2 * H) & 3) == 0;
    if (cat) ASCA_TRY(refresh_dec_w(ctx, m));
    bf16* dqkv16 = cat ? h16(N * ldq) : h16(N * 3 * d);
    bf16* dg16 = cat ? dqkv16 + 3 * d : h16(N * 2 * H);
    const int64_t ld_dq = cat ? ldq : 3 * d, ld_dg = cat ? ldq : 2 * H;
    ASCA_REQUIRE(ctx, dh_ && dx && dxn && d_moe && d_o && d_qkv && d_gate && dx16 && do16 && dqkv16 && dg16,
                 "model_forward_backward: out of memory");
    ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, V, dl16, V, W + m->head16, V, dh_, d, nullptr, 0, BF));
    ASCA_TRY(asca_rmsnorm_bwd(ctx, x, dh_, dx, N, d, 1e-6f));
    const int64_t blocks_nd = ceil_div64(N * d, 256);
    for (int64_t li = L - 1; li >= 0; --li) {
        const Lyr& w = m->lay[li];
        const Lyr& w16 = m->lay16[li];
        Act& a = acts[li];
        ASCA_TRY((acc ? asca_moe_bwd_acc : asca_moe_bwd)(ctx, a.xn, W + w16.w1, W + w16.w2, a.pre_p, a.hid_p, dx, perm, offs, N, d, F, E, BF, G + w.w1,
                                  G + w.b1, G + w.w2, G + w.b2, dxn));
        ASCA_TRY(grad_ready(ctx, m, w.w1, (li + 1 < L ? m->lay[li + 1].w_qkv : m->n_params) - w.w1));   // the block's experts
        // d_mid = dx + rmsnorm_bwd(x_mid, dxn), with its bf16 copy: one pass where the rows fit the warp kernel
        const int rc_join = asca_rmsnorm_bwd_add_cast(ctx, a.x_mid, dxn, dx, dx, dx16, N, d, 1e-6f);
        if (rc_join != ASCA_ERR_UNSUPPORTED) {
            ASCA_TRY(rc_join);
        } else if (vec4) {
            ASCA_TRY(asca_rmsnorm_bwd(ctx, a.x_mid, dxn, d_moe, N, d, 1e-6f));
            add_cast4_kernel<<<add_grid, 256, 0, ctx->stream>>>(dx, d_moe, dx, dx16, N * d / 4);
            ASCA_CHECK_LAUNCH(ctx);
        } else {
            ASCA_TRY(asca_rmsnorm_bwd(ctx, a.x_mid, dxn, d_moe, N, d, 1e-6f));
            add_kernel<<<(unsigned)blocks_nd, 256, 0, ctx->stream>>>(dx, d_moe, dx, N * d);
            ctx->launches++;
            ASCA_TRY(asca_cast_bf16(ctx, dx, dx16, N * d));
        }
        {   // d_o = d_mid Wo^T, wanted as bf16 only (the delta backward's input)
            gemm_tc::Args t{};
            t.mode = ASCA_NT; t.A = dx16; t.lda = d; t.a_rows = N; t.a_cols = d;
            t.B = W + w16.w_o; t.ldb = d; t.b_rows = d; t.b_cols = d;
            t.C = d_o; t.ldc = d; t.M = (int)N; t.N = (int)d; t.K = (int)d;
            t.group_dim = gemm_tc::GROUP_NONE; t.epi = gemm_tc::EPI_NONE;
            t.C2 = do16; t.ldc2 = d; t.c2_only = 1;
            if (asca_tc_enabled() && gemm_tc::supported(t)) {
                ASCA_TRY(gemm_tc::launch(ctx, t));
            } else {
                ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, d, dx16, d, W + w16.w_o, d, d_o, d, nullptr, 0, BF));
                ASCA_TRY(asca_cast_bf16(ctx, d_o, do16, N * d));
            }
        }
        ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, d, N, a.o, d, dx16, d, G + w.w_o, d, nullptr, acc, BF));
        ASCA_TRY(asca_colsum(ctx, dx, d, N, d, G + w.b_o, acc));
        ASCA_TRY(asca_delta_bwd(ctx, a.q, a.k, a.v, a.al, a.be, a.qn, a.kn, do16, a.ckpt, B, T, H, dh, CH, BF, d_qkv, d_gate));
        bool bqkv_done = false;   // the d_qkv bias gradient was taken in the cast pass
        if (cat) {
            {   // bf16 copy of d_qkv and its column sums (the b_qkv gradient) in one pass over the 3 d wide f32 matrix
                const int64_t cols = 3 * d, col_blocks = ceil_div64(cols, 1024);
                int64_t n_slabs = std::max<int64_t>(1, std::min<int64_t>(ceil_div64(148 * 8, col_blocks), ceil_div64(N, 64)));
                const int64_t rps = ceil_div64(N, n_slabs);
                n_slabs = ceil_div64(N, rps);
                void* part;
                ASCA_TRY(asca_malloc(ctx, (size_t)n_slabs * cols * 4 + 256, &part));
                cast_colsum_kernel<<<dim3((unsigned)col_blocks, (unsigned)n_slabs), 256, 0, ctx->stream>>>(d_qkv, (int)cols, N, rps, dqkv16, ldq,
                                                                                                         (float*)part);
                colsum_finish_kernel<<<(unsigned)ceil_div64(cols, 256), 256, 0, ctx->stream>>>((const float*)part, (int)n_slabs, (int)cols,
                                                                                              G + w.b_qkv, acc);
                const cudaError_t le = cudaGetLastError();
                asca_free(ctx, part);
                ASCA_CUDA(ctx, le);
                ctx->launches += 2;
                bqkv_done = true;
            }
            cast_cols_kernel<<<(unsigned)std::min<int64_t>(ceil_div64(N * 2 * H / 4, 256), 148 * 16), 256, 0, ctx->stream>>>(
                d_gate, (int)(2 * H / 4), N * 2 * H / 4, dg16, ldq);
            ctx->launches += 1;
            ASCA_CUDA(ctx, cudaGetLastError());
        } else {
            ASCA_TRY(asca_cast_bf16(ctx, d_qkv, dqkv16, N * 3 * d));
            ASCA_TRY(asca_cast_bf16(ctx, d_gate, dg16, N * 2 * H));
        }
        ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, 3 * d, N, a.x_in, d, dqkv16, ld_dq, G + w.w_qkv, 3 * d, nullptr, acc, BF));
        if (!bqkv_done) ASCA_TRY(asca_colsum(ctx, d_qkv, 3 * d, N, 3 * d, G + w.b_qkv, acc));
        ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, 2 * H, N, a.x_in, d, dg16, ld_dg, G + w.w_gate, 2 * H, nullptr, acc, BF));
        ASCA_TRY(asca_colsum(ctx, d_gate, 2 * H, N, 2 * H, G + w.b_gate, acc));
        if (cat) {   // dx += [d_qkv | d_gate] [W_qkv | W_gate]^T
            ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, ldq, dqkv16, ldq, m->dec_w + li * d * ldq, ldq, dx, d, nullptr, 1, BF));
        } else {
            ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, 3 * d, dqkv16, 3 * d, W + w16.w_qkv, 3 * d, dx, d, nullptr, 1, BF));
            ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, 2 * H, dg16, 2 * H, W + w16.w_gate, 2 * H, dx, d, nullptr, 1, BF));
        }
        ASCA_TRY(grad_ready(ctx, m, w.w_qkv, w.w1 - w.w_qkv));   // the block's projections
    }
    if (!acc) ASCA_CUDA(ctx, cudaMemsetAsync(G + m->embed, 0, (size_t)V * d * 4, ctx->stream));
    ASCA_TRY(asca_embed_bwd(ctx, dx, ids, N, d, V, G + m->embed));
    ASCA_TRY(grad_ready(ctx, m, 0, m->lay[0].w_qkv));   // embedding + head
    ASCA_CUDA(ctx, cudaGetLastError());
    return asca_ctx_sync(ctx);
}

extern "C" {

int asca_colsum(asca_ctx* ctx, const float* src, int64_t ld, int64_t rows, int64_t cols, float* out, int accumulate) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, src && out && rows >= 0 && cols > 0 && ld >= cols, "colsum: bad arguments");
    if (rows == 0) {
        if (!accumulate) ASCA_CUDA(ctx, cudaMemsetAsync(out, 0, (size_t)cols * 4, ctx->stream));
        return ASCA_OK;
    }
    // enough row slices to fill the GPU, at least 256 rows each
    const int64_t col_blocks = ceil_div64(cols, 32);
    int64_t n_slices = ceil_div64(148 * 8, col_blocks);
    if (n_slices > ceil_div64(rows, 256)) n_slices = ceil_div64(rows, 256);
    if (n_slices < 1) n_slices = 1;
    const int64_t rps = ceil_div64(rows, n_slices);
    n_slices = ceil_div64(rows, rps);
    // partial sums from the block pool, not the context's scratch area: callers (the expert-FFN backward) may
    // be holding that; the block goes back to the pool at once and is reused only by later work on the stream
    void* ws;
    ASCA_TRY(asca_malloc(ctx, (size_t)n_slices * cols * 4 + 256, &ws));
    colsum_slices_kernel<<<dim3((unsigned)col_blocks, (unsigned)n_slices), 256, 0, ctx->stream>>>(src, ld, rows, (int)cols, rps,
                                                                                               (float*)ws);
    ctx->launches++;
    colsum_finish_kernel<<<(unsigned)ceil_div64(cols, 256), 256, 0, ctx->stream>>>((const float*)ws, (int)n_slices, (int)cols, out,
                                                                                  accumulate);
    const cudaError_t le = cudaGetLastError();
    asca_free(ctx, ws);
    ASCA_CUDA(ctx, le);
    ctx->launches++;
    return ASCA_OK;
}

int asca_cross_entropy(asca_ctx* ctx, const float* logits, const uint32_t* targets, int64_t N, int64_t V,
                       float* dlogits, float* loss) {
    return cross_entropy_scaled(ctx, logits, targets, N, V, dlogits, loss, 1.0f);
}

// grad_scale multiplies dlogits only (1 / micro-batches under gradient accumulation); the loss stays the token mean
static int cross_entropy_scaled(asca_ctx* ctx, const float* logits, const uint32_t* targets, int64_t N, int64_t V,
                                float* dlogits, float* loss, float grad_scale) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, logits && targets && loss && N > 0 && V > 0, "cross_entropy: bad arguments");
    void* ws;
    ASCA_TRY(asca_workspace(ctx, (size_t)N * 4 + 256, &ws));
    cross_entropy_kernel<<<(unsigned)ceil_div64(N, 8), 256, 0, ctx->stream>>>(logits, targets, N, (int)V, dlogits,
                                                                              (float*)ws, grad_scale / (float)N);
    ASCA_CHECK_LAUNCH(ctx);
    mean_kernel<<<1, 1024, 0, ctx->stream>>>((const float*)ws, N, 1.0f / (float)N, loss);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_embed_fwd(asca_ctx* ctx, const float* table, const uint32_t* ids, int64_t N, int64_t d, float* x) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, table && ids && x && N >= 0 && d > 0, "embed_fwd: bad arguments");
    if (N == 0) return ASCA_OK;
    embed_fwd_kernel<<<(unsigned)ceil_div64(N, 8), 256, 0, ctx->stream>>>(table, ids, N, (int)d, x);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_embed_bwd(asca_ctx* ctx, const float* dx, const uint32_t* ids, int64_t N, int64_t d, int64_t vocab,
                   float* d_table) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dx && ids && d_table && N >= 0 && d > 0 && vocab > 0 && vocab < 65536, "embed_bwd: bad arguments");
    if (N == 0) return ASCA_OK;
    if ((d & 3) == 0 && (reinterpret_cast<uintptr_t>(dx) & 15) == 0)
        embed_bwd_ballot_kernel<<<dim3((unsigned)vocab, (unsigned)ceil_div64(d, 256)), 256, 0, ctx->stream>>>(dx, ids, N, (int)d, d_table);
    else
        embed_bwd_kernel<<<dim3((unsigned)vocab, (unsigned)ceil_div64(d, 128)), 128, 0, ctx->stream>>>(dx, ids, N, (int)d, d_table);
    ASCA_CHECK_LAUNCH(ctx);
    return ASCA_OK;
}

int asca_model_create(asca_ctx* ctx, int64_t vocab, int64_t d, int64_t H, int64_t L, int64_t E, int64_t F,
                      asca_model** out) {
    if (!ctx || !out) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, vocab > 0 && d > 0 && H > 0 && L > 0 && E > 0 && F > 0 && d % H == 0, "model_create: bad config");
    const int64_t dh = d / H;
    if (dh != 16 && dh != 32 && dh != 64 && dh != 128)
        return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "model_create: d/H must be 16, 32, 64 or 128");
    asca_model* m = new asca_model();
    m->vocab = vocab; m->d = d; m->H = H; m->L = L; m->E = E; m->F = F;
    int64_t o = 0, o16 = 0;
    auto take = [&](int64_t n, int64_t* at16) {
        const int64_t at = o;
        m->seg_off.push_back(at);
        m->seg16.push_back(o16);
        *at16 = o16;
        o += n;
        o16 += (n + 7) & ~(int64_t)7;
        return at;
    };
    m->embed = take(vocab * d, &m->embed16);
    m->head = take(d * vocab, &m->head16);
    for (int64_t i = 0; i < L; ++i) {
        Lyr y, z;
        y.w_qkv = take(d * 3 * d, &z.w_qkv); y.b_qkv = take(3 * d, &z.b_qkv);
        y.w_gate = take(d * 2 * H, &z.w_gate); y.b_gate = take(2 * H, &z.b_gate);
        y.w_o = take(d * d, &z.w_o); y.b_o = take(d, &z.b_o);
        y.w1 = take(d * E * F, &z.w1); y.b1 = take(E * F, &z.b1);
        y.w2 = take(E * F * d, &z.w2); y.b2 = take(d, &z.b2);
        m->lay.push_back(y);
        m->lay16.push_back(z);
    }
    m->seg_off.push_back(o);
    m->n_params = o;
    m->n16 = o16;
    float** bufs[4] = {&m->params, &m->grads, &m->m, &m->v};
    for (auto b : bufs) {
        if (cudaMalloc((void**)b, (size_t)o * 4) != cudaSuccess) {
            asca_model_destroy(ctx, m);
            return asca_fail(ctx, ASCA_ERR_OOM, "model_create: cannot allocate %lld parameters", (long long)o);
        }
        cudaMemsetAsync(*b, 0, (size_t)o * 4, ctx->stream);
    }
    *out = m;
    return ASCA_OK;
}

int asca_model_destroy(asca_ctx* ctx, asca_model* m) {
    if (!m) return ASCA_OK;
    if (ctx) cudaStreamSynchronize(ctx->stream);
    if (m->dp) asca_dp_free(m);   // before the buffers its copies and collectives touch
    for (float* b : {m->params, m->grads, m->m, m->v})
        if (b) cudaFree(b);
    if (m->params16) cudaFree(m->params16);
    if (m->dec_w) cudaFree(m->dec_w);
    if (m->dec_b) cudaFree(m->dec_b);
    if (m->dec_pk) cudaFree(m->dec_pk);
    delete m;
    return ASCA_OK;
}

int64_t asca_model_num_params(const asca_model* m) { return m ? m->n_params : 0; }

int asca_model_buffers(asca_model* m, float** params, float** grads, float** adam_m, float** adam_v) {
    if (!m) return ASCA_ERR_ARG;
    if (params) *params = m->params;
    if (grads) {
        materialize_zero_grads(nullptr, m);
        *grads = m->grads;
    }
    if (adam_m) *adam_m = m->m;
    if (adam_v) *adam_v = m->v;
    return ASCA_OK;
}

int asca_model_set_compute(asca_ctx* ctx, asca_model* m, int dtype) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, dtype == ASCA_F32 || dtype == ASCA_BF16, "model_set_compute: unknown dtype %d", dtype);
    m->compute = dtype;
    return ASCA_OK;
}

int asca_model_set_fused_head(asca_model* m, int on) {
    if (!m) return ASCA_ERR_ARG;
    m->fused_head = on != 0;
    return ASCA_OK;
}

int asca_model_set_fused_qkv(asca_model* m, int on) {
    if (!m) return ASCA_ERR_ARG;
    m->fused_qkv = on != 0;
    return ASCA_OK;
}

int asca_model_set_grad_scale(asca_model* m, float scale) {
    if (!m) return ASCA_ERR_ARG;
    m->grad_scale = scale;
    return ASCA_OK;
}

int asca_model_set_grad_hook(asca_model* m, asca_grad_ready_fn fn, void* user) {
    if (!m) return ASCA_ERR_ARG;
    m->grad_hook = fn;
    m->grad_hook_user = user;
    return ASCA_OK;
}

int asca_model_adam_counter(asca_model* m, const uint32_t* set, uint32_t* get) {
    if (!m) return ASCA_ERR_ARG;
    if (set) m->adam_counter = *set;
    if (get) *get = m->adam_counter;
    return ASCA_OK;
}

int asca_model_params_changed(asca_model* m) {
    if (!m) return ASCA_ERR_ARG;
    m->params16_stale = true;
    m->dec_stale = true;
    m->dec_pk_stale = true;
    return ASCA_OK;
}

int asca_model_set_params_host(asca_ctx* ctx, asca_model* m, const float* params) {
    if (!ctx || !m || !params) return ASCA_ERR_ARG;
    m->adam_counter = 0;
    m->master_stale = false;
    ASCA_TRY(asca_dp_wait_all(ctx, m));
    ASCA_CUDA(ctx, cudaMemsetAsync(m->m, 0, (size_t)m->n_params * 4, ctx->stream));
    ASCA_CUDA(ctx, cudaMemsetAsync(m->v, 0, (size_t)m->n_params * 4, ctx->stream));
    m->params16_stale = true;
    m->dec_stale = true;
    m->dec_pk_stale = true;
    return asca_memcpy_h2d(ctx, m->params, params, (size_t)m->n_params * 4);
}

int asca_model_get_host(asca_ctx* ctx, asca_model* m, float* params, float* grads) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, !(params && m->master_stale),
                 "model_get: after a sharded optimizer step the master weights of other ranks' chunks are stale on this "
                 "rank; call asca_model_dp_gather_master first");
    if (params) ASCA_TRY(asca_memcpy_d2h(ctx, params, m->params, (size_t)m->n_params * 4));
    if (grads) {
        ASCA_TRY(materialize_zero_grads(ctx, m));
        ASCA_TRY(asca_memcpy_d2h(ctx, grads, m->grads, (size_t)m->n_params * 4));
    }
    return ASCA_OK;
}

int asca_model_zero_grads(asca_ctx* ctx, asca_model* m) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    m->grads_zero_pending = true;
    return ASCA_OK;
}


int asca_model_forward_backward_host(asca_ctx* ctx, asca_model* m, const uint32_t* ids_h, const uint32_t* tg_h,
                                     int64_t B, int64_t T, float* loss_h, float* logits_h) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, ids_h && tg_h && loss_h && B > 0 && T > 0, "model_forward_backward: bad arguments");
    const int64_t N = B * T, d = m->d, H = m->H, dh = d / H, E = m->E, F = m->F, V = m->vocab, L = m->L;
    const int64_t CH = 64;
    for (int64_t i = 0; i < N; ++i)
        ASCA_REQUIRE(ctx, ids_h[i] < (uint32_t)V && tg_h[i] < (uint32_t)V, "model_forward_backward: id out of range");
    if (m->compute == ASCA_BF16) return forward_backward_bf16(ctx, m, ids_h, tg_h, B, T, loss_h, logits_h);
    float* P = m->params;
    float* G = m->grads;
    const int acc = m->grads_zero_pending ? 0 : 1;   // first backward after zero_grads: overwrite
    m->grads_zero_pending = false;
    Bufs bf(ctx);
    uint32_t* ids = (uint32_t*)bf.f(N);
    uint32_t* tg = (uint32_t*)bf.f(N);
    int32_t* perm = (int32_t*)bf.f(N);
    int32_t* offs = (int32_t*)bf.f(E + 1);
    ASCA_REQUIRE(ctx, ids && tg && perm && offs, "model_forward_backward: out of memory");
    ASCA_CUDA(ctx, cudaMemcpyAsync(ids, ids_h, (size_t)N * 4, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_CUDA(ctx, cudaMemcpyAsync(tg, tg_h, (size_t)N * 4, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_TRY(asca_moe_dispatch(ctx, ids, N, E, perm, offs, nullptr));   // same routing for every layer

    struct Act {
        float *x_in, *q, *k, *v, *qn, *kn, *al, *be, *o, *ckpt, *x_mid, *xn, *pre_p, *hid_p;
    };
    std::vector<Act> acts(L);
    const int64_t nck = asca_delta_ckpt_floats(B, T, H, dh, CH);
    float* x = bf.f(N * d);
    float* qkv = bf.f(N * 3 * d);
    float* gate = bf.f(N * 2 * H);
    float* y = bf.f(N * d);
    float* mo = bf.f(N * d);
    ASCA_REQUIRE(ctx, x && qkv && gate && y && mo, "model_forward_backward: out of memory");
    ASCA_TRY(asca_embed_fwd(ctx, P + m->embed, ids, N, d, x));
    // ---- forward (rust/src/model.rs:651-700)
    for (int64_t li = 0; li < L; ++li) {
        const Lyr& w = m->lay[li];
        Act& a = acts[li];
        a.x_in = bf.f(N * d); a.q = bf.f(N * d); a.k = bf.f(N * d); a.v = bf.f(N * d);
        a.qn = bf.f(N * H); a.kn = bf.f(N * H); a.al = bf.f(N * H); a.be = bf.f(N * H);
        a.o = bf.f(N * d); a.ckpt = bf.f(nck); a.x_mid = bf.f(N * d); a.xn = bf.f(N * d);
        a.pre_p = bf.f(N * F); a.hid_p = bf.f(N * F);
        ASCA_REQUIRE(ctx, a.x_in && a.q && a.k && a.v && a.qn && a.kn && a.al && a.be && a.o && a.ckpt && a.x_mid && a.xn &&
                              a.pre_p && a.hid_p, "model_forward_backward: out of memory");
        ASCA_CUDA(ctx, cudaMemcpyAsync(a.x_in, x, (size_t)N * d * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, 3 * d, d, x, d, P + w.w_qkv, 3 * d, qkv, 3 * d, P + w.b_qkv, 0, ASCA_F32));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, 2 * H, d, x, d, P + w.w_gate, 2 * H, gate, 2 * H, P + w.b_gate, 0, ASCA_F32));
        ASCA_TRY(asca_delta_prep(ctx, qkv, gate, N, H, dh, a.q, a.k, a.v, a.qn, a.kn, a.al, a.be));
        ASCA_TRY(asca_delta_fwd(ctx, a.q, a.k, a.v, a.al, a.be, B, T, H, dh, CH, ASCA_F32, a.o, nullptr, nullptr, a.ckpt));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, d, d, a.o, d, P + w.w_o, d, y, d, P + w.b_o, 0, ASCA_F32));
        ASCA_TRY(asca_residual_rmsnorm(ctx, x, y, a.x_mid, a.xn, N, d, 1e-6f));
        ASCA_TRY(asca_moe_fwd(ctx, a.xn, P + w.w1, P + w.b1, P + w.w2, P + w.b2, perm, offs, N, d, F, E, ASCA_F32, mo,
                              a.pre_p, a.hid_p));
        ASCA_TRY(asca_residual_rmsnorm(ctx, a.x_mid, mo, x, nullptr, N, d, 1e-6f));   // x_out
    }
    float* h_final = bf.f(N * d);
    float* logits = bf.f(N * V);
    float* dlogits = bf.f(N * V);
    float* loss_d = bf.f(1);
    ASCA_REQUIRE(ctx, h_final && logits && dlogits && loss_d, "model_forward_backward: out of memory");
    ASCA_TRY(asca_rmsnorm_fwd(ctx, x, h_final, nullptr, N, d, 1e-6f));
    ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, V, d, h_final, d, P + m->head, V, logits, V, nullptr, 0, ASCA_F32));
    if (logits_h) ASCA_CUDA(ctx, cudaMemcpyAsync(logits_h, logits, (size_t)N * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
    // ---- backward (rust/src/model.rs:744-794)
    ASCA_TRY(cross_entropy_scaled(ctx, logits, tg, N, V, dlogits, loss_d, m->grad_scale));
    ASCA_CUDA(ctx, cudaMemcpyAsync(loss_h, loss_d, 4, cudaMemcpyDeviceToHost, ctx->stream));
    ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, V, N, h_final, d, dlogits, V, G + m->head, V, nullptr, acc, ASCA_F32));
    float* dh_ = bf.f(N * d);
    float* dx = bf.f(N * d);
    float* dxn = bf.f(N * d);
    float* d_moe = bf.f(N * d);
    float* d_o = bf.f(N * d);
    float* d_qkv = bf.f(N * 3 * d);
    float* d_gate = bf.f(N * 2 * H);
    ASCA_REQUIRE(ctx, dh_ && dx && dxn && d_moe && d_o && d_qkv && d_gate, "model_forward_backward: out of memory");
    ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, V, dlogits, V, P + m->head, V, dh_, d, nullptr, 0, ASCA_F32));
    ASCA_TRY(asca_rmsnorm_bwd(ctx, x, dh_, dx, N, d, 1e-6f));   // x = x_out of the last layer
    const int64_t blocks_nd = ceil_div64(N * d, 256);
    for (int64_t li = L - 1; li >= 0; --li) {
        const Lyr& w = m->lay[li];
        Act& a = acts[li];
        // HashMoe::backward: gradients accumulate into the flat buffer
        ASCA_TRY((acc ? asca_moe_bwd_acc : asca_moe_bwd)(ctx, a.xn, P + w.w1, P + w.w2, a.pre_p, a.hid_p, dx, perm, offs, N, d, F, E, ASCA_F32,
                                  G + w.w1, G + w.b1, G + w.w2, G + w.b2, dxn));
        ASCA_TRY(grad_ready(ctx, m, w.w1, (li + 1 < L ? m->lay[li + 1].w_qkv : m->n_params) - w.w1));   // the block's experts
        ASCA_TRY(asca_rmsnorm_bwd(ctx, a.x_mid, dxn, d_moe, N, d, 1e-6f));
        add_kernel<<<(unsigned)blocks_nd, 256, 0, ctx->stream>>>(dx, d_moe, dx, N * d);   // d_mid
        ctx->launches++;
        // DeltaBlock::backward (rust/src/delta.rs:615-674)
        ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, d, dx, d, P + w.w_o, d, d_o, d, nullptr, 0, ASCA_F32));
        ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, d, N, a.o, d, dx, d, G + w.w_o, d, nullptr, acc, ASCA_F32));
        ASCA_TRY(asca_colsum(ctx, dx, d, N, d, G + w.b_o, acc));
        ASCA_TRY(asca_delta_bwd(ctx, a.q, a.k, a.v, a.al, a.be, a.qn, a.kn, d_o, a.ckpt, B, T, H, dh, CH, ASCA_F32, d_qkv,
                                d_gate));
        ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, 3 * d, N, a.x_in, d, d_qkv, 3 * d, G + w.w_qkv, 3 * d, nullptr, acc, ASCA_F32));
        ASCA_TRY(asca_colsum(ctx, d_qkv, 3 * d, N, 3 * d, G + w.b_qkv, acc));
        ASCA_TRY(asca_gemm(ctx, ASCA_TN, d, 2 * H, N, a.x_in, d, d_gate, 2 * H, G + w.w_gate, 2 * H, nullptr, acc, ASCA_F32));
        ASCA_TRY(asca_colsum(ctx, d_gate, 2 * H, N, 2 * H, G + w.b_gate, acc));
        // dx = d_mid + d_qkv Wqkv^T + d_gate Wg^T   (accumulate onto d_mid in place)
        ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, 3 * d, d_qkv, 3 * d, P + w.w_qkv, 3 * d, dx, d, nullptr, 1, ASCA_F32));
        ASCA_TRY(asca_gemm(ctx, ASCA_NT, N, d, 2 * H, d_gate, 2 * H, P + w.w_gate, 2 * H, dx, d, nullptr, 1, ASCA_F32));
        ASCA_TRY(grad_ready(ctx, m, w.w_qkv, w.w1 - w.w_qkv));   // the block's projections
    }
    if (!acc) ASCA_CUDA(ctx, cudaMemsetAsync(G + m->embed, 0, (size_t)V * d * 4, ctx->stream));
    ASCA_TRY(asca_embed_bwd(ctx, dx, ids, N, d, V, G + m->embed));
    ASCA_TRY(grad_ready(ctx, m, 0, m->lay[0].w_qkv));   // embedding + head
    ASCA_CUDA(ctx, cudaGetLastError());
    return asca_ctx_sync(ctx);
}

int asca_model_adamw_step(asca_ctx* ctx, asca_model* m, float lr, float beta1, float beta2, float eps, float wd) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_TRY(materialize_zero_grads(ctx, m));
    const int n_seg = (int)m->seg_off.size() - 1;
    std::vector<float> lr_t(n_seg), eps_t(n_seg);
    auto powi = [](float b, int e) {   // f32 exponentiation by squaring, as `f32::powi` lowers
        float r = 1.0f, x = b;
        while (e > 0) {
            if (e & 1) r *= x;
            x *= x;
            e >>= 1;
        }
        return r;
    };
    for (int i = 0; i < n_seg; ++i) {
        m->adam_counter += 1;   // once per tensor (rust/src/tensor.rs:393)
        const float bc1 = 1.0f - powi(beta1, (int)m->adam_counter), bc2 = 1.0f - powi(beta2, (int)m->adam_counter);
        lr_t[i] = lr * sqrtf(bc1 / bc2);
        eps_t[i] = eps * sqrtf(bc2);
    }
    // bf16 mode with an unpadded copy: the update writes the bf16 weights itself
    const bool fuse = m->compute == ASCA_BF16 && m->params16 && m->n16 == m->n_params;
    m->params16_stale = !fuse;
    m->dec_stale = true;
    m->dec_pk_stale = true;
    return asca_adamw_segmented_cast(ctx, m->params, m->grads, m->m, m->v, m->seg_off.data(), lr_t.data(), eps_t.data(), n_seg,
                                     beta1, beta2, lr * wd, fuse ? (void*)m->params16 : nullptr);
}

// One optimizer step restricted to n sorted, disjoint slices [lo[i], hi[i]) of the flat buffer (a rank's share under a
// sharded optimizer: its parts of the large tensors, and whatever small tensors every rank updates). Every tensor gets
// the step number asca_model_adamw_step would give it; the counter advances as for a full step when `advance` is set
// (a step may be issued as several calls, the last one advancing). bf16 mode with an
// unpadded bf16 copy only (the update writes that copy for the slices; the caller exchanges the rest).
int asca_model_adamw_slices(asca_ctx* ctx, asca_model* m, float lr, float beta1, float beta2, float eps, float wd, const int64_t* lo,
                            const int64_t* hi, int n, int advance) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, lo && hi && n > 0, "model_adamw_slices: bad arguments");
    ASCA_REQUIRE(ctx, m->compute == ASCA_BF16 && m->params16 && m->n16 == m->n_params,
                 "model_adamw_slices: needs bf16 compute mode with an unpadded bf16 weight copy");
    ASCA_TRY(materialize_zero_grads(ctx, m));
    ASCA_TRY(refresh_params16(ctx, m));
    const int n_seg = (int)m->seg_off.size() - 1;
    auto powi = [](float b, int e) {
        float r = 1.0f, x = b;
        while (e > 0) {
            if (e & 1) r *= x;
            x *= x;
            e >>= 1;
        }
        return r;
    };
    int64_t prev = 0;
    for (int s = 0; s < n; ++s) {
        ASCA_REQUIRE(ctx, lo[s] >= prev && hi[s] > lo[s] && hi[s] <= m->n_params && (lo[s] & 3) == 0,
                     "model_adamw_slices: slices must be sorted, disjoint, inside the buffer and start at multiples of 4");
        prev = hi[s];
        std::vector<int64_t> off{0};
        std::vector<float> lr_t, eps_t;
        for (int i = 0; i < n_seg; ++i) {
            const int64_t a = std::max(lo[s], m->seg_off[i]), b = std::min(hi[s], m->seg_off[i + 1]);
            if (a >= b) continue;
            const int t = (int)(m->adam_counter + (uint32_t)i + 1u);
            const float bc1 = 1.0f - powi(beta1, t), bc2 = 1.0f - powi(beta2, t);
            off.push_back(b - lo[s]);
            lr_t.push_back(lr * sqrtf(bc1 / bc2));
            eps_t.push_back(eps * sqrtf(bc2));
        }
        ASCA_TRY(asca_adamw_segmented_cast(ctx, m->params + lo[s], m->grads + lo[s], m->m + lo[s], m->v + lo[s], off.data(), lr_t.data(),
                                           eps_t.data(), (int)lr_t.size(), beta1, beta2, lr * wd, m->params16 + lo[s]));
    }
    if (advance) m->adam_counter += (uint32_t)n_seg;   // the last call of an optimizer step
    m->dec_stale = true;
    m->dec_pk_stale = true;
    return ASCA_OK;
}

// Device address of the bf16 weight copy (bf16 compute mode; same element offsets as the f32 buffer when unpadded).
int asca_model_params16(asca_ctx* ctx, asca_model* m, void** out, int64_t* n16) {
    if (!ctx || !m || !out) return ASCA_ERR_ARG;
    ASCA_TRY(refresh_params16(ctx, m));
    ASCA_TRY(asca_dp_wait_all(ctx, m));
    *out = m->params16;
    if (n16) *n16 = m->n16;
    return ASCA_OK;
}

// Chunked prefill: the forward of Model::forward (rust/src/model.rs:651-690) over n_streams prompts of T tokens at
// once, keeping only what a decoder needs -- the recurrent state after the last token, per block, head and stream,
// written into the decode state -- and the logits of each stream's last token. The reference prefills by stepping the
// decoder token by token (rust/src/main.rs:367-371); the result is the same state (stepping equals the full forward,
// rust/tests/decode_parity.rs), reached with T-token products and the chunked scan instead of T decode steps.
// The incoming `state` is the initial state (zeros for a fresh stream), so a prompt may be fed in several calls.
int asca_model_prefill_host(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids_h, int64_t ns, int64_t T,
                            float* logits_h, uint32_t* next_h) {
    typedef __nv_bfloat16 bf16;
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, state && ids_h && ns > 0 && T > 0, "model_prefill: bad arguments");
    const int64_t N = ns * T, d = m->d, H = m->H, dh = d / H, E = m->E, F = m->F, V = m->vocab, L = m->L;
    ASCA_REQUIRE(ctx, N < (1ll << 31), "model_prefill: too many tokens in one call");
    for (int64_t i = 0; i < N; ++i) ASCA_REQUIRE(ctx, ids_h[i] < (uint32_t)V, "model_prefill: id out of range");
    const bool bfm = m->compute == ASCA_BF16;
    const int DT = bfm ? ASCA_BF16 : ASCA_F32;
    if (bfm) {
        ASCA_TRY(refresh_params16(ctx, m));
        ASCA_TRY(asca_dp_wait_all(ctx, m));
    }
    const float* P = m->params;
    const bf16* W = m->params16;
    Bufs bf(ctx);
    auto h16 = [&](int64_t n) { return (bf16*)bf.f((n + 1) / 2); };
    uint32_t* ids = (uint32_t*)bf.f(N);
    int32_t* perm = (int32_t*)bf.f(N);
    int32_t* offs = (int32_t*)bf.f(E + 1);
    int32_t* last = (int32_t*)bf.f(ns);
    uint32_t* nxt = (uint32_t*)bf.f(ns);
    float *x = bf.f(N * d), *qkv = bf.f(N * 3 * d), *gate = bf.f(N * 2 * H), *y = bf.f(N * d), *x_mid = bf.f(N * d), *mo = bf.f(N * d);
    float *qn = bf.f(N * H), *kn = bf.f(N * H), *al = bf.f(N * H), *be = bf.f(N * H), *pre_p = bf.f(N * F);
    float* s_fin = bf.f(ns * H * dh * dh);
    float *xl = bf.f(ns * d), *hf = bf.f(ns * d), *logits = bf.f(ns * V);
    // activations a product reads: bf16 in bf16 mode, f32 otherwise (same element counts)
    auto act = [&](int64_t n) { return bfm ? (void*)h16(n) : (void*)bf.f(n); };
    void *x_in = bfm ? act(N * d) : nullptr, *q = act(N * d), *k = act(N * d), *v = act(N * d), *o = act(N * d), *xn = act(N * d),
         *hid_p = act(N * F), *hf_in = bfm ? act(ns * d) : nullptr;
    ASCA_REQUIRE(ctx, ids && perm && offs && last && nxt && x && qkv && gate && y && x_mid && mo && qn && kn && al && be && pre_p &&
                          s_fin && xl && hf && logits && q && k && v && o && xn && hid_p && (!bfm || (x_in && hf_in)),
                 "model_prefill: out of memory");
    ASCA_CUDA(ctx, cudaMemcpyAsync(ids, ids_h, (size_t)N * 4, cudaMemcpyHostToDevice, ctx->stream));
    {
        std::vector<int32_t> lh(ns);
        for (int64_t s_ = 0; s_ < ns; ++s_) lh[s_] = (int32_t)(s_ * T + T - 1);
        ASCA_CUDA(ctx, cudaMemcpyAsync(last, lh.data(), (size_t)ns * 4, cudaMemcpyHostToDevice, ctx->stream));
        ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // lh leaves scope
    }
    ASCA_TRY(asca_moe_dispatch(ctx, ids, N, E, perm, offs, nullptr));
    ASCA_TRY(asca_embed_fwd(ctx, P + m->embed, ids, N, d, x));
    const size_t st_layer = (size_t)ns * H * dh * dh;
    for (int64_t li = 0; li < L; ++li) {
        const Lyr& w = m->lay[li];
        const Lyr& w16 = m->lay16[li];
        const void* xi = x;
        if (bfm) {
            ASCA_TRY(asca_cast_bf16(ctx, x, x_in, N * d));
            xi = x_in;
        }
        const void *Wqkv = bfm ? (const void*)(W + w16.w_qkv) : (const void*)(P + w.w_qkv), *Wg = bfm ? (const void*)(W + w16.w_gate) : (const void*)(P + w.w_gate),
                   *Wo = bfm ? (const void*)(W + w16.w_o) : (const void*)(P + w.w_o), *W1 = bfm ? (const void*)(W + w16.w1) : (const void*)(P + w.w1),
                   *W2 = bfm ? (const void*)(W + w16.w2) : (const void*)(P + w.w2);
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, 3 * d, d, xi, d, Wqkv, 3 * d, qkv, 3 * d, P + w.b_qkv, 0, DT));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, 2 * H, d, xi, d, Wg, 2 * H, gate, 2 * H, P + w.b_gate, 0, DT));
        if (bfm) ASCA_TRY(asca_delta_prep_bf16(ctx, qkv, gate, N, H, dh, q, k, v, qn, kn, al, be));
        else ASCA_TRY(asca_delta_prep(ctx, qkv, gate, N, H, dh, (float*)q, (float*)k, (float*)v, qn, kn, al, be));
        float* st = state + (size_t)li * st_layer;
        ASCA_TRY(asca_delta_fwd(ctx, q, k, v, al, be, ns, T, H, dh, 64, DT, o, st, s_fin, nullptr));
        ASCA_CUDA(ctx, cudaMemcpyAsync(st, s_fin, st_layer * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, N, d, d, o, d, Wo, d, y, d, P + w.b_o, 0, DT));
        if (bfm) ASCA_TRY(asca_residual_rmsnorm_bf16(ctx, x, y, x_mid, xn, N, d, 1e-6f));
        else ASCA_TRY(asca_residual_rmsnorm(ctx, x, y, x_mid, (float*)xn, N, d, 1e-6f));
        ASCA_TRY(asca_moe_fwd(ctx, xn, W1, P + w.b1, W2, P + w.b2, perm, offs, N, d, F, E, DT, mo, pre_p, hid_p));
        ASCA_TRY(asca_residual_rmsnorm(ctx, x_mid, mo, x, nullptr, N, d, 1e-6f));
    }
    // the head on each stream's last token only
    ASCA_TRY(asca_gather_rows(ctx, x, last, ns, d, xl));
    if (bfm) {
        ASCA_TRY(asca_residual_rmsnorm_bf16(ctx, xl, nullptr, nullptr, hf_in, ns, d, 1e-6f));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, V, d, hf_in, d, W + m->head16, V, logits, V, nullptr, 0, DT));
    } else {
        ASCA_TRY(asca_rmsnorm_fwd(ctx, xl, hf, nullptr, ns, d, 1e-6f));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, V, d, hf, d, P + m->head, V, logits, V, nullptr, 0, DT));
    }
    if (logits_h) ASCA_CUDA(ctx, cudaMemcpyAsync(logits_h, logits, (size_t)ns * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (next_h) {
        argmax_kernel<<<(unsigned)ceil_div64(ns, 8), 256, 0, ctx->stream>>>(logits, ns, (int)V, nxt);
        ASCA_CHECK_LAUNCH(ctx);
        ASCA_CUDA(ctx, cudaMemcpyAsync(next_h, nxt, (size_t)ns * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return asca_ctx_sync(ctx);
}

int asca_model_decode_greedy_host(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids_h, int64_t ns, int64_t n_steps,
                                  uint32_t* tokens_h) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, state && ids_h && tokens_h && ns > 0 && n_steps > 0, "model_decode_greedy: bad arguments");
    for (int64_t i = 0; i < ns; ++i) ASCA_REQUIRE(ctx, ids_h[i] < (uint32_t)m->vocab, "model_decode_greedy: id out of range");
    if (m->compute == ASCA_BF16) return decode_step_bf16(ctx, m, state, ids_h, ns, nullptr, nullptr, n_steps, tokens_h);
    const uint32_t* cur = ids_h;   // f32 mode: the single-step path, token by token
    for (int64_t t = 0; t < n_steps; ++t) {
        ASCA_TRY(asca_model_decode_step_host(ctx, m, state, cur, ns, nullptr, tokens_h + t * ns));
        cur = tokens_h + t * ns;
    }
    return ASCA_OK;
}

int asca_model_decode_step_host(asca_ctx* ctx, asca_model* m, float* state, const uint32_t* ids_h, int64_t ns,
                                float* logits_h, uint32_t* next_h) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, state && ids_h && ns > 0, "model_decode_step: bad arguments");
    const int64_t d = m->d, H = m->H, dh = d / H, E = m->E, F = m->F, V = m->vocab;
    for (int64_t i = 0; i < ns; ++i) ASCA_REQUIRE(ctx, ids_h[i] < (uint32_t)V, "model_decode_step: id out of range");
    if (m->compute == ASCA_BF16) return decode_step_bf16(ctx, m, state, ids_h, ns, logits_h, next_h);
    float* P = m->params;
    Bufs bf(ctx);
    uint32_t* ids = (uint32_t*)bf.f(ns);
    uint32_t* nxt = (uint32_t*)bf.f(ns);
    float *x = bf.f(ns * d), *qkv = bf.f(ns * 3 * d), *gate = bf.f(ns * 2 * H), *o = bf.f(ns * d), *y = bf.f(ns * d),
          *x_mid = bf.f(ns * d), *mo = bf.f(ns * d), *hf = bf.f(ns * d), *logits = bf.f(ns * V);
    ASCA_REQUIRE(ctx, ids && nxt && x && qkv && gate && o && y && x_mid && mo && hf && logits, "model_decode_step: out of memory");
    ASCA_CUDA(ctx, cudaMemcpyAsync(ids, ids_h, (size_t)ns * 4, cudaMemcpyHostToDevice, ctx->stream));
    ASCA_TRY(asca_embed_fwd(ctx, P + m->embed, ids, ns, d, x));
    for (int64_t li = 0; li < m->L; ++li) {
        const Lyr& w = m->lay[li];
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, 3 * d, d, x, d, P + w.w_qkv, 3 * d, qkv, 3 * d, P + w.b_qkv, 0, ASCA_F32));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, 2 * H, d, x, d, P + w.w_gate, 2 * H, gate, 2 * H, P + w.b_gate, 0, ASCA_F32));
        ASCA_TRY(asca_delta_step(ctx, qkv, nullptr, nullptr, gate, nullptr, state + li * ns * H * dh * dh, ns, H, dh, 1, o));
        ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, d, d, o, d, P + w.w_o, d, y, d, P + w.b_o, 0, ASCA_F32));
        ASCA_TRY(asca_residual_rmsnorm(ctx, x, y, x_mid, nullptr, ns, d, 1e-6f));
        ASCA_TRY(asca_moe_step(ctx, x_mid, ids, P + w.w1, P + w.b1, P + w.w2, P + w.b2, ns, d, F, E, ASCA_F32, mo));
        ASCA_TRY(asca_residual_rmsnorm(ctx, x_mid, mo, x, nullptr, ns, d, 1e-6f));
    }
    ASCA_TRY(asca_rmsnorm_fwd(ctx, x, hf, nullptr, ns, d, 1e-6f));
    ASCA_TRY(asca_gemm(ctx, ASCA_NN, ns, V, d, hf, d, P + m->head, V, logits, V, nullptr, 0, ASCA_F32));
    if (logits_h) ASCA_CUDA(ctx, cudaMemcpyAsync(logits_h, logits, (size_t)ns * V * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (next_h) {
        argmax_kernel<<<(unsigned)ceil_div64(ns, 8), 256, 0, ctx->stream>>>(logits, ns, (int)V, nxt);
        ASCA_CHECK_LAUNCH(ctx);
        ASCA_CUDA(ctx, cudaMemcpyAsync(next_h, nxt, (size_t)ns * 4, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return asca_ctx_sync(ctx);
}

}  // extern "C"
