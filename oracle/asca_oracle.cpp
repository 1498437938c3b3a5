// CPU oracle: a C++17 restatement of the reference's f32 CPU path for the Delta Memory
// block, the hash-routed MoE, the tensor engine they sit on, and the model glue.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. Only the test suite, the smoke check and
// the benchmark's CPU-baseline leg may load it; the CUDA library never calls into it.
//
// PINNING: the reference (MythEclipse/asca, a dependency-free Rust crate) ships no golden vectors
// or known-answer tests for this path and cannot be built where this oracle is built (no Rust
// toolchain). The oracle is pinned (a) on a GPU against the reference's own CUDA kernels,
// compiled unmodified by oracle/build_ref.py (tests/test_reference_pin.py: delta forward and
// backward, GEMMs, RMSNorm, SiLU, cross-entropy), and (b) by re-running the reference's own
// self-consistency gates on it (tests/test_oracle_gates.py: finite-difference gradchecks, batch
// parity, decode parity, the independent scalar scan of `asca gpu`). The hash dispatch, the
// composed MoE layer, AdamW and the model glue have no reference GPU kernel or fixture and are
// pinned by (b) only.
//
// Every function cites the reference lines it follows (paths relative to the reference
// repository root). Arithmetic order follows the reference: f32 throughout, fused
// multiply-add exactly where the reference's AVX2 helpers use `_mm256_fmadd_ps`
// (rust/src/simd.rs:114-206) and plain mul+add elsewhere (build with -ffp-contract=off).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

namespace {

int g_threads = 0;  // 0 = hardware concurrency

// rust/src/tensor.rs:16-28 (num_threads; ASCA_THREADS override)
int num_threads() {
    if (g_threads > 0) return g_threads;
    if (const char* e = std::getenv("ASCA_THREADS")) {
        int n = std::atoi(e);
        if (n >= 1) return n;
    }
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

// Run `jobs` closures the way `std::thread::scope` does in the reference (one fresh thread
// per job). With more jobs than cores the OS time-slices them, as it does for the reference.
// To keep huge job counts (one per (head, sequence)) from exhausting the host, jobs are
// handed to at most `cap` workers; each job still runs start-to-finish on one thread, so
// results are identical.
void run_jobs(size_t n_jobs, const std::function<void(size_t)>& fn, int cap = 0) {
    if (n_jobs == 0) return;
    size_t workers = cap > 0 ? (size_t)cap : n_jobs;
    workers = std::min(workers, n_jobs);
    if (workers <= 1) {
        for (size_t j = 0; j < n_jobs; ++j) fn(j);
        return;
    }
    std::vector<std::thread> th;
    th.reserve(workers);
    for (size_t w = 0; w < workers; ++w)
        th.emplace_back([&, w]() {
            for (size_t j = w; j < n_jobs; j += workers) fn(j);
        });
    for (auto& t : th) t.join();
}

// ---------------------------------------------------------------- simd.rs restated
// rust/src/simd.rs:136-154 (axpy_avx2): FMA on full 8-lane groups, mul+add on the tail.
inline void axpy(float* dst, float a, const float* src, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) dst[i + j] = std::fmaf(a, src[i + j], dst[i + j]);
    for (; i < n; ++i) dst[i] += a * src[i];
}
// rust/src/simd.rs:156-182 (dot_avx2): 8 partial sums with FMA, then the horizontal sum
// (hi+lo, movehl, shuffle) and a scalar tail.
inline float dot(const float* a, const float* b, size_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) acc[j] = std::fmaf(a[i + j], b[i + j], acc[j]);
    float s0 = acc[4] + acc[0], s1 = acc[5] + acc[1], s2 = acc[6] + acc[2], s3 = acc[7] + acc[3];
    s0 = s0 + s2;
    s1 = s1 + s3;
    float total = s0 + s1;
    for (; i < n; ++i) total += a[i] * b[i];
    return total;
}
// rust/src/simd.rs:94-111 (scale_avx2)
inline void scale(float* dst, float a, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] *= a;
}
// rust/src/simd.rs:114-134 (scale_axpy_avx2): dst = fma(b, src, a*dst) on full groups.
inline void scale_axpy(float* dst, float a, float b, const float* src, size_t n) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) dst[i + j] = std::fmaf(b, src[i + j], a * dst[i + j]);
    for (; i < n; ++i) dst[i] = a * dst[i] + b * src[i];
}

// rust/src/tensor.rs:245-248
inline float sigmoidf(float x) { return 1.0f / (1.0f + std::exp(-x)); }
// rust/src/model.rs:79-85
inline float siluf(float x) { return x / (1.0f + std::exp(-x)); }

// ---------------------------------------------------------------- tensor.rs restated
constexpr size_t PAR_MIN_MAC = 1u << 18;   // rust/src/tensor.rs:33
constexpr size_t PAR_MIN_ADAM = 1u << 14;  // rust/src/tensor.rs:35

// rust/src/tensor.rs:91-146 (Mat::matmul CPU path): row-chunked threads, k-ascending axpy,
// zero-skip on A entries.
void matmul(const float* A, const float* B, float* C, size_t n, size_t k, size_t m) {
    std::fill(C, C + n * m, 0.0f);
    auto rows = [&](size_t lo, size_t hi) {
        for (size_t i = lo; i < hi; ++i) {
            const float* a = A + i * k;
            float* o = C + i * m;
            for (size_t p = 0; p < k; ++p) {
                float ap = a[p];
                if (ap == 0.0f) continue;
                axpy(o, ap, B + p * m, m);
            }
        }
    };
    size_t nt = (size_t)num_threads();
    size_t mac = n * m * k;
    if (nt <= 1 || mac < PAR_MIN_MAC || n < nt * 2) {
        rows(0, n);
        return;
    }
    size_t chunk = (n + nt - 1) / nt;
    size_t parts = (n + chunk - 1) / chunk;
    run_jobs(parts, [&](size_t ci) { rows(ci * chunk, std::min(n, (ci + 1) * chunk)); });
}
// rust/src/tensor.rs:151-177 (matmul_ta CPU path): single thread, k outer.
void matmul_ta(const float* A, const float* B, float* C, size_t k, size_t m, size_t n) {
    std::fill(C, C + m * n, 0.0f);
    for (size_t p = 0; p < k; ++p) {
        const float* a = A + p * m;
        const float* b = B + p * n;
        for (size_t i = 0; i < m; ++i) {
            float ai = a[i];
            if (ai == 0.0f) continue;
            axpy(C + i * n, ai, b, n);
        }
    }
}
// rust/src/tensor.rs:180-201 (matmul_t CPU path): C[i][j] = dot(A row i, B row j).
void matmul_t(const float* A, const float* B, float* C, size_t n, size_t k, size_t m) {
    for (size_t i = 0; i < n; ++i)
        for (size_t j = 0; j < m; ++j) C[i * m + j] = dot(A + i * k, B + j * k, k);
}
// rust/src/tensor.rs:214-222
void transpose(const float* A, float* At, size_t rows, size_t cols) {
    for (size_t i = 0; i < rows; ++i)
        for (size_t j = 0; j < cols; ++j) At[j * rows + i] = A[i * cols + j];
}
// rust/src/tensor.rs:225-234
void add_row_bias(float* X, const float* b, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) X[r * cols + c] += b[c];
}
// rust/src/tensor.rs:251-271
void rmsnorm_rows(const float* x, float* y, float* inv_out, size_t rows, size_t cols, float eps) {
    for (size_t r = 0; r < rows; ++r) {
        const float* row = x + r * cols;
        float ms = dot(row, row, cols) / (float)cols;
        float inv = 1.0f / std::sqrt(ms + eps);
        if (inv_out) inv_out[r] = inv;
        for (size_t c = 0; c < cols; ++c) y[r * cols + c] = row[c] * inv;
    }
}
// rust/src/tensor.rs:274-297
void rmsnorm_rows_backward(const float* x, const float* dy, float* dx, size_t rows, size_t cols,
                           float eps) {
    for (size_t r = 0; r < rows; ++r) {
        const float* row = x + r * cols;
        const float* dyr = dy + r * cols;
        float ms = dot(row, row, cols) / (float)cols;
        float inv = 1.0f / std::sqrt(ms + eps);
        float mean = dot(dyr, row, cols) * inv;
        mean /= (float)cols;
        for (size_t c = 0; c < cols; ++c) dx[r * cols + c] = inv * (dyr[c] - row[c] * inv * mean);
    }
}

// rust/src/tensor.rs:299-337 (xorshift128+ with Box-Muller, cosine branch only)
struct Rng {
    uint64_t s0, s1;
    explicit Rng(uint64_t seed) {
        s0 = (seed * 0x9E3779B97F4A7C15ull) | 1ull;
        s1 = ((seed ^ 0xDEADBEEFCAFEF00Dull) * 0xBF58476D1CE4E5B9ull) | 1ull;
    }
    uint64_t next_u64() {
        uint64_t x = s0, y = s1;
        s0 = y;
        x ^= x << 23;
        s1 = x ^ y ^ (x >> 17) ^ (y >> 26);
        return s1 + y;
    }
    float uniform() { return (float)(next_u64() >> 40) / (float)(1u << 24); }
    float normal() {
        float u1 = std::max(uniform(), 1e-7f);
        float u2 = uniform();
        return std::sqrt(-2.0f * std::log(u1)) * std::cos(2.0f * 3.14159265358979323846f * u2);
    }
    size_t below(size_t n) { return (size_t)(next_u64() % (uint64_t)n); }
};

// rust/src/model.rs:69-77
inline uint32_t hash_route(uint32_t id, uint32_t n_experts) {
    uint32_t h = id * 0x9E3779B1u;
    h ^= h >> 15;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    return (uint32_t)((size_t)h % (size_t)n_experts);
}

// ---------------------------------------------------------------- delta.rs restated
// One (head, sequence) chain of the forward scan. rust/src/delta.rs:275-318.
// `states` (nullable) receives S before every step plus the final S, (seq+1)*dh*dh floats.
void scan_chain(const float* q, const float* k, const float* v, const float* alpha,
                const float* beta, size_t seq, size_t H, size_t dh, size_t hh, size_t row0,
                float* o_rows /* (.., H*dh) */, float* states, float* s_final) {
    const size_t d = H * dh, off = hh * dh;
    std::vector<float> s(dh * dh, 0.0f), sk(dh), u(dh);
    for (size_t t = 0; t < seq; ++t) {
        size_t r = row0 + t;
        if (states) std::memcpy(states + t * dh * dh, s.data(), dh * dh * sizeof(float));
        const float* kt = k + r * d + off;
        const float* vt = v + r * d + off;
        const float* qt = q + r * d + off;
        float a = alpha[r * H + hh], b = beta[r * H + hh];
        std::fill(sk.begin(), sk.end(), 0.0f);
        for (size_t ai = 0; ai < dh; ++ai) {
            float ka = kt[ai];
            if (ka == 0.0f) continue;
            const float* srow = &s[ai * dh];
            for (size_t i = 0; i < dh; ++i) sk[i] += srow[i] * ka;
        }
        for (size_t i = 0; i < dh; ++i) u[i] = b * (vt[i] - a * sk[i]);
        for (size_t ai = 0; ai < dh; ++ai)
            for (size_t i = 0; i < dh; ++i) s[ai * dh + i] = a * s[ai * dh + i] + kt[ai] * u[i];
        float* ot = o_rows + r * d + off;
        for (size_t i = 0; i < dh; ++i) {
            float acc = 0.0f;
            for (size_t ai = 0; ai < dh; ++ai) acc += s[ai * dh + i] * qt[ai];
            ot[i] = acc;
        }
    }
    if (states) std::memcpy(states + seq * dh * dh, s.data(), dh * dh * sizeof(float));
    if (s_final) std::memcpy(s_final, s.data(), dh * dh * sizeof(float));
}

// One (head, sequence) chain of the BPTT. rust/src/delta.rs:476-572. Writes the chain's
// rows of d_q/d_k/d_v (N x d, pre L2-norm-backward) and d_alpha/d_beta (N x H).
void bptt_chain(const float* states, const float* q, const float* k, const float* v,
                const float* alpha, const float* beta, const float* d_o, size_t seq, size_t H,
                size_t dh, size_t hh, size_t row0, float* d_q, float* d_k, float* d_v,
                float* d_alpha, float* d_beta) {
    const size_t d = H * dh, off = hh * dh, dd = dh * dh;
    std::vector<float> ds(dd, 0.0f), ds_prev(dd, 0.0f), sk(dh), u(dh), dq(dh), dk(dh), du(dh),
        dsk(dh);
    for (size_t tt = seq; tt-- > 0;) {
        size_t t = tt, r = row0 + t;
        std::fill(dk.begin(), dk.end(), 0.0f);
        const float* s_t = states + (t + 1) * dd;
        const float* s_prev = states + t * dd;
        const float* qt = q + r * d + off;
        const float* kt = k + r * d + off;
        const float* vt = v + r * d + off;
        const float* do_t = d_o + r * d + off;
        float a = alpha[r * H + hh], b = beta[r * H + hh];
        for (size_t ai = 0; ai < dh; ++ai) dq[ai] = dot(do_t, s_t + ai * dh, dh);
        for (size_t ai = 0; ai < dh; ++ai) {
            d_q[r * d + off + ai] = dq[ai];
            axpy(&ds[ai * dh], qt[ai], do_t, dh);
        }
        std::fill(sk.begin(), sk.end(), 0.0f);
        for (size_t ai = 0; ai < dh; ++ai) {
            float ka = kt[ai];
            if (ka != 0.0f) axpy(sk.data(), ka, s_prev + ai * dh, dh);
        }
        for (size_t i = 0; i < dh; ++i) u[i] = b * (vt[i] - a * sk[i]);
        float dalpha = dot(ds.data(), s_prev, dd);
        float dbeta = 0.0f;
        for (size_t ai = 0; ai < dh; ++ai) dk[ai] += dot(&ds[ai * dh], u.data(), dh);
        std::fill(du.begin(), du.end(), 0.0f);
        for (size_t ai = 0; ai < dh; ++ai) {
            float ka = kt[ai];
            if (ka != 0.0f) axpy(du.data(), ka, &ds[ai * dh], dh);
        }
        for (size_t idx = 0; idx < dd; ++idx) ds_prev[idx] = a * ds[idx];
        for (size_t i = 0; i < dh; ++i) {
            dbeta += du[i] * (vt[i] - a * sk[i]);
            d_v[r * d + off + i] = b * du[i];
            dsk[i] = -b * a * du[i];
            dalpha += -b * du[i] * sk[i];
        }
        for (size_t ai = 0; ai < dh; ++ai) {
            dk[ai] += dot(s_prev + ai * dh, dsk.data(), dh);
            axpy(&ds_prev[ai * dh], kt[ai], dsk.data(), dh);
        }
        for (size_t ai = 0; ai < dh; ++ai) d_k[r * d + off + ai] = dk[ai];
        d_alpha[r * H + hh] = dalpha;
        d_beta[r * H + hh] = dbeta;
        ds.swap(ds_prev);
    }
}

// rust/src/delta.rs:678-698
void norm_backward(const float* y, const float* norms, float* dmat, size_t rows, size_t H,
                   size_t dh) {
    const size_t d = H * dh;
    for (size_t t = 0; t < rows; ++t)
        for (size_t hh = 0; hh < H; ++hh) {
            size_t off = hh * dh;
            float s = norms[t * H + hh];
            float dt = 0.0f;
            for (size_t c = 0; c < dh; ++c) dt += y[t * d + off + c] * dmat[t * d + off + c];
            for (size_t c = 0; c < dh; ++c)
                dmat[t * d + off + c] = (dmat[t * d + off + c] - y[t * d + off + c] * dt) / s;
        }
}

// rust/src/delta.rs:421-613 (bptt_cpu), restructured only in memory: each (head, sequence)
// job recomputes its own state history with the forward scan instead of reading a global
// (T+1)*dh^2-per-chain table, which at B8 H16 T4096 dh128 would be 34 GB. Arithmetic per
// chain is the reference's.
void delta_bptt(const float* q, const float* k, const float* v, const float* alpha,
                const float* beta, const float* qn, const float* kn, const float* d_o, size_t B,
                size_t seq, size_t H, size_t dh, float* d_qkv, float* d_gate, int max_workers) {
    const size_t N = B * seq, d = H * dh;
    std::vector<float> d_q(N * d, 0.0f), d_k(N * d, 0.0f), d_v(N * d, 0.0f), d_a(N * H, 0.0f),
        d_b(N * H, 0.0f);
    run_jobs(
        H * B,
        [&](size_t j) {
            size_t hh = j / B, bi = j % B;
            std::vector<float> states((seq + 1) * dh * dh);
            std::vector<float> o_tmp;  // scan_chain writes o; discard into a scratch
            o_tmp.resize(seq * d);
            // shift pointers so scan_chain's `row0 + t` indexing lands in o_tmp rows [0,seq)
            scan_chain(q, k, v, alpha, beta, seq, H, dh, hh, bi * seq,
                       o_tmp.data() - bi * seq * d, states.data(), nullptr);
            bptt_chain(states.data(), q, k, v, alpha, beta, d_o, seq, H, dh, hh, bi * seq,
                       d_q.data(), d_k.data(), d_v.data(), d_a.data(), d_b.data());
        },
        max_workers);
    norm_backward(q, qn, d_q.data(), N, H, dh);
    norm_backward(k, kn, d_k.data(), N, H, dh);
    for (size_t r = 0; r < N; ++r)
        for (size_t c = 0; c < d; ++c) {
            d_qkv[r * 3 * d + c] = d_q[r * d + c];
            d_qkv[r * 3 * d + d + c] = d_k[r * d + c];
            d_qkv[r * 3 * d + 2 * d + c] = d_v[r * d + c];
        }
    for (size_t r = 0; r < N; ++r)
        for (size_t hh = 0; hh < H; ++hh) {
            float al = alpha[r * H + hh], be = beta[r * H + hh];
            d_gate[r * 2 * H + hh] = d_a[r * H + hh] * al * (1.0f - al);
            d_gate[r * 2 * H + H + hh] = d_b[r * H + hh] * be * (1.0f - be);
        }
}

struct DeltaParams {  // views into a flat parameter / gradient buffer
    float *w_qkv, *b_qkv, *w_gate, *b_gate, *w_o, *b_o;
};
struct DeltaCache {
    std::vector<float> x, qkv, q, k, v, gate, alpha, beta, qn, kn, o;
    size_t batch = 0, seq = 0;
};

// rust/src/delta.rs:121-207 (DeltaBlock::forward)
void delta_block_forward(const DeltaParams& p, const float* x, size_t N, size_t batch, size_t d,
                         size_t H, float* y, DeltaCache& c) {
    const size_t dh = d / H, seq = N / batch;
    c.batch = batch;
    c.seq = seq;
    c.x.assign(x, x + N * d);
    c.qkv.resize(N * 3 * d);
    matmul(x, p.w_qkv, c.qkv.data(), N, d, 3 * d);
    add_row_bias(c.qkv.data(), p.b_qkv, N, 3 * d);
    c.q.resize(N * d);
    c.k.resize(N * d);
    c.v.resize(N * d);
    for (size_t r = 0; r < N; ++r)
        for (size_t cc = 0; cc < d; ++cc) {
            c.q[r * d + cc] = c.qkv[r * 3 * d + cc];
            c.k[r * d + cc] = c.qkv[r * 3 * d + d + cc];
            c.v[r * d + cc] = c.qkv[r * 3 * d + 2 * d + cc];
        }
    c.qn.resize(N * H);
    c.kn.resize(N * H);
    for (size_t r = 0; r < N; ++r)
        for (size_t hh = 0; hh < H; ++hh)
            for (int which = 0; which < 2; ++which) {
                float* seg = (which == 0 ? c.q.data() : c.k.data()) + r * d + hh * dh;
                float ss = 0.0f;
                for (size_t i = 0; i < dh; ++i) ss += seg[i] * seg[i];
                float n = std::max(std::sqrt(ss), 1e-8f);
                for (size_t i = 0; i < dh; ++i) seg[i] /= n;
                (which == 0 ? c.qn : c.kn)[r * H + hh] = n;
            }
    c.gate.resize(N * 2 * H);
    matmul(x, p.w_gate, c.gate.data(), N, d, 2 * H);
    add_row_bias(c.gate.data(), p.b_gate, N, 2 * H);
    c.alpha.resize(N * H);
    c.beta.resize(N * H);
    for (size_t r = 0; r < N; ++r)
        for (size_t hh = 0; hh < H; ++hh) {
            c.alpha[r * H + hh] = sigmoidf(c.gate[r * 2 * H + hh]);
            c.beta[r * H + hh] = sigmoidf(c.gate[r * 2 * H + H + hh]);
        }
    c.o.assign(N * d, 0.0f);
    // rust/src/delta.rs:269-321: one thread per head, sequences looped inside.
    run_jobs(H, [&](size_t hh) {
        for (size_t bi = 0; bi < batch; ++bi)
            scan_chain(c.q.data(), c.k.data(), c.v.data(), c.alpha.data(), c.beta.data(), seq, H, dh,
                       hh, bi * seq, c.o.data(), nullptr, nullptr);
    });
    matmul(c.o.data(), p.w_o, y, N, d, d);
    add_row_bias(y, p.b_o, N, d);
}

// rust/src/delta.rs:615-674 (DeltaBlock::backward). `g` = gradient views (accumulated +=).
void delta_block_backward(const DeltaParams& p, const DeltaParams& g, const DeltaCache& c,
                          const float* dy, size_t N, size_t d, size_t H, float* dx) {
    const size_t dh = d / H;
    std::vector<float> d_o(N * d), tmp(d * d);
    matmul_t(dy, p.w_o, d_o.data(), N, d, d);
    matmul_ta(c.o.data(), dy, tmp.data(), N, d, d);
    for (size_t i = 0; i < d * d; ++i) g.w_o[i] += 1.0f * tmp[i];
    for (size_t r = 0; r < N; ++r)
        for (size_t cc = 0; cc < d; ++cc) g.b_o[cc] += dy[r * d + cc];
    std::vector<float> d_qkv(N * 3 * d), d_gate(N * 2 * H);
    delta_bptt(c.q.data(), c.k.data(), c.v.data(), c.alpha.data(), c.beta.data(), c.qn.data(),
               c.kn.data(), d_o.data(), c.batch, c.seq, H, dh, d_qkv.data(), d_gate.data(), 0);
    std::vector<float> xt(d * N);
    transpose(c.x.data(), xt.data(), N, d);
    std::vector<float> dw(d * 3 * d);
    matmul(xt.data(), d_qkv.data(), dw.data(), d, N, 3 * d);
    for (size_t i = 0; i < dw.size(); ++i) g.w_qkv[i] += 1.0f * dw[i];
    for (size_t r = 0; r < N; ++r)
        for (size_t cc = 0; cc < 3 * d; ++cc) g.b_qkv[cc] += d_qkv[r * 3 * d + cc];
    std::vector<float> dwg(d * 2 * H);
    matmul(xt.data(), d_gate.data(), dwg.data(), d, N, 2 * H);
    for (size_t i = 0; i < dwg.size(); ++i) g.w_gate[i] += 1.0f * dwg[i];
    for (size_t r = 0; r < N; ++r)
        for (size_t cc = 0; cc < 2 * H; ++cc) g.b_gate[cc] += d_gate[r * 2 * H + cc];
    std::vector<float> wt(3 * d * d), wgt(2 * H * d), dx2(N * d);
    transpose(p.w_qkv, wt.data(), d, 3 * d);
    matmul(d_qkv.data(), wt.data(), dx, N, 3 * d, d);
    transpose(p.w_gate, wgt.data(), d, 2 * H);
    matmul(d_gate.data(), wgt.data(), dx2.data(), N, 2 * H, d);
    for (size_t i = 0; i < N * d; ++i) dx[i] += 1.0f * dx2[i];
}

// rust/src/delta.rs:341-411 (DeltaBlock::step). The reference holds the normalised q,k in
// [f32; 64] scratch and so panics for dh > 64; the oracle uses heap scratch with identical
// arithmetic so that larger heads can be checked too.
void delta_block_step(const DeltaParams& p, const float* x, size_t d, size_t H, float* states,
                      float* y) {
    const size_t dh = d / H;
    std::vector<float> qkv(3 * d), gate(2 * H), o(d, 0.0f), sk(dh), u(dh), qn(dh), kn(dh);
    matmul(x, p.w_qkv, qkv.data(), 1, d, 3 * d);
    add_row_bias(qkv.data(), p.b_qkv, 1, 3 * d);
    matmul(x, p.w_gate, gate.data(), 1, d, 2 * H);
    add_row_bias(gate.data(), p.b_gate, 1, 2 * H);
    for (size_t hh = 0; hh < H; ++hh) {
        size_t off = hh * dh;
        float a = sigmoidf(gate[hh]), b = sigmoidf(gate[H + hh]);
        float qq = 0.0f, kk = 0.0f;
        for (size_t i = 0; i < dh; ++i) {
            float qv = qkv[off + i], kv = qkv[d + off + i];
            qq += qv * qv;
            kk += kv * kv;
        }
        float qi = 1.0f / std::max(std::sqrt(qq), 1e-8f);
        float ki = 1.0f / std::max(std::sqrt(kk), 1e-8f);
        for (size_t i = 0; i < dh; ++i) {
            qn[i] = qkv[off + i] * qi;
            kn[i] = qkv[d + off + i] * ki;
        }
        float* s = states + hh * dh * dh;
        std::fill(sk.begin(), sk.end(), 0.0f);
        for (size_t ai = 0; ai < dh; ++ai) {
            float ka = kn[ai];
            if (ka == 0.0f) continue;
            axpy(sk.data(), ka, s + ai * dh, dh);
        }
        for (size_t i = 0; i < dh; ++i) u[i] = b * (qkv[2 * d + off + i] - a * sk[i]);
        for (size_t ai = 0; ai < dh; ++ai) {
            float ka = kn[ai];
            if (ka == 0.0f) {
                scale(s + ai * dh, a, dh);
                continue;
            }
            scale_axpy(s + ai * dh, a, ka, u.data(), dh);
        }
        for (size_t i = 0; i < dh; ++i) {
            float acc = 0.0f;
            for (size_t ai = 0; ai < dh; ++ai) acc += s[ai * dh + i] * qn[ai];
            o[off + i] = acc;
        }
    }
    matmul(o.data(), p.w_o, y, 1, d, d);
    add_row_bias(y, p.b_o, 1, d);
}

// ---------------------------------------------------------------- model.rs: HashMoe
struct MoeParams {
    float *w1, *b1, *w2, *b2;  // w1 (d, E*F); b1 (E*F); w2 (E*F, d); b2 (d)
};
struct MoeCache {
    std::vector<float> x, xn, pre, hidden;
    std::vector<std::vector<size_t>> buckets;
};
constexpr float EPS = 1e-6f;  // rust/src/model.rs:14

// rust/src/model.rs:190-193
void build_buckets(const uint32_t* ids, size_t N, size_t E, std::vector<std::vector<size_t>>& b) {
    b.assign(E, {});
    for (size_t t = 0; t < N; ++t) b[hash_route(ids[t], (uint32_t)E)].push_back(t);
}

// Expert FFN forward on already-normalised rows. rust/src/model.rs:237-293.
void moe_ffn_forward(const MoeParams& p, const float* xn, size_t N, size_t d, size_t F, size_t E,
                     const std::vector<std::vector<size_t>>& buckets, float* out, float* pre_all,
                     float* hid_all) {
    std::fill(out, out + N * d, 0.0f);
    run_jobs(E, [&](size_t e) {
        const auto& rows = buckets[e];
        size_t n = rows.size();
        if (n == 0) return;
        std::vector<float> pre(n * F), hidden(n * F), o(n * d);
        const float* b1 = p.b1 + e * F;
        for (size_t i = 0; i < n; ++i) std::memcpy(&pre[i * F], b1, F * sizeof(float));
        for (size_t c = 0; c < d; ++c) {
            const float* w1row = p.w1 + c * (E * F) + e * F;
            for (size_t i = 0; i < n; ++i) {
                float xc = xn[rows[i] * d + c];
                if (xc == 0.0f) continue;
                axpy(&pre[i * F], xc, w1row, F);
            }
        }
        for (size_t i = 0; i < n; ++i) {
            for (size_t j = 0; j < F; ++j) hidden[i * F + j] = siluf(pre[i * F + j]);
            std::memcpy(&o[i * d], p.b2, d * sizeof(float));
        }
        for (size_t j = 0; j < F; ++j) {
            const float* w2row = p.w2 + (e * F + j) * d;
            for (size_t i = 0; i < n; ++i) {
                float hj = hidden[i * F + j];
                if (hj == 0.0f) continue;
                axpy(&o[i * d], hj, w2row, d);
            }
        }
        for (size_t i = 0; i < n; ++i) {
            size_t t = rows[i];
            if (pre_all) std::memcpy(pre_all + t * F, &pre[i * F], F * sizeof(float));
            if (hid_all) std::memcpy(hid_all + t * F, &hidden[i * F], F * sizeof(float));
            std::memcpy(out + t * d, &o[i * d], d * sizeof(float));
        }
    });
}

// rust/src/model.rs:187-306 (HashMoe::forward, CPU path)
void moe_forward(const MoeParams& p, const float* x, const uint32_t* ids, size_t N, size_t d,
                 size_t F, size_t E, float* out, MoeCache& c) {
    build_buckets(ids, N, E, c.buckets);
    c.x.assign(x, x + N * d);
    c.xn.resize(N * d);
    rmsnorm_rows(x, c.xn.data(), nullptr, N, d, EPS);
    c.pre.assign(N * F, 0.0f);
    c.hidden.assign(N * F, 0.0f);
    moe_ffn_forward(p, c.xn.data(), N, d, F, E, c.buckets, out, c.pre.data(), c.hidden.data());
}

// Expert FFN backward up to dxn. rust/src/model.rs:363-495.
void moe_ffn_backward(const MoeParams& p, const MoeParams& g, const float* xn, const float* pre_r,
                      const float* hidden_r, const std::vector<std::vector<size_t>>& buckets,
                      const float* dout, size_t N, size_t d, size_t F, size_t E, float* dxn) {
    std::fill(dxn, dxn + N * d, 0.0f);
    struct Job {
        std::vector<float> dpre, dw1, dw2, db1, db2, dxn;
    };
    std::vector<Job> jobs(E);
    run_jobs(E, [&](size_t e) {
        const auto& rows = buckets[e];
        size_t n = rows.size();
        Job& jb = jobs[e];
        if (n == 0) return;
        jb.dpre.assign(n * F, 0.0f);
        jb.dw1.assign(d * F, 0.0f);
        jb.dw2.assign(F * d, 0.0f);
        jb.db1.assign(F, 0.0f);
        jb.db2.assign(d, 0.0f);
        jb.dxn.assign(n * d, 0.0f);
        for (size_t t : rows) {
            const float* dr = dout + t * d;
            for (size_t j = 0; j < F; ++j) {
                float hj = hidden_r[t * F + j];
                if (hj == 0.0f) continue;
                axpy(&jb.dw2[j * d], hj, dr, d);
            }
            for (size_t c = 0; c < d; ++c) jb.db2[c] += dr[c];
        }
        for (size_t i = 0; i < n; ++i) {
            const float* dr = dout + rows[i] * d;
            for (size_t j = 0; j < F; ++j) jb.dpre[i * F + j] = dot(dr, p.w2 + (e * F + j) * d, d);
        }
        for (size_t i = 0; i < n; ++i)
            for (size_t j = 0; j < F; ++j) {
                float pre = pre_r[rows[i] * F + j];
                float sg = 1.0f / (1.0f + std::exp(-pre));
                float dh = jb.dpre[i * F + j] * (sg * (1.0f + pre * (1.0f - sg)));
                jb.db1[j] += dh;
                jb.dpre[i * F + j] = dh;
            }
        for (size_t c = 0; c < d; ++c) {
            const float* w1row = p.w1 + c * (E * F) + e * F;
            float* gw = &jb.dw1[c * F];
            for (size_t i = 0; i < n; ++i) {
                float xc = xn[rows[i] * d + c];
                if (xc == 0.0f) continue;
                axpy(gw, xc, &jb.dpre[i * F], F);
            }
            for (size_t i = 0; i < n; ++i) jb.dxn[i * d + c] += dot(&jb.dpre[i * F], w1row, F);
        }
    });
    for (size_t e = 0; e < E; ++e) {
        const Job& jb = jobs[e];
        if (jb.dw1.empty()) continue;
        for (size_t j = 0; j < F; ++j)
            for (size_t c = 0; c < d; ++c) g.w2[(e * F + j) * d + c] += jb.dw2[j * d + c];
        for (size_t c = 0; c < d; ++c)
            for (size_t j = 0; j < F; ++j) g.w1[c * (E * F) + e * F + j] += jb.dw1[c * F + j];
        for (size_t j = 0; j < F; ++j) g.b1[e * F + j] += jb.db1[j];
        for (size_t c = 0; c < d; ++c) g.b2[c] += jb.db2[c];
        for (size_t i = 0; i < buckets[e].size(); ++i)
            for (size_t c = 0; c < d; ++c) dxn[buckets[e][i] * d + c] += jb.dxn[i * d + c];
    }
}

// rust/src/model.rs:339-497 (HashMoe::backward, CPU path)
void moe_backward(const MoeParams& p, const MoeParams& g, const MoeCache& c, const float* dout,
                  size_t N, size_t d, size_t F, size_t E, float* dx) {
    std::vector<float> dxn(N * d);
    moe_ffn_backward(p, g, c.xn.data(), c.pre.data(), c.hidden.data(), c.buckets, dout, N, d, F, E,
                     dxn.data());
    rmsnorm_rows_backward(c.x.data(), dxn.data(), dx, N, d, EPS);
}

// rust/src/model.rs:309-337 (HashMoe::step)
void moe_step(const MoeParams& p, const float* x, uint32_t id, size_t d, size_t F, size_t E,
              float* out) {
    std::vector<float> xn(d), pre(F);
    rmsnorm_rows(x, xn.data(), nullptr, 1, d, EPS);
    size_t e = hash_route(id, (uint32_t)E);
    std::memcpy(pre.data(), p.b1 + e * F, F * sizeof(float));
    for (size_t c = 0; c < d; ++c) {
        float xc = xn[c];
        if (xc == 0.0f) continue;
        axpy(pre.data(), xc, p.w1 + c * (E * F) + e * F, F);
    }
    for (auto& v : pre) v = siluf(v);
    std::memcpy(out, p.b2, d * sizeof(float));
    for (size_t j = 0; j < F; ++j) axpy(out, pre[j], p.w2 + (e * F + j) * d, d);
}

// ---------------------------------------------------------------- model.rs: Model
struct Config {
    size_t vocab, d, H, L, E, F;
};
// Parameter order rust/src/model.rs:593-609: embed, head, then per layer
// w_qkv, b_qkv, w_gate, b_gate, w_o, b_o, w1, b1, w2, b2.
struct Layout {
    size_t embed, head;
    struct Lyr {
        size_t w_qkv, b_qkv, w_gate, b_gate, w_o, b_o, w1, b1, w2, b2;
    };
    std::vector<Lyr> layers;
    size_t total;
    std::vector<size_t> tensor_off, tensor_len;  // in parameter order
};
Layout make_layout(const Config& c) {
    Layout l;
    size_t o = 0;
    auto take = [&](size_t n) {
        size_t at = o;
        l.tensor_off.push_back(at);
        l.tensor_len.push_back(n);
        o += n;
        return at;
    };
    l.embed = take(c.vocab * c.d);
    l.head = take(c.d * c.vocab);
    for (size_t i = 0; i < c.L; ++i) {
        Layout::Lyr y;
        y.w_qkv = take(c.d * 3 * c.d);
        y.b_qkv = take(3 * c.d);
        y.w_gate = take(c.d * 2 * c.H);
        y.b_gate = take(2 * c.H);
        y.w_o = take(c.d * c.d);
        y.b_o = take(c.d);
        y.w1 = take(c.d * c.E * c.F);
        y.b1 = take(c.E * c.F);
        y.w2 = take(c.E * c.F * c.d);
        y.b2 = take(c.d);
        l.layers.push_back(y);
    }
    l.total = o;
    return l;
}
DeltaParams delta_view(float* base, const Layout::Lyr& y) {
    return {base + y.w_qkv, base + y.b_qkv, base + y.w_gate, base + y.b_gate, base + y.w_o,
            base + y.b_o};
}
MoeParams moe_view(float* base, const Layout::Lyr& y) {
    return {base + y.w1, base + y.b1, base + y.w2, base + y.b2};
}

struct LayerCache {
    DeltaCache dc;
    MoeCache mc;
    std::vector<float> x_out;
};

// rust/src/model.rs:651-700 (Model::forward); returns logits (N x vocab).
void model_forward(const Config& c, const Layout& l, float* params, const uint32_t* ids, size_t N,
                   size_t batch, std::vector<LayerCache>& caches, std::vector<float>& h_final,
                   float* logits) {
    const size_t d = c.d;
    std::vector<float> x(N * d);
    for (size_t t = 0; t < N; ++t)
        std::memcpy(&x[t * d], params + l.embed + ids[t] * d, d * sizeof(float));
    caches.resize(c.L);
    std::vector<float> dy(N * d), dm(N * d), x_mid(N * d);
    for (size_t li = 0; li < c.L; ++li) {
        DeltaParams dp = delta_view(params, l.layers[li]);
        MoeParams mp = moe_view(params, l.layers[li]);
        delta_block_forward(dp, x.data(), N, batch, d, c.H, dy.data(), caches[li].dc);
        for (size_t i = 0; i < N * d; ++i) x_mid[i] = x[i] + 1.0f * dy[i];
        moe_forward(mp, x_mid.data(), ids, N, d, c.F, c.E, dm.data(), caches[li].mc);
        for (size_t i = 0; i < N * d; ++i) x[i] = x_mid[i] + 1.0f * dm[i];
        caches[li].x_out = x;
    }
    h_final.resize(N * d);
    rmsnorm_rows(x.data(), h_final.data(), nullptr, N, d, EPS);
    matmul(h_final.data(), params + l.head, logits, N, d, c.vocab);
}

// rust/src/model.rs:804-844 (cpu_cross_entropy): per-thread row chunks, partial losses
// summed in chunk order.
float cross_entropy(const float* logits, const uint32_t* targets, size_t N, size_t V,
                    float* dlogits) {
    size_t nt = (size_t)std::max(num_threads(), 1);
    float inv = 1.0f / (float)N;
    size_t chunk = (N + nt - 1) / nt;
    size_t parts = std::max<size_t>((N + chunk - 1) / chunk, 1);
    std::vector<float> loss_parts(parts, 0.0f);
    run_jobs(parts, [&](size_t ci) {
        size_t start = ci * chunk, end = std::min(N, start + chunk);
        float lsum = 0.0f;
        for (size_t t = start; t < end; ++t) {
            const float* row = logits + t * V;
            float mx = -INFINITY;
            for (size_t cc = 0; cc < V; ++cc) mx = std::max(mx, row[cc]);
            float sum = 0.0f;
            for (size_t cc = 0; cc < V; ++cc) sum += std::exp(row[cc] - mx);
            float lse = mx + std::log(sum);
            lsum += lse - row[targets[t]];
            float* drow = dlogits + t * V;
            for (size_t cc = 0; cc < V; ++cc) drow[cc] = std::exp(row[cc] - lse) * inv;
            drow[targets[t]] -= inv;
        }
        loss_parts[ci] = lsum;
    });
    float loss = 0.0f;
    for (float v : loss_parts) loss += v;
    return loss * inv;
}

// rust/src/model.rs:703-718 (Model::loss): batch = 1, serial sum.
float loss_only(const float* logits, const uint32_t* targets, size_t N, size_t V) {
    float loss = 0.0f;
    for (size_t t = 0; t < N; ++t) {
        const float* row = logits + t * V;
        float mx = -INFINITY;
        for (size_t cc = 0; cc < V; ++cc) mx = std::max(mx, row[cc]);
        float sum = 0.0f;
        for (size_t cc = 0; cc < V; ++cc) sum += std::exp(row[cc] - mx);
        loss += mx + std::log(sum) - row[targets[t]];
    }
    return loss / (float)N;
}

// rust/src/model.rs:744-794 (Model::backward, host-logits path)
float model_backward(const Config& c, const Layout& l, float* params, float* grads,
                     const uint32_t* ids, const uint32_t* targets, size_t N,
                     std::vector<LayerCache>& caches, const std::vector<float>& h_final,
                     const float* logits) {
    const size_t d = c.d, V = c.vocab;
    std::vector<float> dlogits(N * V);
    float loss = cross_entropy(logits, targets, N, V, dlogits.data());
    std::vector<float> d_head(d * V), dh(N * d);
    matmul_ta(h_final.data(), dlogits.data(), d_head.data(), N, d, V);
    matmul_t(dlogits.data(), params + l.head, dh.data(), N, V, d);
    for (size_t i = 0; i < d * V; ++i) grads[l.head + i] += 1.0f * d_head[i];
    std::vector<float> dx(N * d), d_moe(N * d), d_delta(N * d);
    rmsnorm_rows_backward(caches.back().x_out.data(), dh.data(), dx.data(), N, d, EPS);
    for (size_t li = c.L; li-- > 0;) {
        DeltaParams dp = delta_view(params, l.layers[li]), dg = delta_view(grads, l.layers[li]);
        MoeParams mp = moe_view(params, l.layers[li]), mg = moe_view(grads, l.layers[li]);
        moe_backward(mp, mg, caches[li].mc, dx.data(), N, d, c.F, c.E, d_moe.data());
        for (size_t i = 0; i < N * d; ++i) dx[i] += 1.0f * d_moe[i];  // d_mid
        delta_block_backward(dp, dg, caches[li].dc, dx.data(), N, d, c.H, d_delta.data());
        for (size_t i = 0; i < N * d; ++i) dx[i] += 1.0f * d_delta[i];  // d_in
    }
    for (size_t t = 0; t < N; ++t)
        for (size_t cc = 0; cc < d; ++cc) grads[l.embed + ids[t] * d + cc] += dx[t * d + cc];
    return loss;
}

// `f32::powi` restated: repeated multiplication by squaring is what LLVM's powi lowers to;
// the oracle uses it so the bias corrections do not depend on libm's powf.
float powi(float b, int e) {
    float r = 1.0f;
    float x = b;
    int n = e;
    while (n > 0) {
        if (n & 1) r *= x;
        x *= x;
        n >>= 1;
    }
    return r;
}

}  // namespace

// =================================================================== C ABI
extern "C" {

void orc_set_threads(int n) { g_threads = n; }
int orc_num_threads() { return num_threads(); }

// ---- Rng (rust/src/tensor.rs:299-337). State = two u64 words owned by the caller.
void orc_rng_new(uint64_t seed, uint64_t* state) {
    Rng r(seed);
    state[0] = r.s0;
    state[1] = r.s1;
}
void orc_rng_normal(uint64_t* state, float scale, float* out, size_t n) {
    Rng r(0);
    r.s0 = state[0];
    r.s1 = state[1];
    for (size_t i = 0; i < n; ++i) out[i] = r.normal() * scale;
    state[0] = r.s0;
    state[1] = r.s1;
}
void orc_rng_uniform(uint64_t* state, float* out, size_t n) {
    Rng r(0);
    r.s0 = state[0];
    r.s1 = state[1];
    for (size_t i = 0; i < n; ++i) out[i] = r.uniform();
    state[0] = r.s0;
    state[1] = r.s1;
}
void orc_rng_below(uint64_t* state, uint64_t bound, uint32_t* out, size_t n) {
    Rng r(0);
    r.s0 = state[0];
    r.s1 = state[1];
    for (size_t i = 0; i < n; ++i) out[i] = (uint32_t)r.below((size_t)bound);
    state[0] = r.s0;
    state[1] = r.s1;
}

// ---- tensor engine
void orc_matmul(const float* A, const float* B, float* C, size_t M, size_t K, size_t N) {
    matmul(A, B, C, M, K, N);
}
void orc_matmul_ta(const float* A, const float* B, float* C, size_t K, size_t M, size_t N) {
    matmul_ta(A, B, C, K, M, N);
}
void orc_matmul_t(const float* A, const float* B, float* C, size_t M, size_t K, size_t N) {
    matmul_t(A, B, C, M, K, N);
}
void orc_rmsnorm_fwd(const float* x, float* y, float* inv, size_t rows, size_t cols, float eps) {
    rmsnorm_rows(x, y, inv, rows, cols, eps);
}
void orc_rmsnorm_bwd(const float* x, const float* dy, float* dx, size_t rows, size_t cols,
                     float eps) {
    rmsnorm_rows_backward(x, dy, dx, rows, cols, eps);
}
// One tensor's AdamW update given the already-derived per-tensor scalars, i.e. the loop body
// of rust/src/tensor.rs:444-453 (what the reference's Gpu::adamw_update receives).
void orc_adamw_apply(float* p, const float* g, float* m, float* v, size_t n, float lr_t, float b1,
                     float b2, float eps_t, float wd_eff) {
    for (size_t i = 0; i < n; ++i) {
        float gi = g[i];
        m[i] = b1 * m[i] + (1.0f - b1) * gi;
        v[i] = b2 * v[i] + (1.0f - b2) * gi * gi;
        float upd = m[i] / (std::sqrt(v[i]) + eps_t);
        p[i] -= wd_eff * p[i];
        p[i] -= lr_t * upd;
    }
}
// Per-tensor scalars of rust/src/tensor.rs:393-402 at counter t (after the increment).
void orc_adamw_scalars(float lr, float b1, float b2, float eps, float wd, uint32_t t, float* lr_t,
                       float* eps_t, float* wd_eff) {
    float bc1 = 1.0f - powi(b1, (int)t);
    float bc2 = 1.0f - powi(b2, (int)t);
    *lr_t = lr * std::sqrt(bc1 / bc2);
    *eps_t = eps * std::sqrt(bc2);
    *wd_eff = lr * wd;
}

// ---- hash routing and the dispatch permutation
uint32_t orc_hash_route(uint32_t id, uint32_t n_experts) { return hash_route(id, n_experts); }
// perm = concat_e buckets[e] (token indices, ascending inside each expert);
// offsets[e] = start of expert e in perm, offsets[E] = N; route[t] = expert of token t.
void orc_moe_dispatch(const uint32_t* ids, size_t N, size_t E, int32_t* perm, int32_t* offsets,
                      int32_t* route) {
    std::vector<std::vector<size_t>> b;
    build_buckets(ids, N, E, b);
    size_t o = 0;
    for (size_t e = 0; e < E; ++e) {
        offsets[e] = (int32_t)o;
        for (size_t t : b[e]) {
            perm[o++] = (int32_t)t;
            if (route) route[t] = (int32_t)e;
        }
    }
    offsets[E] = (int32_t)o;
}

// ---- delta rule, isolated op (inputs as Gpu::delta_scan receives them: q,k normalised)
// states: nullable, layout ((h*B)+b)*(seq+1)*dh*dh as rust/kernels/asca.cu:275.
// s_final: nullable, layout ((b*H)+h)*dh*dh.
void orc_delta_scan(const float* q, const float* k, const float* v, const float* alpha,
                    const float* beta, size_t B, size_t seq, size_t H, size_t dh, float* o,
                    float* states, float* s_final, int per_chain_threads) {
    if (per_chain_threads) {
        run_jobs(
            H * B,
            [&](size_t j) {
                size_t hh = j / B, bi = j % B;
                scan_chain(q, k, v, alpha, beta, seq, H, dh, hh, bi * seq, o,
                           states ? states + (hh * B + bi) * (seq + 1) * dh * dh : nullptr,
                           s_final ? s_final + (bi * H + hh) * dh * dh : nullptr);
            },
            num_threads());
        return;
    }
    run_jobs(H, [&](size_t hh) {  // the reference's partitioning: one thread per head
        for (size_t bi = 0; bi < B; ++bi)
            scan_chain(q, k, v, alpha, beta, seq, H, dh, hh, bi * seq, o,
                       states ? states + (hh * B + bi) * (seq + 1) * dh * dh : nullptr,
                       s_final ? s_final + (bi * H + hh) * dh * dh : nullptr);
    });
}
// Outputs as Gpu::delta_bwd_dev returns them: d_qkv (N x 3d) after the L2-norm backward,
// d_gate (N x 2H) after the sigmoid backward. max_workers bounds concurrent chains (each
// holds a (seq+1)*dh*dh history); 0 = one thread per chain as in the reference.
void orc_delta_bptt(const float* q, const float* k, const float* v, const float* alpha,
                    const float* beta, const float* qn, const float* kn, const float* d_o,
                    size_t B, size_t seq, size_t H, size_t dh, float* d_qkv, float* d_gate,
                    int max_workers) {
    delta_bptt(q, k, v, alpha, beta, qn, kn, d_o, B, seq, H, dh, d_qkv, d_gate, max_workers);
}
// The independent scalar scan that `asca gpu` uses to check the device kernel
// (rust/src/main.rs:887-928): a second, simpler statement of the recurrence for one chain.
void orc_delta_scan_scalar(const float* q, const float* k, const float* v, const float* alpha,
                           const float* beta, size_t B, size_t seq, size_t H, size_t dh, float* o) {
    const size_t d = H * dh;
    for (size_t bi = 0; bi < B; ++bi)
        for (size_t hh = 0; hh < H; ++hh) {
            std::vector<float> s(dh * dh, 0.0f), sk(dh), u(dh);
            for (size_t t = 0; t < seq; ++t) {
                size_t r = bi * seq + t, off = hh * dh;
                float a = alpha[r * H + hh], b = beta[r * H + hh];
                for (size_t i = 0; i < dh; ++i) {
                    float acc = 0.0f;
                    for (size_t a2 = 0; a2 < dh; ++a2) acc += s[a2 * dh + i] * k[r * d + off + a2];
                    sk[i] = acc;
                }
                for (size_t i = 0; i < dh; ++i) u[i] = b * (v[r * d + off + i] - a * sk[i]);
                for (size_t a2 = 0; a2 < dh; ++a2)
                    for (size_t i = 0; i < dh; ++i)
                        s[a2 * dh + i] = a * s[a2 * dh + i] + k[r * d + off + a2] * u[i];
                for (size_t i = 0; i < dh; ++i) {
                    float acc = 0.0f;
                    for (size_t a2 = 0; a2 < dh; ++a2) acc += s[a2 * dh + i] * q[r * d + off + a2];
                    o[r * d + off + i] = acc;
                }
            }
        }
}

// ---- delta block (projections + scan), parameters passed as six separate arrays
struct orc_delta_cache {
    DeltaCache c;
};
orc_delta_cache* orc_delta_block_forward(const float* w_qkv, const float* b_qkv,
                                         const float* w_gate, const float* b_gate,
                                         const float* w_o, const float* b_o, const float* x,
                                         size_t N, size_t batch, size_t d, size_t H, float* y) {
    auto* h = new orc_delta_cache();
    DeltaParams p{(float*)w_qkv, (float*)b_qkv, (float*)w_gate, (float*)b_gate, (float*)w_o,
                  (float*)b_o};
    delta_block_forward(p, x, N, batch, d, H, y, h->c);
    return h;
}
// Copies cached intermediates out (any pointer may be null).
void orc_delta_cache_get(const orc_delta_cache* h, float* q, float* k, float* v, float* alpha,
                         float* beta, float* qn, float* kn, float* o) {
    auto cp = [](float* dst, const std::vector<float>& s) {
        if (dst) std::memcpy(dst, s.data(), s.size() * sizeof(float));
    };
    cp(q, h->c.q);
    cp(k, h->c.k);
    cp(v, h->c.v);
    cp(alpha, h->c.alpha);
    cp(beta, h->c.beta);
    cp(qn, h->c.qn);
    cp(kn, h->c.kn);
    cp(o, h->c.o);
}
void orc_delta_block_backward(const orc_delta_cache* h, const float* w_qkv, const float* w_gate,
                              const float* w_o, const float* dy, size_t N, size_t d, size_t H,
                              float* g_w_qkv, float* g_b_qkv, float* g_w_gate, float* g_b_gate,
                              float* g_w_o, float* g_b_o, float* dx) {
    DeltaParams p{(float*)w_qkv, nullptr, (float*)w_gate, nullptr, (float*)w_o, nullptr};
    DeltaParams g{g_w_qkv, g_b_qkv, g_w_gate, g_b_gate, g_w_o, g_b_o};
    delta_block_backward(p, g, h->c, dy, N, d, H, dx);
}
void orc_delta_cache_free(orc_delta_cache* h) { delete h; }
void orc_delta_block_step(const float* w_qkv, const float* b_qkv, const float* w_gate,
                          const float* b_gate, const float* w_o, const float* b_o, const float* x,
                          size_t d, size_t H, float* states, float* y) {
    DeltaParams p{(float*)w_qkv, (float*)b_qkv, (float*)w_gate, (float*)b_gate, (float*)w_o,
                  (float*)b_o};
    delta_block_step(p, x, d, H, states, y);
}
// Scan-only decode step on already-normalised q,k (what a decode kernel computes per head):
// rust/src/delta.rs:377-406. S layout (stream, head, dh, dh), updated in place.
void orc_delta_step_core(const float* q, const float* k, const float* v, const float* alpha,
                         const float* beta, float* S, size_t n_streams, size_t H, size_t dh,
                         float* o) {
    const size_t d = H * dh;
    run_jobs(
        n_streams,
        [&](size_t s_i) {
            std::vector<float> sk(dh), u(dh);
            for (size_t hh = 0; hh < H; ++hh) {
                size_t off = s_i * d + hh * dh;
                float a = alpha[s_i * H + hh], b = beta[s_i * H + hh];
                float* s = S + (s_i * H + hh) * dh * dh;
                std::fill(sk.begin(), sk.end(), 0.0f);
                for (size_t ai = 0; ai < dh; ++ai) {
                    float ka = k[off + ai];
                    if (ka == 0.0f) continue;
                    axpy(sk.data(), ka, s + ai * dh, dh);
                }
                for (size_t i = 0; i < dh; ++i) u[i] = b * (v[off + i] - a * sk[i]);
                for (size_t ai = 0; ai < dh; ++ai) {
                    float ka = k[off + ai];
                    if (ka == 0.0f) {
                        scale(s + ai * dh, a, dh);
                        continue;
                    }
                    scale_axpy(s + ai * dh, a, ka, u.data(), dh);
                }
                for (size_t i = 0; i < dh; ++i) {
                    float acc = 0.0f;
                    for (size_t ai = 0; ai < dh; ++ai) acc += s[ai * dh + i] * q[off + ai];
                    o[off + i] = acc;
                }
            }
        },
        num_threads());
}

// ---- hash MoE
// FFN on normalised rows with caller-supplied dispatch (what Gpu::moe_forward_dev receives).
// pre/hidden: nullable (N x F), token order.
void orc_moe_ffn_forward(const float* xn, const float* w1, const float* b1, const float* w2,
                         const float* b2, const uint32_t* ids, size_t N, size_t d, size_t F,
                         size_t E, float* out, float* pre, float* hidden) {
    std::vector<std::vector<size_t>> b;
    build_buckets(ids, N, E, b);
    MoeParams p{(float*)w1, (float*)b1, (float*)w2, (float*)b2};
    moe_ffn_forward(p, xn, N, d, F, E, b, out, pre, hidden);
}
// Gradients are accumulated (+=) into d_w1,d_b1,d_w2,d_b2; dxn is overwritten.
void orc_moe_ffn_backward(const float* xn, const float* w1, const float* w2, const float* pre,
                          const float* hidden, const uint32_t* ids, const float* dout, size_t N,
                          size_t d, size_t F, size_t E, float* d_w1, float* d_b1, float* d_w2,
                          float* d_b2, float* dxn) {
    std::vector<std::vector<size_t>> b;
    build_buckets(ids, N, E, b);
    MoeParams p{(float*)w1, nullptr, (float*)w2, nullptr};
    MoeParams g{d_w1, d_b1, d_w2, d_b2};
    moe_ffn_backward(p, g, xn, pre, hidden, b, dout, N, d, F, E, dxn);
}
// Whole layer incl. the internal RMSNorm (HashMoe::forward / backward).
void orc_moe_forward(const float* x, const float* w1, const float* b1, const float* w2,
                     const float* b2, const uint32_t* ids, size_t N, size_t d, size_t F, size_t E,
                     float* out) {
    MoeParams p{(float*)w1, (float*)b1, (float*)w2, (float*)b2};
    MoeCache c;
    moe_forward(p, x, ids, N, d, F, E, out, c);
}
void orc_moe_forward_backward(const float* x, const float* w1, const float* b1, const float* w2,
                              const float* b2, const uint32_t* ids, const float* dout, size_t N,
                              size_t d, size_t F, size_t E, float* out, float* d_w1, float* d_b1,
                              float* d_w2, float* d_b2, float* dx) {
    MoeParams p{(float*)w1, (float*)b1, (float*)w2, (float*)b2};
    MoeParams g{d_w1, d_b1, d_w2, d_b2};
    MoeCache c;
    moe_forward(p, x, ids, N, d, F, E, out, c);
    moe_backward(p, g, c, dout, N, d, F, E, dx);
}
void orc_moe_step(const float* x, const float* w1, const float* b1, const float* w2,
                  const float* b2, uint32_t id, size_t d, size_t F, size_t E, float* out) {
    MoeParams p{(float*)w1, (float*)b1, (float*)w2, (float*)b2};
    moe_step(p, x, id, d, F, E, out);
}

// ---- whole model on a flat parameter buffer (order rust/src/model.rs:593-609)
size_t orc_model_num_params(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F) {
    return make_layout({vocab, d, H, L, E, F}).total;
}
size_t orc_model_num_tensors(size_t L) { return 2 + 10 * L; }
void orc_model_tensor_table(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                            uint64_t* offs, uint64_t* lens) {
    Layout l = make_layout({vocab, d, H, L, E, F});
    for (size_t i = 0; i < l.tensor_off.size(); ++i) {
        offs[i] = l.tensor_off[i];
        lens[i] = l.tensor_len[i];
    }
}
// rust/src/model.rs:560-587 + rust/src/delta.rs:64-94 + rust/src/model.rs:88-101: draw order
// embed(0.02), head(sqrt(1/d)), per layer w_qkv, w_gate, w_o (sqrt(1/d)), w1 (sqrt(1/d)),
// w2 (sqrt(1/F)); b_gate = -2 / -1; other biases zero. Leaves the rng state advanced so the
// caller can keep drawing ids from the same stream like the reference tests do.
void orc_model_init(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                    uint64_t* rng_state, float* params) {
    Config c{vocab, d, H, L, E, F};
    Layout l = make_layout(c);
    Rng r(0);
    r.s0 = rng_state[0];
    r.s1 = rng_state[1];
    std::fill(params, params + l.total, 0.0f);
    auto fill = [&](size_t off, size_t n, float sc) {
        for (size_t i = 0; i < n; ++i) params[off + i] = r.normal() * sc;
    };
    fill(l.embed, vocab * d, 0.02f);
    fill(l.head, d * vocab, std::sqrt(1.0f / (float)d));
    for (size_t li = 0; li < L; ++li) {
        const auto& y = l.layers[li];
        fill(y.w_qkv, d * 3 * d, std::sqrt(1.0f / (float)d));
        fill(y.w_gate, d * 2 * H, std::sqrt(1.0f / (float)d));
        fill(y.w_o, d * d, std::sqrt(1.0f / (float)d));
        for (size_t j = 0; j < H; ++j) {
            params[y.b_gate + j] = -2.0f;
            params[y.b_gate + H + j] = -1.0f;
        }
        fill(y.w1, d * E * F, std::sqrt(1.0f / (float)d));
        fill(y.w2, E * F * d, std::sqrt(1.0f / (float)F));
    }
    rng_state[0] = r.s0;
    rng_state[1] = r.s1;
}
// forward (+ optional logits copy-out) then backward; grads accumulated (+=). Returns loss.
float orc_model_forward_backward(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                                 const float* params, float* grads, const uint32_t* ids,
                                 const uint32_t* targets, size_t N, size_t batch,
                                 float* logits_out) {
    Config c{vocab, d, H, L, E, F};
    Layout l = make_layout(c);
    std::vector<LayerCache> caches;
    std::vector<float> h_final, logits(N * vocab);
    model_forward(c, l, (float*)params, ids, N, batch, caches, h_final, logits.data());
    if (logits_out) std::memcpy(logits_out, logits.data(), logits.size() * sizeof(float));
    if (!grads) return loss_only(logits.data(), targets, N, vocab);
    return model_backward(c, l, (float*)params, grads, ids, targets, N, caches, h_final,
                          logits.data());
}
void orc_model_forward(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                       const float* params, const uint32_t* ids, size_t N, size_t batch,
                       float* logits) {
    Config c{vocab, d, H, L, E, F};
    Layout l = make_layout(c);
    std::vector<LayerCache> caches;
    std::vector<float> h_final;
    model_forward(c, l, (float*)params, ids, N, batch, caches, h_final, logits);
}
// rust/src/model.rs:703-718 (Model::loss: forward with batch=1, serial CE sum)
float orc_model_loss(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                     const float* params, const uint32_t* ids, const uint32_t* targets, size_t N) {
    std::vector<float> logits(N * vocab);
    orc_model_forward(vocab, d, H, L, E, F, params, ids, N, 1, logits.data());
    return loss_only(logits.data(), targets, N, vocab);
}
// rust/src/model.rs:631-649 (Model::step). state: (L, H, dh, dh) fp32, updated in place.
void orc_model_step(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                    const float* params, uint32_t id, float* state, float* logits) {
    Config c{vocab, d, H, L, E, F};
    Layout l = make_layout(c);
    float* P = (float*)params;
    const size_t dh = d / H;
    std::vector<float> x(P + l.embed + id * d, P + l.embed + (id + 1) * d), dy(d), dm(d), hf(d);
    for (size_t li = 0; li < L; ++li) {
        delta_block_step(delta_view(P, l.layers[li]), x.data(), d, H, state + li * H * dh * dh,
                         dy.data());
        for (size_t i = 0; i < d; ++i) x[i] += 1.0f * dy[i];
        moe_step(moe_view(P, l.layers[li]), x.data(), id, d, F, E, dm.data());
        for (size_t i = 0; i < d; ++i) x[i] += 1.0f * dm[i];
    }
    rmsnorm_rows(x.data(), hf.data(), nullptr, 1, d, EPS);
    matmul(hf.data(), P + l.head, logits, 1, d, vocab);
}
// rust/src/model.rs:798-802 + rust/src/tensor.rs:392-472: one optimizer step = update() per
// tensor in parameter order; the counter advances once PER TENSOR. `counter` in/out.
void orc_model_adamw_step(size_t vocab, size_t d, size_t H, size_t L, size_t E, size_t F,
                          float* params, const float* grads, float* m, float* v, float lr, float b1,
                          float b2, float eps, float wd, uint32_t* counter) {
    Layout l = make_layout({vocab, d, H, L, E, F});
    for (size_t i = 0; i < l.tensor_off.size(); ++i) {
        *counter += 1;
        float lr_t, eps_t, wd_eff;
        orc_adamw_scalars(lr, b1, b2, eps, wd, *counter, &lr_t, &eps_t, &wd_eff);
        size_t off = l.tensor_off[i], n = l.tensor_len[i];
        size_t nt = (size_t)std::max(num_threads(), 1);
        if (nt <= 1 || n < PAR_MIN_ADAM) {
            orc_adamw_apply(params + off, grads + off, m + off, v + off, n, lr_t, b1, b2, eps_t,
                            wd_eff);
        } else {
            size_t chunk = (n + nt - 1) / nt, parts = (n + chunk - 1) / chunk;
            run_jobs(parts, [&](size_t ci) {
                size_t lo = ci * chunk, hi = std::min(n, lo + chunk);
                orc_adamw_apply(params + off + lo, grads + off + lo, m + off + lo, v + off + lo,
                                hi - lo, lr_t, b1, b2, eps_t, wd_eff);
            });
        }
    }
}

}  // extern "C"
