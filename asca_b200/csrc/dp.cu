// Data-parallel training: the one exchange the path needs, behind the C ABI.
//
// The path shards by sequence (chains, token rows and decode streams never read another rank's data; heads and
// experts stay local), so training needs exactly one exchange per step: the mean of the flat gradient buffer over
// the ranks (the property rust/tests/batch_parity.rs pins: batch = B equals the mean of B x batch = 1). It runs as
// NCCL collectives on a side stream owned by the model's data-parallel state, queued from inside the backward as
// each range of the gradient buffer is final, so that the transfer of one block's gradients runs under the
// backward of the blocks before it. Two optimizers:
//   replicated  every range is all-reduced (mean), every rank applies the same AdamW update;
//   sharded     the experts' W1 / W2 (98 % of the parameters at the training configuration) are reduce-scattered
//               instead (half the bytes), a rank updates its 1/N chunk of them plus every small tensor, and the
//               updated bf16 chunks are all-gathered into every rank's bf16 weight copy. The all-gather is queued
//               block by block, first block first, and the NEXT forward waits for a block's weights only when it
//               reaches that block's expert products, so the gather runs under the forward.
// NCCL is loaded at run time (dlopen) on the first asca_comm_* call: a single-GPU user of the library needs no NCCL
// at all, and a process that already holds a copy (a framework's) shares it. No peer-memory loads and no multicast
// loads of our own; NCCL moves the bytes.
#include "model.cuh"

#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace {

// The slice of NCCL's C API this file uses, declared here so that building the library needs no NCCL header.
// Values are those of nccl.h 2.10 and later (ncclAvg exists since 2.10).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { NCCL_SUM = 0, NCCL_AVG = 4 };
enum { NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9 };

struct Nccl {
    void* handle = nullptr;
    int (*GetVersion)(int*) = nullptr;
    int (*GetUniqueId)(ncclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    std::string error;
};

Nccl* nccl() {
    static Nccl n;
    static bool tried = false;
    if (tried) return &n;
    tried = true;
    const char* env = getenv("ASCA_NCCL_LIB");
    if (env && *env) n.handle = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
    if (!n.handle) n.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // a copy the process already holds
    if (!n.handle) n.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.handle) n.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!n.handle) {
        n.error = "cannot load libnccl.so.2 (set ASCA_NCCL_LIB to its path)";
        return &n;
    }
    bool ok = true;
    auto sym = [&](const char* name) {
        void* p = dlsym(n.handle, name);
        if (!p) {
            ok = false;
            n.error = std::string("libnccl lacks ") + name;
        }
        return p;
    };
    n.GetVersion = (decltype(n.GetVersion))sym("ncclGetVersion");
    n.GetUniqueId = (decltype(n.GetUniqueId))sym("ncclGetUniqueId");
    n.CommInitRank = (decltype(n.CommInitRank))sym("ncclCommInitRank");
    n.CommDestroy = (decltype(n.CommDestroy))sym("ncclCommDestroy");
    n.GetErrorString = (decltype(n.GetErrorString))sym("ncclGetErrorString");
    n.AllReduce = (decltype(n.AllReduce))sym("ncclAllReduce");
    n.ReduceScatter = (decltype(n.ReduceScatter))sym("ncclReduceScatter");
    n.AllGather = (decltype(n.AllGather))sym("ncclAllGather");
    n.GroupStart = (decltype(n.GroupStart))sym("ncclGroupStart");
    n.GroupEnd = (decltype(n.GroupEnd))sym("ncclGroupEnd");
    if (!ok) {
        n.handle = nullptr;
        return &n;
    }
    int v = 0;
    if (n.GetVersion(&v) != ncclSuccess || v < 21000) {
        n.error = "libnccl is older than 2.10 (no ncclAvg)";
        n.handle = nullptr;
    }
    return &n;
}

}  // namespace

struct asca_comm {
    ncclComm_t comm = nullptr;
    int nranks = 1, rank = 0, device = 0;
    cudaStream_t side = nullptr;     // every collective of this communicator runs here
    cudaEvent_t ev = nullptr;        // hand-over between the context's stream and the side stream
};

#define ASCA_NCCL(ctx, call)                                                                                   \
    do {                                                                                                       \
        int r__ = (call);                                                                                      \
        if (r__ != ncclSuccess)                                                                                \
            return asca_fail((ctx), ASCA_ERR_CUDA, "NCCL error %d (%s) at %s:%d", r__, nccl()->GetErrorString(r__), \
                             __FILE__, __LINE__);                                                              \
    } while (0)

// The data-parallel state of one model.
struct asca_dp {
    asca_comm* comm = nullptr;
    int sharded = 0;
    bool armed = false;             // the next backward queues its exchanges
    bool exchange_open = false;     // collectives queued since the last finish
    struct Big { int64_t off, n; int layer; };
    std::vector<Big> big;           // the sharded tensors in buffer order
    struct Group { std::vector<int64_t> lo, hi; int big; };   // update ranges issued together, then big's all-gather
    std::vector<Group> groups;
    // per block: the all-gather of its bf16 expert weights, pending until the next forward reaches the block
    std::vector<cudaEvent_t> ag_done, fwd_reach;
    std::vector<char> ag_pending, ag_timed;
    // the events the forward of the step being timed waited on (ag_done of the step before), for the timeline
    std::vector<cudaEvent_t> ag_waited;
    std::vector<char> waited_timed;
    // timeline of the last step (CUDA events, read by asca_model_dp_timeline)
    cudaEvent_t t_bwd_end = nullptr, t_comm_end = nullptr, t_adam_start = nullptr, t_adam_end = nullptr, t_ag_end = nullptr;
    bool have_step = false;
    float last_exposed_gather_ms = 0.0f;
};

namespace {

int side_after_compute(asca_ctx* ctx, asca_comm* c) {
    ASCA_CUDA(ctx, cudaEventRecord(c->ev, ctx->stream));
    ASCA_CUDA(ctx, cudaStreamWaitEvent(c->side, c->ev, 0));
    return ASCA_OK;
}
int compute_after_side(asca_ctx* ctx, asca_comm* c) {
    ASCA_CUDA(ctx, cudaEventRecord(c->ev, c->side));
    ASCA_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, c->ev, 0));
    return ASCA_OK;
}

// The sharded tensors of a model at `nranks`: W1 and W2 of every block whose size 4 * nranks divides (a chunk then
// starts on a 16-byte boundary in both the f32 and the bf16 buffer).
void plan_big(const asca_model* m, int nranks, std::vector<asca_dp::Big>* big) {
    big->clear();
    if (nranks <= 1) return;
    for (int li = 0; li < (int)m->L; ++li) {
        const Lyr& w = m->lay[li];
        const int64_t n = m->d * m->E * m->F;
        if (n % (4 * (int64_t)nranks) != 0) continue;
        big->push_back({w.w1, n, li});
        big->push_back({w.w2, n, li});
    }
}

// The ranges `rank` updates: its chunk of every sharded tensor and every other tensor whole; adjacent ranges merged.
void plan_slices(const asca_model* m, const std::vector<asca_dp::Big>& big, int nranks, int rank, std::vector<int64_t>* lo,
                 std::vector<int64_t>* hi) {
    lo->clear();
    hi->clear();
    size_t b = 0;
    for (size_t i = 0; i + 1 < m->seg_off.size(); ++i) {
        int64_t a = m->seg_off[i], e = m->seg_off[i + 1];
        if (b < big.size() && big[b].off == a) {
            const int64_t c = big[b].n / nranks;
            a = big[b].off + rank * c;
            e = a + c;
            ++b;
        }
        if (!lo->empty() && hi->back() == a) hi->back() = e;
        else {
            lo->push_back(a);
            hi->push_back(e);
        }
    }
}

}  // namespace

extern "C" {

int asca_comm_unique_id(asca_ctx* ctx, void* id128) {
    if (!id128) return asca_fail(ctx, ASCA_ERR_ARG, "comm_unique_id: null buffer");
    Nccl* n = nccl();
    if (!n->handle) return asca_fail(ctx, ASCA_ERR_UNSUPPORTED, "%s", n->error.c_str());
    ncclUniqueId id;
    ASCA_NCCL(ctx, n->GetUniqueId(&id));
    memcpy(id128, &id, sizeof id);
    return ASCA_OK;
}

int asca_comm_init(asca_ctx* ctx, int nranks, int rank, const void* id128, asca_comm** out) {
    if (!ctx || !out) return ASCA_ERR_ARG;
    *out = nullptr;
    ASCA_REQUIRE(ctx, nranks >= 1 && rank >= 0 && rank < nranks, "comm_init: rank %d of %d", rank, nranks);
    asca_comm* c = new asca_comm();
    c->nranks = nranks;
    c->rank = rank;
    c->device = ctx->device;
    cudaSetDevice(ctx->device);
    if (cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev, cudaEventDisableTiming) != cudaSuccess) {
        delete c;
        return asca_fail(ctx, ASCA_ERR_CUDA, "comm_init: cannot create the side stream");
    }
    if (nranks > 1) {
        Nccl* n = nccl();
        if (!n->handle || !id128) {
            cudaStreamDestroy(c->side);
            cudaEventDestroy(c->ev);
            delete c;
            return asca_fail(ctx, n->handle ? ASCA_ERR_ARG : ASCA_ERR_UNSUPPORTED, "%s",
                             n->handle ? "comm_init: null unique id" : n->error.c_str());
        }
        ncclUniqueId id;
        memcpy(&id, id128, sizeof id);
        int r = n->CommInitRank(&c->comm, nranks, id, rank);
        if (r != ncclSuccess) {
            cudaStreamDestroy(c->side);
            cudaEventDestroy(c->ev);
            delete c;
            return asca_fail(ctx, ASCA_ERR_CUDA, "NCCL error %d (%s) in ncclCommInitRank", r, n->GetErrorString(r));
        }
    }
    *out = c;
    return ASCA_OK;
}

int asca_comm_destroy(asca_ctx* ctx, asca_comm* c) {
    if (!c) return ASCA_OK;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->side);
    if (c->comm) nccl()->CommDestroy(c->comm);
    cudaEventDestroy(c->ev);
    cudaStreamDestroy(c->side);
    delete c;
    (void)ctx;
    return ASCA_OK;
}

int asca_comm_info(const asca_comm* c, int* nranks, int* rank) {
    if (!c) return ASCA_ERR_ARG;
    if (nranks) *nranks = c->nranks;
    if (rank) *rank = c->rank;
    return ASCA_OK;
}

int asca_allreduce_grads(asca_ctx* ctx, asca_comm* c, float* flat_grad, int64_t n, const int64_t* bucket_off,
                         int n_buckets) {
    if (!ctx || !c) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, flat_grad && n >= 0, "allreduce_grads: bad buffer");
    if (c->nranks == 1 || n == 0) return ASCA_OK;
    const int64_t whole[2] = {0, n};
    if (!bucket_off || n_buckets <= 0) {
        bucket_off = whole;
        n_buckets = 1;
    }
    ASCA_REQUIRE(ctx, bucket_off[0] == 0 && bucket_off[n_buckets] == n, "allreduce_grads: the buckets must tile [0, n)");
    for (int b = 0; b < n_buckets; ++b)
        ASCA_REQUIRE(ctx, bucket_off[b + 1] >= bucket_off[b], "allreduce_grads: bucket offsets must ascend");
    ASCA_TRY(side_after_compute(ctx, c));
    Nccl* nc = nccl();
    for (int b = n_buckets - 1; b >= 0; --b) {   // the backward finishes the end of the buffer first
        const int64_t lo = bucket_off[b], len = bucket_off[b + 1] - lo;
        if (len > 0) ASCA_NCCL(ctx, nc->AllReduce(flat_grad + lo, flat_grad + lo, (size_t)len, NCCL_FLOAT32, NCCL_AVG, c->comm, c->side));
    }
    return compute_after_side(ctx, c);
}

int asca_dp_shard_plan(int64_t vocab, int64_t d, int64_t H, int64_t L, int64_t E, int64_t F, int nranks, int rank,
                       int64_t* lo, int64_t* hi, int capacity, int* n_slices, int64_t* big_off, int64_t* big_len,
                       int big_capacity, int* n_big) {
    if (vocab <= 0 || d <= 0 || H <= 0 || L <= 0 || E <= 0 || F <= 0 || nranks < 1 || rank < 0 || rank >= nranks) return ASCA_ERR_ARG;
    asca_model m;
    m.vocab = vocab; m.d = d; m.H = H; m.L = L; m.E = E; m.F = F;
    int64_t o = 0;
    auto take = [&](int64_t n) {
        const int64_t at = o;
        m.seg_off.push_back(at);
        o += n;
        return at;
    };
    take(vocab * d);
    take(d * vocab);
    for (int64_t i = 0; i < L; ++i) {
        Lyr y;
        y.w_qkv = take(d * 3 * d); y.b_qkv = take(3 * d); y.w_gate = take(d * 2 * H); y.b_gate = take(2 * H);
        y.w_o = take(d * d); y.b_o = take(d); y.w1 = take(d * E * F); y.b1 = take(E * F); y.w2 = take(E * F * d); y.b2 = take(d);
        m.lay.push_back(y);
    }
    m.seg_off.push_back(o);
    m.n_params = o;
    std::vector<asca_dp::Big> big;
    plan_big(&m, nranks, &big);
    std::vector<int64_t> l, h;
    plan_slices(&m, big, nranks, rank, &l, &h);
    if (n_slices) *n_slices = (int)l.size();
    if (n_big) *n_big = (int)big.size();
    if ((lo || hi) && (int)l.size() > capacity) return ASCA_ERR_ARG;
    if ((big_off || big_len) && (int)big.size() > big_capacity) return ASCA_ERR_ARG;
    for (size_t i = 0; i < l.size(); ++i) {
        if (lo) lo[i] = l[i];
        if (hi) hi[i] = h[i];
    }
    for (size_t i = 0; i < big.size(); ++i) {
        if (big_off) big_off[i] = big[i].off;
        if (big_len) big_len[i] = big[i].n;
    }
    return ASCA_OK;
}

int asca_model_dp_attach(asca_ctx* ctx, asca_model* m, asca_comm* comm, int sharded) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    if (m->dp) {
        ASCA_TRY(asca_dp_wait_all(ctx, m));
        cudaStreamSynchronize(m->dp->comm->side);
        asca_dp_free(m);
    }
    if (!comm) return ASCA_OK;
    ASCA_REQUIRE(ctx, comm->device == ctx->device, "model_dp_attach: the communicator belongs to another device");
    if (sharded && comm->nranks > 1)
        ASCA_REQUIRE(ctx, m->compute == ASCA_BF16 && m->n16 == m->n_params,
                     "model_dp_attach: the sharded optimizer needs bf16 compute mode with an unpadded bf16 weight copy");
    asca_dp* dp = new asca_dp();
    dp->comm = comm;
    dp->sharded = sharded && comm->nranks > 1;
    cudaSetDevice(ctx->device);
    if (dp->sharded) {
        plan_big(m, comm->nranks, &dp->big);
        std::vector<int64_t> lo, hi;
        plan_slices(m, dp->big, comm->nranks, comm->rank, &lo, &hi);
        // the update is issued tensor group by tensor group, so that a sharded tensor's all-gather can start while
        // the next group is being updated: cut the ranges at the sharded tensors' ends
        size_t k = 0;
        int64_t carry_lo = -1;
        for (size_t b = 0; b <= dp->big.size(); ++b) {
            const int64_t cut = b < dp->big.size() ? dp->big[b].off + dp->big[b].n : m->n_params;
            asca_dp::Group g;
            g.big = b < dp->big.size() ? (int)b : -1;
            while (k < lo.size() && (carry_lo >= 0 ? carry_lo : lo[k]) < cut) {
                const int64_t a = carry_lo >= 0 ? carry_lo : lo[k];
                if (hi[k] <= cut) {
                    g.lo.push_back(a);
                    g.hi.push_back(hi[k]);
                    carry_lo = -1;
                    ++k;
                } else {
                    g.lo.push_back(a);
                    g.hi.push_back(cut);
                    carry_lo = cut;
                }
            }
            dp->groups.push_back(g);
        }
        dp->ag_done.resize(m->L);
        dp->ag_waited.resize(m->L);
        dp->fwd_reach.resize(m->L);
        dp->ag_pending.assign(m->L, 0);
        dp->ag_timed.assign(m->L, 0);
        dp->waited_timed.assign(m->L, 0);
        for (int64_t i = 0; i < m->L; ++i) {
            cudaEventCreate(&dp->ag_done[i]);
            cudaEventCreate(&dp->ag_waited[i]);
            cudaEventCreate(&dp->fwd_reach[i]);
        }
    }
    for (cudaEvent_t* e : {&dp->t_bwd_end, &dp->t_comm_end, &dp->t_adam_start, &dp->t_adam_end, &dp->t_ag_end}) cudaEventCreate(e);
    m->dp = dp;
    return ASCA_OK;
}

int asca_model_dp_arm(asca_model* m, int on) {
    if (!m || !m->dp) return ASCA_ERR_ARG;
    m->dp->armed = on != 0;
    return ASCA_OK;
}

int asca_model_dp_step(asca_ctx* ctx, asca_model* m, float lr, float beta1, float beta2, float eps, float wd) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, m->dp, "model_dp_step: no communicator attached");
    asca_dp* dp = m->dp;
    asca_comm* c = dp->comm;
    ASCA_TRY(asca_dp_wait_all(ctx, m));   // a gather of the previous step nobody waited for
    // wait for the exchanges queued by the backward
    ASCA_CUDA(ctx, cudaEventRecord(dp->t_bwd_end, ctx->stream));
    ASCA_CUDA(ctx, cudaEventRecord(dp->t_comm_end, c->side));
    ASCA_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, dp->t_comm_end, 0));
    dp->exchange_open = false;
    dp->armed = false;
    ASCA_CUDA(ctx, cudaEventRecord(dp->t_adam_start, ctx->stream));
    if (!dp->sharded) {
        ASCA_TRY(asca_model_adamw_step(ctx, m, lr, beta1, beta2, eps, wd));
        ASCA_CUDA(ctx, cudaEventRecord(dp->t_adam_end, ctx->stream));
        ASCA_CUDA(ctx, cudaEventRecord(dp->t_ag_end, ctx->stream));
        dp->have_step = true;
        return ASCA_OK;
    }
    {
        void* p16 = nullptr;   // the bf16 copy exists and is current
        ASCA_TRY(asca_model_params16(ctx, m, &p16, nullptr));
    }
    // the forward of this step waited on the previous step's gather events: keep them for the timeline and record
    // this step's gathers into the other set
    std::swap(dp->ag_done, dp->ag_waited);
    dp->waited_timed = dp->ag_timed;
    dp->ag_timed.assign(dp->ag_timed.size(), 0);
    Nccl* nc = nccl();
    int last = -1;
    for (size_t i = 0; i < dp->groups.size(); ++i)
        if (!dp->groups[i].lo.empty()) last = (int)i;
    for (size_t i = 0; i < dp->groups.size(); ++i) {
        const asca_dp::Group& g = dp->groups[i];
        if (!g.lo.empty())
            ASCA_TRY(asca_model_adamw_slices(ctx, m, lr, beta1, beta2, eps, wd, g.lo.data(), g.hi.data(), (int)g.lo.size(), (int)i == last));
        if (g.big >= 0) {
            const asca_dp::Big& b = dp->big[g.big];
            const int64_t chunk = b.n / c->nranks;
            ASCA_TRY(side_after_compute(ctx, c));
            ASCA_NCCL(ctx, nc->AllGather(m->params16 + b.off + c->rank * chunk, m->params16 + b.off, (size_t)chunk, NCCL_BFLOAT16,
                                         c->comm, c->side));
            const bool last_of_layer = (size_t)g.big + 1 == dp->big.size() || dp->big[g.big + 1].layer != b.layer;
            if (last_of_layer) {
                ASCA_CUDA(ctx, cudaEventRecord(dp->ag_done[b.layer], c->side));
                dp->ag_pending[b.layer] = 1;
            }
        }
    }
    ASCA_CUDA(ctx, cudaEventRecord(dp->t_adam_end, ctx->stream));
    ASCA_CUDA(ctx, cudaEventRecord(dp->t_ag_end, c->side));
    m->master_stale = true;
    dp->have_step = true;
    return ASCA_OK;
}

int asca_model_dp_gather_master(asca_ctx* ctx, asca_model* m) {
    if (!ctx || !m) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, m->dp, "model_dp_gather_master: no communicator attached");
    asca_dp* dp = m->dp;
    asca_comm* c = dp->comm;
    ASCA_TRY(asca_dp_wait_all(ctx, m));
    if (dp->sharded) {
        Nccl* nc = nccl();
        ASCA_TRY(side_after_compute(ctx, c));
        for (float* buf : {m->params, m->m, m->v})
            for (const asca_dp::Big& b : dp->big) {
                const int64_t chunk = b.n / c->nranks;
                ASCA_NCCL(ctx, nc->AllGather(buf + b.off + c->rank * chunk, buf + b.off, (size_t)chunk, NCCL_FLOAT32, c->comm, c->side));
            }
        ASCA_TRY(compute_after_side(ctx, c));
    }
    m->master_stale = false;
    return asca_ctx_sync(ctx);
}

int asca_model_dp_timeline(asca_ctx* ctx, asca_model* m, float* ms4) {
    if (!ctx || !m || !ms4) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, m->dp && m->dp->have_step, "model_dp_timeline: no step recorded");
    asca_dp* dp = m->dp;
    ASCA_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ASCA_CUDA(ctx, cudaStreamSynchronize(dp->comm->side));
    float exch = 0, adam = 0, tail = 0;
    ASCA_CUDA(ctx, cudaEventElapsedTime(&exch, dp->t_bwd_end, dp->t_comm_end));
    ASCA_CUDA(ctx, cudaEventElapsedTime(&adam, dp->t_adam_start, dp->t_adam_end));
    ASCA_CUDA(ctx, cudaEventElapsedTime(&tail, dp->t_adam_end, dp->t_ag_end));
    float exposed = 0;
    for (size_t i = 0; i < dp->waited_timed.size(); ++i)
        if (dp->waited_timed[i]) {
            float t = 0;
            if (cudaEventElapsedTime(&t, dp->fwd_reach[i], dp->ag_waited[i]) == cudaSuccess && t > 0) exposed += t;
        }
    cudaGetLastError();
    dp->last_exposed_gather_ms = exposed;
    ms4[0] = exch > 0 ? exch : 0;     // the backward's end waited this long for the gradient exchange
    ms4[1] = adam;                    // the optimizer update (this rank's share)
    ms4[2] = tail > 0 ? tail : 0;     // the weight all-gather ran this long past the update
    ms4[3] = exposed;                 // the forward that followed waited this long for gathered weights
    return ASCA_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ called from the model's dataflow (model.cu)
int asca_dp_grad_ready(asca_ctx* ctx, asca_model* m, int64_t off, int64_t cnt) {
    asca_dp* dp = m->dp;
    if (!dp || !dp->armed || dp->comm->nranks == 1 || cnt <= 0) return ASCA_OK;
    asca_comm* c = dp->comm;
    Nccl* nc = nccl();
    ASCA_TRY(side_after_compute(ctx, c));
    float* g = m->grads;
    ASCA_NCCL(ctx, nc->GroupStart());
    int64_t pos = off;
    const int64_t end = off + cnt;
    for (const asca_dp::Big& b : dp->big) {   // cut the range at the sharded tensors inside it
        if (b.off < off || b.off + b.n > end) continue;
        if (b.off > pos) ASCA_NCCL(ctx, nc->AllReduce(g + pos, g + pos, (size_t)(b.off - pos), NCCL_FLOAT32, NCCL_AVG, c->comm, c->side));
        const int64_t chunk = b.n / c->nranks;
        ASCA_NCCL(ctx, nc->ReduceScatter(g + b.off, g + b.off + c->rank * chunk, (size_t)chunk, NCCL_FLOAT32, NCCL_AVG, c->comm, c->side));
        pos = b.off + b.n;
    }
    if (pos < end) ASCA_NCCL(ctx, nc->AllReduce(g + pos, g + pos, (size_t)(end - pos), NCCL_FLOAT32, NCCL_AVG, c->comm, c->side));
    ASCA_NCCL(ctx, nc->GroupEnd());
    dp->exchange_open = true;
    return ASCA_OK;
}

int asca_dp_before_expert_weights(asca_ctx* ctx, asca_model* m, int64_t layer) {
    asca_dp* dp = m->dp;
    if (!dp || dp->ag_pending.empty() || !dp->ag_pending[layer]) return ASCA_OK;
    ASCA_CUDA(ctx, cudaEventRecord(dp->fwd_reach[layer], ctx->stream));
    ASCA_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, dp->ag_done[layer], 0));
    dp->ag_pending[layer] = 0;
    dp->ag_timed[layer] = 1;
    return ASCA_OK;
}

int asca_dp_wait_all(asca_ctx* ctx, asca_model* m) {
    asca_dp* dp = m->dp;
    if (!dp) return ASCA_OK;
    for (size_t i = 0; i < dp->ag_pending.size(); ++i)
        if (dp->ag_pending[i]) {
            ASCA_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, dp->ag_done[i], 0));
            dp->ag_pending[i] = 0;
            dp->ag_timed[i] = 0;
        }
    return ASCA_OK;
}

void asca_dp_free(asca_model* m) {
    asca_dp* dp = m->dp;
    if (!dp) return;
    for (cudaEvent_t e : dp->ag_done) cudaEventDestroy(e);
    for (cudaEvent_t e : dp->ag_waited) cudaEventDestroy(e);
    for (cudaEvent_t e : dp->fwd_reach) cudaEventDestroy(e);
    for (cudaEvent_t e : {dp->t_bwd_end, dp->t_comm_end, dp->t_adam_start, dp->t_adam_end, dp->t_ag_end})
        if (e) cudaEventDestroy(e);
    delete dp;
    m->dp = nullptr;
}
