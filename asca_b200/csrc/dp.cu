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
// loads of our own; NCCL moves the bytes -- or, as an option for the sharded tensors, the copy engines do
// (asca_model_dp_peer_export / _open: peer buffers mapped through CUDA IPC, one cudaMemcpyAsync and one flag store per
// chunk and peer, a bounded poll and a rank-ordered sum on the receiving side; see struct asca_dp).
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
    // Copy-engine transport for the sharded tensors (asca_model_dp_peer_export / _open): the peers' staging, flag and bf16
    // weight buffers mapped through CUDA IPC. A gradient chunk travels as one cudaMemcpyAsync per peer into that peer's
    // staging slot for this rank, followed by a flag (the step number) written into the peer's flag array; the owner of
    // the chunk waits for the flags of all peers (a bounded poll) and sums the slots in rank order. Updated bf16 chunks
    // travel the same way straight into the peers' weight copies. No SM is held while bytes move.
    bool ce = false;
    bool ce_gather = false;                  // the bf16 all-gather on the copy engines too (ASCA_DP_CE_GATHER=1); default: NCCL
    float* stage = nullptr;                  // [(nranks - 1) sources][stage_per_src] incoming gradient chunks
    int* flags = nullptr;                    // [2 kinds][big tensors][nranks]: last step whose chunk from that rank has landed
    std::vector<float*> peer_stage;
    std::vector<int*> peer_flags;
    std::vector<__nv_bfloat16*> peer_p16;
    std::vector<int64_t> stage_off;          // offset (floats) of big tensor i inside one source's staging area
    int64_t stage_per_src = 0;
    static constexpr int N_PUSH = 8;         // copies in flight at once (a single copy does not fill the NVLink ports)
    cudaStream_t push[N_PUSH] = {};
    cudaEvent_t push_ev[N_PUSH] = {}, piece_ev[N_PUSH] = {};
    bool push_open = false;                  // copies queued that the next writer of their sources has not yet waited for
    int step_no = 0;
};

namespace {

// ---- copy-engine transport: the three small kernels
// Peer store of a landed-chunk flag; runs on the stream that carried the chunk, after it.
__global__ void ce_flag_kernel(int* flag, int step) {
    __threadfence_system();
    *reinterpret_cast<volatile int*>(flag) = step;
    __threadfence_system();
}
// Waits until every peer's flag for tensor `t` has reached `step` (lane = rank). Bounded: gives up after `limit` cycles and
// raises the error word; the kernels behind it then run on whatever has landed and the host sees ASCA_ERR_DEVICE.
__global__ void ce_wait_kernel(const int* flags, int nranks, int self, int step, long long limit, int* err_word) {
    const int r = threadIdx.x;
    if (r >= nranks || r == self) return;
    const volatile int* f = flags + r;
    const long long t0 = clock64();
    while (*f < step) {
        if (clock64() - t0 > limit) {
            atomicExch(err_word, 401);
            break;
        }
        __nanosleep(500);
    }
    __threadfence_system();
}
// own[i] = (sum over ranks, in rank order, of that rank's chunk) * scale; the peers' chunks sit in the staging slots.
__global__ void __launch_bounds__(256) ce_reduce_kernel(float* __restrict__ own, const float* __restrict__ stage, int64_t stage_per_src,
                                                        int64_t n4, int nranks, int self, float scale) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int r = 0; r < nranks; ++r) {
            const float4 v = r == self ? reinterpret_cast<const float4*>(own)[i]
                                       : reinterpret_cast<const float4*>(stage + (int64_t)(r < self ? r : r - 1) * stage_per_src)[i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(own)[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
    }
}
constexpr long long CE_WAIT_CYCLES = 40000000000ll;   // about 20 s: ranks may be seconds apart in their first step

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

// The push streams start after whatever the context's stream has queued so far.
int push_after_compute(asca_ctx* ctx, asca_dp* dp) {
    ASCA_CUDA(ctx, cudaEventRecord(dp->comm->ev, ctx->stream));
    for (int i = 0; i < asca_dp::N_PUSH; ++i) ASCA_CUDA(ctx, cudaStreamWaitEvent(dp->push[i], dp->comm->ev, 0));
    return ASCA_OK;
}
// The context's stream waits for every copy the push streams hold (before the copies' sources are written again).
int compute_after_push(asca_ctx* ctx, asca_dp* dp) {
    if (!dp->push_open) return ASCA_OK;
    for (int i = 0; i < asca_dp::N_PUSH; ++i) {
        ASCA_CUDA(ctx, cudaEventRecord(dp->push_ev[i], dp->push[i]));
        ASCA_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, dp->push_ev[i], 0));
    }
    dp->push_open = false;
    return ASCA_OK;
}
// This rank's chunk-for-p of sharded tensor `bi` to every peer p (kind 0: f32 gradient chunk p into p's staging slot for
// this rank; kind 1: this rank's updated bf16 chunk into p's weight copy), each followed by the landed-chunk flag.
int ce_push(asca_ctx* ctx, asca_model* m, asca_dp* dp, int bi, int kind) {
    const asca_dp::Big& b = dp->big[bi];
    const int N = dp->comm->nranks, me = dp->comm->rank;
    const int64_t chunk = b.n / N;
    const int step = dp->step_no + 1;
    // a peer's chunk goes as `pieces` copies on different streams, so that about N_PUSH copies are in flight whatever N is
    const int pieces = std::max(1, asca_dp::N_PUSH / (N - 1));
    const size_t esz = kind == 0 ? 4 : 2;
    for (int k = 1; k < N; ++k) {
        const int p = (me + k) % N;
        char* dst = kind == 0 ? reinterpret_cast<char*>(dp->peer_stage[p] + (int64_t)(me < p ? me : me - 1) * dp->stage_per_src + dp->stage_off[bi])
                              : reinterpret_cast<char*>(dp->peer_p16[p] + b.off + me * chunk);
        const char* src = kind == 0 ? reinterpret_cast<const char*>(m->grads + b.off + p * chunk)
                                    : reinterpret_cast<const char*>(m->params16 + b.off + me * chunk);
        const size_t bytes = (size_t)chunk * esz, piece = ((bytes / pieces) + 255) & ~(size_t)255;
        const int s0 = ((k - 1) * pieces) % asca_dp::N_PUSH;
        for (int j = 0; j < pieces; ++j) {
            const size_t lo = (size_t)j * piece, n = lo < bytes ? std::min(piece, bytes - lo) : 0;
            const int sj = (s0 + j) % asca_dp::N_PUSH;
            if (n) ASCA_CUDA(ctx, cudaMemcpyAsync(dst + lo, src + lo, n, cudaMemcpyDefault, dp->push[sj]));
            if (j > 0) {   // the flag's stream learns of the other pieces
                ASCA_CUDA(ctx, cudaEventRecord(dp->piece_ev[sj], dp->push[sj]));
                ASCA_CUDA(ctx, cudaStreamWaitEvent(dp->push[s0], dp->piece_ev[sj], 0));
            }
        }
        ce_flag_kernel<<<1, 1, 0, dp->push[s0]>>>(dp->peer_flags[p] + ((size_t)kind * dp->big.size() + bi) * N + me, step);
        ASCA_CUDA(ctx, cudaGetLastError());
    }
    dp->push_open = true;
    return ASCA_OK;
}
// On the side stream: wait for every peer's chunk of tensor `bi` (kind as above).
int ce_wait(asca_ctx* ctx, asca_dp* dp, int bi, int kind) {
    const int N = dp->comm->nranks;
    ce_wait_kernel<<<1, 32 * ((N + 31) / 32), 0, dp->comm->side>>>(dp->flags + ((size_t)kind * dp->big.size() + bi) * N, N, dp->comm->rank,
                                                                   dp->step_no + 1, CE_WAIT_CYCLES, ctx->err_word);
    ASCA_CUDA(ctx, cudaGetLastError());
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

int asca_model_dp_peer_export(asca_ctx* ctx, asca_model* m, void* blob256) {
    if (!ctx || !m || !blob256) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, m->dp && m->dp->sharded && m->dp->comm->nranks > 1 && !m->dp->big.empty(),
                 "model_dp_peer_export: needs the sharded optimizer on more than one rank");
    asca_dp* dp = m->dp;
    const int N = dp->comm->nranks;
    cudaSetDevice(ctx->device);
    if (!dp->stage) {
        dp->stage_off.clear();
        dp->stage_per_src = 0;
        for (const asca_dp::Big& b : dp->big) {
            dp->stage_off.push_back(dp->stage_per_src);
            dp->stage_per_src += b.n / N;
        }
        const size_t n_flags = 2 * dp->big.size() * (size_t)N;
        if (cudaMalloc((void**)&dp->stage, (size_t)(N - 1) * dp->stage_per_src * 4) != cudaSuccess ||
            cudaMalloc((void**)&dp->flags, n_flags * 4) != cudaSuccess)
            return asca_fail(ctx, ASCA_ERR_OOM, "model_dp_peer_export: cannot allocate the staging area (%.1f GB)",
                             (double)(N - 1) * dp->stage_per_src * 4 / 1e9);
        ASCA_CUDA(ctx, cudaMemset(dp->flags, 0, n_flags * 4));
    }
    {
        void* p16 = nullptr;   // the bf16 copy must exist before its handle does
        ASCA_TRY(asca_model_params16(ctx, m, &p16, nullptr));
    }
    char* out = static_cast<char*>(blob256);
    memset(out, 0, 256);
    cudaIpcMemHandle_t h;
    ASCA_CUDA(ctx, cudaIpcGetMemHandle(&h, dp->stage));
    memcpy(out, &h, sizeof h);
    ASCA_CUDA(ctx, cudaIpcGetMemHandle(&h, dp->flags));
    memcpy(out + 64, &h, sizeof h);
    ASCA_CUDA(ctx, cudaIpcGetMemHandle(&h, m->params16));
    memcpy(out + 128, &h, sizeof h);
    const int64_t sps = dp->stage_per_src;
    memcpy(out + 192, &sps, 8);
    return ASCA_OK;
}

int asca_model_dp_peer_open(asca_ctx* ctx, asca_model* m, const void* blobs, int nranks) {
    if (!ctx || !m || !blobs) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, m->dp && m->dp->stage && nranks == m->dp->comm->nranks, "model_dp_peer_open: export first, and pass one blob per rank");
    asca_dp* dp = m->dp;
    const int N = nranks, me = dp->comm->rank;
    cudaSetDevice(ctx->device);
    dp->peer_stage.assign(N, nullptr);
    dp->peer_flags.assign(N, nullptr);
    dp->peer_p16.assign(N, nullptr);
    const char* in = static_cast<const char*>(blobs);
    for (int p = 0; p < N; ++p) {
        if (p == me) continue;
        const char* b = in + (size_t)p * 256;
        int64_t sps = 0;
        memcpy(&sps, b + 192, 8);
        ASCA_REQUIRE(ctx, sps == dp->stage_per_src, "model_dp_peer_open: rank %d was built for another model or world size", p);
        cudaIpcMemHandle_t h;
        void* ptr = nullptr;
        memcpy(&h, b, sizeof h);
        ASCA_CUDA(ctx, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        dp->peer_stage[p] = static_cast<float*>(ptr);
        memcpy(&h, b + 64, sizeof h);
        ASCA_CUDA(ctx, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        dp->peer_flags[p] = static_cast<int*>(ptr);
        memcpy(&h, b + 128, sizeof h);
        ASCA_CUDA(ctx, cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        dp->peer_p16[p] = static_cast<__nv_bfloat16*>(ptr);
    }
    for (int i = 0; i < asca_dp::N_PUSH; ++i) {
        ASCA_CUDA(ctx, cudaStreamCreateWithFlags(&dp->push[i], cudaStreamNonBlocking));
        ASCA_CUDA(ctx, cudaEventCreateWithFlags(&dp->push_ev[i], cudaEventDisableTiming));
        ASCA_CUDA(ctx, cudaEventCreateWithFlags(&dp->piece_ev[i], cudaEventDisableTiming));
    }
    dp->ce = true;
    {
        const char* e = getenv("ASCA_DP_CE_GATHER");
        dp->ce_gather = e && e[0] == '1';
    }
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
    if (dp->ce) ASCA_TRY(compute_after_push(ctx, dp));   // this rank's chunks have left: the update may rewrite their sources
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
            const bool last_of_layer = (size_t)g.big + 1 == dp->big.size() || dp->big[g.big + 1].layer != b.layer;
            if (dp->ce && dp->ce_gather) {
                ASCA_TRY(push_after_compute(ctx, dp));
                ASCA_TRY(ce_push(ctx, m, dp, g.big, 1));
                if (last_of_layer)   // the block's chunks of every peer have landed in this rank's copy
                    for (int bj = 0; bj <= g.big; ++bj)
                        if (dp->big[bj].layer == b.layer) ASCA_TRY(ce_wait(ctx, dp, bj, 1));
            } else {
                ASCA_TRY(side_after_compute(ctx, c));
                ASCA_NCCL(ctx, nc->AllGather(m->params16 + b.off + c->rank * chunk, m->params16 + b.off, (size_t)chunk, NCCL_BFLOAT16,
                                             c->comm, c->side));
            }
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
    ++dp->step_no;
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
    if (dp->ce) {   // the sharded tensors inside the range travel on the copy engines
        bool any = false;
        for (size_t bi = 0; bi < dp->big.size(); ++bi) {
            const asca_dp::Big& b = dp->big[bi];
            if (b.off < off || b.off + b.n > off + cnt) continue;
            if (!any) ASCA_TRY(push_after_compute(ctx, dp));
            any = true;
            ASCA_TRY(ce_push(ctx, m, dp, (int)bi, 0));
        }
        for (size_t bi = 0; bi < dp->big.size(); ++bi) {
            const asca_dp::Big& b = dp->big[bi];
            if (b.off < off || b.off + b.n > off + cnt) continue;
            const int64_t chunk = b.n / c->nranks;
            ASCA_TRY(ce_wait(ctx, dp, (int)bi, 0));
            ce_reduce_kernel<<<(unsigned)std::min<int64_t>((chunk / 4 + 255) / 256, 148 * 8), 256, 0, c->side>>>(
                g + b.off + c->rank * chunk, dp->stage + dp->stage_off[bi], dp->stage_per_src, chunk / 4, c->nranks, c->rank,
                1.0f / (float)c->nranks);
            ASCA_CUDA(ctx, cudaGetLastError());
        }
    }
    ASCA_NCCL(ctx, nc->GroupStart());
    int64_t pos = off;
    const int64_t end = off + cnt;
    for (const asca_dp::Big& b : dp->big) {   // cut the range at the sharded tensors inside it
        if (b.off < off || b.off + b.n > end) continue;
        if (b.off > pos) ASCA_NCCL(ctx, nc->AllReduce(g + pos, g + pos, (size_t)(b.off - pos), NCCL_FLOAT32, NCCL_AVG, c->comm, c->side));
        const int64_t chunk = b.n / c->nranks;
        if (!dp->ce)
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
    if (dp && dp->ce) ASCA_TRY(compute_after_push(ctx, dp));   // before this step's backward rewrites the gradient buffer
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
    // Everything this rank queued has run: in particular its polls for the peers' chunks, so no peer copy into this
    // rank's buffers is still on its way when they are freed below (a peer frees only after the same waits on its side).
    if (dp->comm && dp->comm->side) cudaStreamSynchronize(dp->comm->side);
    for (cudaEvent_t e : dp->ag_done) cudaEventDestroy(e);
    for (cudaEvent_t e : dp->ag_waited) cudaEventDestroy(e);
    for (cudaEvent_t e : dp->fwd_reach) cudaEventDestroy(e);
    for (cudaEvent_t e : {dp->t_bwd_end, dp->t_comm_end, dp->t_adam_start, dp->t_adam_end, dp->t_ag_end})
        if (e) cudaEventDestroy(e);
    for (int i = 0; i < asca_dp::N_PUSH; ++i) {
        if (dp->push[i]) {
            cudaStreamSynchronize(dp->push[i]);
            cudaStreamDestroy(dp->push[i]);
        }
        if (dp->push_ev[i]) cudaEventDestroy(dp->push_ev[i]);
        if (dp->piece_ev[i]) cudaEventDestroy(dp->piece_ev[i]);
    }
    for (float* p : dp->peer_stage) if (p) cudaIpcCloseMemHandle(p);
    for (int* p : dp->peer_flags) if (p) cudaIpcCloseMemHandle(p);
    for (__nv_bfloat16* p : dp->peer_p16) if (p) cudaIpcCloseMemHandle(p);
    if (dp->stage) cudaFree(dp->stage);
    if (dp->flags) cudaFree(dp->flags);
    delete dp;
    m->dp = nullptr;
}
