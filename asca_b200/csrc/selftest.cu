// Self-test of the give-up path every tensor-core kernel shares: a wait on an mbarrier that nothing will ever
// complete must run out, raise the context's error word, release the TMEM the CTA holds and return -- leaving the
// context usable. The production kernels use the same mbar_wait with a limit of about two seconds; here the limit comes
// from the host (a few thousand cycles) so that the path can be exercised in microseconds without hanging anything.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

__global__ void __launch_bounds__(64) wait_timeout_kernel(long long limit_cycles, int* err_word, int* report) {
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(&bar, 1);     // one arrival expected; nobody arrives
        tc::mbar_fence_init();
    }
    if (warp == 0) tc::tmem_alloc(&tmem_slot, 32);   // hold some TMEM, as a real kernel does while it waits
    tc::tcgen05_fence_before();
    __syncthreads();
    tc::tcgen05_fence_after();
    bool ok = true;
    if (threadIdx.x == 32)   // the role that waits (a consumer warp's elected thread in the real kernels)
        ok = tc::mbar_wait_limit(&bar, 0, &abort_flag, err_word, 77, limit_cycles);
    __syncthreads();
    if (threadIdx.x == 32) report[0] = ok ? 1 : 2;             // 2 = gave up, as it must
    if (threadIdx.x == 0) report[1] = abort_flag;              // the other roles see the abort flag
    tc::tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_slot, 32);            // and the TMEM goes back
}

}  // namespace

extern "C" int asca_selftest_wait_timeout(asca_ctx* ctx, int64_t limit_cycles, int* gave_up, int* abort_seen) {
    if (!ctx) return ASCA_ERR_ARG;
    ASCA_REQUIRE(ctx, limit_cycles > 0 && limit_cycles <= 100000000, "selftest_wait_timeout: the limit must be 1 .. 1e8 cycles");
    void* ws;
    ASCA_TRY(asca_workspace(ctx, 256, &ws));
    int* report = (int*)ws;
    ASCA_CUDA(ctx, cudaMemsetAsync(report, 0, 8, ctx->stream));
    wait_timeout_kernel<<<1, 64, 0, ctx->stream>>>((long long)limit_cycles, ctx->err_word, report);
    ASCA_CHECK_LAUNCH(ctx);
    int host[2] = {0, 0};
    ASCA_CUDA(ctx, cudaMemcpyAsync(host, report, 8, cudaMemcpyDeviceToHost, ctx->stream));
    const int rc = asca_ctx_sync(ctx);   // reads (and clears) the error word: ASCA_ERR_DEVICE is the expected answer
    if (gave_up) *gave_up = host[0] == 2;
    if (abort_seen) *abort_seen = host[1];
    return rc;
}
