// Self-test of the bounded-wait machinery every kernel of the library relies on: a wait that cannot be
// satisfied must run out, leave its code in the context's status word and return, so that the context
// stays usable.  Nothing here traps, faults or spins without a limit.
#include "internal.h"
#include "ptx.cuh"

namespace b200 {

// One warp.  Lane 0 initialises an mbarrier that expects one arrival, and nobody ever arrives: the
// wait gives up after limit_ns, records KST_WAIT_SELFTEST and raises the CTA's abort flag, which is what
// lets the other lanes (the "other roles" of a real kernel) fall through to the common exit.
__global__ void __launch_bounds__(32) selftest_wait_kernel(int* d_status, unsigned long long limit_ns, int* gave_up) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncwarp();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, d_status, KST_WAIT_SELFTEST, &abort_flag, limit_ns);
    __syncwarp();
    if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = ok ? 0 : (abort_flag ? 1 : 2);
}

} // namespace b200

using namespace b200;

extern "C" int b200_selftest_bounded_wait(b200_ctx* ctx, int64_t limit_ns, int* gave_up_dev) {
    B200_REQUIRE(ctx, B200_EINVAL, "selftest_bounded_wait: null ctx");
    B200_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, B200_EINVAL,
                 "selftest_bounded_wait: limit %lld ns outside (0, 100 ms]", (long long)limit_ns);
    B200_CUDA(cudaSetDevice(ctx->device));
    selftest_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, (unsigned long long)limit_ns, gave_up_dev);
    ctx->launches++;
    B200_CUDA(cudaGetLastError());
    return B200_OK;
}
