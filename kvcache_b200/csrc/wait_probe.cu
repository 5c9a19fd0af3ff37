// A kernel whose only wait cannot end: one thread waits, with the bounded wait every TMA / tcgen05 kernel of this
// package uses (tc::mbar_wait), on an mbarrier that nothing ever arrives on.  The wait runs out of polls, the kernel
// sets the time-out bit of the error word and returns normally - which is how a stalled pipeline shows itself to the
// host (CudaKernels.check_errors) instead of hanging the device.  Built with a short poll limit (KVB_SPIN_LIMIT) so
// that it ends within milliseconds.  The reference has no device-side waits and no counterpart of this.
#include "tc_common.cuh"

namespace {

__global__ void wait_probe_kernel(int* __restrict__ err, int* __restrict__ outcome) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool arrived = tc::mbar_wait(&bar, 0);      // phase 0 never completes: nobody arrives
        if (!arrived) atomicOr(err, tc::KVB_DEV_TIMEOUT);
        outcome[0] = arrived ? 1 : 2;                     // 2: the wait gave up after SPIN_LIMIT polls
        outcome[1] = (int)tc::SPIN_LIMIT;
    }
}

}  // namespace

KVB_API int kvb_wait_probe(int* err, int* outcome, void* stream) {
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(err, outcome);
    return kvb_launch_status();
}
