// Self-test of the failure-detection chain, without any fault: a kernel whose CTAs wait, with a short
// limit, on an mbarrier that nothing ever completes.  The wait runs out, the CTA reports a code through
// the device status word and sets the launch-wide abort flag exactly as the attention kernels do; CTAs
// that start after the flag is set skip their wait.  The context stays usable.
#include "kfa_common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace kfa {
namespace {

__global__ void __launch_bounds__(64) wait_probe(int* status, int* abort_flag, long long limit, int* skipped) {
    __shared__ uint64_t never;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = *reinterpret_cast<volatile int*>(abort_flag) != 0 ? 90 : 0;
        mbar_init(&never, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (abort_word != 0) {
        if (threadIdx.x == 0) atomicAdd(skipped, 1);  // an earlier CTA gave up: nothing to do
    } else if (threadIdx.x == 32) {
        mbar_wait_limit(&never, 0, &abort_word, 1, limit);
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_word != 0 && abort_word != 90) {
        *status = 9000 + abort_word;
        *reinterpret_cast<volatile int*>(abort_flag) = 1;
    }
}

}  // namespace

cudaError_t launch_wait_probe(int* status, int* abort_flag, long long limit, int ctas, int* skipped, cudaStream_t st) {
    wait_probe<<<ctas, 64, 0, st>>>(status, abort_flag, limit, skipped);
    return cudaGetLastError();
}

}  // namespace kfa
