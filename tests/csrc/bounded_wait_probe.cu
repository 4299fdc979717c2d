// Test-only kernel (built by tests/test_gpu_bounded_wait.py, never shipped with the package):
// one thread waits with kl::mbar_wait, the bounded wait of the tensor-core kernels, on an
// mbarrier at which nothing ever arrives, with a limit of 4,096 polls.  The wait must give up,
// raise the CTA's abort flag and write its code into the device's status word; the kernel then
// returns normally.  Nothing traps, faults or spins without a limit.
#include "tcgen05.cuh"

namespace {
__global__ void bounded_wait_probe_kernel(int* status, int where, int* result) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        kl::mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = kl::mbar_wait(&bar, 0, &abort_flag, status, where, 1u << 12);
        result[0] = ok ? 1 : 0;
        result[1] = abort_flag;
        // a second role that looks at the flag gives up at once, without writing a second code
        result[2] = kl::mbar_wait(&bar, 0, &abort_flag, status, where + 1, 1u << 12) ? 1 : 0;
    }
}
}  // namespace

KL_API int kl_test_bounded_wait(int* status, int where, int* result, cudaStream_t stream) {
    bounded_wait_probe_kernel<<<1, 32, 0, stream>>>(status, where, result);
    KL_LAUNCH_CHECK();
    return KL_OK;
}
