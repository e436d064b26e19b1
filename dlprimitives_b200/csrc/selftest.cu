// Self-test of the bounded device-side waits.
//
// Every mbarrier wait of the tensor-core kernels gives up after a time limit: the waiting thread raises the CTA's
// abort flag and leaves a code in the device status word, every other role sees the flag at its next wait and
// leaves its loop, and the kernel ends normally, so the context stays usable and dlp_device_status() reports
// DLP_TIMEOUT.  This file lets that path be exercised without disturbing a real kernel: a one-CTA kernel whose
// first warp waits on a barrier that nothing ever arrives at (it runs into the limit), and whose second warp
// starts waiting on another such barrier half a limit later and must be released by the abort flag rather than
// by its own limit.
#include "tc_device.cuh"

namespace dlp {
namespace {

__global__ void __launch_bounds__(64, 1) wait_expiry_kernel(int *status, int *observed)
{
    __shared__ unsigned long long never[2];
    __shared__ int abort_flag;
    if(threadIdx.x == 0) {
        tc::mbar_init(&never[0], 1);
        tc::mbar_init(&never[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // warp 1 starts its wait half a limit later than warp 0, so that its own limit cannot be the one that ends it
    if(warp == 1) {
        const long long start = tc::global_ns();
        while(tc::global_ns() - start < tc::WAIT_LIMIT_NS / 2) __nanosleep(1000);
    }
    const long long t0 = tc::global_ns();
    // warp 0 runs into the time limit; warp 1 is let go by the abort flag warp 0 raises
    const bool ok = tc::warp_wait(&never[warp], 0, &abort_flag, status, DLP_SELFTEST_WAIT_CODE + warp, lane);
    const long long waited = tc::global_ns() - t0;
    if(lane == 0) {
        observed[2 * warp] = ok ? 1 : 0;
        observed[2 * warp + 1] = int(waited / 1000000);     // milliseconds spent in the wait
    }
}

} // namespace
} // namespace dlp

using namespace dlp;

extern "C" dlp_status dlp_selftest_wait_expiry(int observed[4], void *stream)
{
    DLP_REQUIRE(observed != nullptr, "null result pointer");
    int *status = device_status_word();
    if(!status) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    int *dev = nullptr;
    DLP_CUDA_OK(cudaMalloc((void **)&dev, 4 * sizeof(int)));
    cudaError_t e = cudaMemsetAsync(dev, 0xff, 4 * sizeof(int), (cudaStream_t)stream);
    if(e == cudaSuccess) {
        wait_expiry_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status, dev);
        count_launch();
        e = cudaPeekAtLastError();
    }
    if(e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if(e == cudaSuccess) e = cudaMemcpy(observed, dev, 4 * sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(dev);
    return check_cuda(e, "wait_expiry_kernel");
}
