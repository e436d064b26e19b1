// Self-tests and probes: the bounded device-side waits, and the tensor pipe's own TF32 rate.
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

// ---- raw tensor-core rate: every CTA's one issuing thread sends `iters` x 16 tcgen05.mma.kind::tf32 (M = 128, N = 128, K = 8,
// A from tensor memory, B from shared memory: the operand placement of the contraction kernels) over zeroed operands and
// waits for the last to retire.  Nothing is loaded or stored: the time is the tensor pipe's.
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, int *status)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ unsigned long long done;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    unsigned char *smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    for(int i = threadIdx.x; i < 128 * 32; i += 128) reinterpret_cast<float *>(smem)[i] = 0.0f;      // one B tile: 128 rows x 128 bytes
    if(threadIdx.x == 0) {
        tc::mbar_init(&done, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    tc::fence_proxy_async_shared();
    const int warp = threadIdx.x >> 5;
    if(warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&tmem_base_s;
    // zero the A columns this test reads (tensor memory is not cleared on allocation): lanes = rows, 32 columns from 256
    {
        uint32_t z[16];
        #pragma unroll
        for(int i = 0; i < 16; i++) z[i] = 0u;
        const uint32_t t = tmem_base + (uint32_t(warp * 32) << 16) + 256;
        tc::tmem_st16(t, z);
        tc::tmem_st16(t + 16, z);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    if(threadIdx.x == 0) {
        constexpr uint32_t idesc = tc::instr_desc_tf32(128);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
        const uint64_t bdesc = (uint64_t(DESC_HI) << 32) | (((tc::smem_u32(smem) & 0x3FFFF) >> 4) | (1u << 16));
        const uint32_t d = tmem_base, a = tmem_base + 256;
        for(int i = 0; i < iters; i++) {
            #pragma unroll
            for(int j = 0; j < 16; j++)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                             ::"r"(d), "r"(a + (j & 3) * 8), "l"(bdesc + 2 * (j & 3)), "r"(idesc), "r"(1) : "memory");
        }
        tc::mma_commit(tc::smem_u32(&done));
        tc::mbar_wait(&done, 0, &abort_flag, status, DLP_SELFTEST_WAIT_CODE + 10);
    }
    tc::tc_fence_before();
    __syncthreads();
    if(warp == 0) {
        tc::tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

} // namespace
} // namespace dlp

using namespace dlp;

extern "C" dlp_status dlp_tf32_mma_rate(double *tflops, void *stream)
{
    DLP_REQUIRE(tflops != nullptr, "null result pointer");
    int *status = device_status_word();
    if(!status) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    const int smem = 1024 + 128 * 128;
    const int ctas = sm_count(), iters = 4000;            // 64 000 MMAs of 64 cycles each per SM: about 2 ms
    cudaEvent_t e0, e1;
    DLP_CUDA_OK(cudaEventCreate(&e0));
    DLP_CUDA_OK(cudaEventCreate(&e1));
    cudaStream_t s = (cudaStream_t)stream;
    mma_rate_kernel<<<ctas, 128, smem, s>>>(200, status);                        // warm-up
    cudaError_t e = cudaEventRecord(e0, s);
    mma_rate_kernel<<<ctas, 128, smem, s>>>(iters, status);
    count_launch(2);
    if(e == cudaSuccess) e = cudaEventRecord(e1, s);
    if(e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.0f;
    if(e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if(e == cudaSuccess) e = cudaPeekAtLastError();
    DLP_CUDA_OK(e);
    *tflops = ms > 0.0f ? double(ctas) * iters * 16 * (2.0 * 128 * 128 * 8) / (ms * 1e9) : 0.0;
    return DLP_OK;
}

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
