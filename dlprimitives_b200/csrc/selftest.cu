// Self-tests and probes: the bounded device-side waits, the tensor pipe's own TF32 rate, and what an MMA issuing scheme costs.
//
// Every mbarrier wait of the tensor-core kernels gives up after a time limit: the waiting thread raises the CTA's
// abort flag and leaves a code in the device status word, every other role sees the flag at its next wait and
// leaves its loop, and the kernel ends normally, so the context stays usable and dlp_device_status() reports
// DLP_TIMEOUT.  This file lets that path be exercised without disturbing a real kernel: a one-CTA kernel whose
// first warp waits on a barrier that nothing ever arrives at (it runs into the limit), and whose second warp
// starts waiting on another such barrier half a limit later and must be released by the abort flag rather than
// by its own limit.
#include "tc_device.cuh"
#include <mutex>

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


// ---- what the issuing warp's own bookkeeping costs.  MMA-only as above (zeroed operands, nothing loaded or stored),
// but with the k-block structure of the contraction kernels: twelve MMAs (hi/lo) per k-block on a 4-stage ring of A
// columns and B tiles, a commit per k-block, an accumulator commit every eight.  Every barrier the loop waits on is
// complete from the start (a barrier no phase of which has completed answers a wait for parity 1 at once), so what is
// timed is the issuing scheme alone:
//   0  one thread, no waits                       1  whole warp, lanes 0..2 each wait on one barrier, vote, fence, elect
//   2  whole warp, every lane tests the same barriers (uniform instructions): A columns per k-block, accumulator per tile
//   3  two issuer warps taking pairs of k-blocks in turn (named-barrier handoff between tcgen05 fences)
// CTA 0 reports clock cycles per k-block.
__device__ long long g_issue_probe_out[2];

template<int N, int SCHEME>
__global__ void __launch_bounds__(128, 1) issue_probe_kernel(int total, int *status)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ unsigned long long done, released, full_a[4], full_b[4], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag_s;
    unsigned char *smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int B_TILE_BYTES = N * 128, B_STAGE_BYTES = 2 * B_TILE_BYTES, STAGES = 4, CHUNK_KB = 8;
    for(int i = threadIdx.x; i < STAGES * B_STAGE_BYTES / 4; i += 128) reinterpret_cast<float *>(smem)[i] = 0.0f;
    if(threadIdx.x == 0) {
        tc::mbar_init(&done, 1);
        tc::mbar_init(&released, 1);
        for(int i = 0; i < 4; i++) { tc::mbar_init(&full_a[i], 1); tc::mbar_init(&full_b[i], 1); }
        for(int i = 0; i < 2; i++) tc::mbar_init(&acc_empty[i], 1);
        abort_flag_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    tc::fence_proxy_async_shared();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int *abort_flag = &abort_flag_s;
    if(warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(&tmem_base_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&tmem_base_s;
    {
        // zero the A ring (columns 256..511): tensor memory is not cleared on allocation
        uint32_t z[16];
        #pragma unroll
        for(int i = 0; i < 16; i++) z[i] = 0u;
        const uint32_t t = tmem_base + (uint32_t(warp * 32) << 16) + 256;
        for(int c = 0; c < 256; c += 16) tc::tmem_st16(t + c, z);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    constexpr uint32_t idesc = tc::instr_desc_tf32(N);
    constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
    const uint32_t ring_base = ((tc::smem_u32(smem) & 0x3FFFF) >> 4) | (1u << 16);
    const uint32_t released_bar = tc::smem_u32(&released), done_bar = tc::smem_u32(&done);
    const bool issuer = SCHEME == 3 ? warp < 2 : (SCHEME == 0 ? threadIdx.x == 0 : warp == 0);
    if(issuer) {
        const int me = warp;
        uint32_t it = 0, step = 0, s = 0, chunk = 0;
        int in_chunk = 0;
        bool dead = false;
        const long long t0 = clock64();
        #pragma unroll 1
        while(it < uint32_t(total)) {
            const uint32_t buf = chunk & 1;
            const bool pair = SCHEME == 3 && (s & 1) == 0 && in_chunk + 2 <= CHUNK_KB;
            const int n = pair ? 2 : 1;
            const bool closes_chunk = in_chunk + n == CHUNK_KB;
            if(SCHEME != 3 || int(step & 1) == me) {
                if(SCHEME == 1) {
                    bool ok = true;
                    if(lane == 0) ok = tc::mbar_wait(&full_a[s], 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 20);
                    else if(lane == 1) ok = tc::mbar_wait(&full_b[s], 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 21);
                    else if(lane == 2 && in_chunk == 0) ok = tc::mbar_wait(&acc_empty[buf], 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 22);
                    if(!__all_sync(0xffffffffu, ok)) dead = true;
                }
                else if(SCHEME == 2) {
                    // the pointwise kernel's loop with resident weights: the A columns every k-block, the B tiles only during the
                    // first work item, the accumulator when a tile opens (each test with its vote costs about 130 cycles)
                    bool ok = tc::warp_wait_ready(&full_a[s], 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 20, lane);
                    if(ok && it < 8) ok = tc::warp_wait_ready(&full_b[s], 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 21, lane);
                    if(ok && in_chunk == 0) ok = tc::warp_wait_ready(&acc_empty[buf], 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 22, lane);
                    if(!ok) dead = true;
                }
                else if(SCHEME == 3) {
                    // as the contraction kernel: lanes 0, 1 the first stage's two barriers, lanes 2, 3 the second's, lane 4 the accumulator
                    const bool mine = lane < 2 || (lane < 4 && pair) || (lane == 4 && in_chunk == 0);
                    const uint32_t bar = lane == 4 ? tc::smem_u32(&acc_empty[buf]) : tc::smem_u32(lane & 1 ? &full_b[0] : &full_a[0]) + 8 * (s + (lane >> 1));
                    const bool ok = mine ? tc::mbar_wait(bar, 1, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 23) : true;
                    if(!__all_sync(0xffffffffu, ok)) dead = true;
                }
                const uint32_t d = tmem_base + buf * N, a = tmem_base + 256 + s * 64;
                const uint32_t bhi = ring_base + s * (B_STAGE_BYTES >> 4), blo = bhi + (B_TILE_BYTES >> 4);
                uint32_t ah[2][4], al[2][4];
                uint64_t bh[2][4], bl[2][4];
                #pragma unroll
                for(int h = 0; h < 2; h++)
                    #pragma unroll
                    for(int j = 0; j < 4; j++) {
                        ah[h][j] = a + h * 64 + 8 * j;
                        al[h][j] = a + h * 64 + 32 + 8 * j;
                        bh[h][j] = (uint64_t(DESC_HI) << 32) | (bhi + h * (B_STAGE_BYTES >> 4) + 2 * j);
                        bl[h][j] = (uint64_t(DESC_HI) << 32) | (blo + h * (B_STAGE_BYTES >> 4) + 2 * j);
                    }
                if(SCHEME == 3 && step > 0) asm volatile("bar.sync %0, 64;" ::"r"(3 + int((step - 1) & 1)) : "memory");
                if(SCHEME != 0) tc::tc_fence_after();
                if(!dead && (SCHEME == 0 || tc::elect_one())) {
                    tc::mma_kblock(d, ah[0], al[0], bh[0], bl[0], idesc, in_chunk != 0);
                    if(pair) tc::mma_kblock(d, ah[1], al[1], bh[1], bl[1], idesc, 1u);
                }
                if(SCHEME != 0) __syncwarp();
                if(SCHEME == 3) {
                    tc::tc_fence_before();
                    asm volatile("bar.arrive %0, 64;" ::"r"(3 + int(step & 1)) : "memory");
                }
                if(!dead && (SCHEME == 0 || tc::elect_one())) {
                    tc::mma_commit(released_bar);                  // stands for the release of the stage(s): nobody waits on it
                    if(closes_chunk) tc::mma_commit(released_bar);
                }
                if(SCHEME != 0) __syncwarp();
            }
            step++;
            it += n;
            s = (s + n) & (STAGES - 1);
            in_chunk = closes_chunk ? 0 : in_chunk + n;
            chunk = closes_chunk ? chunk + 1 : chunk;
        }
        if(SCHEME == 3 && step > 0 && int(step & 1) == me) asm volatile("bar.sync %0, 64;" ::"r"(3 + int((step - 1) & 1)) : "memory");
        if(lane == 0 && warp == 0 && blockIdx.x == 0) {
            g_issue_probe_out[0] = clock64() - t0;
            g_issue_probe_out[1] = it;
        }
    }
    tc::tc_fence_before();
    __syncthreads();
    tc::tc_fence_after();
    // everything issued retires (bounded) before tensor memory goes away: one commit per issuing thread
    if(lane == 0 && (warp == 0 || (SCHEME == 3 && warp == 1))) {
        unsigned long long *bar = warp == 0 ? &done : &acc_empty[1];
        tc::mma_commit(tc::smem_u32(bar));
        tc::mbar_wait(bar, 0, abort_flag, status, DLP_SELFTEST_WAIT_CODE + 24);
    }
    (void)done_bar;
    tc::tc_fence_before();
    __syncthreads();
    if(warp == 0) {
        tc::tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

template<int N, int SCHEME>
dlp_status run_issue_probe(double *cycles, int *status, cudaStream_t s)
{
    const int smem = 1024 + 4 * 2 * N * 128, total = 8 * 800;
    static std::mutex mutex;
    {
        std::lock_guard<std::mutex> lock(mutex);
        DLP_CUDA_OK(cudaFuncSetAttribute(issue_probe_kernel<N, SCHEME>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    issue_probe_kernel<N, SCHEME><<<sm_count(), 128, smem, s>>>(8 * 20, status);          // warm-up
    issue_probe_kernel<N, SCHEME><<<sm_count(), 128, smem, s>>>(total, status);
    count_launch(2);
    DLP_CUDA_OK(cudaPeekAtLastError());
    DLP_CUDA_OK(cudaStreamSynchronize(s));
    long long out[2] = { 0, 0 };
    DLP_CUDA_OK(cudaMemcpyFromSymbol(out, g_issue_probe_out, sizeof(out)));
    *cycles = out[1] > 0 ? double(out[0]) / double(out[1]) : 0.0;
    return DLP_OK;
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

extern "C" dlp_status dlp_tf32_issue_probe(int scheme, int n, double *cycles_per_kblock, void *stream)
{
    DLP_REQUIRE(cycles_per_kblock != nullptr, "null result pointer");
    DLP_REQUIRE(scheme >= 0 && scheme <= 3 && (n == 64 || n == 128), "scheme 0..3, n 64 or 128");
    int *status = device_status_word();
    if(!status) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    cudaStream_t s = (cudaStream_t)stream;
    switch(scheme * 2 + (n == 128 ? 1 : 0)) {
    case 0: return run_issue_probe<64, 0>(cycles_per_kblock, status, s);
    case 1: return run_issue_probe<128, 0>(cycles_per_kblock, status, s);
    case 2: return run_issue_probe<64, 1>(cycles_per_kblock, status, s);
    case 3: return run_issue_probe<128, 1>(cycles_per_kblock, status, s);
    case 4: return run_issue_probe<64, 2>(cycles_per_kblock, status, s);
    case 5: return run_issue_probe<128, 2>(cycles_per_kblock, status, s);
    case 6: return run_issue_probe<64, 3>(cycles_per_kblock, status, s);
    default: return run_issue_probe<128, 3>(cycles_per_kblock, status, s);
    }
}
