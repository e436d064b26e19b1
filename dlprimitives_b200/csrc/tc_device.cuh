// Device-side building blocks shared by the tensor-core kernels: mbarrier waits with a time limit, bulk and
// tensor-map copies, tcgen05 (tensor memory, MMA issue, commit) wrappers.
#pragma once
#include "contraction.cuh"

namespace dlp {
namespace tc {

constexpr long long WAIT_LIMIT_NS = 400ll * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Barrier waits take the barrier either as a pointer or as its 32-bit shared-space address.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, uint32_t parity) { return mbar_try_wait(smem_u32(bar), parity); }
// non-blocking: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ long long global_ns()
{
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait by one thread.  Returns false when the CTA is aborting or the time limit ran out
// (then it raises the abort).
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int *abort_flag, int *status, int code)
{
    #pragma unroll 1
    for(int i = 0; i < 32; i++)
        if(mbar_try_wait(bar, parity)) return true;
    const long long t0 = global_ns();
    #pragma unroll 1
    for(uint32_t i = 0;; i++) {
        if(mbar_try_wait(bar, parity)) return true;
        __nanosleep(32);
        if((i & 63) == 63) {
            if(*(volatile int *)abort_flag) return false;
            if(global_ns() - t0 > WAIT_LIMIT_NS) {
                *(volatile int *)abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *abort_flag, int *status, int code)
{
    if(mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, code);
}
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, int *abort_flag, int *status, int code)
{
    return mbar_wait(smem_u32(bar), parity, abort_flag, status, code);
}
// The same for a whole warp: one lane polls (32 lanes polling one barrier serialise), all get the answer.
__device__ __forceinline__ bool warp_wait(unsigned long long *bar, uint32_t parity, int *abort_flag, int *status, int code, int lane)
{
    int ok = 1;
    __syncwarp();
    if(lane == 0) ok = mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
}
// For a converged warp that expects the barrier to be complete already: every lane tries it (one uniform instruction, no
// divergent path: a few cycles); only when it is not complete does one lane settle down to poll.
__device__ __forceinline__ bool warp_wait_ready(unsigned long long *bar, uint32_t parity, int *abort_flag, int *status, int code, int lane)
{
    if(__all_sync(0xffffffffu, mbar_try_wait(smem_u32(bar), parity))) return true;
    return warp_wait(bar, parity, abort_flag, status, code, lane);
}

// A read-only load that stays where it is written (the compiler keeps it ahead of the waits that follow): for operands
// asked for early so that their trip to L2 is over by the time they are used.
__device__ __forceinline__ float ldg_early(const float *p)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "elect.sync _|p, 0xffffffff;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Contiguous bulk copy global -> shared (both 16-byte aligned, size a multiple of 16); completion is
// counted in bytes on the mbarrier.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptors (K-major tile, 128-byte rows, 128B swizzle) are put together where the
// MMAs are issued: address >> 4 in the low word with the leading byte offset field set to 1 (unused for
// swizzled K-major), and in the high word the stride byte offset (8-row groups 1024 bytes apart),
// descriptor version 1 (sm_100) and layout type 2 (SWIZZLE_128B).
// Instruction descriptor: fp32 accumulate, TF32 x TF32, both operands K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t instr_desc_tf32(int bn)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}
// The twelve MMAs of one k-block (four K=8 steps x three products), small terms first.  d: the
// accumulator; ah / al: tensor-memory addresses of the hi / lo columns of A for each K=8 step;
// bh / bl: shared-memory descriptors of the hi / lo tile of B for each step.  The operands come in
// ready-made so that the caller can compute them in warp-uniform code.
__device__ __forceinline__ void mma_kblock(uint32_t d, const uint32_t (&ah)[4], const uint32_t (&al)[4], const uint64_t (&bh)[4],
                                           const uint64_t (&bl)[4], uint32_t idesc, uint32_t accumulate_first)
{
    asm volatile("{\n\t"
                 ".reg .pred p, t;\n\t"
                 "setp.ne.b32 p, %18, 0;\n\t"
                 "setp.eq.b32 t, 0, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%5], %9, %17, p;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %13, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %9, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%6], %10, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%2], %14, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%2], %10, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%7], %11, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%3], %15, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%3], %11, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%8], %12, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%4], %16, %17, t;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%4], %12, %17, t;\n\t"
                 "}"
                 ::"r"(d), "r"(ah[0]), "r"(ah[1]), "r"(ah[2]), "r"(ah[3]), "r"(al[0]), "r"(al[1]), "r"(al[2]), "r"(al[3]),
                   "l"(bh[0]), "l"(bh[1]), "l"(bh[2]), "l"(bh[3]), "l"(bl[0]), "l"(bl[1]), "l"(bl[2]), "l"(bl[3]),
                   "r"(idesc), "r"(accumulate_first) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar)   // bar: shared-space address of the mbarrier
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                 "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[16]) { tmem_ld16(taddr, v); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                   "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                   "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ bool act_is_clamp(int act) { return act == DLP_ACT_IDENTITY || act == DLP_ACT_RELU || act == DLP_ACT_RELU6; }
__device__ __forceinline__ float2 act_clamp(int act)
{
    return make_float2(act == DLP_ACT_IDENTITY ? -INFINITY : 0.0f, act == DLP_ACT_RELU6 ? 6.0f : INFINITY);
}

// ---- tensor-map (TMA) copies of one box of a 3-D tensor; the map lives in kernel parameter space
__device__ __forceinline__ void tma_load_3d(void *dst, const void *tmap, int x, int y, int z, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void *tmap, int x, int y, int z, const void *src)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(src)) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N of this thread's most recent bulk groups may still be reading their shared-memory source
template<int N> __device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template<int N> __device__ __forceinline__ void bulk_wait_group() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// makes shared-memory writes of this thread visible to the copy engines (before a bulk store reads them)
__device__ __forceinline__ void fence_proxy_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

} // namespace tc
} // namespace dlp
