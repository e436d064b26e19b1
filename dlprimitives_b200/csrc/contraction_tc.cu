// Dense contraction on the sm_100a tensor cores with fp32 accuracy (3xTF32).
//
//   D[row, col] = sum_k A(row, k) * B(col, k),   rows = output pixels, cols = output channels.
//
// Every fp32 operand value v is split as  hi = v with the low 13 mantissa bits cleared (exactly a
// TF32 number) and lo = v - hi (exact in fp32).  The kernel accumulates  hi_a*hi_b + lo_a*hi_b +
// hi_a*lo_b  in one fp32 accumulator, dropping only lo_a*lo_b (relative size 2^-22).
//
// Data flow per CTA (persistent, one CTA per SM, 128-row x BN-column output tiles):
//   * B (weights, pre-packed hi/lo planes, K-major, padded) : TMA -> 128B-swizzled shared memory ring
//   * A (activations) : loader warps read the caller's NCHW tensor directly (implicit im2col, no
//     re-layout in memory), split each value in registers and write hi/lo with tcgen05.st into a
//     ring of tensor-memory columns.  The MMA therefore takes A from tensor memory and B from
//     shared memory, which keeps the shared-memory read traffic of the three products at one
//     operand instead of two.
//   * one thread issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8), accumulators live in tensor
//     memory, double-buffered so the epilogue of a tile overlaps the main loop of the next one
//   * epilogue warps read the accumulator with tcgen05.ld, apply bias / activation / residual /
//     beta and store straight to NCHW (32 consecutive pixels per warp store) or row-major.
//
// All mbarrier waits are bounded: a wait that gives up records a code in the device status word,
// raises the CTA's abort flag, and every role then leaves its loop; the CTA drains its bulk copies
// and frees its tensor memory before it returns.
#include "contraction.cuh"
#include <cuda.h>
#include <mutex>
#include <cstdlib>

namespace dlp {

namespace tc {

constexpr int BM = 128;              // rows per tile = tensor-memory lanes
constexpr int BK = 32;               // K per pipeline stage: 32 fp32 = one 128-byte swizzle row
constexpr int STAGES = 4;
constexpr int A_COL_BASE = 256;      // tensor-memory columns [0,256) hold two accumulators, [256,512) the A ring
constexpr int TMEM_COLS = 512;
constexpr int NUM_LOADER_WARPS = 8;  // 4 lane quadrants x 2 alternating stage groups
constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_EPI0 = 2, WARP_LOAD0 = 6;
constexpr int NUM_WARPS = WARP_LOAD0 + NUM_LOADER_WARPS;
constexpr int NUM_THREADS = NUM_WARPS * 32;
constexpr long long WAIT_LIMIT_NS = 400ll * 1000 * 1000;

// codes left in the device status word
enum { ST_TMA_EMPTY = 101, ST_MMA_FULL_B = 102, ST_MMA_FULL_A = 103, ST_MMA_ACC = 104, ST_EPI_ACC = 105, ST_LOAD_EMPTY = 106,
       ST_DRAIN = 107 };

struct Shared {
    unsigned long long full_b[STAGES];
    unsigned long long full_a[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned long long drain;
    uint32_t tmem_base;
    int abort_flag;
    uint32_t tma_issued;     // k-blocks whose bulk copies were issued
    uint32_t mma_consumed;   // k-blocks whose full_b barrier the MMA thread has passed
};

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
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ long long global_ns()
{
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  Returns false when the CTA is aborting or the time limit ran out (then it raises the abort).
__device__ __noinline__ bool mbar_wait_slow(unsigned long long *bar, uint32_t parity, Shared *sh, int *status, int code)
{
    long long t0 = global_ns();
    for(uint32_t i = 0;; i++) {
        if(mbar_try_wait(bar, parity)) return true;
        __nanosleep(64);
        if((i & 63) == 63) {
            if(*(volatile int *)&sh->abort_flag) return false;
            if(global_ns() - t0 > WAIT_LIMIT_NS) {
                *(volatile int *)&sh->abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, uint32_t parity, Shared *sh, int *status, int code)
{
    #pragma unroll 1
    for(int i = 0; i < 16; i++)
        if(mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, sh, status, code);
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int c0, int c1, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"((unsigned long long)map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor for a K-major tile with 128-byte rows and the 128B swizzle:
// 8-row groups are 1024 bytes apart (SBO), descriptor version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t addr)
{
    uint64_t d = 0;
    d |= uint64_t((addr & 0x3FFFF) >> 4);
    d |= uint64_t(1) << 16;             // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;     // stride byte offset
    d |= uint64_t(1) << 46;             // version
    d |= uint64_t(2) << 61;             // SWIZZLE_128B
    return d;
}
// Instruction descriptor: fp32 accumulate, TF32 x TF32, both operands K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t instr_desc_tf32(int bn)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(BM >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned long long *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                 "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
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
// Lean store of 32 accumulator columns of one row: y = clamp(acc + bias) [then clamp(y + s*residual)].
template<bool BIAS, bool RES>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], float *y0, const float *r0, long long cs, const float *b0,
                                            float2 clamp, float res_scale, float2 post_clamp)
{
    #pragma unroll
    for(int j = 0; j < 32; j++) {
        float a = __uint_as_float(v[j]);
        if(BIAS) a += __ldg(b0 + j);
        a = fminf(fmaxf(a, clamp.x), clamp.y);
        if(RES) {
            a = a + res_scale * __ldg(r0 + j * cs);
            a = fminf(fmaxf(a, post_clamp.x), post_clamp.y);
        }
        y0[j * cs] = a;
    }
}

// Position of a loader in the CTA's sequence of k-blocks (the sequence runs on across tiles).
struct Cursor {
    long long tile;
    int kb;
    uint32_t it;
};

template<int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
contraction_tf32x3_kernel(const __grid_constant__ CUtensorMap b_map, const Contraction p, int n_pad, int kblocks, int n_tiles,
                          long long num_tiles, int *status, int dbg)
{
    extern __shared__ unsigned char smem_raw[];
    // B ring first, 1024-byte aligned as the 128B swizzle requires; barriers after it.
    unsigned char *smem = (unsigned char *)((uintptr_t(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int B_TILE_BYTES = BN * BK * 4;          // one hi or lo tile
    constexpr int STAGE_BYTES = 2 * B_TILE_BYTES;
    Shared *sh = (Shared *)(smem + STAGES * STAGE_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if(threadIdx.x == 0) {
        for(int s = 0; s < STAGES; s++) {
            mbar_init(&sh->full_b[s], 1);
            mbar_init(&sh->full_a[s], 4);
            mbar_init(&sh->empty[s], 1);
        }
        for(int a = 0; a < 2; a++) {
            mbar_init(&sh->acc_full[a], 1);
            mbar_init(&sh->acc_empty[a], 4);
        }
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        sh->tma_issued = 0;
        sh->mma_consumed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&sh->tmem_base;

    if(warp == WARP_TMA) {
        // ------------------------------------------------------------------ B producer
        if(lane == 0) {
            uint32_t it = 0;
            bool live = true;
            for(long long tile = blockIdx.x; tile < num_tiles && live; tile += gridDim.x) {
                const int n0 = int(tile % n_tiles) * BN;
                for(int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    if(!mbar_wait(&sh->empty[s], ((it / STAGES) & 1) ^ 1, sh, status, ST_TMA_EMPTY)) { live = false; break; }
                    mbar_arrive_expect_tx(&sh->full_b[s], STAGE_BYTES);
                    unsigned char *dst = smem + s * STAGE_BYTES;
                    tma_load_2d(dst, &b_map, kb * BK, n0, &sh->full_b[s]);
                    tma_load_2d(dst + B_TILE_BYTES, &b_map, kb * BK, n_pad + n0, &sh->full_b[s]);
                    *(volatile uint32_t *)&sh->tma_issued = it + 1;
                }
            }
        }
    }
    else if(warp == WARP_MMA) {
        // ------------------------------------------------------------------ MMA issuer
        if(lane == 0) {
            constexpr uint32_t idesc = instr_desc_tf32(BN);
            uint32_t it = 0, tile_iter = 0;
            bool live = true;
            for(long long tile = blockIdx.x; tile < num_tiles && live; tile += gridDim.x, tile_iter++) {
                const uint32_t acc = tile_iter & 1;
                if(!mbar_wait(&sh->acc_empty[acc], ((tile_iter >> 1) & 1) ^ 1, sh, status, ST_MMA_ACC)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for(int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if(!mbar_wait(&sh->full_b[s], ph, sh, status, ST_MMA_FULL_B)) { live = false; break; }
                    *(volatile uint32_t *)&sh->mma_consumed = it + 1;
                    if(!mbar_wait(&sh->full_a[s], ph, sh, status, ST_MMA_FULL_A)) { live = false; break; }
                    tc_fence_after();
                    const uint32_t b_hi = smem_u32(smem + s * STAGE_BYTES);
                    const uint32_t b_lo = b_hi + B_TILE_BYTES;
                    const uint32_t a_hi = tmem_base + A_COL_BASE + s * 64;
                    const uint32_t a_lo = a_hi + 32;
                    #pragma unroll
                    for(int j = 0; j < BK / 8; j++) {
                        const uint64_t dhi = smem_desc_k128(b_hi + j * 32), dlo = smem_desc_k128(b_lo + j * 32);
                        // small terms first, the dominant product last
                        if(dbg & 4) continue;
                        mma_tf32_ts(d_tmem, a_lo + j * 8, dhi, idesc, (kb | j) != 0);
                        mma_tf32_ts(d_tmem, a_hi + j * 8, dlo, idesc, 1);
                        mma_tf32_ts(d_tmem, a_hi + j * 8, dhi, idesc, 1);
                    }
                    mma_commit(&sh->empty[s]);   // frees the B stage and the A columns once these MMAs retire
                }
                if(live) mma_commit(&sh->acc_full[acc]);
            }
        }
    }
    else if(warp >= WARP_EPI0 && warp < WARP_LOAD0) {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3;                     // tensor-memory lanes this warp may touch
        uint32_t tile_iter = 0;
        // identity / relu / relu6 are a clamp; with no per-row bias and no beta the whole epilogue is
        // add, clamp, (residual, clamp,) store.  Anything else takes the general path.
        const float2 clamp = act_clamp(p.act), post_clamp = act_clamp(p.post_act);
        const bool epi_fast = act_is_clamp(p.act) && act_is_clamp(p.post_act) && p.bias_mode != DLP_GEMM_BIAS_M && p.beta == 0.0f;
        for(long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, tile_iter++) {
            const uint32_t acc = tile_iter & 1;
            const long long m_tile = tile / n_tiles;
            const int n0 = int(tile % n_tiles) * BN;
            const long long row = m_tile * BM + quad * 32 + lane;
            const RowInfo r = make_row(p, row);
            __syncwarp();
            if(!__all_sync(0xffffffffu, mbar_wait(&sh->acc_full[acc], (tile_iter >> 1) & 1, sh, status, ST_EPI_ACC))) break;
            tc_fence_after();
            // Everything that does not depend on the column is hoisted out of the store loop: the
            // epilogue has to drain 128 x BN values per tile with only four warps.
            const long long col_stride = p.out_mode == OUT_NCHW ? (long long)p.plane : 1ll;
            float *y_row = p.y + r.out + (long long)n0 * col_stride;
            const float *res_row = p.residual ? p.residual + r.out + (long long)n0 * col_stride : nullptr;
            #pragma unroll 1
            for(int c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                __syncwarp();
                tmem_ld32(tmem_base + (uint32_t(quad * 32) << 16) + acc * BN + c * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if(c == BN / 32 - 1) {
                    // accumulator fully read: hand it back before the global stores
                    tc_fence_before();
                    __syncwarp();
                    if(lane == 0) mbar_arrive(&sh->acc_empty[acc]);
                }
                const int col0 = n0 + c * 32;
                const int ncols = p.cols - col0;           // columns of this chunk inside the matrix
                if(!r.valid || ncols <= 0 || (dbg & 2)) continue;
                float *y0 = y_row + (long long)(c * 32) * col_stride;
                if(epi_fast && ncols >= 32) {
                    const float *b0 = p.bias + col0;
                    if(res_row) {
                        const float *r0 = res_row + (long long)(c * 32) * col_stride;
                        if(p.bias_mode == DLP_GEMM_BIAS_N) store_chunk<true, true>(v, y0, r0, col_stride, b0, clamp, p.residual_scale, post_clamp);
                        else store_chunk<false, true>(v, y0, r0, col_stride, b0, clamp, p.residual_scale, post_clamp);
                    }
                    else {
                        if(p.bias_mode == DLP_GEMM_BIAS_N) store_chunk<true, false>(v, y0, nullptr, col_stride, b0, clamp, 0.0f, post_clamp);
                        else store_chunk<false, false>(v, y0, nullptr, col_stride, b0, clamp, 0.0f, post_clamp);
                    }
                }
                else {
                    #pragma unroll 4
                    for(int j = 0; j < 32; j++)
                        if(j < ncols) p.y[out_index(p, r, col0 + j)] = finish_output(p, r, row, col0 + j, __uint_as_float(v[j]));
                }
            }
        }
    }
    else {
        // ------------------------------------------------------------------ A loaders
        const int quad = warp & 3;                       // tensor-memory lanes this warp may touch
        const int group = (warp - WARP_LOAD0) >> 2;      // this warp handles k-blocks with (it & 1) == group
        const int row_in_tile = quad * 32 + lane;
        long long loaded_tile = -1;
        RowInfo r;
        r.valid = false; r.base = 0; r.iy0 = r.ix0 = 0; r.out = 0;

        auto advance = [&](Cursor &c, int steps) {
            c.kb += steps;
            c.it += steps;
            while(c.kb >= kblocks) { c.kb -= kblocks; c.tile += gridDim.x; }
        };
        // Issue the 32 loads of one k-block for this thread's row; nothing waits on them here.
        auto issue_loads = [&](const Cursor &c, float (&buf)[BK]) {
            if(c.tile != loaded_tile) {
                loaded_tile = c.tile;
                r = make_row(p, (c.tile / n_tiles) * BM + row_in_tile);
            }
            const int k0 = c.kb * BK;
            if(p.a_mode == A_STRIDED) {
                const float *src = p.a + r.base + (long long)k0 * p.a_k_stride;
                #pragma unroll
                for(int i = 0; i < BK; i++) {
                    const bool ok = r.valid && (k0 + i) < p.k && !(dbg & 1);
                    buf[i] = ok ? __ldg(src + (long long)i * p.a_k_stride) : 0.0f;
                }
            }
            else {
                const float *src = p.a + r.base;
                const int2 *tab = reinterpret_cast<const int2 *>(p.ktab + k0);
                #pragma unroll
                for(int i = 0; i < BK; i++) {
                    const int2 t = __ldg(tab + i);
                    const int iy = r.iy0 + (t.y >> 16), ix = r.ix0 + (t.y & 0xffff);
                    const bool ok = r.valid && unsigned(iy) < unsigned(p.in_h) && unsigned(ix) < unsigned(p.in_w);
                    buf[i] = ok ? __ldg(src + t.x) : 0.0f;
                }
            }
        };
        // Split the values and publish them as the A operand of stage (it % STAGES).
        auto publish = [&](const Cursor &c, const float (&buf)[BK]) -> bool {
            const int s = c.it % STAGES;
            __syncwarp();
            if(!__all_sync(0xffffffffu, mbar_wait(&sh->empty[s], ((c.it / STAGES) & 1) ^ 1, sh, status, ST_LOAD_EMPTY))) return false;
            tc_fence_after();
            const uint32_t t_hi = tmem_base + (uint32_t(quad * 32) << 16) + A_COL_BASE + s * 64;
            #pragma unroll
            for(int h = 0; h < 2; h++) {
                uint32_t hi[16], lo[16];
                #pragma unroll
                for(int i = 0; i < 16; i++) {
                    const float v = buf[h * 16 + i];
                    const uint32_t hb = __float_as_uint(v) & 0xffffe000u;
                    hi[i] = hb;
                    lo[i] = __float_as_uint(v - __uint_as_float(hb));
                }
                tmem_st16(t_hi + h * 16, hi);
                tmem_st16(t_hi + 32 + h * 16, lo);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(&sh->full_a[s]);
            return true;
        };

        // Two register buffers: the loads of this warp's next k-block are in flight while the
        // current one is split and stored.
        float buf_a[BK], buf_b[BK];
        Cursor cur;
        cur.tile = blockIdx.x; cur.kb = 0; cur.it = 0;
        advance(cur, group);
        if(cur.tile < num_tiles) issue_loads(cur, buf_a);
        while(cur.tile < num_tiles) {
            Cursor nxt = cur;
            advance(nxt, 2);
            if(nxt.tile < num_tiles) issue_loads(nxt, buf_b);
            if(!publish(cur, buf_a)) break;
            cur = nxt;
            if(cur.tile >= num_tiles) break;
            advance(nxt, 2);
            if(nxt.tile < num_tiles) issue_loads(nxt, buf_a);
            if(!publish(cur, buf_b)) break;
            cur = nxt;
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if(*(volatile int *)&sh->abort_flag) {
        // A wait gave up somewhere.  Let the bulk copies and tensor-core work already issued finish
        // (bounded), so nothing is still writing shared or tensor memory when the CTA goes away.
        if(threadIdx.x == 0) {
            const uint32_t issued = *(volatile uint32_t *)&sh->tma_issued;
            for(uint32_t it = *(volatile uint32_t *)&sh->mma_consumed; it < issued; it++) {
                const long long t0 = global_ns();
                while(!mbar_try_wait(&sh->full_b[it % STAGES], (it / STAGES) & 1)) {
                    __nanosleep(256);
                    if(global_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(status, 0, ST_DRAIN); break; }
                }
            }
        }
        if(warp == WARP_MMA && lane == 0) {
            mma_commit(&sh->drain);
            const long long t0 = global_ns();
            while(!mbar_try_wait(&sh->drain, 0)) {
                __nanosleep(256);
                if(global_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(status, 0, ST_DRAIN); break; }
            }
        }
        __syncthreads();
    }
    if(warp == WARP_MMA) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// Pack B(col, k) into two padded K-major planes: hi (TF32-exact) then lo (the remainder).
__global__ void prepack_hi_lo_kernel(const float *__restrict__ b, long long col_stride, long long k_stride, int cols, int k,
                                     int n_pad, int k_pad, float *__restrict__ packed)
{
    const long long total = (long long)n_pad * k_pad;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int n = int(idx / k_pad), kk = int(idx - (long long)n * k_pad);
        float v = 0.0f;
        if(n < cols && kk < k) v = __ldg(b + n * col_stride + kk * k_stride);
        const float hi = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        packed[idx] = hi;
        packed[total + idx] = v - hi;
    }
}

} // namespace tc

// ---------------------------------------------------------------------------------------------- host

TcPacked tc_packed_layout(int cols, int k)
{
    TcPacked L;
    L.bn = cols <= 32 ? 32 : (cols <= 64 ? 64 : 128);
    L.n_pad = round_up(cols, L.bn);
    L.k_pad = round_up(k, tc::BK);
    return L;
}

dlp_status tc_prepack(const TcPacked &L, const float *b, long long b_col_stride, long long b_k_stride, int cols, int k,
                      float *packed, cudaStream_t stream)
{
    const long long total = (long long)L.n_pad * L.k_pad;
    const int threads = 256;
    const int blocks = int(std::min<long long>(ceil_div<long long>(total, threads), 8 * sm_count()));
    tc::prepack_hi_lo_kernel<<<blocks, threads, 0, stream>>>(b, b_col_stride, b_k_stride, cols, k, L.n_pad, L.k_pad, packed);
    DLP_LAUNCH_OK("prepack_hi_lo_kernel");
    return DLP_OK;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

template<int BN>
dlp_status launch_bn(const Contraction &p, const TcPacked &L, const CUtensorMap &map, cudaStream_t stream)
{
    const int smem = 1024 + tc::STAGES * 2 * BN * tc::BK * 4 + int(sizeof(tc::Shared));
    static bool configured = false;   // per instantiation; the attribute is per function, set once per process
    if(!configured) {
        DLP_CUDA_OK(cudaFuncSetAttribute(tc::contraction_tf32x3_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured = true;
    }
    const long long m_tiles = ceil_div<long long>(p.rows, tc::BM);
    const int n_tiles = L.n_pad / BN;
    const long long num_tiles = m_tiles * n_tiles;
    const int grid = int(std::min<long long>(num_tiles, sm_count()));
    int *status = device_status_word();
    if(!status) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    tc::contraction_tf32x3_kernel<BN><<<grid, tc::NUM_THREADS, smem, stream>>>(map, p, L.n_pad, L.k_pad / tc::BK, n_tiles, num_tiles,
                                                                              status, getenv("DLP_DBG") ? atoi(getenv("DLP_DBG")) : 0);
    DLP_LAUNCH_OK("contraction_tf32x3_kernel");
    return DLP_OK;
}
} // namespace

dlp_status launch_contraction_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream)
{
    if(p.rows <= 0 || p.cols <= 0) return DLP_OK;
    EncodeTiledFn enc = encode_tiled();
    if(!enc) return fail(DLP_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    if(reinterpret_cast<uintptr_t>(packed) % 16 != 0) return fail(DLP_INVALID_ARGUMENT, "packed weights must be 16-byte aligned");
    CUtensorMap map;
    const cuuint64_t dims[2] = { cuuint64_t(L.k_pad), cuuint64_t(2) * L.n_pad };
    const cuuint64_t strides[1] = { cuuint64_t(L.k_pad) * sizeof(float) };
    const cuuint32_t box[2] = { cuuint32_t(tc::BK), cuuint32_t(L.bn) };
    const cuuint32_t elem[2] = { 1, 1 };
    CUresult rc = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(packed), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(rc != CUDA_SUCCESS) return fail(DLP_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(rc)));
    switch(L.bn) {
    case 32: return launch_bn<32>(p, L, map, stream);
    case 64: return launch_bn<64>(p, L, map, stream);
    case 128: return launch_bn<128>(p, L, map, stream);
    }
    return fail(DLP_INVALID_ARGUMENT, "unsupported column tile");
}

} // namespace dlp
