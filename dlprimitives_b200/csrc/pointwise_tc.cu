// 1x1, stride-1 convolution on the sm_100a tensor cores (3xTF32, fp32 in and out) for the shapes whose time is
// memory traffic, not arithmetic: few input channels (K <= 256) over large planes.  Same arithmetic and the
// same packed weights as contraction_tf32x3_kernel; what differs is how the bytes move.
//
//   * An output tile is 128 consecutive pixels of ONE image x BN output channels (tiles never straddle images:
//     the last tile of an image is clipped), so every operand of a tile is a box of a 3-D tensor
//     [pixels, channels, images] and the copy engines can move it:
//       - A: one tensor-map copy per k-block (128 pixels x 32 input channels, 16 KB) into a shared-memory ring,
//         issued by one thread several k-blocks ahead; rows beyond the image arrive as zeros.  Converter warps
//         read their row from shared memory, split each value into its TF32 part and the remainder and write
//         both to the tensor-memory ring the MMAs read.  No thread computes an address or waits on a global load.
//       - B (packed weights): with few input channels the whole column tile's weights fit in shared memory and
//         a CTA works on one column tile throughout, so they are copied once per CTA and stay; otherwise they
//         stream through a ring, one bulk copy per k-block.
//       - residual operand: a tensor-map copy per 32 channels of the tile into one of three epilogue buffers,
//         issued by its own thread as soon as a buffer is free (up to two groups ahead of the epilogue warps).
//       - result: the epilogue warps read the accumulator from tensor memory, add bias / activation / residual,
//         write the finished 128 x 32 block into the same epilogue buffer and one thread stores it with a
//         tensor-map copy, which clips the pixels beyond the image and the channels beyond the tensor.
//   * Roles (20 warps): warp 0 A copies, warp 1 MMA issue, warp 2 residual copies, warp 3 B copies (then second MMA issuer when the weights are resident; warp 2 is when they stream and there is no residual), warps 8-15 converters
//     (two groups taking k-blocks in turn), warps 4-7 and 16-19 two sets of epilogue warps that take the 32-channel groups of a tile in turn (the tile's
//     time is its epilogue: each set has its own block barrier, its own storing thread and its own stores in flight).
//   * Every wait is bounded (device status word + abort flag, as in the general kernel); each copy-issuing
//     thread waits for its own copies before it leaves, and tensor memory is freed on every path.
//
// Reference: the 1x1 fast path of src/kernels/sgemm.cl:71-134 / src/core/conv.cpp:59-80 (is_1x1 tiling).
#include "tc_device.cuh"
#include <cuda.h>
#include <algorithm>
#include <mutex>
#include <vector>
#include <cstring>

namespace dlp {
namespace pw {

using namespace tc;

constexpr int BM = 128, BK = 32;
constexpr int T_STAGES = 4;                 // tensor-memory ring of A (and the B ring when the weights stream)
// Shared memory is shared out per launch: the weights take what they need (resident: the column tile's whole K, at most
// 128 KB; streaming: four stages), the rest goes to the ring the tensor-map copies of A land in (s_stages x 16 KB) and
// to the epilogue buffers (e_bufs x 16 KB: residual in, result out, 128 pixels x 32 channels each).
constexpr int MAX_S_STAGES = 6, MAX_E_BUFS = 8;
constexpr int MAX_B_BYTES = 128 * 1024;
constexpr int MAX_B_STAGES = 16;
constexpr int A_STAGE_BYTES = BM * BK * 4;
constexpr int E_BUF_BYTES = BM * 32 * 4;
constexpr int A_COL_BASE = 256, TMEM_COLS = 512;
constexpr int WARP_A = 0, WARP_MMA = 1, WARP_RES = 2, WARP_B = 3, WARP_ACC0 = 4, WARP_CONV0 = 8, WARP_ACC1 = 16;
constexpr int NUM_WARPS = 20, NUM_THREADS = NUM_WARPS * 32;
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int SMEM_FIXED = 1024 + 1024;     // alignment slack + the barrier block

// codes left in the device status word
enum { ST_A_EMPTY = 201, ST_B_EMPTY = 202, ST_RES_EMPTY = 203, ST_CONV_FULL = 204, ST_CONV_EMPTY = 205, ST_MMA_A = 206, ST_MMA_B = 207,
       ST_MMA_ACC = 208, ST_EPI_ACC = 209, ST_EPI_BUF = 210, ST_DRAIN = 211 };

struct Shared {
    unsigned long long sa_full[MAX_S_STAGES];  // a tensor-map copy of A landed in the shared-memory ring
    unsigned long long sa_empty[MAX_S_STAGES]; // ... and the four converter warps of its k-block have read it
    unsigned long long full_a[T_STAGES];       // the k-block's hi/lo columns are written to tensor memory (4 converter warps)
    unsigned long long full_b[MAX_B_STAGES];   // a B stage landed
    unsigned long long empty[T_STAGES];        // the MMAs of a k-block retired: its tensor-memory columns (and B stage) are free
    unsigned long long acc_full[2], acc_empty[2];
    unsigned long long e_full[MAX_E_BUFS];     // residual operand landed in an epilogue buffer
    unsigned long long e_empty[MAX_E_BUFS];    // the store of an epilogue buffer has read it
    unsigned long long drain;
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Shared) <= 1024, "barrier block");

struct Params {
    int plane;              // pixels per image (H*W)
    int cols;               // output channels of this launch
    int kblocks;            // ceil(K / 32), at most 8
    int tiles_per_image;    // ceil(plane / 128)
    int n_tiles;            // column tiles
    long long num_items;    // images * tiles_per_image * n_tiles
    int resident;           // the weights of a CTA's column tile are copied once and stay in shared memory
    int b_bytes;            // shared memory set aside for the weights
    int s_stages, e_bufs;   // depth of the A ring and number of epilogue buffers
    const float *bias;      // per output channel or null
    int act, post_act;
    int has_res;
    float res_scale;
};

struct Item {
    int b, pix0, n_tile;
};
__device__ __forceinline__ Item decode(long long item, const Params &q)
{
    Item w;
    const long long m_tile = item / q.n_tiles;
    w.n_tile = int(item - m_tile * q.n_tiles);
    w.b = int(m_tile / q.tiles_per_image);
    w.pix0 = int(m_tile - (long long)w.b * q.tiles_per_image) * BM;
    return w;
}

// Barrier 1 + set of the CTA, for the 128 threads of a set of epilogue warps, with an AND vote riding on it.
__device__ __forceinline__ bool epilogue_barrier_all(bool ok, int set)
{
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbar.red.and.pred p, %2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"(uint32_t(ok)), "r"(1 + set) : "memory");
    return r != 0;
}

// A copy-issuing thread waits (bounded) for the last `depth` copies it armed before it leaves: nothing may still be
// writing shared memory when the CTA ends.  count: copies issued; the n-th copy used barrier n % depth, phase n / depth.
__device__ __forceinline__ void drain_own(unsigned long long *bars, int depth, uint32_t count, int *status)
{
    for(uint32_t n = count > uint32_t(depth) ? count - depth : 0; n < count; n++) {
        const long long t0 = global_ns();
        while(!mbar_try_wait(&bars[n % depth], (n / depth) & 1)) {
            __nanosleep(256);
            if(global_ns() - t0 > WAIT_LIMIT_NS) { atomicCAS(status, 0, ST_DRAIN); break; }
        }
    }
}

template<int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
pointwise_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                        const __grid_constant__ CUtensorMap tm_res, const float *__restrict__ packed, const Params q, int *status)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int B_TILE_BYTES = BN * BK * 4;
    constexpr int B_STAGE_BYTES = 2 * B_TILE_BYTES;              // hi tile, then lo tile
    static_assert(MAX_B_BYTES / B_STAGE_BYTES <= MAX_B_STAGES, "barrier array");
    constexpr int GROUPS = BN / 32;
    const int S_STAGES = q.s_stages, E_BUFS = q.e_bufs;
    Shared *sh = reinterpret_cast<Shared *>(smem);
    unsigned char *b_region = smem + 1024;
    unsigned char *a_ring = b_region + q.b_bytes;
    float *e_bufs = reinterpret_cast<float *>(a_ring + S_STAGES * A_STAGE_BYTES);
    int *abort_flag = &sh->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = q.kblocks;
    // a warp with nothing else to do issues MMAs too: the B warp once resident weights are in, else the residual warp of a launch without residual
    const int second_issuer = q.resident ? WARP_B : (q.has_res ? -1 : WARP_RES);
    const long long my_items = blockIdx.x < q.num_items ? (q.num_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if(threadIdx.x == 0) {
        for(int s = 0; s < MAX_S_STAGES; s++) { mbar_init(&sh->sa_full[s], 1); mbar_init(&sh->sa_empty[s], 4); }
        for(int s = 0; s < T_STAGES; s++) { mbar_init(&sh->full_a[s], 4); mbar_init(&sh->empty[s], 1); }
        for(int s = 0; s < MAX_B_STAGES; s++) mbar_init(&sh->full_b[s], 1);
        for(int a = 0; a < 2; a++) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 4 * (GROUPS > 1 ? 2 : 1)); }
        for(int e = 0; e < MAX_E_BUFS; e++) { mbar_init(&sh->e_full[e], 1); mbar_init(&sh->e_empty[e], 1); }
        mbar_init(&sh->drain, 2);
        sh->abort_flag = 0;
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

    if(warp == WARP_B) {
        // ------------------------------------------------------------------ B copies
        if(lane == 0) {
            if(q.resident) {
                // the CTA's column tile never changes: its k-blocks go to stages 0 .. kblocks-1 once
                if(my_items > 0) {
                    const Item w = decode(blockIdx.x, q);
                    const float *src = packed + (long long)w.n_tile * kblocks * (B_STAGE_BYTES / 4);
                    for(int kb = 0; kb < kblocks; kb++) {
                        mbar_arrive_expect_tx(&sh->full_b[kb], B_STAGE_BYTES);
                        bulk_load(b_region + kb * B_STAGE_BYTES, src + (long long)kb * (B_STAGE_BYTES / 4), B_STAGE_BYTES, &sh->full_b[kb]);
                    }
                    for(int kb = 0; kb < kblocks; kb++) drain_own(&sh->full_b[kb], 1, 1, status);
                }
            }
            else {
                uint32_t it = 0;
                bool live = true;
                for(long long item = blockIdx.x; item < q.num_items && live; item += gridDim.x) {
                    const Item w = decode(item, q);
                    const float *src = packed + (long long)w.n_tile * kblocks * (B_STAGE_BYTES / 4);
                    for(int kb = 0; kb < kblocks; kb++, it++) {
                        const int s = it % T_STAGES;
                        if(!mbar_wait(&sh->empty[s], ((it / T_STAGES) & 1) ^ 1, abort_flag, status, ST_B_EMPTY)) { live = false; break; }
                        mbar_arrive_expect_tx(&sh->full_b[s], B_STAGE_BYTES);
                        bulk_load(b_region + s * B_STAGE_BYTES, src + (long long)kb * (B_STAGE_BYTES / 4), B_STAGE_BYTES, &sh->full_b[s]);
                    }
                }
                drain_own(sh->full_b, T_STAGES, it, status);
            }
        }
    }
    __syncwarp();

    if(warp == WARP_A) {
        // ------------------------------------------------------------------ A copies
        if(lane == 0) {
            uint32_t it = 0;
            bool live = true;
            for(long long item = blockIdx.x; item < q.num_items && live; item += gridDim.x) {
                const Item w = decode(item, q);
                for(int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % S_STAGES;
                    if(!mbar_wait(&sh->sa_empty[s], ((it / S_STAGES) & 1) ^ 1, abort_flag, status, ST_A_EMPTY)) { live = false; break; }
                    mbar_arrive_expect_tx(&sh->sa_full[s], A_STAGE_BYTES);
                    tma_load_3d(a_ring + s * A_STAGE_BYTES, &tm_x, w.pix0, kb * BK, w.b, &sh->sa_full[s]);
                }
            }
            drain_own(sh->sa_full, S_STAGES, it, status);
        }
    }
    else if(warp == WARP_RES && q.has_res) {
        // ------------------------------------------------------------------ residual copies
        if(lane == 0) {
            uint32_t j = 0;
            bool live = true;
            for(long long item = blockIdx.x; item < q.num_items && live; item += gridDim.x) {
                const Item w = decode(item, q);
                for(int g = 0; g < GROUPS; g++, j++) {
                    const int e = j % E_BUFS;
                    if(!mbar_wait(&sh->e_empty[e], ((j / E_BUFS) & 1) ^ 1, abort_flag, status, ST_RES_EMPTY)) { live = false; break; }
                    mbar_arrive_expect_tx(&sh->e_full[e], E_BUF_BYTES);
                    tma_load_3d(e_bufs + e * (E_BUF_BYTES / 4), &tm_res, w.pix0, w.n_tile * BN + g * 32, w.b, &sh->e_full[e]);
                }
            }
            drain_own(sh->e_full, E_BUFS, j, status);
        }
    }
    else if(warp == WARP_MMA || warp == second_issuer) {
        // ------------------------------------------------------------------ MMA issuers
        // The issuing thread blocks in tcgen05.mma at the tensor core's pace (its queue is short), so whatever else it
        // executes between k-blocks is time the tensor core idles, and one thread cannot issue faster than an MMA per
        // 45 cycles (a 64-column MMA is 32 cycles of work).  So: the whole warp runs the loop with uniform control flow
        // (operands stay in uniform registers); every lane tests the same barriers, one uniform instruction each (a lane
        // per barrier is three divergent paths: 400 cycles per k-block even when all are complete); an iteration takes two
        // k-blocks where it can; and a warp that has nothing else to do -- the B warp once resident weights are in, the
        // residual warp of a launch without residual -- is a second issuer: the two take the iterations in turn, one waiting for its stages and building its operands
        // while the other's MMAs go out (a named barrier carries the turn, tcgen05 fences around it keep the MMAs of
        // the two threads in order).  A warp whose wait gave up keeps taking its turns without issuing.
        constexpr uint32_t idesc = instr_desc_tf32(BN);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO, version 1, SWIZZLE_128B
        const uint32_t region_base = ((smem_u32(b_region) & 0x3FFFF) >> 4) | (1u << 16);
        const bool two = second_issuer >= 0;
        const int me = warp == WARP_MMA ? 0 : 1;
        const uint32_t total = uint32_t(my_items * kblocks);
        uint32_t it = 0, step = 0, item_i = 0;
        int kb = 0;
        bool dead = false;
        #pragma unroll 1
        while(it < total) {
            const uint32_t s = it % T_STAGES, phase = (it / T_STAGES) & 1;
            const uint32_t buf = item_i & 1;
            const bool pair = (s & 1) == 0 && kb + 2 <= kblocks;
            const int n = pair ? 2 : 1;
            const bool closes = kb + n == kblocks;
            if(!two || int(step & 1) == me) {
                const uint32_t sb = q.resident ? uint32_t(kb) : s;
                if(!dead) {
                    bool ok = warp_wait_ready(&sh->full_a[s], phase, abort_flag, status, ST_MMA_A, lane);
                    if(ok && pair) ok = warp_wait_ready(&sh->full_a[s + 1], phase, abort_flag, status, ST_MMA_A, lane);
                    if(!q.resident || item_i == 0) {
                        if(ok) ok = warp_wait_ready(&sh->full_b[sb], q.resident ? 0u : phase, abort_flag, status, ST_MMA_B, lane);
                        if(ok && pair) ok = warp_wait_ready(&sh->full_b[sb + 1], q.resident ? 0u : phase, abort_flag, status, ST_MMA_B, lane);
                    }
                    if(ok && kb == 0) ok = warp_wait_ready(&sh->acc_empty[buf], ((item_i >> 1) & 1) ^ 1, abort_flag, status, ST_MMA_ACC, lane);
                    if(!ok) dead = true;
                }
                const uint32_t d = tmem_base + buf * BN, a = tmem_base + A_COL_BASE + s * 64;
                const uint32_t bhi = region_base + sb * (B_STAGE_BYTES >> 4), blo = bhi + (B_TILE_BYTES >> 4);
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
                // my turn: the other warp has issued the iteration before this one
                if(two && step > 0) asm volatile("bar.sync %0, 64;" ::"r"(3 + int((step - 1) & 1)) : "memory");
                tc_fence_after();
                if(!dead && elect_one()) {
                    mma_kblock(d, ah[0], al[0], bh[0], bl[0], idesc, kb != 0);
                    if(pair) mma_kblock(d, ah[1], al[1], bh[1], bl[1], idesc, 1u);
                }
                __syncwarp();
                if(two) {
                    tc_fence_before();
                    asm volatile("bar.arrive %0, 64;" ::"r"(3 + int(step & 1)) : "memory");      // the other warp's turn
                }
                if(!dead && elect_one()) {
                    mma_commit(smem_u32(&sh->empty[s]));
                    if(pair) mma_commit(smem_u32(&sh->empty[s + 1]));
                    if(closes) mma_commit(smem_u32(&sh->acc_full[buf]));
                }
                __syncwarp();
            }
            step++;
            it += n;
            kb += n;
            if(kb == kblocks) { kb = 0; item_i++; }
        }
        // the last turn handed over is taken by nobody: meet it so that both barriers are left balanced
        if(two && step > 0 && int(step & 1) == me) asm volatile("bar.sync %0, 64;" ::"r"(3 + int((step - 1) & 1)) : "memory");
    }
    else if(warp == WARP_B || warp == WARP_RES) {
        // nothing more for this warp: the B warp's one thread has issued its copies above; no residual operand in this launch
    }
    else if(warp < WARP_CONV0 || warp >= WARP_ACC1) {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3;
        const int set = warp >= WARP_ACC1 ? 1 : 0;                 // which of the two sets of epilogue warps
        constexpr int SETS = GROUPS > 1 ? 2 : 1;
        if(set >= SETS) goto teardown;                            // a 32-channel tile has one group: the second set has no work
        const int row = quad * 32 + lane;
        const float2 clamp = act_clamp(q.act), post_clamp = act_clamp(q.post_act);
        const bool lean = act_is_clamp(q.act) && act_is_clamp(q.post_act);
        const bool storer = (warp == WARP_ACC0 || warp == WARP_ACC1) && lane == 0;
        const bool release_at_once = q.has_res || E_BUFS < 2 * SETS;
        bool live = true;
        long long i = 0;
        for(long long item = blockIdx.x; item < q.num_items && live; item += gridDim.x, i++) {
            const Item w = decode(item, q);
            const uint32_t buf = uint32_t(i) & 1;
            // bias of the 32-channel groups this set takes (one coalesced load per group and warp, handed round by shuffles below):
            // asked for before the wait for the accumulator -- the shared-memory carve-out leaves no L1 to speak of, and a trip
            // to L2 in front of every group was a sixth of the tile's time
            float bias_g[2] = { 0.0f, 0.0f };
            #pragma unroll
            for(int u = 0; u < 2; u++) {
                const int col = w.n_tile * BN + (set + u * SETS) * 32 + lane;
                if(set + u * SETS < GROUPS && q.bias && col < q.cols) bias_g[u] = ldg_early(q.bias + col);
            }
            // A wait that gives up must not leave the other epilogue warps alone at the block barrier below: a warp
            // that failed keeps walking the groups without touching anything, and the barrier itself carries the
            // vote that ends the loop for all four warps together.
            bool ok = warp_wait(&sh->acc_full[buf], (uint32_t(i) >> 1) & 1, abort_flag, status, ST_EPI_ACC, lane);
            tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + buf * BN;
            #pragma unroll 1
            for(int g = set; g < GROUPS; g += SETS) {
                const uint32_t j = uint32_t(i) * GROUPS + g;        // the group's number in the CTA's sequence: picks its buffer
                const int e = j % E_BUFS;
                const int col0 = w.n_tile * BN + g * 32;
                if(ok) {
                    uint32_t v[32];
                    tmem_ld(taddr + g * 32, v);
                    const float bias_lane = g == set ? bias_g[0] : bias_g[1];
                    // the buffer: with a residual it arrives filled by the copy thread, otherwise it only has to be free
                    ok = q.has_res ? warp_wait(&sh->e_full[e], (j / E_BUFS) & 1, abort_flag, status, ST_EPI_BUF, lane)
                                   : warp_wait(&sh->e_empty[e], ((j / E_BUFS) & 1) ^ 1, abort_flag, status, ST_EPI_BUF, lane);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if(g + SETS >= GROUPS) {
                        // this warp's last read of the accumulator
                        tc_fence_before();
                        __syncwarp();
                        if(lane == 0) mbar_arrive(&sh->acc_empty[buf]);
                    }
                    if(ok) {
                        float *slot = e_bufs + e * (E_BUF_BYTES / 4) + row;      // (channel c of the group, this row) at slot[c * 128]
                        if(lean) {
                            #pragma unroll
                            for(int c = 0; c < 32; c++) {
                                float a = __uint_as_float(v[c]);
                                a += __shfl_sync(0xffffffffu, bias_lane, c);
                                a = fminf(fmaxf(a, clamp.x), clamp.y);
                                if(q.has_res) a = fminf(fmaxf(a + q.res_scale * slot[c * BM], post_clamp.x), post_clamp.y);
                                slot[c * BM] = a;
                            }
                        }
                        else {
                            #pragma unroll
                            for(int c = 0; c < 32; c++) {
                                float a = __uint_as_float(v[c]);
                                a += __shfl_sync(0xffffffffu, bias_lane, c);
                                a = apply_act(a, q.act);
                                if(q.has_res) a = apply_act(a + q.res_scale * slot[c * BM], q.post_act);
                                slot[c * BM] = a;
                            }
                        }
                        fence_proxy_async_shared();
                    }
                }
                // the four epilogue warps meet: the block is complete (or somebody gave up)
                if(!epilogue_barrier_all(ok, set)) { live = false; break; }
                if(storer) {
                    tma_store_3d(&tm_y, w.pix0, col0, w.b, e_bufs + e * (E_BUF_BYTES / 4));
                    bulk_commit_group();
                    if(release_at_once) {
                        // once the store has read the buffer it can take the residual operand of a later group: the sooner the
                        // copy thread learns of it, the further ahead of the epilogue its copies run
                        bulk_wait_group_read<0>();
                        mbar_arrive(&sh->e_empty[e]);
                    }
                    else {
                        // nobody is waiting to fill the buffer: let this store read on and hand back the set's previous one
                        bulk_wait_group_read<1>();
                        if(j >= uint32_t(SETS)) mbar_arrive(&sh->e_empty[(j - SETS) % E_BUFS]);
                    }
                }
            }
        }
        if(storer) bulk_wait_group<0>();
    }
    else {
        // ------------------------------------------------------------------ converters
        const int quad = warp & 3, group = (warp - WARP_CONV0) >> 2;
        const int row = quad * 32 + lane;
        const uint32_t total = uint32_t(my_items * kblocks);
        #pragma unroll 1
        for(uint32_t it = group; it < total; it += 2) {
            const int sa = it % S_STAGES, st = it % T_STAGES;
            if(!warp_wait(&sh->sa_full[sa], (it / S_STAGES) & 1, abort_flag, status, ST_CONV_FULL, lane)) break;
            const float *src = reinterpret_cast<const float *>(a_ring + sa * A_STAGE_BYTES) + row;    // [channel][pixel]
            float buf[BK];
            #pragma unroll
            for(int k = 0; k < BK; k++) buf[k] = src[k * BM];
            // Split: the tensor core reads only the TF32 part of an fp32 word, so the value itself serves as "hi";
            // lo = v - tf32(v) goes to the 32 columns after it.
            uint32_t lo[BK];
            #pragma unroll
            for(int k = 0; k < BK; k++) lo[k] = __float_as_uint(buf[k] - __uint_as_float(__float_as_uint(buf[k]) & 0xffffe000u));
            // the values are in registers: the shared-memory stage can take the next copy
            __syncwarp();
            if(lane == 0) mbar_arrive(&sh->sa_empty[sa]);
            if(!warp_wait(&sh->empty[st], ((it / T_STAGES) & 1) ^ 1, abort_flag, status, ST_CONV_EMPTY, lane)) break;
            tc_fence_after();
            const uint32_t t_hi = tmem_base + (uint32_t(quad * 32) << 16) + A_COL_BASE + st * 64;
            #pragma unroll
            for(int h = 0; h < 2; h++) {
                uint32_t hi16[16], lo16[16];
                #pragma unroll
                for(int k = 0; k < 16; k++) { hi16[k] = __float_as_uint(buf[h * 16 + k]); lo16[k] = lo[h * 16 + k]; }
                tmem_st16(t_hi + h * 16, hi16);
                tmem_st16(t_hi + 32 + h * 16, lo16);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(&sh->full_a[st]);
        }
    }

    // ---------------------------------------------------------------------- teardown
teardown:
    tc_fence_before();
    __syncthreads();
    if(*(volatile int *)abort_flag) {
        // a wait gave up: let the MMAs already issued retire (bounded) before tensor memory goes away
        // (a commit covers the MMAs of the thread that executes it: one from each issuer, or two from the only one)
        if(warp == second_issuer && elect_one()) mma_commit(smem_u32(&sh->drain));
        if(warp == WARP_MMA && elect_one()) {
            mma_commit(smem_u32(&sh->drain));
            if(second_issuer < 0) mma_commit(smem_u32(&sh->drain));
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

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn()
{
    static std::mutex mutex;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if(!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess && res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [pixels, channels, images] view of an NCHW tensor (or of a channel range of it); box = 128 pixels x 32 channels.
static dlp_status make_map(CUtensorMap &m, const float *base, int plane, int channels, long long batch_stride, int images)
{
    EncodeTiledFn enc = encode_fn();
    if(!enc) return fail(DLP_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = { cuuint64_t(plane), cuuint64_t(channels), cuuint64_t(images) };
    cuuint64_t strides[2] = { cuuint64_t(plane) * 4, cuuint64_t(batch_stride) * 4 };
    cuuint32_t box[3] = { cuuint32_t(BM), 32, 1 }, elem[3] = { 1, 1, 1 };
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS) return fail(DLP_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return DLP_OK;
}

template<int BN>
static dlp_status launch_bn(const CUtensorMap &tx, const CUtensorMap &ty, const CUtensorMap &tr, const float *packed, const Params &q,
                            cudaStream_t stream)
{
    {
        static std::mutex mutex;
        static std::vector<char> configured;          // by device ordinal: the attribute belongs to the function in that device's context
        int dev = 0;
        DLP_CUDA_OK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mutex);
        if(size_t(dev) >= configured.size()) configured.resize(size_t(dev) + 1, 0);
        if(!configured[dev]) {
            DLP_CUDA_OK(cudaFuncSetAttribute(pointwise_tf32x3_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
            configured[dev] = 1;
        }
    }
    int *status = device_status_word();
    if(!status) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    const int grid = int(std::min<long long>(q.num_items, sm_count()));
    Params r = q;
    constexpr int b_stage_bytes = 2 * BN * BK * 4;
    r.resident = q.kblocks * b_stage_bytes <= MAX_B_BYTES && grid % q.n_tiles == 0;
    r.b_bytes = (r.resident ? q.kblocks : T_STAGES) * b_stage_bytes;
    // the rest of shared memory in 16 KB units: split between the A ring and the epilogue buffers
    const int avail = (SMEM_LIMIT - SMEM_FIXED - r.b_bytes) / A_STAGE_BYTES;
    if(avail <= 6) {
        // full weights region: a residual operand needs the buffers more than A needs depth
        r.s_stages = q.has_res ? 2 : 4;
        r.e_bufs = avail - r.s_stages;
    }
    else {
        r.s_stages = std::min(MAX_S_STAGES - 1, avail / 2);
        r.e_bufs = std::min(MAX_E_BUFS, avail - r.s_stages);
    }
    const int smem_bytes = SMEM_FIXED + r.b_bytes + (r.s_stages + r.e_bufs) * A_STAGE_BYTES;
    pointwise_tf32x3_kernel<BN><<<grid, NUM_THREADS, smem_bytes, stream>>>(tx, ty, tr, packed, r, status);
    DLP_LAUNCH_OK("pointwise_tf32x3_kernel");
    return DLP_OK;
}

} // namespace pw

bool pointwise_tc_eligible(const Contraction &p, const TcPacked &L)
{
    if(p.a_mode != A_STRIDED || p.plane < pw::BM || p.out_mode != OUT_NCHW) return false;
    if(p.plane % 4 != 0 || p.in_h * p.in_w != p.plane || p.a_k_stride != p.plane) return false;    // 1x1, stride 1: output pixel = input pixel
    if(L.k_pad / pw::BK > 8) return false;                                    // one partial accumulator
    if(p.beta != 0.0f || p.bias_mode == DLP_GEMM_BIAS_M) return false;
    if(p.rows % p.plane != 0 || p.rows / p.plane >= (1ll << 31)) return false;
    // the clipped last tile of every image is computed in full: worth it while that costs little (measured on 14x14
    // planes, 31 % of the rows clipped: 128 -> 512 channels 0.063 -> 0.054 ms with this kernel, 256 -> 1024 0.189 -> 0.205 ms)
    const int tpi = ceil_div(p.plane, pw::BM);
    const int clip_limit = L.k_pad / pw::BK <= 4 ? 135 : 115;
    if((long long)tpi * pw::BM * 100 > (long long)p.plane * clip_limit) return false;
    const uintptr_t align = reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.y) | reinterpret_cast<uintptr_t>(p.residual);
    if(align % 16 != 0 || (p.a_batch_stride % 4) != 0) return false;
    return true;
}

dlp_status launch_pointwise_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream)
{
    const int images = int(p.rows / p.plane);
    CUtensorMap tx, ty, tr;
    dlp_status st = pw::make_map(tx, p.a, p.plane, p.k, p.a_batch_stride, images);
    if(st != DLP_OK) return st;
    const long long out_batch_stride = (long long)p.out_channels_total * p.plane;
    st = pw::make_map(ty, p.y, p.plane, p.cols, out_batch_stride, images);
    if(st != DLP_OK) return st;
    st = pw::make_map(tr, p.residual ? p.residual : p.y, p.plane, p.cols, out_batch_stride, images);
    if(st != DLP_OK) return st;
    pw::Params q;
    memset(&q, 0, sizeof(q));
    q.plane = p.plane;
    q.cols = p.cols;
    q.kblocks = L.k_pad / pw::BK;
    q.tiles_per_image = ceil_div(p.plane, pw::BM);
    q.n_tiles = L.n_pad / L.bn;
    q.num_items = (long long)images * q.tiles_per_image * q.n_tiles;
    q.bias = p.bias_mode == DLP_GEMM_BIAS_N ? p.bias : nullptr;
    q.act = p.act;
    q.post_act = p.post_act;
    q.has_res = p.residual != nullptr;
    q.res_scale = p.residual_scale;
    switch(L.bn) {
    case 32: return pw::launch_bn<32>(tx, ty, tr, packed, q, stream);
    case 64: return pw::launch_bn<64>(tx, ty, tr, packed, q, stream);
    case 128: return pw::launch_bn<128>(tx, ty, tr, packed, q, stream);
    default: return fail(DLP_INVALID_ARGUMENT, "unsupported column tile");
    }
}

} // namespace dlp
