// Convolutions with up to 64 output channels over wide rows, on the sm_100a tensor cores (3xTF32, fp32 in and out), with
// the input fetched by the copy engines: the 7x7 stem and the 3x3 convolutions of the 56x56 stage.  Same arithmetic, same
// packed weights (tap-block or row-taps order) and the same order of the sum over K as contraction_tf32x3_kernel; what
// differs is how the A operand reaches the tensor core.  There the loader threads fetch every element of every k-block from
// global memory (32 loads per thread and k-block, and their rate sets the kernel's pace whatever the tile width); here
//
//   * an output tile is R whole output rows of ONE image (R * OW <= 128 rows of the MMA; the rest of the 128 is padding),
//     so the input it needs is a box of the 4-D tensor [W, H, channels, images]: rows oy0*S - pad .. of all columns, for 32
//     channels (tap-block order) or all of them (row-taps order).  One tensor-map copy brings that patch into shared memory,
//     zero-filled outside the image -- so no thread tests a bound -- starting four columns left of the image because a
//     tensor-map copy must start on a 16-byte boundary;
//   * every k-block of the tile that reads those channels (nine taps of a 3x3 kernel) is gathered from the patch: converter
//     warps read their row's 32 values from shared memory at offsets that depend only on the tap, split them into the TF32
//     part and the remainder and write both to the tensor-memory ring the MMAs read;
//   * the sum over K is cut into chunks of eight k-blocks as in the general kernel (the tensor core truncates when it adds into
//     its accumulator); the partial sums are added in registers by the epilogue warps, 32 columns per thread;
//   * the result leaves through shared memory and a tensor-map store of R * OW pixels x 32 channels, which clips rows beyond
//     the image.
//   * Roles (20 warps): warp 0 patch copies, warps 1 and 2 MMA issue (in turn), warp 3 weight copies, warps 8-15 converters (two groups taking
//     k-blocks in turn), warps 4-7 and 16-19 two sets of epilogue warps, one per 32 output channels.
//   * Every wait is bounded (device status word + abort flag); each copy-issuing thread waits for its own copies before it
//     leaves, and tensor memory is freed on every path.
//
// Reference: the implicit GEMM of src/kernels/sgemm.cl:95-123 (B(k, n) gathered from x, zero outside the image).
#include "tc_device.cuh"
#include <cuda.h>
#include <algorithm>
#include <mutex>
#include <vector>
#include <cstring>

namespace dlp {
namespace sg {

using namespace tc;

constexpr int BM = 128, BK = 32;
constexpr int T_STAGES = 4;                 // tensor-memory ring of A (and the B ring when the weights stream)
constexpr int CHUNK_KB = 8;                 // k-blocks summed inside the tensor core before the sum moves to fp32 adds
constexpr int MAX_S_STAGES = 4, MAX_E_BUFS = 4;
constexpr int MAX_B_BYTES = 96 * 1024;
constexpr int MAX_B_STAGES = 12;
constexpr int E_BUF_BYTES = BM * 32 * 4;
constexpr int MAX_PATCH_BYTES = 40 * 1024;
constexpr int MAX_KBLOCKS = 40;             // k-blocks per tile (tables in the barrier block)
constexpr int A_COL_BASE = 256, TMEM_COLS = 512;
constexpr int WARP_A = 0, WARP_MMA = 1, WARP_MMA2 = 2, WARP_B = 3, WARP_ACC0 = 4, WARP_CONV0 = 8, WARP_ACC1 = 16;
constexpr int NUM_WARPS = 20, NUM_THREADS = NUM_WARPS * 32;
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int SMEM_FIXED = 1024 + 1024;     // alignment slack + the barrier block

// codes left in the device status word
enum { ST_A_EMPTY = 301, ST_B_EMPTY = 302, ST_CONV_FULL = 304, ST_CONV_EMPTY = 305, ST_MMA_A = 306, ST_MMA_B = 307,
       ST_MMA_ACC = 308, ST_EPI_ACC = 309, ST_EPI_BUF = 310, ST_DRAIN = 311 };

struct Shared {
    unsigned long long sa_full[MAX_S_STAGES];  // a patch landed in the shared-memory ring
    unsigned long long sa_empty[MAX_S_STAGES]; // ... and the eight converter warps have read their last k-block from it
    unsigned long long full_a[T_STAGES];       // the k-block's hi/lo columns are written to tensor memory (4 converter warps)
    unsigned long long full_b[MAX_B_STAGES];   // a B stage landed
    unsigned long long empty[T_STAGES / 2];    // the MMAs of a pair of k-blocks retired: their tensor-memory columns (and B stages) are free
    unsigned long long acc_full[2], acc_empty[2];
    unsigned long long e_empty[MAX_E_BUFS];    // the store of an epilogue buffer has read it
    unsigned long long drain;
    uint32_t tmem_base;
    int abort_flag;
    // per k-block of a tile: which patch of the tile it reads and where its first value lies in a patch channel; in the
    // row-taps order, per group of eight columns, the offset of its (channel, kernel row) or -1 beyond the last channel
    short kb_patch[MAX_KBLOCKS];
    int kb_offset[MAX_KBLOCKS * 4];
};
static_assert(sizeof(Shared) <= 1024, "barrier block");

struct Params {
    int ow, oh;             // output plane
    int rows_per_tile;      // R: output rows of a tile
    int valid;              // R * ow: rows of the 128 that are output pixels
    int tiles_per_image, n_tiles;
    long long num_items;    // images * tiles_per_image * n_tiles
    int stride, pad, kh, kw, cin;
    int row_taps;           // 0: k-block = (channel block, tap); 1: k-block = four (channel, kernel row) groups of eight columns
    int x_shift;            // the patch starts this many columns left of the image (0 or 4)
    int w_box, h_box, c_box, chan_stride;   // patch box and the floats between two channels of it
    int patch_bytes, slot_bytes;
    int kblocks, cblocks;   // k-blocks per tile; patches per tile
    int resident, b_bytes, s_stages, e_bufs;
    int cols;
    const float *bias;
    int act;
};

struct Item {
    int b, t, n_tile;
};
__device__ __forceinline__ Item decode(long long item, const Params &q)
{
    Item w;
    const long long m_tile = item / q.n_tiles;
    w.n_tile = int(item - m_tile * q.n_tiles);
    w.b = int(m_tile / q.tiles_per_image);
    w.t = int(m_tile - (long long)w.b * q.tiles_per_image);
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

__device__ __forceinline__ void tma_load_4d(void *dst, const void *tmap, int x, int y, int z, int w, unsigned long long *bar)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}

template<int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
staged_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y, const float *__restrict__ packed,
                     const Params q, int *status)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int B_TILE_BYTES = BN * BK * 4;
    constexpr int B_STAGE_BYTES = 2 * B_TILE_BYTES;              // hi tile, then lo tile
    static_assert(MAX_B_BYTES / B_STAGE_BYTES <= MAX_B_STAGES, "barrier array");
    constexpr int GROUPS = BN / 32, SETS = GROUPS;               // one set of epilogue warps per 32 output channels
    static_assert(GROUPS <= 2, "column tiles of 32 or 64");
    const int S_STAGES = q.s_stages, E_BUFS = q.e_bufs;
    Shared *sh = reinterpret_cast<Shared *>(smem);
    unsigned char *b_region = smem + 1024;
    unsigned char *p_ring = b_region + q.b_bytes;
    float *e_bufs = reinterpret_cast<float *>(p_ring + S_STAGES * q.slot_bytes);
    int *abort_flag = &sh->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = q.kblocks;
    const long long my_items = blockIdx.x < q.num_items ? (q.num_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if(threadIdx.x == 0) {
        for(int s = 0; s < MAX_S_STAGES; s++) { mbar_init(&sh->sa_full[s], 1); mbar_init(&sh->sa_empty[s], 8); }
        for(int s = 0; s < T_STAGES; s++) mbar_init(&sh->full_a[s], 4);
        for(int s = 0; s < T_STAGES / 2; s++) mbar_init(&sh->empty[s], 1);
        for(int s = 0; s < MAX_B_STAGES; s++) mbar_init(&sh->full_b[s], 1);
        for(int a = 0; a < 2; a++) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 4 * SETS); }
        for(int e = 0; e < MAX_E_BUFS; e++) mbar_init(&sh->e_empty[e], 1);
        mbar_init(&sh->drain, 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(int(threadIdx.x) < kblocks) {
        const int kb = threadIdx.x, taps = q.kh * q.kw;
        if(q.row_taps) {
            sh->kb_patch[kb] = 0;
            for(int jg = 0; jg < 4; jg++) {
                const int gi = kb * 4 + jg, c = gi / q.kh, ky = gi - c * q.kh;
                sh->kb_offset[kb * 4 + jg] = c < q.cin ? c * q.chan_stride + ky * q.w_box : -1;
            }
        }
        else {
            const int cb = kb / taps, tap = kb - cb * taps, ky = tap / q.kw, kx = tap - ky * q.kw;
            sh->kb_patch[kb] = short(cb);
            sh->kb_offset[kb * 4] = ky * q.w_box + kx;
        }
    }
    if(warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&sh->tmem_base;

    if(warp == WARP_A) {
        // ------------------------------------------------------------------ patch copies
        if(lane == 0) {
            uint32_t pi = 0;
            bool live = true;
            for(long long item = blockIdx.x; item < q.num_items && live; item += gridDim.x) {
                const Item w = decode(item, q);
                const int iy0 = w.t * q.rows_per_tile * q.stride - q.pad;
                for(int cb = 0; cb < q.cblocks; cb++, pi++) {
                    const int s = pi % S_STAGES;
                    if(!mbar_wait(&sh->sa_empty[s], ((pi / S_STAGES) & 1) ^ 1, abort_flag, status, ST_A_EMPTY)) { live = false; break; }
                    mbar_arrive_expect_tx(&sh->sa_full[s], q.patch_bytes);
                    tma_load_4d(p_ring + s * q.slot_bytes, &tm_x, -q.x_shift, iy0, cb * q.c_box, w.b, &sh->sa_full[s]);
                }
            }
            drain_own(sh->sa_full, S_STAGES, pi, status);
        }
    }
    else if(warp == WARP_B) {
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
                        if(!mbar_wait(&sh->empty[s >> 1], ((it / T_STAGES) & 1) ^ 1, abort_flag, status, ST_B_EMPTY)) { live = false; break; }
                        mbar_arrive_expect_tx(&sh->full_b[s], B_STAGE_BYTES);
                        bulk_load(b_region + s * B_STAGE_BYTES, src + (long long)kb * (B_STAGE_BYTES / 4), B_STAGE_BYTES, &sh->full_b[s]);
                    }
                }
                drain_own(sh->full_b, T_STAGES, it, status);
            }
        }
    }
    else if(warp == WARP_MMA || warp == WARP_MMA2) {
        // ------------------------------------------------------------------ MMA issuers
        // As in contraction_tf32x3_kernel: two issuer warps take the iterations in turn (an iteration is a pair of k-blocks
        // when they start on an even stage inside one chunk), the whole warp runs the loop with warp-uniform control flow,
        // lanes 0..4 each watch one barrier, a named barrier carries the turn, and stages are released in pairs.
        constexpr uint32_t idesc = instr_desc_tf32(BN);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO, version 1, SWIZZLE_128B
        const uint32_t region_base = ((smem_u32(b_region) & 0x3FFFF) >> 4) | (1u << 16);
        const uint32_t acc_empty0 = smem_u32(&sh->acc_empty[0]), empty0 = smem_u32(&sh->empty[0]), acc_full0 = smem_u32(&sh->acc_full[0]);
        const uint32_t full_a0 = smem_u32(&sh->full_a[0]), full_b0 = smem_u32(&sh->full_b[0]);
        const uint32_t total = uint32_t(my_items * kblocks);
        uint32_t chunk = 0, s = 0, s_phase = 0, it = 0, step = 0;
        int kb = 0, in_chunk = 0;
        const int me = warp == WARP_MMA ? 0 : 1;
        bool dead = false;
        #pragma unroll 1
        while(it < total) {
            const uint32_t buf = chunk & 1;
            const bool pair = (s & 1) == 0 && in_chunk + 2 <= CHUNK_KB && kb + 2 <= kblocks;
            const int n = pair ? 2 : 1;
            const bool closes_chunk = in_chunk + n == CHUNK_KB || kb + n == kblocks;
            const uint32_t ns = (s + n) & (T_STAGES - 1), nphase = ns < s ? s_phase ^ 1 : s_phase;
            const uint32_t sb = q.resident ? uint32_t(kb) : s;        // the B stage of the first k-block (the second is the next one)
            if(int(step & 1) == me) {
                if(!dead) {
                    // lanes 0, 2: the A columns of the first / second stage; lanes 1, 3: their B stages; lane 4: the accumulator a chunk opens
                    const bool mine = lane < 2 || (lane < 4 && pair) || (lane == 4 && in_chunk == 0);
                    const uint32_t h = lane >> 1;
                    const uint32_t bar = lane == 4 ? acc_empty0 + 8 * buf : (lane & 1 ? full_b0 + 8 * (sb + h) : full_a0 + 8 * (s + h));
                    const uint32_t parity = lane == 4 ? ((chunk >> 1) & 1) ^ 1 : ((lane & 1) && q.resident ? 0u : s_phase);
                    const int code = lane == 4 ? ST_MMA_ACC : (lane & 1 ? ST_MMA_B : ST_MMA_A);
                    const bool ok = mine ? mbar_wait(bar, parity, abort_flag, status, code) : true;
                    if(!__all_sync(0xffffffffu, ok)) dead = true;
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
                const uint32_t accumulate = in_chunk != 0;
                // my turn: the other warp has issued the iteration before this one
                if(step > 0) asm volatile("bar.sync %0, 64;" ::"r"(3 + int((step - 1) & 1)) : "memory");
                tc_fence_after();
                if(!dead && elect_one()) {
                    mma_kblock(d, ah[0], al[0], bh[0], bl[0], idesc, accumulate);
                    if(pair) mma_kblock(d, ah[1], al[1], bh[1], bl[1], idesc, 1u);
                }
                __syncwarp();
                tc_fence_before();
                asm volatile("bar.arrive %0, 64;" ::"r"(3 + int(step & 1)) : "memory");      // the other warp's turn
                if(!dead && elect_one()) {
                    if(pair || (s & 1)) mma_commit(empty0 + 8 * (s >> 1));   // frees the A columns and the B tiles of a pair of stages
                    if(closes_chunk) mma_commit(acc_full0 + 8 * buf);
                }
                __syncwarp();
            }
            step++;
            it += n;
            s = ns;
            s_phase = nphase;
            in_chunk = closes_chunk ? 0 : in_chunk + n;
            kb = kb + n == kblocks ? 0 : kb + n;
            chunk = closes_chunk ? chunk + 1 : chunk;
        }
        // the last turn handed over is taken by nobody: meet it so that both barriers are left balanced
        if(step > 0 && int(step & 1) == me) asm volatile("bar.sync %0, 64;" ::"r"(3 + int((step - 1) & 1)) : "memory");
    }
    else if((warp >= WARP_ACC0 && warp < WARP_CONV0) || warp >= WARP_ACC1) {
        // ------------------------------------------------------------------ accumulate + epilogue
        const int quad = warp & 3;
        const int set = warp >= WARP_ACC1 ? 1 : 0;                 // which 32 output channels of the tile
        if(set >= SETS) goto teardown;
        const int row = quad * 32 + lane;
        const float2 clamp = act_clamp(q.act);
        const bool lean = act_is_clamp(q.act);
        const bool storer = (warp == WARP_ACC0 || warp == WARP_ACC1) && lane == 0;
        const int chunks_per_tile = (kblocks + CHUNK_KB - 1) / CHUNK_KB;
        const int g = set;
        uint32_t chunk = 0;
        bool live = true;
        long long i = 0;
        for(long long item = blockIdx.x; item < q.num_items && live; item += gridDim.x, i++) {
            const Item w = decode(item, q);
            // the bias of the set's 32 channels is asked for now: its trip to L2 is over long before the last chunk is in
            const float bias_lane = q.bias && w.n_tile * BN + g * 32 + lane < q.cols ? ldg_early(q.bias + w.n_tile * BN + g * 32 + lane) : 0.0f;
            float sum[32];
            bool ok = true;
            #pragma unroll 1
            for(int c = 0; c < chunks_per_tile; c++, chunk++) {
                const uint32_t buf = chunk & 1;
                // a warp whose wait gave up keeps walking without touching anything: the block barrier below carries the vote
                if(ok) ok = warp_wait(&sh->acc_full[buf], (chunk >> 1) & 1, abort_flag, status, ST_EPI_ACC, lane);
                if(!ok) continue;
                tc_fence_after();
                uint32_t v[32];
                tmem_ld(tmem_base + (uint32_t(quad * 32) << 16) + buf * BN + g * 32, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if(lane == 0) mbar_arrive(&sh->acc_empty[buf]);
                #pragma unroll
                for(int k = 0; k < 32; k++) sum[k] = c == 0 ? __uint_as_float(v[k]) : sum[k] + __uint_as_float(v[k]);
            }
            const uint32_t j = uint32_t(i) * GROUPS + g;            // the group's number in the CTA's sequence: picks its buffer
            const int e = j % E_BUFS;
            const int col0 = w.n_tile * BN + g * 32;
            if(ok) {
                ok = warp_wait(&sh->e_empty[e], ((j / E_BUFS) & 1) ^ 1, abort_flag, status, ST_EPI_BUF, lane);
                if(ok) {
                    float *slot = e_bufs + e * (E_BUF_BYTES / 4);      // [channel of the group][valid pixels]
                    #pragma unroll
                    for(int c = 0; c < 32; c++) {
                        float a = sum[c] + __shfl_sync(0xffffffffu, bias_lane, c);
                        a = lean ? fminf(fmaxf(a, clamp.x), clamp.y) : apply_act(a, q.act);
                        if(row < q.valid) slot[c * q.valid + row] = a;
                    }
                    fence_proxy_async_shared();
                }
            }
            // the four epilogue warps of the set meet: the block is complete (or somebody gave up)
            if(!epilogue_barrier_all(ok, set)) { live = false; break; }
            if(storer) {
                tma_store_3d(&tm_y, w.t * q.valid, col0, w.b, e_bufs + e * (E_BUF_BYTES / 4));
                bulk_commit_group();
                bulk_wait_group_read<0>();
                mbar_arrive(&sh->e_empty[e]);
            }
        }
        if(storer) bulk_wait_group<0>();
    }
    else if(warp >= WARP_CONV0 && warp < WARP_ACC1) {
        // ------------------------------------------------------------------ converters
        const int quad = warp & 3, group = (warp - WARP_CONV0) >> 2;
        const int row = quad * 32 + lane;
        const bool is_pixel = row < q.valid;
        const int r_l = is_pixel ? row / q.ow : 0, ox = is_pixel ? row - r_l * q.ow : 0;
        const int base = (r_l * q.stride) * q.w_box + ox * q.stride + q.x_shift - q.pad;      // tap (0, 0) of this pixel in a patch channel
        const uint32_t total = uint32_t(my_items * kblocks);
        // position of this group's k-block: first patch of its work item (in the CTA's sequence of patches), k-block within it
        uint32_t patch0 = 0;
        int kb = group;
        while(kb >= kblocks && patch0 < uint32_t(my_items) * q.cblocks) { kb -= kblocks; patch0 += q.cblocks; }
        uint32_t have_patch = 0xffffffffu;
        #pragma unroll 1
        for(uint32_t it = group; it < total; it += 2) {
            const uint32_t patch = patch0 + sh->kb_patch[kb];
            const int sa = int(patch % uint32_t(S_STAGES)), st = it % T_STAGES;
            if(patch != have_patch) {
                if(!warp_wait(&sh->sa_full[sa], (patch / uint32_t(S_STAGES)) & 1, abort_flag, status, ST_CONV_FULL, lane)) break;
                have_patch = patch;
            }
            const float *src = reinterpret_cast<const float *>(p_ring + sa * q.slot_bytes) + base;
            float buf[BK];
            if(q.row_taps) {
                // four (channel, kernel row) groups of eight consecutive columns; groups beyond the last channel are zeros
                #pragma unroll
                for(int jg = 0; jg < 4; jg++) {
                    const int off = sh->kb_offset[kb * 4 + jg];
                    const bool ok = is_pixel && off >= 0;
                    const float *s8 = src + (off >= 0 ? off : 0);
                    #pragma unroll
                    for(int kx = 0; kx < 8; kx++) buf[jg * 8 + kx] = ok ? s8[kx] : 0.0f;
                }
            }
            else {
                const float *s1 = src + sh->kb_offset[kb * 4];
                #pragma unroll
                for(int c = 0; c < BK; c++) { buf[c] = is_pixel ? *s1 : 0.0f; s1 += q.chan_stride; }
            }
            // Split: the tensor core reads only the TF32 part of an fp32 word, so the value itself serves as "hi";
            // lo = v - tf32(v) goes to the 32 columns after it.
            uint32_t lo[BK];
            #pragma unroll
            for(int k = 0; k < BK; k++) lo[k] = __float_as_uint(buf[k] - __uint_as_float(__float_as_uint(buf[k]) & 0xffffe000u));
            // the position of this group's next k-block; when it lies in another patch this warp is done with the current one
            uint32_t next_patch0 = patch0;
            int next_kb = kb + 2;
            while(next_kb >= kblocks) { next_kb -= kblocks; next_patch0 += q.cblocks; }
            if(it + 2 >= total || next_patch0 + sh->kb_patch[next_kb] != patch) {
                __syncwarp();
                if(lane == 0) mbar_arrive(&sh->sa_empty[sa]);
            }
            if(!warp_wait(&sh->empty[st >> 1], ((it / T_STAGES) & 1) ^ 1, abort_flag, status, ST_CONV_EMPTY, lane)) break;
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
            patch0 = next_patch0;
            kb = next_kb;
        }
    }

    // ---------------------------------------------------------------------- teardown
teardown:
    tc_fence_before();
    __syncthreads();
    if(*(volatile int *)abort_flag) {
        // a wait gave up: let the MMAs already issued retire (bounded) before tensor memory goes away
        if(warp == WARP_MMA && elect_one()) {
            mma_commit(smem_u32(&sh->drain));
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

static dlp_status make_map(CUtensorMap &m, const float *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides, const cuuint32_t *box)
{
    EncodeTiledFn enc = encode_fn();
    if(!enc) return fail(DLP_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint32_t elem[4] = { 1, 1, 1, 1 };
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, cuuint32_t(rank), const_cast<float *>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if(r != CUDA_SUCCESS) return fail(DLP_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return DLP_OK;
}

// The geometry of a launch, or false when the problem is not one for this kernel.
static bool plan(const Contraction &p, const TcPacked &L, Params &q)
{
    memset(&q, 0, sizeof(q));
    if(p.a_mode != A_TAPBLOCK && p.a_mode != A_ROWTAPS) return false;
    if(L.bn > 64 || p.out_mode != OUT_NCHW || p.residual != nullptr || p.beta != 0.0f || p.bias_mode == DLP_GEMM_BIAS_M) return false;
    if(p.plane <= 0 || p.out_w <= 0 || p.plane % p.out_w != 0 || p.rows % p.plane != 0 || p.rows / p.plane >= (1ll << 31)) return false;
    if(p.dil_h != 1 || p.dil_w != 1 || p.stride_h != p.stride_w || p.stride_h < 1 || p.stride_h > 2) return false;
    if(p.kh < 1 || p.kw < 1 || p.kh > 8 || p.kw > 8 || p.pad_w > 4 || p.k % (p.kh * p.kw) != 0) return false;
    q.ow = p.out_w; q.oh = p.plane / p.out_w;
    q.stride = p.stride_h; q.pad = p.pad_w; q.kh = p.kh; q.kw = p.kw;
    if(p.pad_h != p.pad_w) return false;
    q.cin = p.k / (p.kh * p.kw);
    if(p.a_batch_stride != (long long)q.cin * p.in_h * p.in_w) return false;        // one group, whole tensor
    q.row_taps = p.a_mode == A_ROWTAPS;
    if(p.in_w % 4 != 0 || q.ow > BM || p.plane % 4 != 0) return false;
    q.rows_per_tile = std::min(BM / q.ow, q.oh);
    q.valid = q.rows_per_tile * q.ow;
    if(q.valid % 4 != 0 || q.valid * 10 < BM * 8) return false;                         // a 16-byte store box; at most a fifth of the MMA rows idle
    q.tiles_per_image = ceil_div(q.oh, q.rows_per_tile);
    q.n_tiles = L.n_pad / L.bn;
    q.num_items = (p.rows / p.plane) * q.tiles_per_image * q.n_tiles;
    q.x_shift = q.pad > 0 ? 4 : 0;
    const int last_col = (q.ow - 1) * q.stride + (q.row_taps ? ROWTAPS_WIDTH : q.kw) - 1 + q.x_shift - q.pad;
    q.w_box = round_up(last_col + 1, 4);
    q.h_box = (q.rows_per_tile - 1) * q.stride + q.kh;
    q.c_box = q.row_taps ? q.cin : 32;
    if(!q.row_taps && q.cin % 32 != 0) return false;
    q.cblocks = q.row_taps ? 1 : q.cin / 32;
    q.chan_stride = q.w_box * q.h_box;
    q.patch_bytes = q.chan_stride * q.c_box * 4;
    q.slot_bytes = round_up(q.patch_bytes, 1024);
    if(q.w_box > 256 || q.h_box > 256 || q.c_box > 256 || q.patch_bytes > MAX_PATCH_BYTES) return false;
    q.kblocks = L.k_pad / BK;
    if(q.kblocks > MAX_KBLOCKS) return false;
    const int kb_per_patch = q.row_taps ? q.kblocks : q.kh * q.kw;
    if(kb_per_patch < 2) return false;                                                   // both converter groups read every patch
    if(!q.row_taps && q.kblocks != q.cblocks * q.kh * q.kw) return false;
    if(q.row_taps && q.kblocks * BK < q.cin * q.kh * ROWTAPS_WIDTH) return false;
    const uintptr_t align = reinterpret_cast<uintptr_t>(p.a) | reinterpret_cast<uintptr_t>(p.y);
    if(align % 16 != 0) return false;
    q.cols = p.cols;
    q.bias = p.bias_mode == DLP_GEMM_BIAS_N ? p.bias : nullptr;
    q.act = p.act;
    return true;
}

template<int BN>
static dlp_status launch_bn(const CUtensorMap &tx, const CUtensorMap &ty, const float *packed, const Params &q, cudaStream_t stream)
{
    {
        static std::mutex mutex;
        static std::vector<char> configured;          // by device ordinal: the attribute belongs to the function in that device's context
        int dev = 0;
        DLP_CUDA_OK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mutex);
        if(size_t(dev) >= configured.size()) configured.resize(size_t(dev) + 1, 0);
        if(!configured[dev]) {
            DLP_CUDA_OK(cudaFuncSetAttribute(staged_tf32x3_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT));
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
    // the rest of shared memory: two epilogue buffers per set of epilogue warps, then as many patches as fit (at most four)
    r.e_bufs = std::min(MAX_E_BUFS, 2 * (BN / 32));
    const int left = SMEM_LIMIT - SMEM_FIXED - r.b_bytes - r.e_bufs * E_BUF_BYTES;
    r.s_stages = std::min(MAX_S_STAGES, left / r.slot_bytes);
    if(r.s_stages < 2) return fail(DLP_INVALID_ARGUMENT, "no room for two input patches");
    const int smem_bytes = SMEM_FIXED + r.b_bytes + r.s_stages * r.slot_bytes + r.e_bufs * E_BUF_BYTES;
    staged_tf32x3_kernel<BN><<<grid, NUM_THREADS, smem_bytes, stream>>>(tx, ty, packed, r, status);
    DLP_LAUNCH_OK("staged_tf32x3_kernel");
    return DLP_OK;
}

} // namespace sg

bool staged_tc_eligible(const Contraction &p, const TcPacked &L)
{
    sg::Params q;
    return sg::plan(p, L, q);
}

dlp_status launch_staged_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream)
{
    sg::Params q;
    if(!sg::plan(p, L, q)) return fail(DLP_INVALID_ARGUMENT, "not a problem for the staged convolution kernel");
    const int images = int(p.rows / p.plane);
    CUtensorMap tx, ty;
    {
        // input as [W, H, channels, images]; box = the patch
        cuuint64_t dims[4] = { cuuint64_t(p.in_w), cuuint64_t(p.in_h), cuuint64_t(q.cin), cuuint64_t(images) };
        cuuint64_t strides[3] = { cuuint64_t(p.in_w) * 4, cuuint64_t(p.in_w) * p.in_h * 4, cuuint64_t(p.a_batch_stride) * 4 };
        cuuint32_t box[4] = { cuuint32_t(q.w_box), cuuint32_t(q.h_box), cuuint32_t(q.c_box), 1 };
        dlp_status st = sg::make_map(tx, p.a, 4, dims, strides, box);
        if(st != DLP_OK) return st;
    }
    {
        // output as [pixels, channels, images]; box = the tile's pixels x 32 channels
        cuuint64_t dims[3] = { cuuint64_t(p.plane), cuuint64_t(p.cols), cuuint64_t(images) };
        cuuint64_t strides[2] = { cuuint64_t(p.plane) * 4, cuuint64_t(p.out_channels_total) * p.plane * 4 };
        cuuint32_t box[3] = { cuuint32_t(q.valid), 32, 1 };
        dlp_status st = sg::make_map(ty, p.y, 3, dims, strides, box);
        if(st != DLP_OK) return st;
    }
    switch(L.bn) {
    case 32: return sg::launch_bn<32>(tx, ty, packed, q, stream);
    case 64: return sg::launch_bn<64>(tx, ty, packed, q, stream);
    default: return fail(DLP_INVALID_ARGUMENT, "unsupported column tile");
    }
}

} // namespace dlp
