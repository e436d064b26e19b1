// Dense contraction on the sm_100a tensor cores with fp32 accuracy (3xTF32).
//
//   D[row, col] = sum_k A(row, k) * B(col, k),   rows = output pixels, cols = output channels.
//
// Every fp32 operand value v is split as  hi = v with the low 13 mantissa bits cleared (exactly a
// TF32 number) and lo = v - hi (exact in fp32).  The kernel accumulates  lo_a*hi_b + hi_a*lo_b +
// hi_a*hi_b, dropping only lo_a*lo_b (relative size 2^-22).
//
// Data flow per CTA (persistent, one CTA per SM, 128-row x BN-column output tiles, K in blocks of 32):
//   * B (weights) is split once, when it is packed: the packed operand is the sequence of pipeline
//     stages (column tile, k-block), each the exact shared-memory image of the k-block's hi tile
//     followed by its lo tile (128B-swizzled).  One contiguous bulk copy per k-block brings a stage
//     into a shared-memory ring, up to four k-blocks ahead of use.
//   * A (activations): loader warps read the caller's NCHW tensor directly (implicit im2col, no
//     re-layout in memory), split each value in registers and write hi/lo with tcgen05.st into a
//     ring of tensor-memory columns.  The MMA takes A from tensor memory and B from shared memory,
//     which keeps the shared-memory read traffic of the three products at one operand.  The tensor
//     core reads only the TF32 part of an fp32 word, so the unsplit value serves as hi.
//   * one elected thread of a warp-uniform loop issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8), twelve
//     per k-block, testing the next k-block's barriers while they go out.
//   * the tensor core adds into its fp32 accumulator with truncation, which over thousands of steps
//     shows up as a systematic shrink of the result.  So a tensor-memory accumulator only ever holds
//     the partial sum of CHUNK_KB k-blocks (two such buffers alternate); accumulate warps add the
//     partial sums into a shared-memory tile with ordinary round-to-nearest fp32 adds, and on the
//     tile's last chunk apply bias / activation / residual / beta and store straight to NCHW
//     (32 consecutive pixels per warp store) or row-major.
//   * variations: tiles of one or two k-blocks borrow a loader group as a second set of epilogue warps;
//     a spare warp hints the next tile's residual operand into L2; problems with too few tiles are cut
//     along K into extra work items whose partial sums a finishing kernel adds in a fixed order.
//
// All mbarrier waits are bounded: a wait that gives up records a code in the device status word,
// raises the CTA's abort flag, and every role then leaves its loop; the CTA drains its bulk copies
// and frees its tensor memory before it returns.
#include "tc_device.cuh"
#include <cstdlib>
#include <cstdio>
#include <mutex>
#include <vector>

namespace dlp {

namespace tc {

constexpr int BM = 128;              // rows per tile = tensor-memory lanes
constexpr int BK = 32;               // K per pipeline stage: 32 fp32 = one 128-byte swizzle row
constexpr int STAGES = 4;            // pipeline depth: A ring in tensor memory (4 x 64 columns), B ring in shared memory
constexpr int A_COL_BASE = 256;      // tensor-memory columns [0,256): two partial accumulators, [256,512): the A ring
constexpr int TMEM_COLS = 512;
constexpr int CHUNK_KB = 8;          // k-blocks summed inside the tensor core before the sum moves to fp32 adds
// Warp roles.  Tensor-memory lanes are tied to (warp index mod 4), so the accumulate and the loader
// warps start at multiples of four (warp 2 prefetches the residual operand into L2, warp 3 is the second MMA issuer).
constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_PREFETCH = 2, WARP_MMA2 = 3, WARP_ACC0 = 4, WARP_LOAD0 = 8;
constexpr int NUM_ACC_WARPS = 4, NUM_LOADER_WARPS = 8;
constexpr int NUM_WARPS = WARP_LOAD0 + NUM_LOADER_WARPS;
constexpr int NUM_THREADS = NUM_WARPS * 32;

// codes left in the device status word
enum { ST_TMA_EMPTY = 101, ST_MMA_FULL_B = 102, ST_MMA_FULL_A = 103, ST_MMA_ACC = 104, ST_EPI_ACC = 105, ST_LOAD_EMPTY = 106,
       ST_DRAIN = 107 };

// Diagnostics are compiled in only with -DDLP_TC_DIAGNOSTICS (the hot loops are tight and share a small
// instruction cache): the timeline (environment variable DLP_TC_TRACE=<file>) and the switches below
// (environment variable DLP_TC_DIAG, for timing experiments; results are wrong with any set).
enum { DIAG_NO_A_LOADS = 1, DIAG_NO_STORES = 2, DIAG_NO_MMA = 4, DIAG_NO_BIAS_LOADS = 8, DIAG_NO_RESIDUAL_LOADS = 16, DIAG_LEAN_NO_STG = 32 };

struct Shared {
    unsigned long long full_b[STAGES];         // the bulk copy of a k-block's B tiles landed
    unsigned long long full_a[STAGES];         // its A columns are written (the 4 loader warps of the k-block's group)
    unsigned long long empty[STAGES / 2];      // the MMAs that read a pair of stages retired: their A columns and B tiles are free
    unsigned long long acc_full[2];            // a chunk's partial sum is complete in tensor memory
    unsigned long long acc_empty[2];           // ... and has been read out (4 accumulate warps)
    unsigned long long drain;
    unsigned long long sums_ready;             // the accumulate warps have reached the last chunk of the CTA's last work item
    uint32_t tmem_base;
    int abort_flag;
    uint32_t tma_issued;     // k-blocks whose bulk copies were issued
    uint32_t mma_consumed;   // the first k-block the MMA issuer has not taken up
    uint32_t epilogue_started;   // work items of this CTA whose partial sums the accumulate warps have begun to read
};

// Lean store of N output columns of one row: y = clamp(acc + bias) [then clamp(y + s*residual)].
template<int N, bool BIAS, bool RES>
__device__ __forceinline__ void store_cols(const float (&v)[N], float *y0, const float (&res)[N], long long cs, const float *b0,
                                           float2 clamp, float res_scale, float2 post_clamp, bool no_bias_loads = false, bool no_stg = false)
{
    #pragma unroll
    for(int j = 0; j < N; j++) {
        float a = v[j];
        if(BIAS) a += no_bias_loads ? 0.25f : __ldg(b0 + j);
        a = fminf(fmaxf(a, clamp.x), clamp.y);
        if(RES) {
            a = a + res_scale * res[j];
            a = fminf(fmaxf(a, post_clamp.x), post_clamp.y);
        }
        if(!no_stg || a == 12345.678f) *y0 = a;
        y0 += cs;
    }
}

#ifdef DLP_TC_DIAGNOSTICS
// timeline buffer of the DLP_TC_TRACE diagnostic (64 k-blocks x 16 slots)
__device__ long long g_trace[64 * 16];
#endif

// work item -> (tile, part of K)
__device__ __forceinline__ void decode_item(long long item, int splits, long long &tile, int &part)
{
    if(splits == 1) { tile = item; part = 0; return; }
    const unsigned t = unsigned(item) / unsigned(splits);      // items fit 32 bits whenever K is split (few tiles)
    tile = t;
    part = int(unsigned(item) - t * unsigned(splits));
}

// Position of a loader in the CTA's sequence of k-blocks (the sequence runs on across tiles).
struct Cursor {
    long long tile;
    int kb;
    uint32_t it;
};

// Split K: when a problem has too few tiles to fill the GPU the launcher cuts K into `splits` equal parts.
// The kernel then sees num_tiles = tiles * splits work items of kblocks = (all k-blocks) / splits each;
// item = tile * splits + part.  Part s reads its own k-blocks of A and B and writes its partial result
// raw to y + s * split_stride (the launcher points y at scratch); a second kernel adds the parts in order.
//
// BN: column tile.  MODE: how the loaders address A (A_GATHER / A_STRIDED / A_TAPBLOCK); a template
// parameter so that each kernel carries one loader only -- the roles share a small instruction cache.
template<int BN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
contraction_tf32x3_kernel(const float *__restrict__ packed, const Contraction p, int kblocks, int n_tiles,
                          long long num_tiles, int splits, long long split_stride, int ktab_smem_entries, int *status, int diag,
                          long long *trace, const TcBatch batch)
{
    // A batch of matrices runs as gridDim.y independent problems: blockIdx.y picks the matrix, whose A and C lie
    // batch.a_stride / batch.y_stride elements further on and whose packed B follows the previous matrix's.
    const long long a_off = blockIdx.y * batch.a_stride, y_off = blockIdx.y * batch.y_stride;
    packed += (long long)blockIdx.y * (2ll * n_tiles * BN) * ((long long)kblocks * splits * BK);
#ifdef DLP_TC_DIAGNOSTICS
    // optional timeline of CTA 0: trace[k-block or chunk][slot] = SM clock at a few points of each role
    // (bits 8.. of diag, when set, select which slots are recorded, so that a measurement can run with few probes)
    const uint32_t trace_slots = trace && blockIdx.x == 0 ? ((diag >> 8) ? uint32_t(diag >> 8) : 0xffffu) : 0u;
#define TC_TRACE(slot, idx) do { if(((trace_slots >> (slot)) & 1u) && (idx) < 64) trace[(idx) * 16 + (slot)] = clock64(); } while(0)
#define TC_DIAG(bit) (diag & (bit))
#else
#define TC_TRACE(slot, idx) do { } while(0)
#define TC_DIAG(bit) false
#endif
    extern __shared__ unsigned char smem_raw[];
    // B ring first, 1024-byte aligned as the 128B swizzle requires; then the fp32 sums, then the barriers.
    // (The offset is applied to the shared array itself so that accesses stay in the shared state space.)
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int B_TILE_BYTES = BN * BK * 4;          // one tile: BN rows of 128 bytes
    constexpr int B_STAGE_BYTES = 2 * B_TILE_BYTES;    // hi tile, then lo tile
    unsigned char *b_ring = smem;
    float *sums = reinterpret_cast<float *>(smem + STAGES * B_STAGE_BYTES);   // [BN][BM]: column-major, a thread owns a row
    Shared *sh = reinterpret_cast<Shared *>(smem + STAGES * B_STAGE_BYTES + BN * BM * 4);
    // gather mode: a copy of the (k -> offset, tap) table when it is small enough (ktab_smem_entries > 0)
    int4 *ktab_s = reinterpret_cast<int4 *>(smem + STAGES * B_STAGE_BYTES + BN * BM * 4 + ((sizeof(Shared) + 15) & ~size_t(15)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Short K (one or two k-blocks per tile): the tile's time is its epilogue, not its MMAs.  Then one loader
    // group feeds all k-blocks and the warps of the other group become a second set of epilogue warps,
    // each set taking every other group of 32 columns.
    const bool short_k = kblocks <= 2 && BN >= 128;
    const int acc_sets = short_k ? 2 : 1;

    if(threadIdx.x == 0) {
        for(int s = 0; s < STAGES; s++) {
            mbar_init(&sh->full_b[s], 1);
            mbar_init(&sh->full_a[s], 4);
        }
        for(int s = 0; s < STAGES / 2; s++) mbar_init(&sh->empty[s], 1);
        for(int a = 0; a < 2; a++) {
            mbar_init(&sh->acc_full[a], 1);
            mbar_init(&sh->acc_empty[a], NUM_ACC_WARPS * acc_sets);
        }
        mbar_init(&sh->drain, 1);
        mbar_init(&sh->sums_ready, NUM_ACC_WARPS);
        sh->abort_flag = 0;
        sh->tma_issued = 0;
        sh->mma_consumed = 0;
        sh->epilogue_started = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(warp == WARP_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if(MODE == A_GATHER || MODE == A_ROWTAPS)
        for(int i = threadIdx.x; i < ktab_smem_entries / 2; i += NUM_THREADS) ktab_s[i] = __ldg(reinterpret_cast<const int4 *>(p.ktab) + i);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t *)&sh->tmem_base;

    // ---- epilogue pieces shared by the accumulate warps and, for a CTA's last work item, the loader warps
    // identity / relu / relu6 are a clamp; with no per-row bias and no beta the whole epilogue is
    // add, clamp, (residual, clamp,) store.  Anything else takes the general path.
    const float2 clamp = act_clamp(p.act), post_clamp = act_clamp(p.post_act);
    const bool epi_fast = act_is_clamp(p.act) && act_is_clamp(p.post_act) && p.bias_mode != DLP_GEMM_BIAS_M && p.beta == 0.0f;
    // The tile is handled 32 columns at a time: two tensor-memory loads under one wait; on the last
    // chunk the residual operand of the same columns is fetched under that wait as well.
    constexpr int G = BN >= 32 ? 32 : 16;
    constexpr int GROUPS = BN / G;
    const int chunks_per_tile = (kblocks + CHUNK_KB - 1) / CHUNK_KB;
    const long long my_items = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // The epilogue of a CTA's last work item has nothing to hide behind.  When that tile is a whole one on the lean path,
    // the loader warps (idle by then) take column groups of its last chunk: group 0 stays with the accumulate warps, 1 and 3
    // go to the first loader group, 2 to the second.  Every side derives the decision from the same CTA-wide values.
    const long long last_item = blockIdx.x + (my_items - 1) * gridDim.x;
    bool tail_help = false;
    if(my_items > 0 && !short_k && GROUPS >= 2 && epi_fast && !TC_DIAG(DIAG_NO_STORES)) {
        long long t;
        int part_unused;
        decode_item(last_item, splits, t, part_unused);
        tail_help = int(t % n_tiles) * BN + BN <= p.cols;
    }
    auto tail_owner = [](int g) { return g == 0 ? 0 : (g == 2 ? 2 : 1); };   // 0: accumulate warps, 1 / 2: loader groups
    struct EpiItem {
        RowInfo r;
        long long row, col_stride;
        int n0, part;
        bool fast, with_res;
        float *y_row;
        const float *res_row;
    };
    auto epi_item = [&](long long item, int row_in_tile) {
        EpiItem e;
        long long tile;
        decode_item(item, splits, tile, e.part);
        e.n0 = int(tile % n_tiles) * BN;
        e.row = (tile / n_tiles) * BM + row_in_tile;
        e.r = make_row(p, e.row, a_off, y_off);
        e.col_stride = p.out_mode == OUT_NCHW ? (long long)p.plane : (p.out_mode == OUT_COL_MAJOR ? p.ldc : 1ll);
        e.fast = epi_fast && e.r.valid && e.n0 + BN <= p.cols && !TC_DIAG(DIAG_NO_STORES);
        e.with_res = e.fast && p.residual != nullptr;
        e.y_row = p.y + e.part * split_stride + e.r.out + (long long)e.n0 * e.col_stride;
        e.res_row = e.with_res ? p.residual + e.r.out + (long long)e.n0 * e.col_stride : nullptr;
        return e;
    };
    // Columns [g*G, g*G+G) of one chunk for the calling thread's row.  release_buf >= 0: after the tensor-memory read the
    // warp hands that partial accumulator back to the MMA issuer.
    auto epi_group = [&](const EpiItem &e, int g, uint32_t taddr, float *my_sums, bool first, bool last, int release_buf, int lane,
                         uint32_t trace_idx) {
        uint32_t v[G];
        float res[G];
        __syncwarp();
        if(warp == WARP_ACC0 && lane == 0) TC_TRACE(9, trace_idx);
        tmem_ld(taddr + g * G, v);
        if(last && e.with_res) {
            // the residual operand of these columns travels while the tensor-memory load does
            const float *rp = e.res_row + (long long)(g * G) * e.col_stride;
            #pragma unroll
            for(int j = 0; j < G; j++) { res[j] = TC_DIAG(DIAG_NO_RESIDUAL_LOADS) ? 0.5f : __ldg(rp); rp += e.col_stride; }
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if(warp == WARP_ACC0 && lane == 0) TC_TRACE(10, trace_idx);
        if(release_buf >= 0) {
            // the partial accumulator is fully read: hand it back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(&sh->acc_empty[release_buf]);
        }
        float x[G];
        float *sg = my_sums + g * G * BM;
        #pragma unroll
        for(int j = 0; j < G; j++) x[j] = first ? __uint_as_float(v[j]) : sg[j * BM] + __uint_as_float(v[j]);
        if(!last) {
            #pragma unroll
            for(int j = 0; j < G; j++) sg[j * BM] = x[j];
            return;
        }
        // ---- last chunk: these columns of the row are final
        const int col0 = e.n0 + g * G;
        if(e.fast) {
            float *y0 = e.y_row + (long long)(g * G) * e.col_stride;
            const float *b0 = p.bias + col0;
            const bool nb = TC_DIAG(DIAG_NO_BIAS_LOADS), ns = TC_DIAG(DIAG_LEAN_NO_STG);
            if(e.with_res) {
                if(p.bias_mode == DLP_GEMM_BIAS_N) store_cols<G, true, true>(x, y0, res, e.col_stride, b0, clamp, p.residual_scale, post_clamp, nb, ns);
                else store_cols<G, false, true>(x, y0, res, e.col_stride, b0, clamp, p.residual_scale, post_clamp, nb, ns);
            }
            else {
                if(p.bias_mode == DLP_GEMM_BIAS_N) store_cols<G, true, false>(x, y0, res, e.col_stride, b0, clamp, 0.0f, post_clamp, nb, ns);
                else store_cols<G, false, false>(x, y0, res, e.col_stride, b0, clamp, 0.0f, post_clamp, nb, ns);
            }
        }
        else {
            // general epilogue: the values pass through the thread's own slots of the sums tile so
            // that this loop can index them (a register array indexed by a loop counter would live
            // in local memory on every path)
            #pragma unroll
            for(int j = 0; j < G; j++) sg[j * BM] = x[j];
            if(e.r.valid && !TC_DIAG(DIAG_NO_STORES)) {
                #pragma unroll 1
                for(int j = 0; j < G; j++)
                    if(col0 + j < p.cols)
                        p.y[e.part * split_stride + out_index(p, e.r, col0 + j)] = finish_output(p, e.r, e.row, col0 + j, sg[j * BM]);
            }
        }
        if(warp == WARP_ACC0 && lane == 0) TC_TRACE(11, trace_idx);
    };

    if(warp == WARP_TMA) {
        // ------------------------------------------------------------------ B producer
        if(lane == 0) {
            uint32_t it = 0;
            bool live = true;
            for(long long item = blockIdx.x; item < num_tiles && live; item += gridDim.x) {
                // the packed operand holds the stages in the order (column tile, k-block), each one the exact
                // shared-memory image of its hi and lo tiles
                long long tile;
                int part;
                decode_item(item, splits, tile, part);
                const float *src = packed + ((long long)(tile % n_tiles) * splits + part) * kblocks * (B_STAGE_BYTES / 4);
                for(int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % STAGES;
                    if(!mbar_wait(&sh->empty[s >> 1], ((it / STAGES) & 1) ^ 1, &sh->abort_flag, status, ST_TMA_EMPTY)) { live = false; break; }
                    TC_TRACE(0, it);
                    mbar_arrive_expect_tx(&sh->full_b[s], B_STAGE_BYTES);
                    bulk_load(b_ring + s * B_STAGE_BYTES, src + (long long)kb * (B_STAGE_BYTES / 4), B_STAGE_BYTES, &sh->full_b[s]);
                    *(volatile uint32_t *)&sh->tma_issued = it + 1;
                }
            }
        }
    }
    else if(warp == WARP_MMA || warp == WARP_MMA2) {
        // ------------------------------------------------------------------ MMA issuers
        // One thread feeds the tensor core, and what it executes per k-block is a dependent scalar chain
        // that has to stay shorter than the tensor core's own time for the k-block.  So:
        //  * the whole warp runs the loop with warp-uniform control flow and every MMA operand is computed
        //    outside the elected region, so the operands can stay in uniform registers;
        //  * lanes 0..2 each watch one barrier of the coming k-block (its A columns, its B tiles, and when it
        //    opens a partial accumulator "read out"); the barriers of k-block it+1 are tested before the
        //    MMAs of k-block it go out and the answer is collected after them, so in the steady state
        //    the issuer never sits in a wait;
        //  * a commit costs about as much as six MMAs, so stages are released in pairs.
        constexpr uint32_t idesc = instr_desc_tf32(BN);
        constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO, version 1, SWIZZLE_128B
        const uint32_t ring_base = ((smem_u32(b_ring) & 0x3FFFF) >> 4) | (1u << 16);
        const uint32_t acc_empty0 = smem_u32(&sh->acc_empty[0]), empty0 = smem_u32(&sh->empty[0]), acc_full0 = smem_u32(&sh->acc_full[0]);
        // the barrier array this lane watches (8 bytes per entry): even lanes the A columns, odd lanes the B tiles
        const uint32_t watch_base = smem_u32(lane & 1 ? &sh->full_b[0] : &sh->full_a[0]);
        const long long my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const uint32_t total = uint32_t(my_tiles * kblocks);
        uint32_t chunk = 0, s = 0, s_phase = 0;           // partial accumulators so far; ring position and parity
        int kb = 0, in_chunk = 0;
        uint32_t it = 0;
        // An iteration takes two k-blocks when they start on an even stage and lie in the same chunk (the usual
        // case): one barrier test, one vote, one release commit and one round of loop bookkeeping for 24 MMAs.
        // Lanes 0,1 watch the first stage, lanes 2,3 the second, lane 4 the read-out of a partial accumulator
        // that the first k-block opens.
        auto pairable = [&](uint32_t st, int ic, int k) { return (st & 1) == 0 && ic + 2 <= CHUNK_KB && k + 2 <= kblocks; };
        // Two issuer warps take the iterations in turn.  A single issuer is a serial chain -- wait for the stages, build
        // the operands, issue (which blocks at the tensor core's own pace: its queue is short), commit, vote, loop -- and
        // everything but the issue leaves the tensor core idle.  With two, warp B waits for its stages and builds its
        // operands while warp A's MMAs go out, and starts the moment A has issued its last one (a named barrier carries
        // the turn; tcgen05 fences around it keep the MMAs of the two threads in order), and A's commits and bookkeeping
        // run under B's MMAs.  Both warps step through the same deterministic sequence of iterations; each acts on every
        // other one.  A warp whose wait gives up keeps taking its turns without issuing, so the other is never left
        // alone at the barrier.
        const int me = warp == WARP_MMA ? 0 : 1;
        uint32_t step = 0;
        bool dead = false;
        #pragma unroll 1
        while(it < total) {
            const uint32_t buf = chunk & 1;
            const bool pair = pairable(s, in_chunk, kb);
            const int n = pair ? 2 : 1;
            const bool closes_chunk = in_chunk + n == CHUNK_KB || kb + n == kblocks;
            const uint32_t ns = (s + n) & (STAGES - 1), nphase = ns < s ? s_phase ^ 1 : s_phase;
            if(int(step & 1) == me) {
                if(!dead) {
                    const bool mine = lane < 2 || (lane < 4 && pair) || (lane == 4 && in_chunk == 0);
                    const uint32_t bar = lane == 4 ? acc_empty0 + 8 * buf : watch_base + 8 * (s + (lane >> 1));
                    const uint32_t parity = lane == 4 ? ((chunk >> 1) & 1) ^ 1 : s_phase;
                    const int code = lane == 4 ? ST_MMA_ACC : (lane & 1 ? ST_MMA_FULL_B : ST_MMA_FULL_A);
                    const bool ok = mine ? mbar_wait(bar, parity, &sh->abort_flag, status, code) : true;
                    if(!__all_sync(0xffffffffu, ok)) dead = true;
                }
                if(lane == 0 && me == 0) TC_TRACE(2, it);
                const uint32_t d = tmem_base + buf * BN, a = tmem_base + A_COL_BASE + s * 64;
                const uint32_t bhi = ring_base + s * (B_STAGE_BYTES >> 4), blo = bhi + (B_TILE_BYTES >> 4);
                uint32_t ah[2][4], al[2][4];
                uint64_t bh[2][4], bl[2][4];
                #pragma unroll
                for(int h = 0; h < 2; h++)
                    #pragma unroll
                    for(int j = 0; j < 4; j++) {
                        // stage h of the pair; K=8 step j: 8 columns further in A, 32 bytes (2 descriptor units) further in the B rows
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
                    if(!TC_DIAG(DIAG_NO_MMA)) {
                        mma_kblock(d, ah[0], al[0], bh[0], bl[0], idesc, accumulate);
                        if(pair) mma_kblock(d, ah[1], al[1], bh[1], bl[1], idesc, 1u);
                    }
                }
                __syncwarp();
                tc_fence_before();
                asm volatile("bar.arrive %0, 64;" ::"r"(3 + int(step & 1)) : "memory");      // the other warp's turn
                if(lane == 0 && me == 0) TC_TRACE(5, it);
                if(!dead && elect_one()) {
                    if(pair || (s & 1)) mma_commit(empty0 + 8 * (s >> 1));   // frees the A columns and the B tiles of a pair of stages
                    if(closes_chunk) mma_commit(acc_full0 + 8 * buf);
                }
                __syncwarp();
                if(lane == 0 && me == 0) TC_TRACE(3, it);
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
        if(lane == 0 && me == 0) *(volatile uint32_t *)&sh->mma_consumed = it;
    }
    else if(warp == WARP_PREFETCH) {
        // ------------------------------------------------------------------ residual prefetcher
        // The epilogue of a tile reads its residual operand with 128 strided loads per thread; from HBM
        // their latency is most of the epilogue's time.  This warp asks for the residual tile of the
        // CTA's next work item to be brought into L2 while the current one is still being computed: one
        // tile ahead.  It only ever gives hints: if its pacing wait runs out it simply stops.
        // Worth it (measured) when a tile has 3 to 8 k-blocks: with fewer the tiles are too short to stay a tile
        // ahead, with more the MMAs hide the epilogue anyway.
        if(p.residual != nullptr && !short_k && kblocks <= CHUNK_KB) {
            // item index i of this CTA is prefetched once the accumulate warps have started on item i - 1
            // (a counter they publish); when this warp has fallen behind it skips to where they are
            uint32_t i = 0;
            for(long long item = blockIdx.x; item < num_tiles; item += gridDim.x, i++) {
                uint32_t started = *(volatile uint32_t *)&sh->epilogue_started;
                for(int tries = 0; started < i && tries < (1 << 14); tries++) {
                    __nanosleep(64);
                    started = *(volatile uint32_t *)&sh->epilogue_started;
                }
                if(started < i) break;              // no progress for a long time: stop giving hints
                if(started > i + 1) continue;       // behind: this tile's residual is being read already
                long long tile;
                int part;
                decode_item(item, splits, tile, part);
                const int n0 = int(tile % n_tiles) * BN;
                const long long row0 = (tile / n_tiles) * BM;
                // every 16th row of the tile (64 bytes apart in a channel plane), and its last row: touches every line
                #pragma unroll 1
                for(int j = 0; j <= BM / 16; j++) {
                    const RowInfo r = make_row(p, row0 + min(16 * j, BM - 1), a_off, y_off);
                    if(!r.valid) break;
                    for(int c = lane; c < BN && n0 + c < p.cols; c += 32)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + out_index(p, r, n0 + c)));
                }
            }
        }
    }
    else if(warp < WARP_ACC0) {
        // (no warp left for this branch)
    }
    else if(warp < WARP_LOAD0 || (short_k && warp >= WARP_LOAD0 + 4)) {
        // ------------------------------------------------------------------ accumulate + epilogue
        const int quad = warp & 3;                          // tensor-memory lanes this warp may touch
        const int acc_set = warp < WARP_LOAD0 ? 0 : 1;      // which of the acc_sets sets of epilogue warps this one is in
        const int row_in_tile = quad * 32 + lane;
        float *my_sums = sums + row_in_tile;                // element (col) at my_sums[col * BM]: conflict-free
        uint32_t chunk = 0, items_begun = 0;
        bool live = true;
        for(long long item = blockIdx.x; item < num_tiles && live; item += gridDim.x) {
            const EpiItem e = epi_item(item, row_in_tile);
            const RowInfo &r = e.r;
            const int n0 = e.n0, part = e.part;
            const long long row = e.row, col_stride = e.col_stride;
            float *y_row = e.y_row;
            // A tile whose last columns lie beyond the matrix takes its own, rolled path: groups of columns that do
            // not exist are skipped and the others go column by column through the lean arithmetic when it applies.
            const bool ragged_tile = n0 + BN > p.cols;
            for(int c = 0; c < chunks_per_tile; c++, chunk++) {
                const uint32_t buf = chunk & 1;
                const bool first = c == 0, last = c == chunks_per_tile - 1;
                // the last chunk of the CTA's last item is shared with the loader warps: every earlier sum of the tile is in place
                const bool shared_tail = tail_help && last && item == last_item;
                if(shared_tail) {
                    __syncwarp();
                    if(lane == 0) mbar_arrive(&sh->sums_ready);
                }
                if(!warp_wait(&sh->acc_full[buf], (chunk >> 1) & 1, &sh->abort_flag, status, ST_EPI_ACC, lane)) { live = false; break; }
                if(c == 0 && warp == WARP_ACC0 && lane == 0) *(volatile uint32_t *)&sh->epilogue_started = ++items_begun;
                tc_fence_after();
                const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + buf * BN;
                if(ragged_tile) {
                    const bool lean = epi_fast && r.valid && !TC_DIAG(DIAG_NO_STORES);
                    #pragma unroll 1
                    for(int g = acc_set; g < GROUPS; g += acc_sets) {
                        const int col0 = n0 + g * G, cols_left = p.cols - col0;        // warp-uniform
                        float *sg = my_sums + g * G * BM;
                        if(cols_left > 0) {
                            uint32_t v[G];
                            __syncwarp();
                            tmem_ld(taddr + g * G, v);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            // the values pass through the thread's own slots of the sums tile so that the rolled loops can index them
                            #pragma unroll
                            for(int j = 0; j < G; j++) sg[j * BM] = first ? __uint_as_float(v[j]) : sg[j * BM] + __uint_as_float(v[j]);
                        }
                        if(g + acc_sets >= GROUPS) {
                            tc_fence_before();
                            __syncwarp();
                            if(lane == 0) mbar_arrive(&sh->acc_empty[buf]);
                        }
                        if(!last || cols_left <= 0) continue;
                        const int ncols = min(cols_left, G);
                        if(lean) {
                            float *y0 = y_row + (long long)(g * G) * col_stride;
                            const float *r0 = p.residual ? p.residual + r.out + (long long)col0 * col_stride : nullptr;
                            #pragma unroll 1
                            for(int j = 0; j < ncols; j++) {
                                float a = sg[j * BM];
                                if(p.bias_mode == DLP_GEMM_BIAS_N) a += __ldg(p.bias + col0 + j);
                                a = fminf(fmaxf(a, clamp.x), clamp.y);
                                if(r0) a = fminf(fmaxf(a + p.residual_scale * __ldg(r0 + (long long)j * col_stride), post_clamp.x), post_clamp.y);
                                y0[(long long)j * col_stride] = a;
                            }
                        }
                        else if(r.valid && !TC_DIAG(DIAG_NO_STORES)) {
                            #pragma unroll 1
                            for(int j = 0; j < ncols; j++)
                                p.y[part * split_stride + out_index(p, r, col0 + j)] = finish_output(p, r, row, col0 + j, sg[j * BM]);
                        }
                    }
                    continue;
                }
                #pragma unroll 1
                for(int g = acc_set; g < GROUPS; g += acc_sets) {
                    if(shared_tail && tail_owner(g) != 0) continue;       // a loader group's columns (nobody waits for this buffer again)
                    epi_group(e, g, taddr, my_sums, first, last, g + acc_sets >= GROUPS ? int(buf) : -1, lane, chunk * GROUPS + g);
                }
            }
        }
    }
    else {
        // ------------------------------------------------------------------ A loaders
        const int quad = warp & 3;                       // tensor-memory lanes this warp may touch
        const int groups = short_k ? 1 : 2;              // loader groups taking the k-blocks in turn
        const int group = (warp - WARP_LOAD0) >> 2;      // this warp handles k-blocks with (it % groups) == group
        const int row_in_tile = quad * 32 + lane;
        long long loaded_tile = -1, loaded_row_tile = 0;      // Cursor::tile counts work items
        int loaded_part = 0;
        RowInfo r;
        r.valid = false; r.base = 0; r.iy0 = r.ix0 = 0; r.out = 0;

        const bool row_vec = MODE == A_STRIDED && p.plane == 0 && p.a_k_stride == 1 && (p.a_row_stride & 3) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.a) & 15) == 0;
        auto advance = [&](Cursor &c, int steps) {
            c.kb += steps;
            c.it += steps;
            while(c.kb >= kblocks) { c.kb -= kblocks; c.tile += gridDim.x; }
        };
        // Issue the 32 loads of one k-block for this thread's row; nothing waits on them here.
        // Per tile the thread works out once whether its row exists and, for a convolution, which of the
        // kernel's taps fall inside the image for its pixel (a bit per tap), so the per-element work is
        // a table entry, a bit test and the load.
        unsigned row_mask = 0, col_mask = 0;     // bit ky / kx: that kernel row / column falls inside the image for this pixel
        auto issue_loads = [&](const Cursor &c, float (&buf)[BK]) {
            if(c.tile != loaded_tile) {
                loaded_tile = c.tile;
                decode_item(c.tile, splits, loaded_row_tile, loaded_part);
                r = make_row(p, (loaded_row_tile / n_tiles) * BM + row_in_tile, a_off, y_off);
                if(TC_DIAG(DIAG_NO_A_LOADS)) r.valid = false;
                row_mask = col_mask = 0;
                if((MODE == A_GATHER || MODE == A_ROWTAPS) && r.valid) {
                    for(int ky = 0; ky < p.kh; ky++)
                        if(unsigned(r.iy0 + ky * p.dil_h) < unsigned(p.in_h)) row_mask |= 1u << ky;
                    for(int kx = 0; kx < p.kw; kx++)
                        if(unsigned(r.ix0 + kx * p.dil_w) < unsigned(p.in_w)) col_mask |= 1u << kx;
                }
            }
            // table entry (ky << 8) | kx -> is that tap inside the image for this thread's pixel
            auto tap_inside = [&](int tap) { return ((row_mask >> (tap >> 8)) & (col_mask >> (tap & 255)) & 1u) != 0; };
            const int kb_all = loaded_part * kblocks + c.kb;       // k-block within the whole of K
            const int k0 = kb_all * BK;
            if(MODE == A_STRIDED) {
                const float *src = p.a + r.base + (long long)k0 * p.a_k_stride;
                if(row_vec && r.valid && k0 + BK <= p.k) {
                    // row-major matrix: the 32 values of a k-block are 128 consecutive bytes of the thread's row
                    const float4 *src4 = reinterpret_cast<const float4 *>(src);
                    #pragma unroll
                    for(int i = 0; i < BK / 4; i++) {
                        const float4 t = __ldg(src4 + i);
                        buf[4 * i] = t.x; buf[4 * i + 1] = t.y; buf[4 * i + 2] = t.z; buf[4 * i + 3] = t.w;
                    }
                }
                else if(r.valid && k0 + BK <= p.k) {
                    #pragma unroll
                    for(int i = 0; i < BK; i++) buf[i] = __ldg(src + (long long)i * p.a_k_stride);
                }
                else {
                    #pragma unroll
                    for(int i = 0; i < BK; i++) {
                        const bool ok = r.valid && (k0 + i) < p.k;
                        buf[i] = ok ? __ldg(src + (long long)i * p.a_k_stride) : 0.0f;
                    }
                }
            }
            else if(MODE == A_TAPBLOCK) {
                const int cb = kb_all / p.num_taps, t = kb_all - cb * p.num_taps;
                const int d = __ldg(p.tap_dydx + t);
                const float *src = p.a + r.base + (long long)(cb * BK) * p.a_k_stride + (d >> 16) * p.in_w + (d & 0xffff);
                if(r.valid && unsigned(r.iy0 + (d >> 16)) < unsigned(p.in_h) && unsigned(r.ix0 + (d & 0xffff)) < unsigned(p.in_w)) {
                    #pragma unroll
                    for(int i = 0; i < BK; i++) buf[i] = __ldg(src + (long long)i * p.a_k_stride);
                }
                else {
                    #pragma unroll
                    for(int i = 0; i < BK; i++) buf[i] = 0.0f;
                }
            }
            else if(MODE == A_ROWTAPS) {
                // four (channel, kernel row) groups of eight consecutive input elements; the table (always in shared
                // memory) gives a group's offset and its kernel row, whose validity bit gates the group's column bits
                const int2 *tab = reinterpret_cast<const int2 *>(ktab_s) + kb_all * (BK / ROWTAPS_WIDTH);
                #pragma unroll
                for(int g = 0; g < BK / ROWTAPS_WIDTH; g++) {
                    const int2 e = tab[g];
                    const float *src = p.a + r.base + e.x;
                    const unsigned cols = ((row_mask >> e.y) & 1u) ? col_mask : 0u;
                    #pragma unroll
                    for(int kx = 0; kx < ROWTAPS_WIDTH; kx++) buf[g * ROWTAPS_WIDTH + kx] = (cols >> kx) & 1u ? __ldg(src + kx) : 0.0f;
                }
            }
            else {
                const float *src = p.a + r.base;
                if(ktab_smem_entries > 0) {
                    // table entries from shared memory, two per load, eight elements at a time: the table reads of a
                    // batch are in flight together instead of each element waiting for its own entry
                    const int4 *tab = ktab_s + k0 / 2;
                    #pragma unroll
                    for(int i0 = 0; i0 < BK; i0 += 8) {
                        int4 e[4];
                        #pragma unroll
                        for(int j = 0; j < 4; j++) e[j] = tab[i0 / 2 + j];
                        #pragma unroll
                        for(int j = 0; j < 4; j++) {
                            buf[i0 + 2 * j] = tap_inside(e[j].y) ? __ldg(src + e[j].x) : 0.0f;
                            buf[i0 + 2 * j + 1] = tap_inside(e[j].w) ? __ldg(src + e[j].z) : 0.0f;
                        }
                    }
                }
                else {
                    const int2 *tab = reinterpret_cast<const int2 *>(p.ktab + k0);
                    #pragma unroll
                    for(int i = 0; i < BK; i++) {
                        const int2 t = __ldg(tab + i);          // offset, tap number (63 = padding beyond K: never valid)
                        const bool ok = tap_inside(t.y);
                        buf[i] = ok ? __ldg(src + t.x) : 0.0f;
                    }
                }
            }
        };
        // Split the values and publish them as the A operand of stage (it % STAGES).  The tensor core reads
        // only the TF32 part of an fp32 word (it ignores the low 13 mantissa bits), so the value itself
        // serves as "hi"; the remainder lo = v - tf32(v) goes to the 32 columns after it.
        auto publish = [&](const Cursor &c, const float (&buf)[BK]) -> bool {
            const int s = c.it % STAGES;
            if(quad == 0 && lane == 0) TC_TRACE(6, c.it);
            if(!warp_wait(&sh->empty[s >> 1], ((c.it / STAGES) & 1) ^ 1, &sh->abort_flag, status, ST_LOAD_EMPTY, lane)) return false;
            if(quad == 0 && lane == 0) TC_TRACE(7, c.it);
            tc_fence_after();
            const uint32_t t_hi = tmem_base + (uint32_t(quad * 32) << 16) + A_COL_BASE + s * 64;
            #pragma unroll
            for(int h = 0; h < 2; h++) {
                uint32_t hi[16], lo[16];
                #pragma unroll
                for(int i = 0; i < 16; i++) {
                    const float v = buf[h * 16 + i];
                    hi[i] = __float_as_uint(v);
                    lo[i] = __float_as_uint(v - __uint_as_float(__float_as_uint(v) & 0xffffe000u));
                }
                tmem_st16(t_hi + h * 16, hi);
                tmem_st16(t_hi + 32 + h * 16, lo);
            }
            if(quad == 0 && lane == 0) TC_TRACE(14, c.it);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            if(quad == 0 && lane == 0) TC_TRACE(15, c.it);
            tc_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(&sh->full_a[s]);
            if(quad == 0 && lane == 0) TC_TRACE(8, c.it);
            return true;
        };

        // Two register buffers: the loads of this warp's next k-block are in flight while the current one
        // is split and stored.  The loop holds one copy of each step and hands the buffer over by moves.
        float cur_buf[BK], nxt_buf[BK];
        Cursor cur, nxt;
        nxt.tile = blockIdx.x; nxt.kb = 0; nxt.it = 0;
        advance(nxt, group);
        cur = nxt;
        bool have_cur = false;
        #pragma unroll 1
        for(;;) {
            const bool more = nxt.tile < num_tiles;
            if(quad == 0 && lane == 0) TC_TRACE(12, nxt.it);
            if(more) issue_loads(nxt, nxt_buf);
            if(quad == 0 && lane == 0) TC_TRACE(13, nxt.it);
            if(have_cur && !publish(cur, cur_buf)) break;
            if(!more) break;
            #pragma unroll
            for(int i = 0; i < BK; i++) cur_buf[i] = nxt_buf[i];
            cur = nxt;
            have_cur = true;
            advance(nxt, groups);
        }
        // ---- the last chunk of the CTA's last work item: this loader group's share of the epilogue
        if(tail_help && !*(volatile int *)&sh->abort_flag) {
            const uint32_t last_chunk = uint32_t(my_items * chunks_per_tile - 1), buf = last_chunk & 1;
            if(warp_wait(&sh->sums_ready, 0, &sh->abort_flag, status, ST_EPI_ACC, lane) &&
               warp_wait(&sh->acc_full[buf], (last_chunk >> 1) & 1, &sh->abort_flag, status, ST_EPI_ACC, lane)) {
                tc_fence_after();
                const EpiItem e = epi_item(last_item, row_in_tile);
                const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + buf * BN;
                #pragma unroll 1
                for(int g = 1; g < GROUPS; g++)
                    if(tail_owner(g) == group + 1) epi_group(e, g, taddr, sums + row_in_tile, chunks_per_tile == 1, true, -1, lane, 0);
            }
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

// Pack B(col, k): zero-padded, split into hi and lo, and laid out as the kernel's shared-memory stages
// (see TcPacked): stage (column tile, k-block) = hi tile then lo tile, each bn rows of 32 floats with the
// 16-byte chunks of a row permuted by the 128-byte swizzle (chunk ^ (row & 7)).
// A thread packs one 16-byte chunk (four consecutive k of one column): the swizzle permutes whole chunks, so the chunk is one
// 16-byte store per tile.  n_major: consecutive threads take consecutive columns (sources whose columns are contiguous),
// otherwise consecutive chunks along k (sources whose k is contiguous, read 16 bytes at a time when aligned).
__global__ void prepack_kernel(const float *__restrict__ b, long long col_stride, long long k_stride, int cols, int k,
                               int n_pad, int k_pad, int bn, int taps, float *__restrict__ packed, long long b_batch_stride, int n_major,
                               int row_kw)
{
    const int chunks = k_pad / 4;
    const long long total = (long long)n_pad * chunks;
    b += blockIdx.y * b_batch_stride;           // a batch of matrices: blockIdx.y picks one, packed one after the other
    packed += blockIdx.y * (2ll * n_pad * k_pad);
    const int kblocks = k_pad / BK;
    const bool vec = !n_major && taps == 0 && row_kw == 0 && k_stride == 1 && (col_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        int n, c;
        if(n_major) { c = int(idx / n_pad); n = int(idx - (long long)c * n_pad); }
        else { n = int(idx / chunks); c = int(idx - (long long)n * chunks); }
        const int kk = c * 4, kb = kk / BK, i = kk % BK;
        float v[4] = { 0.0f, 0.0f, 0.0f, 0.0f };
        if(n < cols) {
            if(vec && kk + 4 <= k) {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(b + n * col_stride + kk));
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            }
            else {
                #pragma unroll
                for(int j = 0; j < 4; j++) {
                    int ks = kk + j;
                    if(taps > 0) {
                        // packed order (channel block, tap, channel in block) <- source order (channel, tap)
                        const int cb = kb / taps, t = kb % taps;
                        ks = (cb * BK + i + j) * taps + t;
                    }
                    bool exists = kk + j < k;
                    if(row_kw > 0) {
                        // packed order (channel, kernel row, column padded to 8) <- source order (channel, kernel row, column)
                        const int g = (kk + j) / ROWTAPS_WIDTH, kx = (kk + j) % ROWTAPS_WIDTH;
                        ks = g * row_kw + kx;
                        exists = kx < row_kw && ks < k;
                    }
                    if(exists) v[j] = __ldg(b + n * col_stride + ks * k_stride);
                }
            }
        }
        float4 hi, lo;
        hi.x = __uint_as_float(__float_as_uint(v[0]) & 0xffffe000u); lo.x = v[0] - hi.x;
        hi.y = __uint_as_float(__float_as_uint(v[1]) & 0xffffe000u); lo.y = v[1] - hi.y;
        hi.z = __uint_as_float(__float_as_uint(v[2]) & 0xffffe000u); lo.z = v[2] - hi.z;
        hi.w = __uint_as_float(__float_as_uint(v[3]) & 0xffffe000u); lo.w = v[3] - hi.w;
        const int tile = n / bn, r = n % bn;
        const long long stage = ((long long)tile * kblocks + kb) * (2 * bn * BK);
        const int off = r * BK + (((i >> 2) ^ (r & 7)) << 2);
        *reinterpret_cast<float4 *>(packed + stage + off) = hi;
        *reinterpret_cast<float4 *>(packed + stage + bn * BK + off) = lo;
    }
}

// Second step of a split-K contraction: add the partial results in a fixed order (so the sum does not
// depend on timing) and apply the epilogue.  Partials are column-major [part][col][rows_pad].
__global__ void split_finish_kernel(const Contraction p, const float *__restrict__ partial, int splits, long long split_stride, long long rows_pad)
{
    const long long total = p.rows * p.cols;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int col = int(idx / p.rows);
        const long long row = idx - (long long)col * p.rows;
        const float *src = partial + (long long)col * rows_pad + row;
        float acc = __ldg(src);
        for(int s = 1; s < splits; s++) acc += __ldg(src + s * split_stride);
        const RowInfo r = make_row(p, row);
        p.y[out_index(p, r, col)] = finish_output(p, r, row, col, acc);
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
                      float *packed, int taps, cudaStream_t stream, int batch, long long b_batch_stride, int row_kw)
{
    const long long total = (long long)L.n_pad * (L.k_pad / 4);
    const int threads = 256;
    const int blocks = int(std::min<long long>(ceil_div<long long>(total, threads), 8 * sm_count()));
    if(batch < 1 || batch > 65535) return fail(DLP_INVALID_ARGUMENT, "a batched product takes 1 to 65535 matrices");
    tc::prepack_kernel<<<dim3(blocks, batch), threads, 0, stream>>>(b, b_col_stride, b_k_stride, cols, k, L.n_pad, L.k_pad, L.bn, taps, packed,
                                                                    b_batch_stride, b_col_stride == 1 && b_k_stride != 1 ? 1 : 0, row_kw);
    DLP_LAUNCH_OK("prepack_kernel");
    return DLP_OK;
}

namespace {
// How many equal parts to cut K into.  Time is counted in k-block periods (about 0.6 us): a CTA works through
// ceil(items / SMs) work items of (k-blocks per part + a fixed cost for pipeline fill and epilogue) each,
// and a split run pays for the finishing kernel.  K is cut only when that model gains a tenth or more.
// The two constants are fitted to timings of batch-32 layer shapes with forced splits (52 to 196 tiles of 16 to 144
// k-blocks): 7 periods per work item, 20 for the second launch and its pass over the partial sums.
int choose_splits(long long rows, const TcPacked &L)
{
    const long long tiles = ceil_div<long long>(rows, tc::BM) * (L.n_pad / L.bn);
    const int kb = L.k_pad / tc::BK, sms = sm_count();
    if(tiles <= 0 || tiles > 4 * sms || kb < 8) return 1;
    const double item_fixed = 7.0, finish = 20.0;
    const double uncut = double(ceil_div<long long>(tiles, sms)) * (kb + item_fixed);
    int best = 1;
    double best_cost = 0.9 * uncut;
    for(int s = 2; s <= 32 && kb / s >= 4; s++) {
        if(kb % s != 0) continue;
        const double cost = double(ceil_div<long long>(tiles * s, sms)) * (kb / s + item_fixed) + finish;
        if(cost < best_cost) { best = s; best_cost = cost; }
    }
    return best;
}

template<int BN, int MODE>
dlp_status launch_bn(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream, int splits, long long split_stride,
                     const TcBatch &batch)
{
    // the gather table rides along in shared memory when it is at most 8 KB (1024 entries: K up to 1024)
    // (row-taps mode: one entry per eight k, always in shared memory; the plan keeps it within 1024 entries)
    const int ktab_entries = MODE == A_ROWTAPS ? L.k_pad / ROWTAPS_WIDTH : (MODE == A_GATHER && L.k_pad <= 1024 && p.ktab != nullptr ? L.k_pad : 0);
    if(MODE == A_ROWTAPS && (p.ktab == nullptr || ktab_entries > 1024)) return fail(DLP_INVALID_ARGUMENT, "row-taps table missing or too long");
    const int smem = 1024 + tc::STAGES * 2 * BN * tc::BK * 4 + BN * tc::BM * 4 + int((sizeof(tc::Shared) + 15) & ~size_t(15)) + ktab_entries * 8;
    const int smem_max = 1024 + tc::STAGES * 2 * BN * tc::BK * 4 + BN * tc::BM * 4 + int((sizeof(tc::Shared) + 15) & ~size_t(15)) + 1024 * 8;
    {
        // The attribute belongs to the function in the current device's context: set it once per (instantiation, device).
        static std::mutex mutex;
        static std::vector<char> configured;          // by device ordinal
        int dev = 0;
        DLP_CUDA_OK(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(mutex);
        if(size_t(dev) >= configured.size()) configured.resize(size_t(dev) + 1, 0);
        if(!configured[dev]) {
            DLP_CUDA_OK(cudaFuncSetAttribute(tc::contraction_tf32x3_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max));
            configured[dev] = 1;
        }
    }
    const long long m_tiles = ceil_div<long long>(p.rows, tc::BM);
    const int n_tiles = L.n_pad / BN;
    const long long num_tiles = m_tiles * n_tiles * splits;     // work items
    const dim3 grid(unsigned(std::min<long long>(num_tiles, sm_count())), unsigned(batch.count));
    int diag = 0;
    long long *trace = nullptr;
#ifdef DLP_TC_DIAGNOSTICS
    static const int diag_env = getenv("DLP_TC_DIAG") ? atoi(getenv("DLP_TC_DIAG")) : 0;
    // DLP_TC_TRACE=<file>: dump the timeline of CTA 0 of every launch (synchronises; diagnostic use only)
    static const char *trace_path = getenv("DLP_TC_TRACE");
    static long long *trace_buf = nullptr;
    if(trace_path && !trace_buf) DLP_CUDA_OK(cudaGetSymbolAddress((void **)&trace_buf, tc::g_trace));
    if(trace_buf) DLP_CUDA_OK(cudaMemsetAsync(trace_buf, 0, 64 * 16 * sizeof(long long), stream));
    diag = diag_env;
    trace = trace_buf;
#endif
    int *status = device_status_word();
    if(!status) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    tc::contraction_tf32x3_kernel<BN, MODE><<<grid, tc::NUM_THREADS, smem, stream>>>(packed, p, L.k_pad / tc::BK / splits, n_tiles, num_tiles,
                                                                                     splits, split_stride, ktab_entries, status, diag, trace, batch);
    DLP_LAUNCH_OK("contraction_tf32x3_kernel");
#ifdef DLP_TC_DIAGNOSTICS
    if(trace) {
        static long long host[64 * 16];
        DLP_CUDA_OK(cudaStreamSynchronize(stream));
        DLP_CUDA_OK(cudaMemcpy(host, trace, sizeof(host), cudaMemcpyDeviceToHost));
        if(FILE *f = fopen(trace_path, "w")) {
            for(int i = 0; i < 64; i++) {
                for(int j = 0; j < 16; j++) fprintf(f, "%lld ", host[i * 16 + j] ? host[i * 16 + j] - host[0] : -1);
                fprintf(f, "\n");
            }
            fclose(f);
        }
    }
#endif
    return DLP_OK;
}
} // namespace

size_t tc_split_scratch_bytes(long long rows, const TcPacked &L)
{
    const int s = choose_splits(rows, L);
    return s > 1 ? size_t(s) * size_t(ceil_div<long long>(rows, tc::BM) * tc::BM) * L.n_pad * sizeof(float) : 0;
}

dlp_status launch_contraction_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream, void *scratch,
                                 size_t scratch_bytes, const TcBatch &batch)
{
    if(p.rows <= 0 || p.cols <= 0 || batch.count <= 0) return DLP_OK;
    if(reinterpret_cast<uintptr_t>(packed) % 16 != 0) return fail(DLP_INVALID_ARGUMENT, "packed weights must be 16-byte aligned");
    if(batch.count > 65535) return fail(DLP_INVALID_ARGUMENT, "a batched product takes at most 65535 matrices");
    int splits = batch.count > 1 ? 1 : choose_splits(p.rows, L);      // the matrices of a batch fill the GPU between them
    if(splits == 1 && batch.count == 1 && pointwise_tc_eligible(p, L)) return launch_pointwise_tc(p, L, packed, stream);
    // (environment variable DLP_TC_NO_STAGED: keep such problems on this file's kernel, for A/B timing and profiling)
    static const bool no_staged = getenv("DLP_TC_NO_STAGED") != nullptr;
    if(splits == 1 && batch.count == 1 && !no_staged && staged_tc_eligible(p, L)) return launch_staged_tc(p, L, packed, stream);
    const long long rows_pad = ceil_div<long long>(p.rows, tc::BM) * tc::BM;
    const long long split_stride = rows_pad * L.n_pad;
    if(splits > 1 && (scratch == nullptr || scratch_bytes < size_t(splits) * split_stride * sizeof(float))) splits = 1;
    Contraction q = p;
    if(splits > 1) {
        // the parts write raw partial sums to the scratch; the epilogue runs in the finishing kernel
        q.y = static_cast<float *>(scratch);
        q.out_mode = OUT_COL_MAJOR;
        q.ldc = rows_pad;
        q.bias = nullptr;
        q.bias_mode = DLP_GEMM_NO_BIAS;
        q.act = DLP_ACT_IDENTITY;
        q.post_act = DLP_ACT_IDENTITY;
        q.beta = 0.0f;
        q.residual = nullptr;
    }
    dlp_status st = DLP_INVALID_ARGUMENT;
    switch(L.bn * 4 + p.a_mode) {
    case 32 * 4 + A_GATHER: st = launch_bn<32, A_GATHER>(q, L, packed, stream, splits, split_stride, batch); break;
    case 32 * 4 + A_STRIDED: st = launch_bn<32, A_STRIDED>(q, L, packed, stream, splits, split_stride, batch); break;
    case 32 * 4 + A_TAPBLOCK: st = launch_bn<32, A_TAPBLOCK>(q, L, packed, stream, splits, split_stride, batch); break;
    case 64 * 4 + A_GATHER: st = launch_bn<64, A_GATHER>(q, L, packed, stream, splits, split_stride, batch); break;
    case 64 * 4 + A_STRIDED: st = launch_bn<64, A_STRIDED>(q, L, packed, stream, splits, split_stride, batch); break;
    case 64 * 4 + A_TAPBLOCK: st = launch_bn<64, A_TAPBLOCK>(q, L, packed, stream, splits, split_stride, batch); break;
    case 128 * 4 + A_GATHER: st = launch_bn<128, A_GATHER>(q, L, packed, stream, splits, split_stride, batch); break;
    case 128 * 4 + A_STRIDED: st = launch_bn<128, A_STRIDED>(q, L, packed, stream, splits, split_stride, batch); break;
    case 128 * 4 + A_TAPBLOCK: st = launch_bn<128, A_TAPBLOCK>(q, L, packed, stream, splits, split_stride, batch); break;
    case 32 * 4 + A_ROWTAPS: st = launch_bn<32, A_ROWTAPS>(q, L, packed, stream, splits, split_stride, batch); break;
    case 64 * 4 + A_ROWTAPS: st = launch_bn<64, A_ROWTAPS>(q, L, packed, stream, splits, split_stride, batch); break;
    case 128 * 4 + A_ROWTAPS: st = launch_bn<128, A_ROWTAPS>(q, L, packed, stream, splits, split_stride, batch); break;
    default: return fail(DLP_INVALID_ARGUMENT, "unsupported column tile");
    }
    if(st != DLP_OK || splits == 1) return st;
    const long long total = p.rows * p.cols;
    const int blocks = int(std::min<long long>(ceil_div<long long>(total, 256), 16 * sm_count()));
    tc::split_finish_kernel<<<blocks, 256, 0, stream>>>(p, static_cast<const float *>(scratch), splits, split_stride, rows_pad);
    DLP_LAUNCH_OK("split_finish_kernel");
    return DLP_OK;
}

} // namespace dlp
