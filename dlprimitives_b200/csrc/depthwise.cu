// Depthwise convolution forward (groups == channels, one filter per channel), stride 1 or 2.
//
// HBM-bound: about 2 flops per byte.  The job is to touch every input and output element once
// with wide coalesced accesses.  In NCHW the planes of consecutive channels are contiguous, and so
// is a band of full-width rows inside a plane, so a CTA's input is one contiguous run of floats: it
// is copied to shared memory with 16-byte loads (whatever W is), the k x k taps are read from there,
// and the outputs (again one contiguous run) are written with coalesced stores.
//   small planes (7x7, 14x14 ...): several whole planes per CTA
//   large planes (56x56, 112x112): one band of output rows of one plane per CTA
// Bias, activation and y = factor*y_old + ... are fused.  The reference's counterpart is
// src/kernels/depthwise_separable_conv.cl (stride 1 only; stride 2 goes to its grouped GEMM).
#include "depthwise.cuh"

namespace dlp {
namespace {

constexpr int THREADS = 256;
constexpr int SMEM_FLOATS = 10240;   // 40 KB staging buffer

struct DwParams {
    const float *x, *w, *bias;
    float *y;
    int channels, H, W, OH, OW;
    int stride, pad, ks;
    int planes;            // batch * channels
    int planes_per_cta;    // > 1 only when a band is the whole plane
    int rows_per_band;     // output rows per CTA
    int bands;             // bands per plane
    int act;
    float factor;
};

// KS, ST: kernel size and stride known at compile time (0, 0: run-time values, any size up to 7).
template<int KS, int ST>
__global__ void __launch_bounds__(THREADS) depthwise_kernel(DwParams p)
{
    __shared__ __align__(16) float tile[SMEM_FLOATS];
    const int ks = KS > 0 ? KS : p.ks;
    const long long plane0 = (long long)(blockIdx.x / p.bands) * p.planes_per_cta;
    const int band = blockIdx.x % p.bands;
    const int np = int(min((long long)p.planes_per_cta, p.planes - plane0));
    const int oy0 = band * p.rows_per_band;
    const int oy1 = min(oy0 + p.rows_per_band, p.OH);
    // input rows this band needs, clipped to the image
    const int iy_lo = max(oy0 * p.stride - p.pad, 0);
    const int iy_hi = min((oy1 - 1) * p.stride - p.pad + ks, p.H);
    const int in_rows = iy_hi - iy_lo;
    const long long plane_elems = (long long)p.H * p.W;
    // contiguous run: np whole planes (bands == 1) or in_rows rows of one plane
    const long long g_begin = plane0 * plane_elems + (long long)iy_lo * p.W;
    const long long g_end = np > 1 ? (plane0 + np) * plane_elems : g_begin + (long long)in_rows * p.W;
    const long long total_in = (long long)p.planes * plane_elems;
    const long long a_begin = g_begin & ~3ll;                   // 16-byte aligned start (x is 16-byte aligned)
    const int shift = int(g_begin - a_begin);
    const int count = int(g_end - a_begin);

    // copy in: four 16-byte loads in flight per thread before their stores, then the ragged rest
    {
        constexpr int U = 4;
        const int safe = int(min((long long)count, total_in - a_begin)) & ~3;      // whole float4s inside the tensor
        int i = threadIdx.x * 4;
        for(; i + (U - 1) * THREADS * 4 < safe; i += U * THREADS * 4) {
            float4 v[U];
            #pragma unroll
            for(int u = 0; u < U; u++) v[u] = __ldg(reinterpret_cast<const float4 *>(p.x + a_begin + i + u * THREADS * 4));
            #pragma unroll
            for(int u = 0; u < U; u++) *reinterpret_cast<float4 *>(tile + i + u * THREADS * 4) = v[u];
        }
        for(; i < count; i += THREADS * 4) {
            const long long gi = a_begin + i;
            if(i + 4 <= safe) *reinterpret_cast<float4 *>(tile + i) = __ldg(reinterpret_cast<const float4 *>(p.x + gi));
            else
                for(int j = 0; j < 4 && gi + j < total_in; j++) tile[i + j] = __ldg(p.x + gi + j);
        }
    }
    __syncthreads();

    const int out_rows = oy1 - oy0;
    if(KS > 0) {
        // A thread takes a patch of CW adjacent output columns by up to R consecutive output rows: the index
        // arithmetic and the filter (kept in registers) are paid once per patch, each input value is read
        // from shared memory once and feeds every output of the patch it belongs to.  Per output the
        // products are added in the same order (ky, then kx) as in the general loop below.
        constexpr int R = 4, CW = 2;
        constexpr int IN_ROWS = (R - 1) * (ST > 0 ? ST : 1) + (KS > 0 ? KS : 1);
        constexpr int IN_COLS = (CW - 1) * (ST > 0 ? ST : 1) + (KS > 0 ? KS : 1);
        const int segs = (out_rows + R - 1) / R, colp = (p.OW + CW - 1) / CW;
        const int items = np * segs * colp;
        for(int it = threadIdx.x; it < items; it += THREADS) {
            const int oxp = it % colp, t2 = it / colp;
            const int seg = t2 % segs, pl = t2 / segs;
            const long long plane = plane0 + pl;
            const int c = int(plane % p.channels);
            float wreg[(KS > 0 ? KS : 1) * (KS > 0 ? KS : 1)];
            #pragma unroll
            for(int i = 0; i < KS * KS; i++) wreg[i] = __ldg(p.w + (long long)c * (KS * KS) + i);
            const int ox0 = oxp * CW, nc = min(CW, p.OW - ox0);
            const int oyb = oy0 + seg * R, nr = min(R, oy1 - oyb);
            const int iyb = oyb * ST - p.pad, ix0 = ox0 * ST - p.pad;
            const float *src = tile + shift + (long long)pl * plane_elems - (long long)iy_lo * p.W;
            unsigned col_ok = 0;      // bit i: input column ix0 + i is inside the image
            #pragma unroll
            for(int i = 0; i < IN_COLS; i++)
                if(unsigned(ix0 + i) < unsigned(p.W)) col_ok |= 1u << i;
            float acc[R][CW];
            #pragma unroll
            for(int j = 0; j < R; j++)
                #pragma unroll
                for(int cc = 0; cc < CW; cc++) acc[j][cc] = 0.0f;
            #pragma unroll
            for(int rr = 0; rr < IN_ROWS; rr++) {
                const int iy = iyb + rr;
                if(rr >= (nr - 1) * ST + KS || unsigned(iy) >= unsigned(p.H)) continue;
                float v[IN_COLS];
                #pragma unroll
                for(int i = 0; i < IN_COLS; i++) v[i] = (col_ok >> i) & 1u ? src[iy * p.W + ix0 + i] : 0.0f;
                #pragma unroll
                for(int j = 0; j < R; j++) {
                    const int ky = rr - j * ST;        // compile-time after unrolling
                    if(ky < 0 || ky >= KS) continue;
                    #pragma unroll
                    for(int cc = 0; cc < CW; cc++)
                        #pragma unroll
                        for(int kx = 0; kx < KS; kx++)
                            if((col_ok >> (cc * ST + kx)) & 1u) acc[j][cc] = fmaf(v[cc * ST + kx], wreg[ky * KS + kx], acc[j][cc]);
                }
            }
            const float b = p.bias ? __ldg(p.bias + c) : 0.0f;
            #pragma unroll
            for(int j = 0; j < R; j++) {
                if(j >= nr) break;
                #pragma unroll
                for(int cc = 0; cc < CW; cc++) {
                    if(cc >= nc) break;
                    float a = acc[j][cc];
                    if(p.bias) a += b;
                    a = apply_act(a, p.act);
                    const long long yi = plane * ((long long)p.OH * p.OW) + (long long)(oyb + j) * p.OW + ox0 + cc;
                    if(p.factor != 0.0f) a += p.factor * p.y[yi];
                    p.y[yi] = a;
                }
            }
        }
        return;
    }
    const int outs_per_plane = out_rows * p.OW;
    const int total_out = np * outs_per_plane;
    for(int o = threadIdx.x; o < total_out; o += THREADS) {
        const int pl = o / outs_per_plane;
        const int rem = o - pl * outs_per_plane;
        const int oy = oy0 + rem / p.OW;
        const int ox = rem % p.OW;
        const long long plane = plane0 + pl;
        const int c = int(plane % p.channels);
        const float *wk = p.w + (long long)c * ks * ks;
        // tile[t] holds global element a_begin + t; element (iy, ix) of this plane sits at src[iy*W + ix]
        const float *src = tile + shift + (long long)pl * plane_elems - (long long)iy_lo * p.W;
        const int iy0 = oy * p.stride - p.pad, ix0 = ox * p.stride - p.pad;
        float acc = 0.0f;
        for(int ky = 0; ky < ks; ky++) {
            const int iy = iy0 + ky;
            if(unsigned(iy) >= unsigned(p.H)) continue;
            for(int kx = 0; kx < ks; kx++) {
                const int ix = ix0 + kx;
                if(unsigned(ix) >= unsigned(p.W)) continue;
                acc = fmaf(src[iy * p.W + ix], __ldg(wk + ky * ks + kx), acc);
            }
        }
        if(p.bias) acc += __ldg(p.bias + c);
        acc = apply_act(acc, p.act);
        const long long yi = plane * ((long long)p.OH * p.OW) + (long long)oy * p.OW + ox;
        if(p.factor != 0.0f) acc += p.factor * p.y[yi];
        p.y[yi] = acc;
    }
}


// 3x3, padding 1, even widths: the register kernel.  No shared memory and no phases: a lane owns V consecutive input
// columns (V = 4 or 2: one 16- or 8-byte load per input row) of one plane over a strip of RS output rows, takes the
// column to its left (and, at stride 1, to its right) from the neighbouring lane by shuffle -- lanes run over (plane,
// column group), and a column group at the edge of a row gets the zero padding instead, so nothing crosses from one plane
// to the next -- and issues all the loads of its strip before the first use.  Per output the products are added in the
// same order (ky, then kx) as in depthwise_kernel; a tap in the padding contributes fmaf(0, w, acc) = acc.
// RS: output rows per strip -- 6 at stride 1, 4 at stride 2, and 7 for stride-2 planes of up to 7 output rows (one strip,
// no input row read twice).
template<int S, int V, int RS>
__global__ void __launch_bounds__(THREADS) depthwise3_reg_kernel(DwParams p, long long groups, int qw, int strips)
{
    constexpr int RI = S * (RS - 1) + 3;      // input rows a strip reads
    constexpr int VO = V / S;                 // outputs per lane and row
    const unsigned full = 0xffffffffu;
    const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if(wid >= ((groups + 31) / 32) * strips) return;
    const int r0 = int(wid % strips) * RS;
    const long long g = (wid / strips) * 32 + lane;
    const bool valid = g < groups;
    const long long pl = valid ? g / qw : 0;
    const int c = valid ? int(g - pl * qw) : 0;
    const int ch = int(pl % p.channels);
    const float *xin = p.x + pl * ((long long)p.H * p.W) + c * V;
    float w[9];
    #pragma unroll
    for(int i = 0; i < 9; i++) w[i] = valid ? __ldg(p.w + ch * 9 + i) : 0.0f;

    float in[RI][V + 2];     // [0]: the column to the left, [1..V]: the lane's own, [V+1]: the column to the right (stride 1)
    bool ok[RI];
    #pragma unroll
    for(int i = 0; i < RI; i++) {
        const int iy = S * r0 - 1 + i;
        ok[i] = valid && iy >= 0 && iy < p.H;
        const float *row = xin + (long long)iy * p.W;
        if(V == 4) {
            const float4 t = ok[i] ? __ldg(reinterpret_cast<const float4 *>(row)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            in[i][1] = t.x; in[i][2] = t.y; in[i][3] = t.z; in[i][4] = t.w;
        }
        else {
            const float2 t = ok[i] ? __ldg(reinterpret_cast<const float2 *>(row)) : make_float2(0.0f, 0.0f);
            in[i][1] = t.x; in[i][2] = t.y;
        }
        // the first and the last lane of the warp have their neighbour in another warp: one more load
        in[i][0] = (ok[i] && lane == 0 && c > 0) ? __ldg(row - 1) : 0.0f;
        in[i][V + 1] = (S == 1 && ok[i] && lane == 31 && c < qw - 1) ? __ldg(row + V) : 0.0f;
    }
    #pragma unroll
    for(int i = 0; i < RI; i++) {
        const float from_left = __shfl_up_sync(full, in[i][V], 1), from_right = __shfl_down_sync(full, in[i][1], 1);
        if(lane > 0) in[i][0] = c > 0 ? from_left : 0.0f;
        if(S == 1 && lane < 31) in[i][V + 1] = c < qw - 1 ? from_right : 0.0f;
    }
    if(!valid) return;
    const float b = p.bias ? __ldg(p.bias + ch) : 0.0f;
    float *yrow = p.y + pl * ((long long)p.OH * p.OW) + c * VO;
    #pragma unroll
    for(int j = 0; j < RS; j++) {
        const int oy = r0 + j;
        if(oy >= p.OH) break;
        float o[VO];
        #pragma unroll
        for(int t = 0; t < VO; t++) {
            float acc = 0.0f;
            #pragma unroll
            for(int ky = 0; ky < 3; ky++)
                #pragma unroll
                for(int kx = 0; kx < 3; kx++) acc = fmaf(in[S * j + ky][S * t + kx], w[ky * 3 + kx], acc);
            if(p.bias) acc += b;
            o[t] = apply_act(acc, p.act);
        }
        float *dst = yrow + (long long)oy * p.OW;
        if(p.factor != 0.0f) {
            #pragma unroll
            for(int t = 0; t < VO; t++) o[t] += p.factor * dst[t];
        }
        if(VO == 4) *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[VO - 1]);
        else if(VO == 2) *reinterpret_cast<float2 *>(dst) = make_float2(o[0], o[VO - 1]);
        else dst[0] = o[0];
    }
}


// 3x3, padding 1, narrow planes (used for W = 7, where a row is 28 bytes, too short for lanes to share): a lane owns a whole
// input ROW.  The rows of all planes form one sequence; a warp takes 32 consecutive rows, of which lanes 1..30 produce output
// and lanes 0 and 31 only supply the row above and below (the warps overlap by two rows).  The columns a lane needs are its
// own registers; the rows above and below come from the neighbouring lanes by shuffle, and a row at the top or bottom of its
// plane takes zeros instead, so nothing crosses planes.  Same order of the nine products per output as depthwise_kernel.
template<int W, int S>
__global__ void __launch_bounds__(THREADS) depthwise3_rows_kernel(DwParams p, long long total_rows)
{
    constexpr int OWC = S == 1 ? W : (W + 1) / 2;          // outputs per row
    const unsigned full = 0xffffffffu;
    const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long R = wid * 30 - 1 + lane;               // this lane's input row in the sequence of all rows
    if(wid * 30 >= total_rows) return;
    const bool have = R >= 0 && R < total_rows;
    const long long plane = have ? R / p.H : 0;
    const int r = have ? int(R - plane * p.H) : 0;
    const int ch = int(plane % p.channels);
    float in[W + 2];                                        // [0] and [W+1]: the padding columns
    in[0] = in[W + 1] = 0.0f;
    const float *src = p.x + R * W;
    if(W % 2 == 0) {
        #pragma unroll
        for(int i = 0; i < W / 2; i++) {
            const float2 t = have ? __ldg(reinterpret_cast<const float2 *>(src) + i) : make_float2(0.0f, 0.0f);
            in[1 + 2 * i] = t.x; in[2 + 2 * i] = t.y;
        }
    }
    else {
        #pragma unroll
        for(int i = 0; i < W; i++) in[1 + i] = have ? __ldg(src + i) : 0.0f;
    }
    float w[9];
    #pragma unroll
    for(int i = 0; i < 9; i++) w[i] = have ? __ldg(p.w + ch * 9 + i) : 0.0f;
    float up[W + 2], down[W + 2];
    up[0] = up[W + 1] = down[0] = down[W + 1] = 0.0f;
    const bool has_up = r > 0, has_down = r < p.H - 1;
    #pragma unroll
    for(int i = 1; i <= W; i++) {
        const float a = __shfl_up_sync(full, in[i], 1), b = __shfl_down_sync(full, in[i], 1);
        up[i] = has_up ? a : 0.0f;
        down[i] = has_down ? b : 0.0f;
    }
    // output rows: every row at stride 1, the even rows at stride 2 (row r = 2 * o is the middle of output row o's window)
    if(!have || lane == 0 || lane == 31 || (S == 2 && (r & 1))) return;
    const int orow = S == 1 ? r : r / 2;
    if(orow >= p.OH) return;
    const float b = p.bias ? __ldg(p.bias + ch) : 0.0f;
    float *dst = p.y + (plane * p.OH + orow) * (long long)p.OW;
    float o[OWC];
    #pragma unroll
    for(int c = 0; c < OWC; c++) {
        float acc = 0.0f;
        #pragma unroll
        for(int kx = 0; kx < 3; kx++) acc = fmaf(up[S * c + kx], w[kx], acc);
        #pragma unroll
        for(int kx = 0; kx < 3; kx++) acc = fmaf(in[S * c + kx], w[3 + kx], acc);
        #pragma unroll
        for(int kx = 0; kx < 3; kx++) acc = fmaf(down[S * c + kx], w[6 + kx], acc);
        if(p.bias) acc += b;
        o[c] = apply_act(acc, p.act);
    }
    if(p.factor != 0.0f) {
        #pragma unroll
        for(int c = 0; c < OWC; c++) o[c] += p.factor * dst[c];
    }
    if(OWC % 2 == 0) {
        #pragma unroll
        for(int c = 0; c < OWC / 2; c++) reinterpret_cast<float2 *>(dst)[c] = make_float2(o[2 * c], o[2 * c + 1]);
    }
    else {
        #pragma unroll
        for(int c = 0; c < OWC; c++) dst[c] = o[c];
    }
}

// 1x1 depthwise (one weight per channel): y = act(w[c] * x + b[c]) [+ factor * y], element by element.  A thread takes four
// consecutive elements (one 16-byte access each way when the plane size is a multiple of 4 and the tensors are aligned),
// U such groups a grid stride apart with their loads issued together; the plane index is a 32-bit division.
__global__ void __launch_bounds__(THREADS) depthwise1_scale_kernel(DwParams p, unsigned total4, unsigned total, int plane, int vec)
{
    constexpr int U = 4;
    const unsigned nthreads = gridDim.x * blockDim.x;
    for(unsigned g0 = blockIdx.x * blockDim.x + threadIdx.x; g0 < total4; g0 += U * nthreads) {
        float v[U][4];
        #pragma unroll
        for(int u = 0; u < U; u++) {
            const unsigned g = g0 + u * nthreads;
            if(g >= total4) continue;
            if(vec) {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(p.x) + g);
                v[u][0] = t.x; v[u][1] = t.y; v[u][2] = t.z; v[u][3] = t.w;
            }
            else
                for(int j = 0; j < 4; j++) v[u][j] = 4 * g + j < total ? __ldg(p.x + 4 * g + j) : 0.0f;
        }
        #pragma unroll
        for(int u = 0; u < U; u++) {
            const unsigned g = g0 + u * nthreads;
            if(g >= total4) continue;
            float o[4];
            // vec: the four elements lie in one plane and share its weight and bias
            unsigned c = ((4 * g) / unsigned(plane)) % unsigned(p.channels);
            float wc = __ldg(p.w + c), bc = p.bias ? __ldg(p.bias + c) : 0.0f;
            #pragma unroll
            for(int j = 0; j < 4; j++) {
                if(!vec && j > 0) {
                    c = ((4 * g + j) / unsigned(plane)) % unsigned(p.channels);
                    wc = __ldg(p.w + c);
                    bc = p.bias ? __ldg(p.bias + c) : 0.0f;
                }
                float a = fmaf(v[u][j], wc, 0.0f);
                if(p.bias) a += bc;
                o[j] = apply_act(a, p.act);
            }
            if(vec) {
                float4 *dst = reinterpret_cast<float4 *>(p.y) + g;
                if(p.factor != 0.0f) {
                    const float4 t = *dst;
                    o[0] += p.factor * t.x; o[1] += p.factor * t.y; o[2] += p.factor * t.z; o[3] += p.factor * t.w;
                }
                *dst = make_float4(o[0], o[1], o[2], o[3]);
            }
            else
                for(int j = 0; j < 4; j++)
                    if(4 * g + j < total) p.y[4 * g + j] = p.factor != 0.0f ? o[j] + p.factor * p.y[4 * g + j] : o[j];
        }
    }
}

} // namespace

bool depthwise_supported(int ks_h, int ks_w, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int in_w)
{
    if(ks_h != ks_w || stride_h != stride_w || pad_h != pad_w || dil_h != 1 || dil_w != 1) return false;
    if(ks_h < 1 || ks_h > 7 || stride_h < 1 || stride_h > 2) return false;
    // one band must fit the staging buffer even at one output row
    return (long long)(ks_h + 1) * in_w + 8 <= SMEM_FLOATS;
}

dlp_status launch_depthwise(const float *x, const float *w, const float *bias, float *y, int batch, int channels, int H, int W,
                            int ks, int stride, int pad, int act, float factor, cudaStream_t stream)
{
    if(reinterpret_cast<uintptr_t>(x) % 16 != 0) return fail(DLP_INVALID_ARGUMENT, "depthwise input must be 16-byte aligned");
    DwParams p;
    p.x = x; p.w = w; p.bias = bias; p.y = y;
    p.channels = channels; p.H = H; p.W = W;
    p.OH = (H + 2 * pad - ks) / stride + 1;
    p.OW = (W + 2 * pad - ks) / stride + 1;
    p.stride = stride; p.pad = pad; p.ks = ks;
    p.planes = batch * channels;
    p.act = act; p.factor = factor;
    if(p.planes <= 0 || p.OH <= 0 || p.OW <= 0) return DLP_OK;
    if(ks == 1 && stride == 1 && pad == 0 && (long long)p.planes * H * W < (1ll << 32) - 4) {
        const unsigned total = unsigned((long long)p.planes * H * W), total4 = (total + 3) / 4;
        const int plane = H * W;
        const int vec = plane % 4 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
        const unsigned blocks = std::max(1u, std::min(ceil_div(total4, unsigned(THREADS * 4)), unsigned(16 * sm_count())));
        depthwise1_scale_kernel<<<blocks, THREADS, 0, stream>>>(p, total4, total, plane, vec);
        DLP_LAUNCH_OK("depthwise1_scale_kernel");
        return DLP_OK;
    }
    // (measured: 1.95 against 1.70 TB/s on the 7x7 rows; on 14x14 planes it is slower than the column kernel below, 1.99 against 2.21)
    if(ks == 3 && pad == 1 && stride == 1 && W == 7 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
        const long long total_rows = (long long)p.planes * H;
        const long long warps = ceil_div<long long>(total_rows, 30);
        const long long blocks = ceil_div<long long>(warps, THREADS / 32);
        if(blocks > 0x7fffffffLL) return fail(DLP_INVALID_ARGUMENT, "depthwise problem too large for one launch");
        depthwise3_rows_kernel<7, 1><<<(unsigned)blocks, THREADS, 0, stream>>>(p, total_rows);
        DLP_LAUNCH_OK("depthwise3_rows_kernel");
        return DLP_OK;
    }
    // (measured on the MobileNetV2 rows: odd widths -- 4-byte loads -- and whole 14-row planes as one strip at stride 1
    // are no faster than the staged kernel or the 6-row strips, so those variants are not kept)
    if(ks == 3 && pad == 1 && W % 2 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
        const int v = W % 4 == 0 ? 4 : 2;
        const int rs = stride == 1 ? 6 : (p.OH <= 7 ? 7 : 4);
        const int qw = W / v;
        const long long groups = (long long)p.planes * qw;
        const int strips = ceil_div(p.OH, rs);
        const long long warps = ceil_div<long long>(groups, 32) * strips;
        const long long blocks = ceil_div<long long>(warps, THREADS / 32);
        if(blocks > 0x7fffffffLL) return fail(DLP_INVALID_ARGUMENT, "depthwise problem too large for one launch");
#define DLP_DW_REG(S, V, RS) depthwise3_reg_kernel<S, V, RS><<<(unsigned)blocks, THREADS, 0, stream>>>(p, groups, qw, strips)
        switch(stride * 1000 + v * 100 + rs) {
        case 1406: DLP_DW_REG(1, 4, 6); break;
        case 1206: DLP_DW_REG(1, 2, 6); break;
        case 2404: DLP_DW_REG(2, 4, 4); break;
        case 2407: DLP_DW_REG(2, 4, 7); break;
        case 2204: DLP_DW_REG(2, 2, 4); break;
        default: DLP_DW_REG(2, 2, 7); break;
        }
#undef DLP_DW_REG
        DLP_LAUNCH_OK("depthwise3_reg_kernel");
        return DLP_OK;
    }
    const long long plane_elems = (long long)H * W;
    const int budget = SMEM_FLOATS - 8;
    if(plane_elems <= budget) {
        p.bands = 1;
        p.rows_per_band = p.OH;
        int ppc = int(budget / plane_elems);
        // several waves of CTAs per SM when the problem allows, so that copy-in and compute phases of different CTAs overlap
        const int want_blocks = 16 * sm_count();
        ppc = std::max(1, std::min(ppc, int(ceil_div<long long>(p.planes, want_blocks))));
        p.planes_per_cta = ppc;
    }
    else {
        p.planes_per_cta = 1;
        int rows = (budget / W - ks) / stride + 1;     // (rows-1)*stride + ks input rows fit
        rows = std::max(1, std::min(rows, p.OH));
        p.rows_per_band = rows;
        p.bands = ceil_div(p.OH, rows);
    }
    const long long blocks = ceil_div<long long>(p.planes, p.planes_per_cta) * p.bands;
    if(blocks > 0x7fffffffLL) return fail(DLP_INVALID_ARGUMENT, "depthwise problem too large for one launch");
    switch(ks * 10 + stride) {
    case 31: depthwise_kernel<3, 1><<<(unsigned)blocks, THREADS, 0, stream>>>(p); break;
    case 32: depthwise_kernel<3, 2><<<(unsigned)blocks, THREADS, 0, stream>>>(p); break;
    case 51: depthwise_kernel<5, 1><<<(unsigned)blocks, THREADS, 0, stream>>>(p); break;
    case 52: depthwise_kernel<5, 2><<<(unsigned)blocks, THREADS, 0, stream>>>(p); break;
    default: depthwise_kernel<0, 0><<<(unsigned)blocks, THREADS, 0, stream>>>(p); break;
    }
    DLP_LAUNCH_OK("depthwise_kernel");
    return DLP_OK;
}

} // namespace dlp
