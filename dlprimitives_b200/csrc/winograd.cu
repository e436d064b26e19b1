// Winograd F(2x2, 3x3) convolution in fp32 on the CUDA cores.
//
// The reference's third convolution algorithm (src/core/conv.cpp:223-297, kernels in
// src/kernels/winograd_fwd.cl): stride 1, padding 1, no dilation, one group.  Two steps, as there:
//   1. filter transform   U = G g G^T        (16 values per (cout, cin); here laid out [xi][cin][cout_pad])
//   2. one fused kernel:  V = B^T d B  per 4x4 input patch,  M[xi] = sum_c V[xi][c] * U[xi][c]  as 16 small
//      GEMMs held in registers,  Y = A^T M A  (2x2 outputs),  + bias, activation, residual, factor.
// with  G = [1 0 0; .5 .5 .5; .5 -.5 .5; 0 0 1],  B^T = [1 0 -1 0; 0 1 1 0; 0 -1 1 0; 0 1 0 -1],
//       A^T = [1 1 1 0; 0 1 -1 -1].
// A CTA owns 32 output tiles (2x2 pixels each, consecutive in (image, tile row, tile column) order) times
// 32 filters and walks the input channels eight at a time.  The arithmetic is plain fp32 FMA, so the
// results differ from the direct sum only by the rounding of the transforms (1e-6 relative).
//
// With the 3xTF32 tensor-core kernel at hand this path is not the fast one on B200 (fp32 FMA peak is a
// third of the 3xTF32 tensor-core rate even after the 2.25x saving in multiplies); it exists so that a
// caller who asks for "winograd" gets that algorithm.
#include "contraction.cuh"

namespace dlp {
namespace {

constexpr int WT = 32;        // output tiles per CTA
constexpr int WF = 32;        // filters per CTA
constexpr int WC = 8;         // input channels per step
constexpr int WTHREADS = 256;

// U[xi][c][o] = (G g G^T)[xi] for filter (o, c); o padded to cout_pad with zeros
__global__ void winograd_filter_transform_kernel(const float *__restrict__ w, float *__restrict__ u, int cin, int cout, int cout_pad)
{
    const long long total = (long long)cin * cout_pad;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int c = int(idx / cout_pad), o = int(idx - (long long)c * cout_pad);
        float g[3][3];
        #pragma unroll
        for(int i = 0; i < 3; i++)
            #pragma unroll
            for(int j = 0; j < 3; j++) g[i][j] = o < cout ? __ldg(w + ((long long)o * cin + c) * 9 + i * 3 + j) : 0.0f;
        float t[4][3];     // G g
        #pragma unroll
        for(int j = 0; j < 3; j++) {
            t[0][j] = g[0][j];
            t[1][j] = 0.5f * (g[0][j] + g[1][j] + g[2][j]);
            t[2][j] = 0.5f * (g[0][j] - g[1][j] + g[2][j]);
            t[3][j] = g[2][j];
        }
        #pragma unroll
        for(int i = 0; i < 4; i++) {
            const float r0 = t[i][0], r1 = 0.5f * (t[i][0] + t[i][1] + t[i][2]), r2 = 0.5f * (t[i][0] - t[i][1] + t[i][2]), r3 = t[i][2];
            u[((long long)(i * 4 + 0) * cin + c) * cout_pad + o] = r0;
            u[((long long)(i * 4 + 1) * cin + c) * cout_pad + o] = r1;
            u[((long long)(i * 4 + 2) * cin + c) * cout_pad + o] = r2;
            u[((long long)(i * 4 + 3) * cin + c) * cout_pad + o] = r3;
        }
    }
}

struct WinogradArgs {
    const float *x, *u, *bias, *residual;
    float *y;
    int batch, cin, cout, cout_pad, h, w;
    int tiles_h, tiles_w;
    long long tiles;          // batch * tiles_h * tiles_w
    int act, post_act;
    float factor, residual_scale;
};

__global__ void __launch_bounds__(WTHREADS)
winograd_f23_kernel(const WinogradArgs a)
{
    __shared__ float Vs[16][WC][WT];
    __shared__ float Us[16][WC][WF];

    const int tid = threadIdx.x;
    const long long tile0 = (long long)blockIdx.x * WT;
    const int f0 = blockIdx.y * WF;

    // loader role: thread = (channel in step, tile in CTA)
    const int lt = tid % WT, lc = tid / WT;
    const long long ltile = tile0 + lt;
    const bool ltile_ok = ltile < a.tiles;
    int lb = 0, ly0 = 0, lx0 = 0;
    if(ltile_ok) {
        const int per_image = a.tiles_h * a.tiles_w;
        lb = int(ltile / per_image);
        const int r = int(ltile - (long long)lb * per_image);
        ly0 = (r / a.tiles_w) * 2 - 1;
        lx0 = (r % a.tiles_w) * 2 - 1;
    }
    // compute role: thread = (pair of tiles, pair of filters)
    const int ct = (tid % 16) * 2, cf = (tid / 16) * 2;

    float acc[16][2][2];
    #pragma unroll
    for(int i = 0; i < 16; i++) acc[i][0][0] = acc[i][0][1] = acc[i][1][0] = acc[i][1][1] = 0.0f;

    for(int c0 = 0; c0 < a.cin; c0 += WC) {
        // input patch -> B^T d B
        {
            const int c = c0 + lc;
            float d[4][4];
            const float *src = a.x + ((long long)lb * a.cin + c) * a.h * a.w;
            #pragma unroll
            for(int i = 0; i < 4; i++)
                #pragma unroll
                for(int j = 0; j < 4; j++) {
                    const int yy = ly0 + i, xx = lx0 + j;
                    const bool ok = ltile_ok && c < a.cin && unsigned(yy) < unsigned(a.h) && unsigned(xx) < unsigned(a.w);
                    d[i][j] = ok ? __ldg(src + (long long)yy * a.w + xx) : 0.0f;
                }
            float t[4][4];   // B^T d
            #pragma unroll
            for(int j = 0; j < 4; j++) {
                t[0][j] = d[0][j] - d[2][j];
                t[1][j] = d[1][j] + d[2][j];
                t[2][j] = d[2][j] - d[1][j];
                t[3][j] = d[1][j] - d[3][j];
            }
            #pragma unroll
            for(int i = 0; i < 4; i++) {
                Vs[i * 4 + 0][lc][lt] = t[i][0] - t[i][2];
                Vs[i * 4 + 1][lc][lt] = t[i][1] + t[i][2];
                Vs[i * 4 + 2][lc][lt] = t[i][2] - t[i][1];
                Vs[i * 4 + 3][lc][lt] = t[i][1] - t[i][3];
            }
        }
        // transformed filters of this channel step: 16 x 8 x 32 values, 16 per thread, coalesced over filters
        #pragma unroll
        for(int i = 0; i < 16 * WC * WF / WTHREADS; i++) {
            const int e = i * WTHREADS + tid;
            const int f = e % WF, c = (e / WF) % WC, xi = e / (WF * WC);
            const bool ok = c0 + c < a.cin;     // cout_pad covers f0 + f
            Us[xi][c][f] = ok ? __ldg(a.u + ((long long)xi * a.cin + c0 + c) * a.cout_pad + f0 + f) : 0.0f;
        }
        __syncthreads();
        #pragma unroll
        for(int xi = 0; xi < 16; xi++)
            #pragma unroll
            for(int c = 0; c < WC; c++) {
                const float2 v = *reinterpret_cast<const float2 *>(&Vs[xi][c][ct]);
                const float2 u = *reinterpret_cast<const float2 *>(&Us[xi][c][cf]);
                acc[xi][0][0] = fmaf(v.x, u.x, acc[xi][0][0]);
                acc[xi][0][1] = fmaf(v.x, u.y, acc[xi][0][1]);
                acc[xi][1][0] = fmaf(v.y, u.x, acc[xi][1][0]);
                acc[xi][1][1] = fmaf(v.y, u.y, acc[xi][1][1]);
            }
        __syncthreads();
    }

    // A^T M A, bias, activation, residual, factor; 2x2 outputs per (tile, filter)
    const int per_image = a.tiles_h * a.tiles_w;
    #pragma unroll
    for(int ti = 0; ti < 2; ti++) {
        const long long tile = tile0 + ct + ti;
        if(tile >= a.tiles) continue;
        const int b = int(tile / per_image);
        const int r = int(tile - (long long)b * per_image);
        const int oy = (r / a.tiles_w) * 2, ox = (r % a.tiles_w) * 2;
        #pragma unroll
        for(int fi = 0; fi < 2; fi++) {
            const int f = f0 + cf + fi;
            if(f >= a.cout) continue;
            float m[4][4];
            #pragma unroll
            for(int i = 0; i < 16; i++) m[i / 4][i % 4] = acc[i][ti][fi];
            float s[2][4];   // A^T M
            #pragma unroll
            for(int j = 0; j < 4; j++) {
                s[0][j] = m[0][j] + m[1][j] + m[2][j];
                s[1][j] = m[1][j] - m[2][j] - m[3][j];
            }
            const float bias = a.bias ? __ldg(a.bias + f) : 0.0f;
            #pragma unroll
            for(int i = 0; i < 2; i++) {
                const float o0 = s[i][0] + s[i][1] + s[i][2], o1 = s[i][1] - s[i][2] - s[i][3];
                #pragma unroll
                for(int j = 0; j < 2; j++) {
                    const int yy = oy + i, xx = ox + j;
                    if(yy >= a.h || xx >= a.w) continue;
                    const long long idx = (((long long)b * a.cout + f) * a.h + yy) * a.w + xx;
                    float v = apply_act((j ? o1 : o0) + bias, a.act);
                    if(a.residual) v = apply_act(v + a.residual_scale * __ldg(a.residual + idx), a.post_act);
                    if(a.factor != 0.0f) v += a.factor * a.y[idx];
                    a.y[idx] = v;
                }
            }
        }
    }
}

} // namespace

size_t winograd_packed_bytes(int cin, int cout)
{
    return size_t(16) * cin * round_up(cout, WF) * sizeof(float);
}

dlp_status winograd_filter_transform(const float *w, float *u, int cin, int cout, cudaStream_t stream)
{
    const int cout_pad = round_up(cout, WF);
    const long long total = (long long)cin * cout_pad;
    const int blocks = int(std::min<long long>(ceil_div<long long>(total, 256), 8 * sm_count()));
    winograd_filter_transform_kernel<<<blocks, 256, 0, stream>>>(w, u, cin, cout, cout_pad);
    DLP_LAUNCH_OK("winograd_filter_transform_kernel");
    return DLP_OK;
}

dlp_status launch_winograd_f23(const float *x, const float *u, const float *bias, float *y, int batch, int cin, int cout, int h, int w,
                               int act, float factor, const float *residual, float residual_scale, int post_act, cudaStream_t stream)
{
    WinogradArgs a;
    a.x = x; a.u = u; a.bias = bias; a.residual = residual; a.y = y;
    a.batch = batch; a.cin = cin; a.cout = cout; a.cout_pad = round_up(cout, WF); a.h = h; a.w = w;
    a.tiles_h = (h + 1) / 2; a.tiles_w = (w + 1) / 2;
    a.tiles = (long long)batch * a.tiles_h * a.tiles_w;
    a.act = act; a.post_act = post_act; a.factor = factor; a.residual_scale = residual_scale;
    if(a.tiles <= 0 || cout <= 0) return DLP_OK;
    const long long gx = ceil_div<long long>(a.tiles, WT);
    if(gx > 0x7fffffffLL) return fail(DLP_INVALID_ARGUMENT, "too many output tiles for one launch");
    dim3 grid((unsigned)gx, (unsigned)(a.cout_pad / WF));
    winograd_f23_kernel<<<grid, WTHREADS, 0, stream>>>(a);
    DLP_LAUNCH_OK("winograd_f23_kernel");
    return DLP_OK;
}

} // namespace dlp
