// Winograd F(2x2, 3x3) convolution with the 16 products on the tensor cores.
//
// The reference's third convolution algorithm (src/core/conv.cpp:223-297, src/kernels/winograd_fwd.cl: 3x3, stride 1,
// padding 1, no dilation, one group) as three launches:
//   1. input transform    V[xi][c][t] = (B^T d B)[xi]   for every 4x4 input patch d of tile t and channel c   (one pass over x)
//   2. sixteen products   M[xi][o][t] = sum_c V[xi][c][t] * U[xi][o][c]   -- ONE launch of the batched 3xTF32 tensor-core
//                         contraction (blockIdx.y = xi; A = V[xi] read as a [tiles x Cin] matrix with the tiles contiguous,
//                         B = U[xi] packed once like any weight matrix, C = M[xi] written column-major so that the tiles
//                         stay contiguous)
//   3. output transform   Y = A^T M A (2x2 outputs per tile) + bias, activation, residual, factor   (one pass over y)
// with  G = [1 0 0; .5 .5 .5; .5 -.5 .5; 0 0 1],  B^T = [1 0 -1 0; 0 1 1 0; 0 -1 1 0; 0 1 0 -1],  A^T = [1 1 1 0; 0 1 -1 -1],
// U = G g G^T computed once when the filters are packed.
// Tiles t run (image, tile row, tile column); a row of V / M is padded to a multiple of 4 tiles.
// The transforms are exact in fp32 up to rounding; the products carry the 3xTF32 error (about 1e-6 relative).
// V and M (16 * tiles * (Cin + Cout) floats) live in the caller's workspace.  They cost 4x the input plus 4x the output
// in HBM traffic each way, which is why the implicit GEMM, not this, is what "auto" picks on this GPU.
#include "contraction.cuh"
#include <algorithm>
#include <cstring>

namespace dlp {
namespace {

// Uraw[xi][o][c] = (G g G^T)[xi] for filter (o, c)
__global__ void wtc_filter_kernel(const float *__restrict__ w, float *__restrict__ u, int cin, int cout)
{
    const long long total = (long long)cin * cout;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        float g[3][3];
        #pragma unroll
        for(int i = 0; i < 9; i++) g[i / 3][i % 3] = __ldg(w + idx * 9 + i);          // idx = o * cin + c
        float t[4][3];
        #pragma unroll
        for(int j = 0; j < 3; j++) {
            t[0][j] = g[0][j];
            t[1][j] = 0.5f * (g[0][j] + g[1][j] + g[2][j]);
            t[2][j] = 0.5f * (g[0][j] - g[1][j] + g[2][j]);
            t[3][j] = g[2][j];
        }
        #pragma unroll
        for(int i = 0; i < 4; i++) {
            const float r[4] = { t[i][0], 0.5f * (t[i][0] + t[i][1] + t[i][2]), 0.5f * (t[i][0] - t[i][1] + t[i][2]), t[i][2] };
            #pragma unroll
            for(int j = 0; j < 4; j++) u[(long long)(i * 4 + j) * total + idx] = r[j];
        }
    }
}

struct Geometry {
    int batch, cin, cout, h, w, tiles_h, tiles_w;
    long long tiles, tiles_pad;
};

// one thread per (channel plane, tile): reads the 4x4 patch, writes the 16 transformed values (tiles contiguous across lanes)
__global__ void wtc_input_kernel(const float *__restrict__ x, float *__restrict__ v, Geometry q)
{
    const long long per_image = (long long)q.tiles_h * q.tiles_w;
    const long long total = q.tiles * q.cin;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int c = int(idx / q.tiles);
        const long long t = idx - (long long)c * q.tiles;
        const int b = int(t / per_image), r = int(t - b * per_image);
        const int ty = r / q.tiles_w, tx = r - ty * q.tiles_w;
        const float *src = x + ((long long)b * q.cin + c) * q.h * q.w;
        float d[4][4];
        #pragma unroll
        for(int i = 0; i < 4; i++) {
            const int iy = 2 * ty - 1 + i;
            #pragma unroll
            for(int j = 0; j < 4; j++) {
                const int ix = 2 * tx - 1 + j;
                d[i][j] = (unsigned(iy) < unsigned(q.h) && unsigned(ix) < unsigned(q.w)) ? __ldg(src + (long long)iy * q.w + ix) : 0.0f;
            }
        }
        float m[4][4];     // B^T d
        #pragma unroll
        for(int j = 0; j < 4; j++) {
            m[0][j] = d[0][j] - d[2][j];
            m[1][j] = d[1][j] + d[2][j];
            m[2][j] = d[2][j] - d[1][j];
            m[3][j] = d[1][j] - d[3][j];
        }
        float *dst = v + (long long)c * q.tiles_pad + t;
        const long long xi_stride = (long long)q.cin * q.tiles_pad;
        #pragma unroll
        for(int i = 0; i < 4; i++) {
            dst[(i * 4 + 0) * xi_stride] = m[i][0] - m[i][2];
            dst[(i * 4 + 1) * xi_stride] = m[i][1] + m[i][2];
            dst[(i * 4 + 2) * xi_stride] = m[i][2] - m[i][1];
            dst[(i * 4 + 3) * xi_stride] = m[i][1] - m[i][3];
        }
    }
}

struct OutArgs {
    const float *bias, *residual;
    float *y;
    int act, post_act;
    float factor, residual_scale;
};

// one thread per (output channel plane, tile): reads the 16 products, writes the 2x2 outputs
__global__ void wtc_output_kernel(const float *__restrict__ mm, Geometry q, OutArgs a)
{
    const long long per_image = (long long)q.tiles_h * q.tiles_w;
    const long long total = q.tiles * q.cout;
    for(long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int o = int(idx / q.tiles);
        const long long t = idx - (long long)o * q.tiles;
        const int b = int(t / per_image), r = int(t - b * per_image);
        const int ty = r / q.tiles_w, tx = r - ty * q.tiles_w;
        const float *src = mm + (long long)o * q.tiles_pad + t;
        const long long xi_stride = (long long)q.cout * q.tiles_pad;
        float m[4][4];
        #pragma unroll
        for(int i = 0; i < 16; i++) m[i / 4][i % 4] = __ldg(src + i * xi_stride);
        float s[2][4];     // A^T M
        #pragma unroll
        for(int j = 0; j < 4; j++) {
            s[0][j] = m[0][j] + m[1][j] + m[2][j];
            s[1][j] = m[1][j] - m[2][j] - m[3][j];
        }
        const float bias = a.bias ? __ldg(a.bias + o) : 0.0f;
        #pragma unroll
        for(int i = 0; i < 2; i++) {
            const int oy = 2 * ty + i;
            if(oy >= q.h) continue;
            const float out[2] = { s[i][0] + s[i][1] + s[i][2], s[i][1] - s[i][2] - s[i][3] };
            #pragma unroll
            for(int j = 0; j < 2; j++) {
                const int ox = 2 * tx + j;
                if(ox >= q.w) continue;
                const long long yi = (((long long)b * q.cout + o) * q.h + oy) * q.w + ox;
                float val = apply_act(out[j] + bias, a.act);
                if(a.residual) val = apply_act(val + a.residual_scale * __ldg(a.residual + yi), a.post_act);
                if(a.factor != 0.0f) val += a.factor * a.y[yi];
                a.y[yi] = val;
            }
        }
    }
}

Geometry geometry(int batch, int cin, int cout, int h, int w)
{
    Geometry q;
    q.batch = batch; q.cin = cin; q.cout = cout; q.h = h; q.w = w;
    q.tiles_h = (h + 1) / 2; q.tiles_w = (w + 1) / 2;
    q.tiles = (long long)batch * q.tiles_h * q.tiles_w;
    q.tiles_pad = round_up<long long>(q.tiles, 4);
    return q;
}

} // namespace

// packed filters: the sixteen packed U[xi] one after the other, then the unpacked U (the pack kernel's input)
size_t winograd_tc_packed_bytes(int cin, int cout)
{
    return 16 * tc_packed_layout(cout, cin).bytes() + size_t(16) * cin * cout * sizeof(float);
}

size_t winograd_tc_workspace_bytes(int batch, int cin, int cout, int h, int w)
{
    const Geometry q = geometry(batch, cin, cout, h, w);
    return size_t(16) * size_t(q.tiles_pad) * size_t(cin + cout) * sizeof(float);
}

dlp_status winograd_tc_filter_transform(const float *w, float *packed, int cin, int cout, cudaStream_t stream)
{
    const TcPacked L = tc_packed_layout(cout, cin);
    float *raw = packed + 16 * (L.bytes() / sizeof(float));
    const long long total = (long long)cin * cout;
    const int blocks = int(std::min<long long>(ceil_div<long long>(total, 256), 8 * sm_count()));
    wtc_filter_kernel<<<blocks, 256, 0, stream>>>(w, raw, cin, cout);
    DLP_LAUNCH_OK("wtc_filter_kernel");
    return tc_prepack(L, raw, cin, 1, cout, cin, packed, 0, stream, 16, total);
}

dlp_status launch_winograd_tc(const float *x, const float *packed, const float *bias, float *y, void *ws, size_t ws_bytes, int batch, int cin,
                              int cout, int h, int w, int act, float factor, const float *residual, float residual_scale, int post_act,
                              cudaStream_t stream)
{
    const Geometry q = geometry(batch, cin, cout, h, w);
    if(q.tiles <= 0 || cout <= 0) return DLP_OK;
    if(q.tiles >= (1ll << 31)) return fail(DLP_INVALID_ARGUMENT, "too many output tiles for one launch");
    if(ws == nullptr || ws_bytes < winograd_tc_workspace_bytes(batch, cin, cout, h, w))
        return fail(DLP_INVALID_ARGUMENT, "workspace smaller than the transformed input and the products need (dlp_conv2d_fwd_workspace() for this batch)");
    float *v = static_cast<float *>(ws);
    float *mm = v + 16ll * q.tiles_pad * cin;
    const int blocks = int(std::min<long long>(ceil_div<long long>(q.tiles * std::max(cin, cout), 256), 32ll * sm_count()));
    wtc_input_kernel<<<blocks, 256, 0, stream>>>(x, v, q);
    DLP_LAUNCH_OK("wtc_input_kernel");

    Contraction p;
    memset(&p, 0, sizeof(p));
    p.rows = q.tiles; p.cols = cout; p.k = cin;
    p.a = v;
    p.a_mode = A_STRIDED;
    p.a_row_stride = 1;
    p.a_k_stride = q.tiles_pad;
    p.y = mm;
    p.out_mode = OUT_COL_MAJOR;
    p.ldc = q.tiles_pad;
    p.bias_mode = DLP_GEMM_NO_BIAS;
    p.act = DLP_ACT_IDENTITY;
    p.post_act = DLP_ACT_IDENTITY;
    TcBatch bt;
    bt.count = 16;
    bt.a_stride = (long long)cin * q.tiles_pad;
    bt.y_stride = (long long)cout * q.tiles_pad;
    dlp_status st = launch_contraction_tc(p, tc_packed_layout(cout, cin), packed, stream, nullptr, 0, bt);
    if(st != DLP_OK) return st;

    OutArgs a;
    a.bias = bias; a.residual = residual; a.y = y; a.act = act; a.post_act = post_act; a.factor = factor; a.residual_scale = residual_scale;
    wtc_output_kernel<<<blocks, 256, 0, stream>>>(mm, q, a);
    DLP_LAUNCH_OK("wtc_output_kernel");
    return DLP_OK;
}

} // namespace dlp
