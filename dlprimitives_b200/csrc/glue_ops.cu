// Bandwidth-bound operators that sit between the convolutions of an inference graph:
// pooling, global pooling, elementwise, activation, softmax, inference batch-norm.
// Semantics follow the reference's CPU operators (cited at each entry point in dlp_cuda.h).
#include "common.cuh"
#include <cfloat>

namespace dlp {
namespace {

__global__ void pooling2d_kernel(const float *__restrict__ x, float *__restrict__ y, long long total, int in_h, int in_w, int out_h,
                                 int out_w, int kh, int kw, int sh, int sw, int ph, int pw, int mode_avg, int include_pad)
{
    for(long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int oc = int(i % out_w);
        const long long t = i / out_w;
        const int orow = int(t % out_h);
        const long long plane = t / out_h;
        const float *src = x + plane * in_h * in_w;
        int row0 = orow * sh - ph, col0 = oc * sw - pw;
        int row1 = row0 + kh, col1 = col0 + kw;
        const int dr_pad = min(row1, in_h + ph) - max(-ph, row0);
        const int dc_pad = min(col1, in_w + pw) - max(-pw, col0);
        row0 = max(row0, 0); col0 = max(col0, 0);
        row1 = min(row1, in_h); col1 = min(col1, in_w);
        float val = mode_avg ? 0.0f : -FLT_MAX;
        for(int r = row0; r < row1; r++)
            for(int c = col0; c < col1; c++) {
                const float v = __ldg(src + r * in_w + c);
                val = mode_avg ? val + v : fmaxf(val, v);
            }
        if(mode_avg) {
            const int dr = row1 - row0, dc = col1 - col0;
            if(dr == kh && dc == kw) val = val * (1.0f / (kh * kw));
            else if(include_pad) val = val / float(dr_pad * dc_pad);
            else val = val * (1.0f / (dr * dc));
        }
        y[i] = val;
    }
}

// Pooling through shared memory: a CTA takes a band of output rows of one plane, reads the input rows
// the band needs once with coalesced (16-byte when aligned) loads, then every thread computes outputs
// from shared memory.  The arithmetic is the same as pooling2d_kernel's, in the same order.
// K, S: kernel size and stride when square and known at compile time (the window loops unroll), 0 = run-time values.
template<int K, int S>
__global__ void pooling2d_band_kernel(const float *__restrict__ x, float *__restrict__ y, long long bands_total, int bands_per_plane,
                                      int band_rows, int in_h, int in_w, int out_h, int out_w, int kh_, int kw_, int sh_, int sw_, int ph,
                                      int pw, int mode_avg, int include_pad, int vec_ok)
{
    const int kh = K ? K : kh_, kw = K ? K : kw_, sh = S ? S : sh_, sw = S ? S : sw_;
    extern __shared__ float tile[];
    for(long long band = blockIdx.x; band < bands_total; band += gridDim.x) {
        const long long plane = band / bands_per_plane;
        const int orow0 = int(band - plane * bands_per_plane) * band_rows;
        const int orows = min(band_rows, out_h - orow0);
        const int irow0 = max(orow0 * sh - ph, 0), irow1 = min((orow0 + orows - 1) * sh - ph + kh, in_h);
        const float *src = x + plane * (long long)in_h * in_w + (long long)irow0 * in_w;
        const int count = (irow1 - irow0) * in_w;
        if(vec_ok) {
            // in_w is a multiple of 4 and x is 16-byte aligned, so every row starts on a 16-byte boundary
            const float4 *src4 = reinterpret_cast<const float4 *>(src);
            float4 *tile4 = reinterpret_cast<float4 *>(tile);
            for(int i = threadIdx.x; i < count / 4; i += blockDim.x) tile4[i] = __ldg(src4 + i);
        }
        else
            for(int i = threadIdx.x; i < count; i += blockDim.x) tile[i] = __ldg(src + i);
        __syncthreads();
        float *dst = y + plane * (long long)out_h * out_w + (long long)orow0 * out_w;
        for(int i = threadIdx.x; i < orows * out_w; i += blockDim.x) {
            const int orel = i / out_w, oc = i - orel * out_w;
            int row0 = (orow0 + orel) * sh - ph, col0 = oc * sw - pw;
            int row1 = row0 + kh, col1 = col0 + kw;
            const int dr_pad = min(row1, in_h + ph) - max(-ph, row0);
            const int dc_pad = min(col1, in_w + pw) - max(-pw, col0);
            row0 = max(row0, 0); col0 = max(col0, 0);
            row1 = min(row1, in_h); col1 = min(col1, in_w);
            float val = mode_avg ? 0.0f : -FLT_MAX;
            if(K) {
                // same elements in the same order as the run-time loops, with the window unrolled
                const int wr0 = (orow0 + orel) * sh - ph, wc0 = oc * sw - pw;
                #pragma unroll
                for(int i2 = 0; i2 < (K ? K : 1); i2++)
                    #pragma unroll
                    for(int j2 = 0; j2 < (K ? K : 1); j2++) {
                        const int r = wr0 + i2, c = wc0 + j2;
                        if(r >= row0 && r < row1 && c >= col0 && c < col1) {
                            const float v = tile[(r - irow0) * in_w + c];
                            val = mode_avg ? val + v : fmaxf(val, v);
                        }
                    }
            }
            else
                for(int r = row0; r < row1; r++)
                    for(int c = col0; c < col1; c++) {
                        const float v = tile[(r - irow0) * in_w + c];
                        val = mode_avg ? val + v : fmaxf(val, v);
                    }
            if(mode_avg) {
                const int dr = row1 - row0, dc = col1 - col0;
                if(dr == kh && dc == kw) val = val * (1.0f / (kh * kw));
                else if(include_pad) val = val / float(dr_pad * dc_pad);
                else val = val * (1.0f / (dr * dc));
            }
            dst[i] = val;
        }
        __syncthreads();
    }
}

// Max pooling 3x3, stride 2, padding 1 over rows of even width, without shared memory: a warp takes 32 output columns
// of a strip of RS output rows.  A lane reads the two input columns 2*oc and 2*oc+1 of every input row of the strip as one
// aligned 8-byte load (a warp reads 256 consecutive bytes), takes column 2*oc-1 from its left neighbour by shuffle, and
// keeps the row maxima in registers; all the strip's loads are issued before the first is used.  Maximum is exact in any
// order, so the result is bit-identical to pooling2d_kernel's.
template<int RS>
__global__ void __launch_bounds__(256) pool_max3s2_kernel(const float *__restrict__ x, float *__restrict__ y, long long items, int col_blocks,
                                                          int strips, int in_h, int in_w, int out_h, int out_w)
{
    const long long item = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if(item >= items) return;
    const int cb = int(item % col_blocks);
    const long long t = item / col_blocks;
    const int strip = int(t % strips);
    const long long plane = t / strips;
    const int oc = cb * 32 + lane, orow0 = strip * RS;
    const bool col_ok = oc < out_w;
    const float *src = x + plane * (long long)in_h * in_w;
    constexpr int ROWS = 2 * RS + 1;
    float2 a[ROWS];
    float left[ROWS];
    #pragma unroll
    for(int r = 0; r < ROWS; r++) {
        const int iy = 2 * orow0 - 1 + r;
        const bool ok = col_ok && iy >= 0 && iy < in_h;
        a[r] = ok ? __ldg(reinterpret_cast<const float2 *>(src + (long long)iy * in_w) + oc) : make_float2(-FLT_MAX, -FLT_MAX);
        // lane 0 has no left neighbour in the warp: column 2*oc-1 is the padding (first block) or one more load
        left[r] = (ok && lane == 0 && oc > 0) ? __ldg(src + (long long)iy * in_w + 2 * oc - 1) : -FLT_MAX;
    }
    float h[ROWS];
    #pragma unroll
    for(int r = 0; r < ROWS; r++) {
        const float from_lane = __shfl_up_sync(0xffffffffu, a[r].y, 1);
        const float l = lane == 0 ? left[r] : from_lane;
        h[r] = fmaxf(fmaxf(l, a[r].x), a[r].y);
    }
    float *dst = y + plane * (long long)out_h * out_w + oc;
    #pragma unroll
    for(int j = 0; j < RS; j++)
        if(col_ok && orow0 + j < out_h) dst[(long long)(orow0 + j) * out_w] = fmaxf(fmaxf(h[2 * j], h[2 * j + 1]), h[2 * j + 2]);
}

// Global pooling of small odd-sized planes: a CTA of 128 threads copies 128 consecutive planes into shared memory with
// coalesced 16-byte loads, then thread t reduces plane t in index order (odd plane size: conflict-free).
__global__ void __launch_bounds__(128) global_pooling_tile_kernel(const float *__restrict__ x, float *__restrict__ y, int planes, int plane_size,
                                                                  int mode_avg)
{
    extern __shared__ float tile[];
    const int plane0 = blockIdx.x * 128, count = min(128, planes - plane0) * plane_size;
    const float *src = x + (long long)plane0 * plane_size;           // 128 * plane_size * 4 bytes per CTA: 16-byte aligned when x is
    const float4 *src4 = reinterpret_cast<const float4 *>(src);
    float4 *tile4 = reinterpret_cast<float4 *>(tile);
    for(int i = threadIdx.x; i < count / 4; i += 128) tile4[i] = __ldg(src4 + i);
    for(int i = (count & ~3) + threadIdx.x; i < count; i += 128) tile[i] = __ldg(src + i);
    __syncthreads();
    if(plane0 + int(threadIdx.x) >= planes) return;
    const float *mine = tile + threadIdx.x * plane_size;
    float v = mode_avg ? 0.0f : -FLT_MAX;
    for(int i = 0; i < plane_size; i++) v = mode_avg ? v + mine[i] : fmaxf(v, mine[i]);
    y[plane0 + threadIdx.x] = mode_avg ? v * (1.0f / plane_size) : v;
}

// one warp per plane
__global__ void global_pooling_kernel(const float *__restrict__ x, float *__restrict__ y, int planes, int plane_size, int mode_avg)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if(warp >= planes) return;
    const float *src = x + (long long)warp * plane_size;
    float v = mode_avg ? 0.0f : -FLT_MAX;
    for(int i = lane; i < plane_size; i += 32) {
        const float a = __ldg(src + i);
        v = mode_avg ? v + a : fmaxf(v, a);
    }
    #pragma unroll
    for(int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, o);
        v = mode_avg ? v + other : fmaxf(v, other);
    }
    if(lane == 0) y[warp] = mode_avg ? v * (1.0f / plane_size) : v;
}

__device__ __forceinline__ float eltwise_op(float a, float b, int op, float c0, float c1)
{
    if(op == 0) return a * c0 + b * c1;
    if(op == 1) return a * b * (c0 * c1);
    return fmaxf(a * c0, b * c1);
}
// c may be a or b (in-place Elementwise): no __restrict__ and no non-coherent loads on the operands
__global__ void elementwise_kernel(const float *a, const float *b, float *c, size_t count, int op, float c0, float c1, int act, int vec_ok)
{
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, step = (size_t)gridDim.x * blockDim.x;
    if(vec_ok) {
        const size_t n4 = count / 4;
        for(size_t i = tid; i < n4; i += step) {
            const float4 u = reinterpret_cast<const float4 *>(a)[i], v = reinterpret_cast<const float4 *>(b)[i];
            float4 r;
            r.x = apply_act(eltwise_op(u.x, v.x, op, c0, c1), act);
            r.y = apply_act(eltwise_op(u.y, v.y, op, c0, c1), act);
            r.z = apply_act(eltwise_op(u.z, v.z, op, c0, c1), act);
            r.w = apply_act(eltwise_op(u.w, v.w, op, c0, c1), act);
            reinterpret_cast<float4 *>(c)[i] = r;
        }
        for(size_t i = n4 * 4 + tid; i < count; i += step) c[i] = apply_act(eltwise_op(a[i], b[i], op, c0, c1), act);
    }
    else
        for(size_t i = tid; i < count; i += step) c[i] = apply_act(eltwise_op(a[i], b[i], op, c0, c1), act);
}

// y may be x (in place)
__global__ void activation_kernel(const float *x, float *y, size_t count, int act)
{
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        y[i] = apply_act(x[i], act);
}

// one CTA per (row, inner) slice; classes strided by `inner`
__global__ void softmax_kernel(const float *x, float *y, int classes, int inner, int log_mode)
{
    __shared__ float red[32];
    const long long slice = blockIdx.x;
    const long long base = (slice / inner) * (long long)classes * inner + slice % inner;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    float m = -FLT_MAX;
    for(int j = tid; j < classes; j += blockDim.x) m = fmaxf(m, x[base + (long long)j * inner]);
    for(int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if(lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for(int i = 1; i < nwarps; i++) m = fmaxf(m, red[i]);
    __syncthreads();
    float s = 0.0f;
    for(int j = tid; j < classes; j += blockDim.x) s += expf(x[base + (long long)j * inner] - m);
    for(int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if(lane == 0) red[warp] = s;
    __syncthreads();
    s = 0.0f;
    for(int i = 0; i < nwarps; i++) s += red[i];
    if(log_mode) {
        const float f = -logf(s);
        for(int j = tid; j < classes; j += blockDim.x) y[base + (long long)j * inner] = x[base + (long long)j * inner] - m + f;
    }
    else {
        const float f = 1.0f / s;
        for(int j = tid; j < classes; j += blockDim.x) y[base + (long long)j * inner] = expf(x[base + (long long)j * inner] - m) * f;
    }
}

__global__ void batchnorm_inference_kernel(const float *x, float *y, size_t count, int features, int plane,
                                           float eps, const float *__restrict__ mean, const float *__restrict__ var,
                                           const float *__restrict__ gamma, const float *__restrict__ beta)
{
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const int f = int((i / plane) % features);
        float a = 1.0f / sqrtf(var[f] + eps);
        float b = -mean[f] * a;
        if(gamma && beta) { a *= gamma[f]; b = gamma[f] * b + beta[f]; }
        y[i] = a * x[i] + b;
    }
}

inline int grid_for(size_t work_items, int threads)
{
    const size_t blocks = (work_items + threads - 1) / threads;
    return int(std::min<size_t>(std::max<size_t>(blocks, 1), size_t(sm_count()) * 16));
}
inline int pool_out(int in_size, int kernel, int pad, int stride, int ceil_mode)
{
    const int padded = in_size + pad * 2;
    const int offset = ceil_mode ? (stride - 1) : 0;
    int size = (padded - kernel + offset) / stride + 1;
    if((size - 1) * stride >= in_size + pad) size--;
    return size;
}

} // namespace
} // namespace dlp

using namespace dlp;

extern "C" {

dlp_status dlp_pooling2d_output_shape(int in_h, int in_w, const int kernel[2], const int stride[2], const int pad[2], int ceil_mode,
                                      int *out_h, int *out_w)
{
    DLP_REQUIRE(kernel && stride && pad && out_h && out_w, "null argument");
    DLP_REQUIRE(kernel[0] > 0 && kernel[1] > 0 && stride[0] > 0 && stride[1] > 0 && pad[0] >= 0 && pad[1] >= 0, "bad pooling geometry");
    DLP_REQUIRE(in_h + 2 * pad[0] >= kernel[0] && in_w + 2 * pad[1] >= kernel[1], "pooling window larger than the padded input");
    *out_h = pool_out(in_h, kernel[0], pad[0], stride[0], ceil_mode);
    *out_w = pool_out(in_w, kernel[1], pad[1], stride[1], ceil_mode);
    return DLP_OK;
}

dlp_status dlp_pooling2d_fwd(const float *x, float *y, int planes, int in_h, int in_w, const int kernel[2], const int stride[2],
                             const int pad[2], int ceil_mode, int mode, int count_include_pad, void *stream)
{
    int oh, ow;
    dlp_status st = dlp_pooling2d_output_shape(in_h, in_w, kernel, stride, pad, ceil_mode, &oh, &ow);
    if(st != DLP_OK) return st;
    DLP_REQUIRE(x && y, "null tensor");
    DLP_REQUIRE(mode == 0 || mode == 1, "mode must be 0 (max) or 1 (avg)");
    const long long total = (long long)planes * oh * ow;
    if(total <= 0) return DLP_OK;
    if(mode == 0 && kernel[0] == 3 && kernel[1] == 3 && stride[0] == 2 && stride[1] == 2 && pad[0] == 1 && pad[1] == 1 && in_w % 2 == 0 &&
       2 * ow <= in_w && reinterpret_cast<uintptr_t>(x) % 8 == 0) {
        constexpr int RS = 4;      // 4-row strips: measured faster than 8 (fewer registers, more warps in flight)
        const int col_blocks = ceil_div(ow, 32), strips = ceil_div(oh, RS);
        const long long items = (long long)planes * col_blocks * strips;
        pool_max3s2_kernel<RS><<<unsigned(ceil_div<long long>(items, 8)), 256, 0, (cudaStream_t)stream>>>(x, y, items, col_blocks, strips, in_h, in_w,
                                                                                                         oh, ow);
        DLP_LAUNCH_OK("pool_max3s2_kernel");
        return DLP_OK;
    }
    // Bands of output rows through shared memory when a useful band fits in 12 KB: each input byte is read
    // from memory once (plus the halo rows between bands), in full lines.
    {
        const size_t row_bytes = size_t(in_w) * sizeof(float);
        int band_rows = 0;
        for(int r = std::min(oh, 16); r >= 1; r--)
            if((size_t(r - 1) * stride[0] + kernel[0]) * row_bytes <= 12 * 1024) { band_rows = r; break; }
        if(band_rows >= 2 && ow >= 16) {
            const int bands_per_plane = (oh + band_rows - 1) / band_rows;
            const long long bands_total = (long long)planes * bands_per_plane;
            const size_t smem = (size_t(band_rows - 1) * stride[0] + kernel[0]) * row_bytes;
            const int vec_ok = in_w % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0;
            const int grid = int(std::min<long long>(bands_total, (long long)sm_count() * 16));
            const bool square = kernel[0] == kernel[1] && stride[0] == stride[1];
#define DLP_POOL_BAND(K, S) pooling2d_band_kernel<K, S><<<grid, 256, smem, (cudaStream_t)stream>>>(x, y, bands_total, bands_per_plane, band_rows, \
            in_h, in_w, oh, ow, kernel[0], kernel[1], stride[0], stride[1], pad[0], pad[1], mode, count_include_pad, vec_ok)
            if(square && kernel[0] == 3 && stride[0] == 2) DLP_POOL_BAND(3, 2);
            else if(square && kernel[0] == 2 && stride[0] == 2) DLP_POOL_BAND(2, 2);
            else if(square && kernel[0] == 3 && stride[0] == 1) DLP_POOL_BAND(3, 1);
            else DLP_POOL_BAND(0, 0);
#undef DLP_POOL_BAND
            DLP_LAUNCH_OK("pooling2d_band_kernel");
            return DLP_OK;
        }
    }
    pooling2d_kernel<<<grid_for(size_t(total), 256), 256, 0, (cudaStream_t)stream>>>(x, y, total, in_h, in_w, oh, ow, kernel[0], kernel[1],
                                                                                      stride[0], stride[1], pad[0], pad[1], mode,
                                                                                      count_include_pad);
    DLP_LAUNCH_OK("pooling2d_kernel");
    return DLP_OK;
}

dlp_status dlp_global_pooling_fwd(const float *x, float *y, int planes, int plane_size, int mode, void *stream)
{
    DLP_REQUIRE(x && y, "null tensor");
    DLP_REQUIRE(plane_size > 0 && (mode == 0 || mode == 1), "bad global pooling arguments");
    if(planes <= 0) return DLP_OK;
    if(plane_size % 2 == 1 && plane_size <= 95 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
        global_pooling_tile_kernel<<<ceil_div(planes, 128), 128, size_t(128) * plane_size * sizeof(float), (cudaStream_t)stream>>>(x, y, planes,
                                                                                                                                plane_size, mode);
        DLP_LAUNCH_OK("global_pooling_tile_kernel");
        return DLP_OK;
    }
    const int threads = 256, warps_per_block = threads / 32;
    global_pooling_kernel<<<ceil_div(planes, warps_per_block), threads, 0, (cudaStream_t)stream>>>(x, y, planes, plane_size, mode);
    DLP_LAUNCH_OK("global_pooling_kernel");
    return DLP_OK;
}

dlp_status dlp_elementwise_fwd(const float *a, const float *b, float *c, size_t count, int op, float coef1, float coef2, int activation,
                               void *stream)
{
    DLP_REQUIRE(a && b && c, "null tensor");
    DLP_REQUIRE(op >= 0 && op <= 2, "op must be 0 (sum), 1 (prod) or 2 (max)");
    if(count == 0) return DLP_OK;
    const int vec_ok = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) % 16) == 0;
    elementwise_kernel<<<grid_for(count / 4 + 1, 256), 256, 0, (cudaStream_t)stream>>>(a, b, c, count, op, coef1, coef2, activation, vec_ok);
    DLP_LAUNCH_OK("elementwise_kernel");
    return DLP_OK;
}

dlp_status dlp_activation_fwd(const float *x, float *y, size_t count, int activation, void *stream)
{
    DLP_REQUIRE(x && y, "null tensor");
    if(count == 0) return DLP_OK;
    activation_kernel<<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>(x, y, count, activation);
    DLP_LAUNCH_OK("activation_kernel");
    return DLP_OK;
}

dlp_status dlp_softmax_fwd(const float *x, float *y, int rows, int classes, int inner, int log_mode, void *stream)
{
    DLP_REQUIRE(x && y, "null tensor");
    DLP_REQUIRE(classes > 0 && inner > 0, "bad softmax shape");
    if(rows <= 0) return DLP_OK;
    const int threads = classes >= 512 ? 256 : (classes >= 128 ? 128 : 32);
    softmax_kernel<<<(unsigned)((long long)rows * inner), threads, 0, (cudaStream_t)stream>>>(x, y, classes, inner, log_mode);
    DLP_LAUNCH_OK("softmax_kernel");
    return DLP_OK;
}

dlp_status dlp_batchnorm_inference_fwd(const float *x, float *y, int batch, int features, int plane, float eps, const float *mean,
                                       const float *var, const float *gamma, const float *beta, void *stream)
{
    DLP_REQUIRE(x && y && mean && var, "null tensor");
    DLP_REQUIRE(features > 0 && plane > 0, "bad batch-norm shape");
    const size_t count = size_t(batch) * features * plane;
    if(count == 0) return DLP_OK;
    batchnorm_inference_kernel<<<grid_for(count, 256), 256, 0, (cudaStream_t)stream>>>(x, y, count, features, plane, eps, mean, var, gamma, beta);
    DLP_LAUNCH_OK("batchnorm_inference_kernel");
    return DLP_OK;
}

} // extern "C"
