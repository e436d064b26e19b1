// One description for every dense contraction on the hot path.
//
// Convolution (implicit GEMM, src/core/conv.cpp:59-80 in the reference), 1x1 convolution, InnerProduct
// and the plain GEMM interface are all   D[row, col] = sum_k  A(row, k) * B(col, k)   with
//   row = an output pixel (batch, oy, ox)  or a row of the GEMM's C,
//   col = an output channel               or a column of C,
//   k   = (input channel, ky, kx)         or the GEMM's K.
// The A side is read straight from the caller's tensor (NCHW activations or a row-major /
// transposed matrix), never re-laid-out in memory; the B side (weights) is either raw or pre-packed.
#pragma once
#include "common.cuh"

namespace dlp {

enum : int {
    A_GATHER = 0,  // general convolution: address = row_base + ktab[k].offset, bounds-checked per tap
    A_STRIDED = 1, // address = row_base + k * a_k_stride (1x1 stride-1 convolution, matrices)
    A_TAPBLOCK = 2, // convolution with channels in blocks of 32: k-block kb = (channel block, tap); the 32 values
                   // of a k-block are one tap of 32 consecutive channels: row_base + tap offset + channel * a_k_stride
    A_ROWTAPS = 3  // convolution with few input channels and a wide kernel (a 7x7 stem): the reduction index is
                   // (channel, kernel row, kernel column padded to 8), so a k-block is four kernel rows of eight
                   // consecutive input elements each: one table entry and one row test per eight loads (tensor-core kernel only)
};
enum : int {
    OUT_NCHW = 0,     // row = (b, pix): y[(b * out_channels_total + col) * out_plane + pix]
    OUT_ROW_MAJOR = 1, // y[row * ldc + col]
    OUT_COL_MAJOR = 2  // y[col * ldc + row]: the scratch layout of split-K partial results
};

struct KTap {
    int offset;  // element offset of reduction index k from the row's base address: c*H*W + dy*W + dx
    int tap;     // FFMA kernel: the kernel tap ky*KW + kx.  Tensor-core kernel: (ky << 8) | kx, and
                 // TAP_PADDING for the zero padding beyond K (a kernel row that never exists)
                 // A_ROWTAPS: one entry per (channel, kernel row): offset of its first column, tap = ky (ROW_PADDING beyond K)
};
constexpr int ROW_PADDING = 31;
constexpr int ROWTAPS_WIDTH = 8;      // kernel columns per (channel, kernel row) group in the A_ROWTAPS order
constexpr int TAP_PADDING = 31 << 8;
constexpr int MAX_KERNEL_SIDE = 30;   // larger kernels (more rows or columns than validity bits) use the FFMA path

struct Contraction {
    // sizes
    long long rows;      // M: batch*OH*OW or GEMM M
    int cols;            // N: output channels of this group or GEMM N
    int k;               // true K
    // A side
    const float *a;
    int a_mode;          // A_GATHER / A_STRIDED
    long long a_k_stride;
    long long a_row_stride;   // A_STRIDED matrices: base = row * a_row_stride (used when plane == 0)
    // convolution geometry (A_GATHER and A_STRIDED with plane > 0)
    int plane;           // OH*OW (0 = matrix addressing)
    int out_w;
    int in_h, in_w;
    int stride_h, stride_w, pad_h, pad_w;
    long long a_batch_stride;  // Cin_total*H*W
    const KTap *ktab;    // k_pad entries
    const int *tap_dydx; // num_taps entries: (dy << 16) | dx displacement of each kernel tap (dilation included)
    int num_taps;
    int kh, kw, dil_h, dil_w;   // kernel size and dilation (tensor-core loaders: which taps fall inside the image)
    // B side, raw form: B(col, k) = b[col * b_col_stride + k * b_k_stride]
    const float *b;
    long long b_col_stride, b_k_stride;
    // output
    float *y;
    int out_mode;
    long long ldc;            // OUT_ROW_MAJOR
    int out_channels_total;   // OUT_NCHW: channels of the whole output tensor
    const float *bias;
    int bias_mode;            // DLP_GEMM_NO_BIAS / BIAS_M (per row) / BIAS_N (per col)
    int act;
    float beta;               // y = beta*y_old + act(...)
    const float *residual;    // optional, same addressing as y
    float residual_scale;
    int post_act;
};

// Row (pixel) coordinates shared by the loaders.
struct RowInfo {
    long long base;  // element offset of the row's first tap (may be "negative" through padding)
    int iy0, ix0;    // input coordinates of tap (0,0)
    long long out;   // element offset of the row in y (without the column term)
    bool valid;
};

// a_off / y_off: element offsets of the matrix a batched product is working on (0 otherwise)
__device__ __forceinline__ RowInfo make_row(const Contraction &p, long long row, long long a_off = 0, long long y_off = 0)
{
    RowInfo r;
    r.valid = row < p.rows;
    if(!r.valid) row = 0;
    if(p.plane > 0) {
        // 32-bit division when it fits: this runs once per tile in every loader and epilogue thread
        int b = p.rows < (1ll << 31) ? int(unsigned(row) / unsigned(p.plane)) : int(row / p.plane);
        int pix = int(row - (long long)b * p.plane);
        int oy = pix / p.out_w;
        int ox = pix - oy * p.out_w;
        r.iy0 = oy * p.stride_h - p.pad_h;
        r.ix0 = ox * p.stride_w - p.pad_w;
        r.base = (long long)b * p.a_batch_stride + (long long)r.iy0 * p.in_w + r.ix0;
        r.out = p.out_mode == OUT_NCHW ? (long long)b * p.out_channels_total * p.plane + pix : (p.out_mode == OUT_COL_MAJOR ? row : row * p.ldc);
    }
    else {
        r.iy0 = r.ix0 = 0;
        r.base = row * p.a_row_stride;
        r.out = p.out_mode == OUT_COL_MAJOR ? row : row * p.ldc;
    }
    r.base += a_off;
    r.out += y_off;
    return r;
}

__device__ __forceinline__ long long out_index(const Contraction &p, const RowInfo &r, int col)
{
    return p.out_mode == OUT_NCHW ? r.out + (long long)col * p.plane : (p.out_mode == OUT_COL_MAJOR ? r.out + (long long)col * p.ldc : r.out + col);
}

__device__ __forceinline__ float finish_output(const Contraction &p, const RowInfo &r, long long row, int col, float acc)
{
    if(p.bias_mode == DLP_GEMM_BIAS_N) acc += __ldg(p.bias + col);
    else if(p.bias_mode == DLP_GEMM_BIAS_M) acc += __ldg(p.bias + row);
    acc = apply_act(acc, p.act);
    long long idx = out_index(p, r, col);
    if(p.residual) acc = apply_act(acc + p.residual_scale * __ldg(p.residual + idx), p.post_act);
    if(p.beta != 0.0f) acc += p.beta * p.y[idx];
    return acc;
}

// launchers (one per translation unit)
// groups: grouped convolution (out_group_channels output channels each) or a batch of matrices (y_group_stride apart in y)
dlp_status launch_contraction_ffma(const Contraction &p, int groups, long long a_group_stride, long long b_group_stride,
                                   int out_group_channels, cudaStream_t stream, long long y_group_stride = 0);

// Pre-packed B for the tensor-core kernel: zero padded and already split into its TF32 part (hi) and
// the remainder (lo).  It is a sequence of pipeline stages in the order (column tile, k-block of 32);
// a stage is the exact shared-memory image the kernel computes from -- the hi tile (bn rows of 32
// floats, 128-byte swizzled) followed by the lo tile -- so one contiguous bulk copy brings it in.
struct TcPacked {
    int bn;         // column tile: 32, 64 or 128
    int n_pad, k_pad;
    size_t bytes() const { return size_t(2) * n_pad * k_pad * sizeof(float); }
};
TcPacked tc_packed_layout(int cols, int k);
// taps > 0 packs in the A_TAPBLOCK order: packed k = ((channel block * taps + tap) * 32 + channel in block)
// batch > 1: that many matrices b_batch_stride elements apart, packed one after the other (L.bytes() each)
// row_kw > 0 packs in the A_ROWTAPS order: packed k = (channel * KH + ky) * 8 + kx  <-  source k = (channel * KH + ky) * row_kw + kx
dlp_status tc_prepack(const TcPacked &L, const float *b, long long b_col_stride, long long b_k_stride, int cols, int k,
                      float *packed, int taps, cudaStream_t stream, int batch = 1, long long b_batch_stride = 0, int row_kw = 0);
// A batch of equal-sized products in one launch: matrix i reads a + i * a_stride, its own packed operand and writes y + i * y_stride.
struct TcBatch {
    int count = 1;
    long long a_stride = 0, y_stride = 0;
};
// Scratch that lets the launcher split K when the problem has too few tiles for the GPU (0: it would not split).
size_t tc_split_scratch_bytes(long long rows, const TcPacked &L);
// scratch may be null or short; the launcher then does not split.
dlp_status launch_contraction_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream, void *scratch = nullptr,
                                 size_t scratch_bytes = 0, const TcBatch &batch = TcBatch());

// 1x1 stride-1 convolutions over large planes with few input channels: a kernel that moves every operand with the copy
// engines (pointwise_tc.cu).  launch_contraction_tc hands eligible problems over by itself.
bool pointwise_tc_eligible(const Contraction &p, const TcPacked &L);
dlp_status launch_pointwise_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream);

// Convolutions with at most 64 output channels over rows of a multiple of four pixels (the 7x7 stem, 3x3 over 64 channels): the
// input patch of a tile of whole output rows comes in by one tensor-map copy per channel block and every tap is gathered from
// shared memory (staged_tc.cu).  launch_contraction_tc hands eligible problems over by itself.
bool staged_tc_eligible(const Contraction &p, const TcPacked &L);
dlp_status launch_staged_tc(const Contraction &p, const TcPacked &L, const float *packed, cudaStream_t stream);

// Winograd F(2x2, 3x3), stride 1, padding 1 (winograd.cu).  u: the transformed filters, winograd_packed_bytes() long.
size_t winograd_packed_bytes(int cin, int cout);
dlp_status winograd_filter_transform(const float *w, float *u, int cin, int cout, cudaStream_t stream);
dlp_status launch_winograd_f23(const float *x, const float *u, const float *bias, float *y, int batch, int cin, int cout, int h, int w,
                               int act, float factor, const float *residual, float residual_scale, int post_act, cudaStream_t stream);

// Winograd F(2x2, 3x3) with the sixteen products on the tensor cores (winograd_tc.cu): transform, one batched 3xTF32
// contraction, transform back.  ws: winograd_tc_workspace_bytes() for the batch.
size_t winograd_tc_packed_bytes(int cin, int cout);
size_t winograd_tc_workspace_bytes(int batch, int cin, int cout, int h, int w);
dlp_status winograd_tc_filter_transform(const float *w, float *packed, int cin, int cout, cudaStream_t stream);
dlp_status launch_winograd_tc(const float *x, const float *packed, const float *bias, float *y, void *ws, size_t ws_bytes, int batch, int cin,
                              int cout, int h, int w, int act, float factor, const float *residual, float residual_scale, int post_act,
                              cudaStream_t stream);

} // namespace dlp
