// Dense contraction in plain fp32 FMA on the CUDA cores.
//
// Same problem description as the tensor-core kernel (contraction.cuh) but with no pre-packing and
// with groups: it serves grouped convolutions that are not depthwise, callers that ask for
// DLP_MATH_FP32_FFMA, and any shape the tensor-core path does not take.  64x64 output tile per CTA,
// 4x4 outputs per thread, K staged through shared memory 16 at a time.
#include "contraction.cuh"

namespace dlp {
namespace {

constexpr int TM = 64, TN = 64, TK = 16, THREADS = 256;

__global__ void __launch_bounds__(THREADS)
contraction_ffma_kernel(Contraction p, long long a_group_stride, long long b_group_stride, int out_group_channels, long long y_group_stride)
{
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];

    const int g = blockIdx.z;
    const float *a = p.a + g * a_group_stride;
    const float *b = p.b + g * b_group_stride;
    const int col_base = g * out_group_channels;   // channel offset of this group in y / bias

    const long long row0 = (long long)blockIdx.x * TM;
    const int col0 = blockIdx.y * TN;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;        // thread owns rows ty*4.., cols tx*4..

    // loader mapping: A tile 16 k x 64 rows -> each thread 4 elements (same row index, 4 k's)
    const int a_row = tid & 63, a_k0 = tid >> 6;   // k = a_k0 + 4*i
    const long long y_off = g * y_group_stride;     // a batch of matrices: where this one's C starts
    const RowInfo ar = make_row(p, row0 + a_row);
    // B tile 16 k x 64 cols -> thread reads k = tid & 15 (contiguous in raw weights), cols (tid >> 4) + 16*i
    const int b_k = tid & 15, b_c0 = tid >> 4;

    float acc[4][4];
    #pragma unroll
    for(int i = 0; i < 4; i++)
        #pragma unroll
        for(int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for(int k0 = 0; k0 < p.k; k0 += TK) {
        #pragma unroll
        for(int i = 0; i < 4; i++) {
            const int kk = k0 + a_k0 + 4 * i;
            float v = 0.0f;
            if(ar.valid && kk < p.k) {
                if(p.a_mode == A_STRIDED)
                    v = __ldg(a + ar.base + (long long)kk * p.a_k_stride);
                else {
                    const KTap t = p.ktab[kk];
                    const int d = __ldg(p.tap_dydx + t.tap);
                    const int iy = ar.iy0 + (d >> 16), ix = ar.ix0 + (d & 0xffff);
                    if(unsigned(iy) < unsigned(p.in_h) && unsigned(ix) < unsigned(p.in_w)) v = __ldg(a + ar.base + t.offset);
                }
            }
            As[a_k0 + 4 * i][a_row] = v;
        }
        #pragma unroll
        for(int i = 0; i < 4; i++) {
            const int c = b_c0 + 16 * i, col = col0 + c, kk = k0 + b_k;
            float v = 0.0f;
            if(col < p.cols && kk < p.k) v = __ldg(b + col * p.b_col_stride + kk * p.b_k_stride);
            Bs[b_k][c] = v;
        }
        __syncthreads();
        #pragma unroll
        for(int kk = 0; kk < TK; kk++) {
            float av[4], bv[4];
            #pragma unroll
            for(int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
            #pragma unroll
            for(int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
            #pragma unroll
            for(int i = 0; i < 4; i++)
                #pragma unroll
                for(int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

    #pragma unroll
    for(int i = 0; i < 4; i++) {
        const long long row = row0 + ty * 4 + i;
        const RowInfo r = make_row(p, row, 0, y_off);
        if(!r.valid) continue;
        #pragma unroll
        for(int j = 0; j < 4; j++) {
            const int col = col0 + tx * 4 + j;
            if(col >= p.cols) continue;
            const int ocol = col_base + col;       // column in the whole output tensor
            p.y[out_index(p, r, ocol)] = finish_output(p, r, row, ocol, acc[i][j]);
        }
    }
}

} // namespace

dlp_status launch_contraction_ffma(const Contraction &p, int groups, long long a_group_stride, long long b_group_stride,
                                   int out_group_channels, cudaStream_t stream, long long y_group_stride)
{
    if(p.rows <= 0 || p.cols <= 0 || groups <= 0) return DLP_OK;
    const long long gx = ceil_div<long long>(p.rows, TM);
    if(gx > 0x7fffffffLL) return fail(DLP_INVALID_ARGUMENT, "too many output rows for one launch");
    dim3 grid((unsigned)gx, (unsigned)ceil_div(p.cols, TN), (unsigned)groups);
    contraction_ffma_kernel<<<grid, THREADS, 0, stream>>>(p, a_group_stride, b_group_stride, out_group_channels, y_group_stride);
    DLP_LAUNCH_OK("contraction_ffma_kernel");
    return DLP_OK;
}

} // namespace dlp
