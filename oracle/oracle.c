/* CPU restatement of the reference's convolution / GEMM forward path.
 * TEST INFRASTRUCTURE ONLY -- see oracle.h.  Parity status: pinned (oracle.h).
 *
 * The arithmetic follows the reference's CPU context operation for operation
 * (same loop nests, same accumulation order, one rounding per multiply and per
 * add, no fused multiply-add), so that on the same inputs the results are
 * bit-identical to the reference library built with its internal BLAS.
 */
#include "oracle.h"
#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>

static int g_threads = 1;
void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int oracle_get_threads(void) { return g_threads; }

/* ---- activations: include/dlprim/cpu/cpu_ops.hpp:16-53 ---- */
void oracle_activation(float *p, size_t n, int activation)
{
    size_t i;
    switch(activation) {
    case ORACLE_ACT_RELU:
        for(i = 0; i < n; i++) p[i] = p[i] > 0.0f ? p[i] : 0.0f;
        break;
    case ORACLE_ACT_TANH:
        for(i = 0; i < n; i++) p[i] = tanhf(p[i]);
        break;
    case ORACLE_ACT_SIGMOID:
        for(i = 0; i < n; i++) p[i] = 1 / (1 + expf(-p[i]));
        break;
    case ORACLE_ACT_RELU6:
        for(i = 0; i < n; i++) { float v = p[i] > 0.0f ? p[i] : 0.0f; p[i] = v < 6.0f ? v : 6.0f; }
        break;
    default:
        break;
    }
}

/* ---- row-major sgemm, four loop orders: src/my_blas/my_cblas.cpp:23-103 ---- */
void oracle_sgemm(int ta, int tb, int M, int N, int K, float alpha, const float *A, int lda,
                  const float *B, int ldb, float beta, float *C, int ldc)
{
    int r, c, k;
    if(beta == 0.0f) {
        for(r = 0; r < M; r++) memset(C + (size_t)ldc * r, 0, sizeof(float) * N);
    }
    else {
        for(r = 0; r < M; r++) for(c = 0; c < N; c++) C[(size_t)ldc * r + c] *= beta;
    }
    if(!ta && !tb) {
        for(r = 0; r < M; r++)
            for(k = 0; k < K; k++) {
                float av = A[(size_t)r * lda + k] * alpha;
                for(c = 0; c < N; c++) C[(size_t)r * ldc + c] += av * B[(size_t)k * ldb + c];
            }
    }
    else if(ta && !tb) {
        for(k = 0; k < K; k++)
            for(r = 0; r < M; r++) {
                float av = A[r + (size_t)lda * k] * alpha;
                for(c = 0; c < N; c++) C[(size_t)r * ldc + c] += av * B[(size_t)k * ldb + c];
            }
    }
    else if(!ta && tb) {
        for(r = 0; r < M; r++)
            for(c = 0; c < N; c++) {
                float acc = C[(size_t)r * ldc + c];
                for(k = 0; k < K; k++) {
                    float bv = B[k + (size_t)ldb * c];
                    float av = A[(size_t)r * lda + k] * alpha;
                    acc += av * bv;
                }
                C[(size_t)r * ldc + c] = acc;
            }
    }
    else {
        for(c = 0; c < N; c++)
            for(k = 0; k < K; k++) {
                float bv = B[k + (size_t)ldb * c] * alpha;
                for(r = 0; r < M; r++) C[(size_t)r * ldc + c] += A[r + (size_t)lda * k] * bv;
            }
    }
}

/* The device GEMM contract, C = beta*C + act(op(A)*op(B) + bias): include/dlprim/gpu/gemm.hpp:15-82.
 * bias_mode 0 none, 1 one value per row of C, 2 one value per column of C. */
void oracle_gemm_bias_act(int ta, int tb, int M, int N, int K, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, const float *bias, int bias_mode, int activation)
{
    float *tmp = (float *)malloc(sizeof(float) * (size_t)M * N);
    int r, c;
    oracle_sgemm(ta, tb, M, N, K, 1.0f, A, lda, B, ldb, 0.0f, tmp, N);
    for(r = 0; r < M; r++)
        for(c = 0; c < N; c++) {
            float v = tmp[(size_t)r * N + c];
            if(bias_mode == 1) v += bias[r];
            else if(bias_mode == 2) v += bias[c];
            tmp[(size_t)r * N + c] = v;
        }
    oracle_activation(tmp, (size_t)M * N, activation);
    for(r = 0; r < M; r++)
        for(c = 0; c < N; c++) {
            float v = tmp[(size_t)r * N + c];
            if(beta != 0.0f) v += beta * C[(size_t)r * ldc + c];
            C[(size_t)r * ldc + c] = v;
        }
    free(tmp);
}

/* ---- InnerProduct::forward_cpu: src/ops/inner_product.cpp:161-184 ---- */
void oracle_inner_product_forward(int batch, int inputs, int outputs, const float *x, const float *w, const float *bias,
                                  int activation, float *y)
{
    int i, j;
    oracle_sgemm(0, 1, batch, outputs, inputs, 1.0f, x, inputs, w, inputs, 0.0f, y, outputs);
    if(bias)
        for(i = 0; i < batch; i++)
            for(j = 0; j < outputs; j++) y[(size_t)i * outputs + j] += 1.0f * bias[j];
    oracle_activation(y, (size_t)batch * outputs, activation);
}

/* ---- Convolution2D::forward_cpu: src/ops/conv2d.cpp:282-409 (im2col), 421-502 ---- */
void oracle_conv2d_output_hw(const oracle_conv2d_desc *d, int *oh, int *ow)
{
    /* src/core/conv.cpp:17-29 */
    *oh = (d->height + 2 * d->pad[0] - d->dilate[0] * (d->kernel[0] - 1) - 1) / d->stride[0] + 1;
    *ow = (d->width + 2 * d->pad[1] - d->dilate[1] * (d->kernel[1] - 1) - 1) / d->stride[1] + 1;
}

/* One image, one group: rows = output pixels, columns = (channel, ky, kx). */
static void im2col_image(const oracle_conv2d_desc *d, int cin_g, int oh, int ow, const float *img, float *mat)
{
    int r, c, ch, ky, kx;
    for(r = 0; r < oh; r++)
        for(c = 0; c < ow; c++) {
            float *row = mat + ((size_t)r * ow + c) * cin_g * d->kernel[0] * d->kernel[1];
            for(ch = 0; ch < cin_g; ch++)
                for(ky = 0; ky < d->kernel[0]; ky++)
                    for(kx = 0; kx < d->kernel[1]; kx++) {
                        int y = r * d->stride[0] - d->pad[0] + ky * d->dilate[0];
                        int x = c * d->stride[1] - d->pad[1] + kx * d->dilate[1];
                        float v = 0.0f;
                        if(y >= 0 && y < d->height && x >= 0 && x < d->width)
                            v = img[((size_t)ch * d->height + y) * d->width + x];
                        *row++ = v;
                    }
        }
}

typedef struct conv_job {
    const oracle_conv2d_desc *d;
    const float *x, *w, *bias;
    float *y;
    int oh, ow, b0, b1, winograd, rc;
} conv_job;

static void conv_image_winograd(const oracle_conv2d_desc *d, int oh, int ow, const float *img, const float *u,
                                const float *bias, float *out);

static void *conv_worker(void *arg)
{
    conv_job *j = (conv_job *)arg;
    const oracle_conv2d_desc *d = j->d;
    int cin_g = d->channels_in / d->groups, cout_g = d->channels_out / d->groups;
    int rows = j->oh * j->ow, cols = cin_g * d->kernel[0] * d->kernel[1];
    size_t in_img = (size_t)d->channels_in * d->height * d->width, out_img = (size_t)d->channels_out * rows;
    float *mat = NULL;
    int b, g, i, p;
    if(!j->winograd) {
        mat = (float *)malloc(sizeof(float) * (size_t)rows * cols);
        if(!mat) { j->rc = -1; return NULL; }
    }
    for(b = j->b0; b < j->b1; b++) {
        if(j->winograd) {
            /* j->w holds the transformed filters [cout][cin][16] */
            conv_image_winograd(d, j->oh, j->ow, j->x + in_img * b, j->w, j->bias, j->y + out_img * b);
            continue;
        }
        for(g = 0; g < d->groups; g++) {
            const float *img = j->x + in_img * b + (size_t)g * cin_g * d->height * d->width;
            float *omg = j->y + out_img * b + (size_t)g * cout_g * rows;
            im2col_image(d, cin_g, j->oh, j->ow, img, mat);
            oracle_sgemm(0, 1, cout_g, rows, cols, 1.0f, j->w + (size_t)g * cout_g * cols, cols, mat, cols, 0.0f, omg, rows);
            if(j->bias)
                for(i = 0; i < cout_g; i++)
                    for(p = 0; p < rows; p++) omg[(size_t)i * rows + p] += 1.0f * j->bias[g * cout_g + i];
        }
    }
    free(mat);
    return NULL;
}

static int conv_run(const oracle_conv2d_desc *d, const float *x, const float *w, const float *bias, float *y, int winograd)
{
    int oh, ow, nt, t, rc = 0;
    conv_job jobs[256];
    pthread_t th[256];
    if(d->groups < 1 || d->channels_in % d->groups || d->channels_out % d->groups) return -1;
    oracle_conv2d_output_hw(d, &oh, &ow);
    if(oh <= 0 || ow <= 0) return -1;
    nt = g_threads < d->batch ? g_threads : d->batch;
    if(nt < 1) nt = 1;
    for(t = 0; t < nt; t++) {
        conv_job j = { d, x, w, bias, y, oh, ow, (int)((long long)d->batch * t / nt), (int)((long long)d->batch * (t + 1) / nt), winograd, 0 };
        jobs[t] = j;
    }
    if(nt == 1)
        conv_worker(&jobs[0]);
    else {
        for(t = 0; t < nt; t++) pthread_create(&th[t], NULL, conv_worker, &jobs[t]);
        for(t = 0; t < nt; t++) pthread_join(th[t], NULL);
    }
    for(t = 0; t < nt; t++) if(jobs[t].rc) rc = jobs[t].rc;
    if(rc) return rc;
    oracle_activation(y, (size_t)d->batch * d->channels_out * oh * ow, d->activation);
    return 0;
}

int oracle_conv2d_forward(const oracle_conv2d_desc *d, const float *x, const float *w, const float *bias, float *y)
{
    return conv_run(d, x, w, bias, y, 0);
}

/* ---- Winograd F(2x2,3x3) restated on the CPU.
 * The reference has this algorithm only as OpenCL (src/kernels/winograd_fwd.cl):
 * filter transform G k G^T :103-135, input transform B^T d B :35-69, output transform
 * A^T m A :138-158, accumulation over input channels in channel order :329-365,
 * then bias and activation :195-222.  3x3, stride 1, pad 1, dilation 1, one group. */
static void winograd_filter(const float *k, float *u)
{
    float gk[3][4];
    int c, i;
    for(c = 0; c < 3; c++) {
        gk[c][0] = k[c];
        gk[c][1] = 0.5f * (k[c] + k[3 + c] + k[6 + c]);
        gk[c][2] = 0.5f * (k[c] - k[3 + c] + k[6 + c]);
        gk[c][3] = k[6 + c];
    }
    for(i = 0; i < 4; i++) {
        u[i * 4 + 0] = gk[0][i];
        u[i * 4 + 1] = 0.5f * (gk[0][i] + gk[1][i] + gk[2][i]);
        u[i * 4 + 2] = 0.5f * (gk[0][i] - gk[1][i] + gk[2][i]);
        u[i * 4 + 3] = gk[2][i];
    }
}
static void winograd_input(float d[4][4], float v[16])
{
    float t[4][4];
    int i;
    for(i = 0; i < 4; i++) {
        t[0][i] = d[0][i] - d[2][i];
        t[1][i] = d[1][i] + d[2][i];
        t[2][i] = d[2][i] - d[1][i];
        t[3][i] = d[1][i] - d[3][i];
    }
    for(i = 0; i < 4; i++) {
        v[i * 4 + 0] = t[i][0] - t[i][2];
        v[i * 4 + 1] = t[i][1] + t[i][2];
        v[i * 4 + 2] = t[i][2] - t[i][1];
        v[i * 4 + 3] = t[i][1] - t[i][3];
    }
}
static void conv_image_winograd(const oracle_conv2d_desc *d, int oh, int ow, const float *img, const float *u,
                                const float *bias, float *out)
{
    int th = (oh + 1) / 2, tw = (ow + 1) / 2, co, ci, ty, tx, i, j;
    size_t plane = (size_t)d->height * d->width;
    float *v = (float *)malloc(sizeof(float) * 16 * (size_t)d->channels_in);
    for(ty = 0; ty < th; ty++)
        for(tx = 0; tx < tw; tx++) {
            for(ci = 0; ci < d->channels_in; ci++) {
                float tile[4][4];
                for(i = 0; i < 4; i++)
                    for(j = 0; j < 4; j++) {
                        int y = ty * 2 - 1 + i, x = tx * 2 - 1 + j;
                        tile[i][j] = (y >= 0 && y < d->height && x >= 0 && x < d->width) ? img[ci * plane + (size_t)y * d->width + x] : 0.0f;
                    }
                winograd_input(tile, v + 16 * (size_t)ci);
            }
            for(co = 0; co < d->channels_out; co++) {
                float m[16], a0[4], a1[4], r[4];
                for(i = 0; i < 16; i++) m[i] = 0.0f;
                for(ci = 0; ci < d->channels_in; ci++) {
                    const float *uu = u + ((size_t)co * d->channels_in + ci) * 16, *vv = v + 16 * (size_t)ci;
                    for(i = 0; i < 16; i++) m[i] += uu[i] * vv[i];
                }
                for(i = 0; i < 4; i++) {
                    a0[i] = m[i] + m[4 + i] + m[8 + i];
                    a1[i] = m[4 + i] - m[8 + i] - m[12 + i];
                }
                r[0] = a0[0] + a0[1] + a0[2];
                r[1] = a0[1] - a0[2] - a0[3];
                r[2] = a1[0] + a1[1] + a1[2];
                r[3] = a1[1] - a1[2] - a1[3];
                for(i = 0; i < 2; i++)
                    for(j = 0; j < 2; j++) {
                        int y = ty * 2 + i, x = tx * 2 + j;
                        if(y < oh && x < ow)
                            out[(size_t)co * oh * ow + (size_t)y * ow + x] = r[i * 2 + j] + (bias ? bias[co] : 0.0f);
                    }
            }
        }
    free(v);
}

int oracle_conv2d_winograd_forward(const oracle_conv2d_desc *d, const float *x, const float *w, const float *bias, float *y)
{
    /* eligibility: src/core/conv.cpp:686-702 */
    float *u;
    size_t n, i;
    int rc;
    if(d->kernel[0] != 3 || d->kernel[1] != 3 || d->stride[0] != 1 || d->stride[1] != 1 || d->pad[0] != 1 || d->pad[1] != 1
       || d->dilate[0] != 1 || d->dilate[1] != 1 || d->groups != 1)
        return -2;
    n = (size_t)d->channels_in * d->channels_out;
    u = (float *)malloc(sizeof(float) * 16 * n);
    if(!u) return -1;
    for(i = 0; i < n; i++) winograd_filter(w + 9 * i, u + 16 * i);
    {
        /* the workers share the transformed filters, passed in place of the raw weights */
        int oh, ow, nt, t;
        conv_job jobs[256];
        pthread_t th[256];
        oracle_conv2d_output_hw(d, &oh, &ow);
        nt = g_threads < d->batch ? g_threads : d->batch;
        if(nt < 1) nt = 1;
        for(t = 0; t < nt; t++) {
            conv_job j = { d, x, u, bias, y, oh, ow, (int)((long long)d->batch * t / nt), (int)((long long)d->batch * (t + 1) / nt), 1, 0 };
            jobs[t] = j;
        }
        for(t = 0; t < nt; t++) pthread_create(&th[t], NULL, conv_worker, &jobs[t]);
        for(t = 0; t < nt; t++) pthread_join(th[t], NULL);
        rc = 0;
        oracle_activation(y, (size_t)d->batch * d->channels_out * oh * ow, d->activation);
    }
    free(u);
    return rc;
}

/* ---- Pooling2D: include/dlprim/core/pool.hpp:17-27, src/ops/pooling.cpp:118-140,282-329 ---- */
int oracle_pooling_output_size(int in_size, int kernel, int pad, int stride, int ceil_mode)
{
    int padded = in_size + pad * 2;
    int offset = ceil_mode ? (stride - 1) : 0;
    int size = (padded - kernel + offset) / stride + 1;
    if((size - 1) * stride >= in_size + pad) size--;
    return size;
}
static int imin(int a, int b) { return a < b ? a : b; }
static int imax(int a, int b) { return a > b ? a : b; }

void oracle_pooling2d_forward(int planes, int in_h, int in_w, const int kernel[2], const int stride[2], const int pad[2],
                              int ceil_mode, int mode_avg, int count_include_pad, const float *x, float *y)
{
    int out_h = oracle_pooling_output_size(in_h, kernel[0], pad[0], stride[0], ceil_mode);
    int out_w = oracle_pooling_output_size(in_w, kernel[1], pad[1], stride[1], ceil_mode);
    float full_factor = 1.0f / (kernel[0] * kernel[1]);
    int p, orow, ocol, r, c;
    for(p = 0; p < planes; p++, x += (size_t)in_h * in_w, y += (size_t)out_h * out_w)
        for(orow = 0; orow < out_h; orow++)
            for(ocol = 0; ocol < out_w; ocol++) {
                int row0 = orow * stride[0] - pad[0], col0 = ocol * stride[1] - pad[1];
                int row1 = row0 + kernel[0], col1 = col0 + kernel[1];
                int dr_pad = imin(row1, in_h + pad[0]) - imax(-pad[0], row0);
                int dc_pad = imin(col1, in_w + pad[1]) - imax(-pad[1], col0);
                int dr, dc;
                float val = mode_avg ? 0.0f : -FLT_MAX;
                row0 = imax(0, row0); col0 = imax(0, col0);
                row1 = imin(row1, in_h); col1 = imin(col1, in_w);
                for(r = row0; r < row1; r++)
                    for(c = col0; c < col1; c++) {
                        float v = x[(size_t)r * in_w + c];
                        if(mode_avg) val = val + v;
                        else val = val > v ? val : v;
                    }
                dr = row1 - row0; dc = col1 - col0;
                if(mode_avg) {
                    if(dr == kernel[0] && dc == kernel[1]) val = val * full_factor;
                    else if(count_include_pad) val = val / (dr_pad * dc_pad);
                    else val = val * (1.0f / (dr * dc));
                }
                y[(size_t)orow * out_w + ocol] = val;
            }
}

/* ---- GlobalPooling::forward_cpu: src/ops/pooling.cpp:427-450 ---- */
void oracle_global_pooling_forward(int planes, int plane_size, int mode_avg, const float *x, float *y)
{
    int p, i;
    float factor = 1.0f / plane_size;
    for(p = 0; p < planes; p++, x += plane_size) {
        if(mode_avg) {
            float sum = 0;
            for(i = 0; i < plane_size; i++) sum += x[i];
            y[p] = sum * factor;
        }
        else {
            float m = x[0];
            for(i = 1; i < plane_size; i++) m = m > x[i] ? m : x[i];
            y[p] = m;
        }
    }
}

/* ---- Elementwise::forward_cpu, same-shape case: src/ops/elementwise.cpp:517-559.  op 0 sum, 1 prod, 2 max ---- */
void oracle_elementwise_forward(size_t n, int op, float c0, float c1, int activation, const float *a, const float *b, float *c)
{
    size_t i;
    if(op == 0) for(i = 0; i < n; i++) c[i] = a[i] * c0 + b[i] * c1;
    else if(op == 1) { float w = c0 * c1; for(i = 0; i < n; i++) c[i] = a[i] * b[i] * w; }
    else for(i = 0; i < n; i++) { float u = a[i] * c0, v = b[i] * c1; c[i] = u > v ? u : v; }
    oracle_activation(c, n, activation);
}

/* ---- Softmax::forward_cpu: src/ops/softmax.cpp:189-222 ---- */
void oracle_softmax_forward(int rows, int classes, int inner, int log_mode, const float *x, float *y)
{
    int i, k, j;
    for(i = 0; i < rows; i++)
        for(k = 0; k < inner; k++) {
            const float *in = x + (size_t)i * classes * inner + k;
            float *out = y + (size_t)i * classes * inner + k;
            float maxv = in[0], sum = 0.0f, factor;
            for(j = 1; j < classes; j++) maxv = in[(size_t)j * inner] > maxv ? in[(size_t)j * inner] : maxv;
            if(log_mode) {
                for(j = 0; j < classes; j++) sum += expf(in[(size_t)j * inner] - maxv);
                factor = -logf(sum);
                for(j = 0; j < classes; j++) out[(size_t)j * inner] = in[(size_t)j * inner] - maxv + factor;
            }
            else {
                for(j = 0; j < classes; j++) sum += out[(size_t)j * inner] = expf(in[(size_t)j * inner] - maxv);
                factor = 1.0f / sum;
                for(j = 0; j < classes; j++) out[(size_t)j * inner] *= factor;
            }
        }
}

/* ---- BatchNorm in inference: src/ops/batch_normalization.cpp:192-228 ---- */
static void bn_coefficients(int features, float eps, const float *mean, const float *var, const float *gamma, const float *beta,
                            float *scale, float *shift)
{
    int i;
    for(i = 0; i < features; i++) {
        float a = 1.0f / sqrtf(var[i] + eps);
        float b = -mean[i] * a;
        if(gamma && beta) { a *= gamma[i]; b = gamma[i] * b + beta[i]; }
        scale[i] = a;
        shift[i] = b;
    }
}
void oracle_batchnorm_inference(int batch, int features, int plane, float eps, const float *mean, const float *var,
                                const float *gamma, const float *beta, const float *x, float *y)
{
    float *a = (float *)malloc(sizeof(float) * features), *b = (float *)malloc(sizeof(float) * features);
    int bt, f, i;
    bn_coefficients(features, eps, mean, var, gamma, beta, a, b);
    for(bt = 0; bt < batch; bt++)
        for(f = 0; f < features; f++)
            for(i = 0; i < plane; i++, x++, y++) *y = a[f] * *x + b[f];
    free(a); free(b);
}

/* Fold an inference BatchNorm that follows a convolution into the convolution's parameters:
 * A, B as above; w'[co,...] = A[co]*w[co,...]; b'[co] = B[co] + A[co]*b[co].  The products are formed
 * in double and rounded once. */
void oracle_fold_batchnorm(int cout, size_t per_channel, float eps, const float *mean, const float *var,
                           const float *gamma, const float *beta, const float *w, const float *bias, float *w_out, float *bias_out)
{
    int co;
    size_t i;
    for(co = 0; co < cout; co++) {
        double a = 1.0 / sqrt((double)var[co] + (double)eps);
        double b = -(double)mean[co] * a;
        if(gamma && beta) { b = (double)gamma[co] * b + (double)beta[co]; a *= (double)gamma[co]; }
        for(i = 0; i < per_channel; i++) w_out[co * per_channel + i] = (float)(a * (double)w[co * per_channel + i]);
        bias_out[co] = (float)(b + (bias ? a * (double)bias[co] : 0.0));
    }
}
