/* CPU restatement of the reference's convolution / GEMM forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing under this directory is part of the
 * product: only the test-suite, the smoke check and the bench's CPU-baseline
 * leg may build or call it, and only as the checker.  The product path is the
 * CUDA library and has no CPU fallback.
 *
 * Parity status: pinned.  The functions here are checked (tests/test_oracle.py)
 * against the PyTorch-generated vectors embedded in the reference's own
 * tests/test_case_inner_product.json, against fixtures regenerated with the
 * reference's tests/make_test_cases_from_pt.py, and bit-for-bit against the
 * reference's own CPU context compiled from its sources (oracle/_ref).
 *
 * All tensors are dense fp32; images are NCHW; file:line citations are paths
 * inside the reference project.
 */
#ifndef DLP_ORACLE_H
#define DLP_ORACLE_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

/* activation codes: include/dlprim/definitions.hpp:278-284 */
enum { ORACLE_ACT_IDENTITY = 0, ORACLE_ACT_RELU = 1, ORACLE_ACT_TANH = 2, ORACLE_ACT_SIGMOID = 3, ORACLE_ACT_RELU6 = 4 };

typedef struct oracle_conv2d_desc {
    int batch, channels_in, height, width;
    int channels_out;
    int kernel[2], stride[2], dilate[2], pad[2];
    int groups;
    int activation;
} oracle_conv2d_desc;

/* worker threads used across independent images (each image's arithmetic is unchanged) */
void oracle_set_threads(int n);
int oracle_get_threads(void);

void oracle_conv2d_output_hw(const oracle_conv2d_desc *d, int *oh, int *ow);
int oracle_conv2d_forward(const oracle_conv2d_desc *d, const float *x, const float *w, const float *bias, float *y);
int oracle_conv2d_winograd_forward(const oracle_conv2d_desc *d, const float *x, const float *w, const float *bias, float *y);
void oracle_sgemm(int trans_a, int trans_b, int M, int N, int K, float alpha, const float *A, int lda,
                  const float *B, int ldb, float beta, float *C, int ldc);
void oracle_gemm_bias_act(int trans_a, int trans_b, int M, int N, int K, const float *A, int lda, const float *B, int ldb,
                          float beta, float *C, int ldc, const float *bias, int bias_mode, int activation);
void oracle_inner_product_forward(int batch, int inputs, int outputs, const float *x, const float *w, const float *bias,
                                  int activation, float *y);
void oracle_activation(float *p, size_t n, int activation);
int oracle_pooling_output_size(int in_size, int kernel, int pad, int stride, int ceil_mode);
void oracle_pooling2d_forward(int planes, int in_h, int in_w, const int kernel[2], const int stride[2], const int pad[2],
                              int ceil_mode, int mode_avg, int count_include_pad, const float *x, float *y);
void oracle_global_pooling_forward(int planes, int plane_size, int mode_avg, const float *x, float *y);
void oracle_elementwise_forward(size_t n, int op, float coef1, float coef2, int activation, const float *a, const float *b, float *c);
void oracle_softmax_forward(int rows, int classes, int inner, int log_mode, const float *x, float *y);
void oracle_batchnorm_inference(int batch, int features, int plane, float eps, const float *mean, const float *var,
                                const float *gamma, const float *beta, const float *x, float *y);
void oracle_fold_batchnorm(int channels_out, size_t weights_per_channel, float eps, const float *mean, const float *var,
                           const float *gamma, const float *beta, const float *w, const float *bias, float *w_out, float *bias_out);

#ifdef __cplusplus
}
#endif
#endif
