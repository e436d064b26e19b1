// Depthwise convolution launcher (depthwise.cu).
#pragma once
#include "common.cuh"

namespace dlp {
bool depthwise_supported(int ks_h, int ks_w, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w, int in_w);
dlp_status launch_depthwise(const float *x, const float *w, const float *bias, float *y, int batch, int channels, int H, int W,
                            int ks, int stride, int pad, int act, float factor, cudaStream_t stream);
}
