// Plan objects behind the opaque handles of dlp_cuda.h (internal to the library).
#pragma once
#include "contraction.cuh"
#include <string>

using dlp::KTap;
using dlp::TcPacked;

enum ConvKernel { CK_TC, CK_FFMA, CK_DEPTHWISE, CK_WINOGRAD };

struct dlp_conv2d_plan {
    dlp_conv2d_desc d;
    std::string algo;        // what Conv2DBase::algo() reports
    std::string kernel;
    ConvKernel kind;
    int out_h, out_w;
    int k;                   // Cin/groups * KH * KW
    bool strided_a;          // 1x1, stride 1, no padding: the taps are a plain stride
    bool winograd_tc = false; // CK_WINOGRAD: the sixteen products run on the tensor cores (winograd_tc.cu), not as fp32 FMA
    bool tapblock;           // tensor-core path with channels in blocks of 32: K runs (channel block, tap, channel)
    bool rowtaps = false;    // tensor-core path for wide kernels over few channels: K runs (channel, kernel row, column padded to 8)
    TcPacked packed;
    KTap *ktab = nullptr;    // device, k_pad entries (gather mode)
    int *tap_dydx = nullptr; // device, one entry per kernel tap
    int num_taps = 0;
    int device = 0;
};

struct dlp_gemm_plan {
    dlp_gemm_desc d;
    bool use_tc;
    std::string kernel;
};

struct dlp_ip_plan {
    dlp_ip_desc d;
    bool use_tc;
    TcPacked packed;
    std::string kernel;
};

