// dlprim::core::Conv2DForward, dlprim::core::IPForward and dlprim::gpu::GEMM over the C ABI.
// The algorithm choice, the kernels and the launches all live behind dlp_cuda.h; these classes only
// translate the reference's object model (tensors, contexts, exceptions) to it.
#include <dlprim/core/conv.hpp>
#include <dlprim/core/ip.hpp>
#include <dlprim/gpu/gemm.hpp>
#include "host_util.hpp"
#include <cuda_runtime.h>

namespace dlprim {
using host::status_check;

namespace core {

Shape Conv2DBase::get_output_shape(Convolution2DConfigBase const &config, Shape const &in)
{
    DLPRIM_CHECK(in.size() == 4);
    DLPRIM_CHECK(int(in[1]) == config.channels_in);
    int ihw[2] = {int(in[2]), int(in[3])};
    int ohw[2];
    for(int i = 0; i < 2; i++)
        ohw[i] = (ihw[i] + 2 * config.pad[i] - config.dilate[i] * (config.kernel[i] - 1) - 1) / config.stride[i] + 1;
    DLPRIM_CHECK(ohw[0] > 0);
    DLPRIM_CHECK(ohw[1] > 0);
    return Shape(in[0], config.channels_out, ohw[0], ohw[1]);
}

namespace {
class Conv2DForwardCuda : public Conv2DForward {
public:
    Conv2DForwardCuda(Context &ctx, Conv2DSettings const &cfg, bool bias, StandardActivations act, std::string const &algo)
        : cfg_(cfg), bias_(bias)
    {
        if(cfg.dtype != float_data) throw NotImplementedError("Only float32 convolution is implemented");
        DLPRIM_CHECK(cfg.shape.size() == 4);
        ctx.activate();
        dlp_conv2d_desc d;
        d.channels_in = cfg.channels_in;
        d.channels_out = cfg.channels_out;
        for(int i = 0; i < 2; i++) {
            d.kernel[i] = cfg.kernel[i];
            d.stride[i] = cfg.stride[i];
            d.dilate[i] = cfg.dilate[i];
            d.pad[i] = cfg.pad[i];
        }
        d.groups = cfg.groups;
        d.batch = int(cfg.shape[0]);
        d.height = int(cfg.shape[2]);
        d.width = int(cfg.shape[3]);
        d.bias = bias ? 1 : 0;
        d.activation = int(act);
        d.algo = algo.c_str();
        d.math_mode = DLP_MATH_AUTO;
        status_check(dlp_conv2d_fwd_create(&d, &plan_));
    }
    ~Conv2DForwardCuda() { dlp_conv2d_fwd_destroy(plan_); }
    char const *algo() const override { return dlp_conv2d_fwd_algo(plan_); }
    char const *kernel_name() const override { return dlp_conv2d_fwd_kernel(plan_); }
    size_t workspace() override { return dlp_conv2d_fwd_workspace(plan_); }
    size_t packed_weights_size() const override { return dlp_conv2d_fwd_packed_bytes(plan_); }

    void enqueue(Tensor &x, Tensor &w, Tensor *bias, Tensor &y, Tensor &ws, float factor, ExecutionContext const &e) override
    {
        check(x, y, bias);
        status_check(dlp_conv2d_fwd_enqueue(plan_, x.device_data<float>(), w.device_data<float>(), bias ? bias->device_data<float>() : nullptr,
                                            y.device_data<float>(), ws.memory_size() ? ws.device_ptr() : nullptr, ws.memory_size(), factor,
                                            int(x.shape()[0]), int(x.shape()[2]), int(x.shape()[3]), e.stream_handle()));
    }
    void pack_weights(Tensor &w, Tensor &packed, ExecutionContext const &e) override
    {
        DLPRIM_CHECK(packed.memory_size() >= packed_weights_size());
        status_check(dlp_conv2d_fwd_prepack(plan_, w.device_data<float>(), packed.device_ptr(), e.stream_handle()));
    }
    void enqueue_packed(Tensor &x, Tensor &packed, Tensor *bias, Tensor &y, Tensor *residual, float residual_scale,
                        StandardActivations post_activation, Tensor *ws, ExecutionContext const &e) override
    {
        check(x, y, bias);
        if(residual) DLPRIM_CHECK(residual->shape() == y.shape());
        const size_t ws_bytes = ws ? ws->memory_size() : 0;
        status_check(dlp_conv2d_fwd_enqueue_packed(plan_, x.device_data<float>(), packed.device_ptr(),
                                                   bias ? bias->device_data<float>() : nullptr, y.device_data<float>(),
                                                   ws_bytes ? ws->device_ptr() : nullptr, ws_bytes, 0.0f,
                                                   residual ? residual->device_data<float>() : nullptr, residual_scale,
                                                   int(post_activation), int(x.shape()[0]), int(x.shape()[2]), int(x.shape()[3]),
                                                   e.stream_handle()));
    }
private:
    void check(Tensor &x, Tensor &y, Tensor *bias)
    {
        DLPRIM_CHECK(x.shape().size() == 4);
        DLPRIM_CHECK(y.shape() == get_output_shape(cfg_, x.shape()));
        DLPRIM_CHECK(bias_ == (bias != nullptr));
    }
    Conv2DSettings cfg_;
    bool bias_;
    dlp_conv2d_plan *plan_ = nullptr;
};

class IPForwardCuda : public IPForward {
public:
    IPForwardCuda(Context &ctx, IPSettings const &cfg, bool bias, StandardActivations act) : cfg_(cfg), bias_(bias)
    {
        if(cfg.dtype != float_data) throw NotImplementedError("Only float32 inner product is implemented");
        ctx.activate();
        dlp_ip_desc d;
        d.inputs = cfg.inputs;
        d.outputs = cfg.outputs;
        d.optimal_batch_size = cfg.optimal_batch_size;
        d.bias = bias ? 1 : 0;
        d.activation = int(act);
        d.math_mode = DLP_MATH_AUTO;
        status_check(dlp_ip_fwd_create(&d, &plan_));
        ws_bytes_ = dlp_ip_fwd_workspace(plan_);
        // IPForward::enqueue has no workspace argument in the reference interface: the scratch for the
        // per-call weight split belongs to this object.
        if(ws_bytes_ > 0) ws_ = Tensor(ctx, Shape(ws_bytes_), uint8_data);
    }
    ~IPForwardCuda() { dlp_ip_fwd_destroy(plan_); }
    char const *kernel_name() const override { return dlp_ip_fwd_kernel(plan_); }
    size_t packed_weights_size() const override { return dlp_ip_fwd_packed_bytes(plan_); }
    void enqueue(Tensor &x, Tensor &w, Tensor *bias, Tensor &y, ExecutionContext const &e) override
    {
        check(x, y, bias);
        status_check(dlp_ip_fwd_enqueue(plan_, x.device_data<float>(), w.device_data<float>(), bias ? bias->device_data<float>() : nullptr,
                                        y.device_data<float>(), ws_bytes_ ? ws_.device_ptr() : nullptr, ws_bytes_, int(x.shape()[0]),
                                        e.stream_handle()));
    }
    void pack_weights(Tensor &w, Tensor &packed, ExecutionContext const &e) override
    {
        DLPRIM_CHECK(packed.memory_size() >= packed_weights_size());
        status_check(dlp_ip_fwd_prepack(plan_, w.device_data<float>(), packed.device_ptr(), e.stream_handle()));
    }
    void enqueue_packed(Tensor &x, Tensor &packed, Tensor *bias, Tensor &y, ExecutionContext const &e) override
    {
        check(x, y, bias);
        status_check(dlp_ip_fwd_enqueue_packed(plan_, x.device_data<float>(), packed.device_ptr(), bias ? bias->device_data<float>() : nullptr,
                                               y.device_data<float>(), ws_bytes_ ? ws_.device_ptr() : nullptr, ws_bytes_, int(x.shape()[0]),
                                               e.stream_handle()));
    }
private:
    void check(Tensor &x, Tensor &y, Tensor *bias)
    {
        DLPRIM_CHECK(int(x.shape().size_no_batch()) == cfg_.inputs);
        DLPRIM_CHECK(y.shape().size() >= 2 && int(y.shape().size_no_batch()) == cfg_.outputs && y.shape()[0] == x.shape()[0]);
        DLPRIM_CHECK(bias_ == (bias != nullptr));
    }
    IPSettings cfg_;
    bool bias_;
    dlp_ip_plan *plan_ = nullptr;
    size_t ws_bytes_ = 0;
    Tensor ws_;
};
} // namespace

std::unique_ptr<Conv2DForward> Conv2DForward::create(Context &ctx, Conv2DSettings const &config, bool bias, StandardActivations activation,
                                                     std::string const &algo)
{
    return std::unique_ptr<Conv2DForward>(new Conv2DForwardCuda(ctx, config, bias, activation, algo));
}
std::unique_ptr<IPForward> IPForward::create(Context &ctx, IPSettings const &config, bool bias, StandardActivations activation)
{
    return std::unique_ptr<IPForward>(new IPForwardCuda(ctx, config, bias, activation));
}

} // namespace core

namespace gpu {
namespace {
class GemmCuda : public GEMM {
public:
    GemmCuda(Context &ctx, bool ta, bool tb, int M, int N, int K, int bias, StandardActivations act) : ctx_(ctx)
    {
        ctx.activate();
        dlp_gemm_desc d;
        d.trans_a = ta; d.trans_b = tb;
        d.m = M; d.n = N; d.k = K;
        d.bias_mode = bias;
        d.activation = int(act);
        d.math_mode = DLP_MATH_AUTO;
        status_check(dlp_gemm_create(&d, &plan_));
        ensure_ws(dlp_gemm_workspace(plan_));
    }
    ~GemmCuda() { dlp_gemm_destroy(plan_); }
    void gemm(int M, int N, int K, DeviceBuffer a, offset_type offset_a, int lda, DeviceBuffer b, offset_type offset_b, int ldb,
              DeviceBuffer c, offset_type offset_c, int ldc, DeviceBuffer bias, offset_type bias_offset, float beta, int size_of_c,
              ExecutionContext const &e) override
    {
        (void)size_of_c;   // the reference needs it for its split-K pre-scale pass; there is none here
        float const *bp = bias ? static_cast<float const *>(bias) + bias_offset : nullptr;
        status_check(dlp_gemm_enqueue(plan_, M, N, K, static_cast<float const *>(a) + offset_a, lda, static_cast<float const *>(b) + offset_b,
                                      ldb, static_cast<float *>(c) + offset_c, ldc, bp, beta, ws_bytes_ ? ws_.device_ptr() : nullptr, ws_bytes_,
                                      e.stream_handle()));
    }
    dlp_gemm_plan *plan() { return plan_; }
    void *ws_ptr() { return ws_bytes_ ? ws_.device_ptr() : nullptr; }
    size_t ws_bytes() const { return ws_bytes_; }
private:
    void ensure_ws(size_t bytes)
    {
        if(bytes > ws_bytes_) {
            ws_ = Tensor(ctx_, Shape(bytes), uint8_data);
            ws_bytes_ = bytes;
        }
    }
    Context ctx_;
    dlp_gemm_plan *plan_ = nullptr;
    Tensor ws_;
    size_t ws_bytes_ = 0;
};
} // namespace

std::unique_ptr<GEMM> GEMM::get_optimal_gemm(Context &ctx, DataType dtype, bool trans_a, bool trans_b, int M, int N, int K, int bias,
                                             StandardActivations act, int im2col_chan)
{
    if(dtype != float_data) throw NotImplementedError("Only float32 GEMM is implemented");
    DLPRIM_CHECK(im2col_chan == 0);   // the convolution path has its own entry point
    return std::unique_ptr<GEMM>(new GemmCuda(ctx, trans_a, trans_b, M, N, K, bias, act));
}

void GEMM::batch_sgemm(DataType dt, bool trans_a, bool trans_b, int Batch, int M, int N, int K, DeviceBuffer a, offset_type offset_a,
                       int batch_stride_a, int lda, DeviceBuffer b, offset_type offset_b, int batch_stride_b, int ldb, DeviceBuffer c,
                       offset_type offset_c, int batch_stride_c, int ldc, float beta, ExecutionContext const &e)
{
    if(dt != float_data) throw NotImplementedError("Only float32 GEMM is implemented");
    int dev = 0;
    host::cuda_check(cudaGetDevice(&dev), "cudaGetDevice");
    Context ctx(Context::cuda, 0, dev);
    GemmCuda g(ctx, trans_a, trans_b, M, N, K, no_bias, StandardActivations::identity);
    status_check(dlp_gemm_batched_enqueue(g.plan(), Batch, M, N, K, static_cast<float const *>(a) + offset_a, batch_stride_a, lda,
                                          static_cast<float const *>(b) + offset_b, batch_stride_b, ldb, static_cast<float *>(c) + offset_c,
                                          batch_stride_c, ldc, beta, g.ws_ptr(), g.ws_bytes(), e.stream_handle()));
    // the scratch of the temporary object must outlive the kernels it was handed to
    e.finish();
}

} // namespace gpu
} // namespace dlprim
