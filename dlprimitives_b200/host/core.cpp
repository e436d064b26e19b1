// dlprim::core::Conv2DForward, dlprim::core::IPForward and dlprim::gpu::GEMM over the C ABI.
// The algorithm choice, the kernels and the launches all live behind dlp_cuda.h; these classes only
// translate the reference's object model (tensors, contexts, exceptions) to it.
#include <dlprim/core/conv.hpp>
#include <dlprim/core/ip.hpp>
#include <dlprim/gpu/gemm.hpp>
#include "host_util.hpp"
#include <cuda_runtime.h>
#include <algorithm>
#include <cstring>

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
        desc_ = d;
        status_check(dlp_gemm_create(&d, &plan_));
        planned_[0] = M; planned_[1] = N; planned_[2] = K;
        ensure_ws(dlp_gemm_workspace(plan_));
    }
    ~GemmCuda() { dlp_gemm_destroy(plan_); }
    void gemm(int M, int N, int K, DeviceBuffer a, offset_type offset_a, int lda, DeviceBuffer b, offset_type offset_b, int ldb,
              DeviceBuffer c, offset_type offset_c, int ldc, DeviceBuffer bias, offset_type bias_offset, float beta, int size_of_c,
              ExecutionContext const &e) override
    {
        (void)size_of_c;   // the reference needs it for its split-K pre-scale pass; there is none here
        if(M > planned_[0] || N > planned_[1] || K > planned_[2]) grow(M, N, K);
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
    // Sizes at call time may exceed the ones the object was made for (the reference's kernels take any size):
    // the scratch for the packed B grows to fit.  Releasing the old scratch waits for the device, so this is the
    // one call that is not asynchronous; calls within the planned sizes never get here.
    void grow(int M, int N, int K)
    {
        dlp_gemm_desc d;
        d.trans_a = desc_.trans_a; d.trans_b = desc_.trans_b;
        d.m = std::max(M, planned_[0]); d.n = std::max(N, planned_[1]); d.k = std::max(K, planned_[2]);
        d.bias_mode = desc_.bias_mode; d.activation = desc_.activation; d.math_mode = desc_.math_mode;
        dlp_gemm_plan *bigger = nullptr;
        status_check(dlp_gemm_create(&d, &bigger));
        dlp_gemm_destroy(plan_);
        plan_ = bigger;
        desc_ = d;
        planned_[0] = d.m; planned_[1] = d.n; planned_[2] = d.k;
        ensure_ws(dlp_gemm_workspace(plan_));
    }
    dlp_gemm_desc desc_;
    int planned_[3];
    Context ctx_;
    dlp_gemm_plan *plan_ = nullptr;
    Tensor ws_;
    size_t ws_bytes_ = 0;
};
// The convolution behind the GEMM interface: gemm() is the call Conv2DForwardGEMM::enqueue makes in the reference.
class ConvGemmCuda : public GEMM {
public:
    ConvGemmCuda(Context &ctx, int M, int K, int kernel[2], int dilate[2], int padding[2], int stride[2], int groups, int src_channels,
                 int src_rows, int src_cols, int tgt_rows, int tgt_cols, int bias, StandardActivations act)
        : ctx_(ctx), plane_(tgt_rows * tgt_cols), src_rows_(src_rows), src_cols_(src_cols)
    {
        ctx.activate();
        DLPRIM_CHECK(bias == no_bias || bias == bias_M);            // a convolution's bias is per output channel
        DLPRIM_CHECK(K == src_channels * kernel[0] * kernel[1]);
        dlp_conv2d_desc d;
        memset(&d, 0, sizeof(d));
        d.channels_in = src_channels * groups;
        d.channels_out = M * groups;
        for(int i = 0; i < 2; i++) { d.kernel[i] = kernel[i]; d.stride[i] = stride[i]; d.dilate[i] = dilate[i]; d.pad[i] = padding[i]; }
        d.groups = groups;
        d.batch = 1;
        d.height = src_rows;
        d.width = src_cols;
        d.bias = bias == bias_M;
        d.activation = int(act);
        d.math_mode = DLP_MATH_AUTO;
        d.algo = "gemm";
        status_check(dlp_conv2d_fwd_create(&d, &plan_));
        d.algo = nullptr;
        desc_ = d;
        planned_batch_ = 1;
    }
    ~ConvGemmCuda() { dlp_conv2d_fwd_destroy(plan_); }
    void gemm(int M, int N, int K, DeviceBuffer a, offset_type offset_a, int lda, DeviceBuffer b, offset_type offset_b, int ldb, DeviceBuffer c,
              offset_type offset_c, int ldc, DeviceBuffer bias, offset_type bias_offset, float beta, int size_of_c,
              ExecutionContext const &e) override
    {
        (void)M; (void)K; (void)lda; (void)ldb; (void)ldc; (void)size_of_c;
        DLPRIM_CHECK(plane_ > 0 && N % plane_ == 0);
        const int batch = N / plane_;
        const size_t need = batch_workspace(batch);
        if(need > ws_bytes_) {
            ws_ = Tensor(ctx_, Shape(need), uint8_data);
            ws_bytes_ = need;
        }
        float const *bp = bias ? static_cast<float const *>(bias) + bias_offset : nullptr;
        status_check(dlp_conv2d_fwd_enqueue(plan_, static_cast<float const *>(b) + offset_b, static_cast<float const *>(a) + offset_a, bp,
                                            static_cast<float *>(c) + offset_c, ws_bytes_ ? ws_.device_ptr() : nullptr, ws_bytes_, beta, batch,
                                            src_rows_, src_cols_, e.stream_handle()));
    }
private:
    // the plan's workspace is sized for the batch it was made with; the part that lets small batches cut K grows with the batch
    size_t batch_workspace(int batch)
    {
        if(batch > planned_batch_) {
            dlp_conv2d_desc d = desc_;
            d.batch = batch;
            d.algo = "gemm";
            dlp_conv2d_plan *bigger = nullptr;
            status_check(dlp_conv2d_fwd_create(&d, &bigger));
            dlp_conv2d_fwd_destroy(plan_);
            plan_ = bigger;
            planned_batch_ = batch;
        }
        return dlp_conv2d_fwd_workspace(plan_);
    }
    Context ctx_;
    dlp_conv2d_plan *plan_ = nullptr;
    dlp_conv2d_desc desc_;
    int plane_, src_rows_, src_cols_;
    int planned_batch_ = 0;
    Tensor ws_;
    size_t ws_bytes_ = 0;
};
} // namespace

std::unique_ptr<GEMM> GEMM::get_optimal_gemm(Context &ctx, DataType dtype, bool trans_a, bool trans_b, int M, int N, int K, int bias,
                                             StandardActivations act, int im2col_chan)
{
    if(dtype != float_data) throw NotImplementedError("Only float32 GEMM is implemented");
    if(im2col_chan != 0) throw NotImplementedError("a convolution GEMM comes from get_optimal_conv_gemm, which knows the geometry");
    return std::unique_ptr<GEMM>(new GemmCuda(ctx, trans_a, trans_b, M, N, K, bias, act));
}

std::unique_ptr<GEMM> GEMM::get_optimal_conv_gemm(Context &ctx, DataType dtype, GemmOpMode op_mode, bool trans_a, bool trans_b, int M, int N,
                                                  int K, int kernel[2], int dilate[2], int padding[2], int stride[2], int groups,
                                                  int src_channels, int src_rows, int src_cols, int tgt_rows, int tgt_cols, int bias,
                                                  StandardActivations act, int im2col_chan)
{
    (void)N;
    if(dtype != float_data) throw NotImplementedError("Only float32 GEMM is implemented");
    if(op_mode != GemmOpMode::forward) throw NotImplementedError("only the forward convolution GEMM is implemented");
    // the forward call of the reference: filters as given, the image operand "transposed" (src/core/conv.cpp:94-96)
    DLPRIM_CHECK(!trans_a && trans_b);
    DLPRIM_CHECK(im2col_chan == 0 || im2col_chan == tgt_rows * tgt_cols);
    return std::unique_ptr<GEMM>(new ConvGemmCuda(ctx, M, K, kernel, dilate, padding, stride, groups, src_channels, src_rows, src_cols,
                                                  tgt_rows, tgt_cols, bias, act));
}

// One launch for the batch (plus the launch that packs every B); the scratch for the packed operands is taken from and
// returned to the stream's memory pool in stream order, so the call neither blocks nor outlives its memory.
void GEMM::batch_sgemm(DataType dt, bool trans_a, bool trans_b, int Batch, int M, int N, int K, DeviceBuffer a, offset_type offset_a,
                       int batch_stride_a, int lda, DeviceBuffer b, offset_type offset_b, int batch_stride_b, int ldb, DeviceBuffer c,
                       offset_type offset_c, int batch_stride_c, int ldc, float beta, ExecutionContext const &e)
{
    if(dt != float_data) throw NotImplementedError("Only float32 GEMM is implemented");
    dlp_gemm_desc d;
    d.trans_a = trans_a; d.trans_b = trans_b;
    d.m = M; d.n = N; d.k = K;
    d.bias_mode = no_bias;
    d.activation = int(StandardActivations::identity);
    d.math_mode = DLP_MATH_AUTO;
    dlp_gemm_plan *plan = nullptr;
    status_check(dlp_gemm_create(&d, &plan));
    const size_t bytes = dlp_gemm_batched_workspace(plan, Batch);
    cudaStream_t stream = static_cast<cudaStream_t>(e.stream_handle());
    void *ws = nullptr;
    cudaError_t err = bytes ? cudaMallocAsync(&ws, bytes, stream) : cudaSuccess;
    dlp_status st = DLP_OK;
    if(err == cudaSuccess)
        st = dlp_gemm_batched_enqueue(plan, Batch, M, N, K, static_cast<float const *>(a) + offset_a, batch_stride_a, lda,
                                      static_cast<float const *>(b) + offset_b, batch_stride_b, ldb, static_cast<float *>(c) + offset_c,
                                      batch_stride_c, ldc, beta, ws, bytes, e.stream_handle());
    if(ws) cudaFreeAsync(ws, stream);
    dlp_gemm_destroy(plan);
    host::cuda_check(err, "cudaMallocAsync");
    status_check(st);
}

} // namespace gpu
} // namespace dlprim
