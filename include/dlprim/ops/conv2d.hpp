// Convolution2D operator (inference): JSON options, shape inference, parameter specs and dispatch to
// core::Conv2DForward.  Same options and shapes as the reference's operator
// (include/dlprim/ops/conv2d.hpp:18-100, src/ops/conv2d.cpp:27-237).
#pragma once
#include <dlprim/operator.hpp>
#include <dlprim/core/conv.hpp>

namespace dlprim {

struct DLPRIM_API Convolution2DConfig : public Convolution2DConfigBase {
    bool bias = true;
    StandardActivations activation = StandardActivations::identity;
    std::string fwd_algo = "auto";   ///< "auto", "gemm", "winograd" or "depthwise_separable"
    static Convolution2DConfig from_json(json::value const &v);
};

class DLPRIM_API Convolution2D : public Operator {
public:
    Convolution2D(Context &ctx, Convolution2DConfig const &cfg);
    ~Convolution2D();
    char const *operator_type() const override { return "Convolution2D"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters,
               size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
    void parameters_changed() override { packed_valid_ = false; }
    void cache_packed_parameters(bool v) override { cache_packed_ = v; packed_valid_ = false; }

    /// Inference extension used by Net's graph optimiser: this convolution followed by
    /// Elementwise("sum", coef2 = residual_scale, activation = post_activation) in one kernel.
    void forward_fused(Tensor &x, Tensor &y, std::vector<Tensor> &parameters, Tensor &workspace, Tensor &residual,
                       float residual_scale, StandardActivations post_activation, ExecutionContext const &ctx);

    Convolution2DConfig const &config() const { return config_; }
    Shape get_output_shape(Shape const &in);
    /// "gemm", "winograd" or "depthwise_separable"; valid after setup().
    char const *algo() const { return conv_ ? conv_->algo() : ""; }
    char const *kernel_name() const { return conv_ ? conv_->kernel_name() : ""; }
private:
    void setup_algo(Shape const &in);
    void ensure_packed(Tensor &w, ExecutionContext const &e);
    Convolution2DConfig config_;
    DataType dtype_ = float_data;
    Shape in_shape_;
    size_t ws_size_ = 0;
    std::unique_ptr<core::Conv2DForward> conv_;
    bool cache_packed_ = false, packed_valid_ = false;
    Tensor packed_;
    void *packed_source_ = nullptr;
};

} // namespace dlprim
