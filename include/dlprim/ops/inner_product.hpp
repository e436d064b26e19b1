// InnerProduct operator (inference):  y[B, outputs] = act(x[B, inputs] * W[outputs, inputs]^T + b).
// Same options and shapes as the reference's operator (include/dlprim/ops/inner_product.hpp:16-72,
// src/ops/inner_product.cpp:24-159).
#pragma once
#include <dlprim/operator.hpp>
#include <dlprim/core/ip.hpp>

namespace dlprim {

struct DLPRIM_API InnerProductConfig {
    int inputs = -1;    ///< -1: deduced from the input shape at setup
    int outputs = -1;
    bool bias = true;
    StandardActivations activation = StandardActivations::identity;
    static InnerProductConfig from_json(json::value const &v);
};

class DLPRIM_API InnerProduct : public Operator {
public:
    InnerProduct(Context &ctx, InnerProductConfig const &cfg);
    ~InnerProduct();
    char const *operator_type() const override { return "InnerProduct"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters,
               size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
    void parameters_changed() override { packed_valid_ = false; }
    void cache_packed_parameters(bool v) override { cache_packed_ = v; packed_valid_ = false; }
    InnerProductConfig const &config() const { return config_; }
    char const *kernel_name() const { return ip_ ? ip_->kernel_name() : ""; }
private:
    InnerProductConfig config_;
    DataType dtype_ = float_data;
    std::unique_ptr<core::IPForward> ip_;
    bool cache_packed_ = false, packed_valid_ = false;
    Tensor packed_;
    void *packed_source_ = nullptr;
};

} // namespace dlprim
