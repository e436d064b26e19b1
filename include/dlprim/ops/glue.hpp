// The bandwidth-bound operators an inference graph needs between convolutions, forward only:
// Pooling2D, GlobalPooling, Elementwise, Activation, Softmax, BatchNorm (inference form), and the
// alias generators Flatten / Squeeze / Reshape.  Options follow the reference's JSON schema
// (docs/network_json_format.md); the semantics follow its CPU operators, cited per class.
#pragma once
#include <dlprim/operator.hpp>

namespace dlprim {

/// src/ops/pooling.cpp:19-38,282-329
class DLPRIM_API Pooling2D : public Operator {
public:
    struct Config {
        enum Mode { max = 0, avg = 1 } mode = max;
        int kernel[2] = {1, 1};
        int stride[2] = {1, 1};
        int pad[2] = {0, 0};
        bool ceil_mode = false;
        bool count_include_pad = false;
        static Config from_json(json::value const &v);
    };
    Pooling2D(Context &ctx, Config const &cfg) : Operator(ctx), config_(cfg) {}
    char const *operator_type() const override { return "Pooling2D"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
private:
    Shape calc_shape(Shape const &in) const;
    Config config_;
};

/// include/dlprim/ops/pooling.hpp:17-24, src/ops/pooling.cpp:427-450 (the default mode is max)
class DLPRIM_API GlobalPooling : public Operator {
public:
    struct Config {
        enum Mode { max = 0, avg = 1 } mode = max;
        static Config from_json(json::value const &v);
    };
    GlobalPooling(Context &ctx, Config const &cfg) : Operator(ctx), config_(cfg) {}
    char const *operator_type() const override { return "GlobalPooling"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
private:
    Config config_;
};

/// src/ops/elementwise.cpp:19-35,517-559; operands must have the same shape on this path
class DLPRIM_API Elementwise : public Operator {
public:
    struct Config {
        enum Operation { elementwise_sum = 0, elementwise_prod = 1, elementwise_max = 2 } op = elementwise_sum;
        float coeff[2] = {1.0f, 1.0f};
        StandardActivations activation = StandardActivations::identity;
        static Config from_json(json::value const &v);
    };
    Elementwise(Context &ctx, Config const &cfg) : Operator(ctx), config_(cfg) {}
    char const *operator_type() const override { return "Elementwise"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
    Config const &config() const { return config_; }
private:
    Config config_;
};

/// src/ops/activation.cpp:18-23,53-110
class DLPRIM_API Activation : public Operator {
public:
    struct Config {
        StandardActivations activation = StandardActivations::identity;
        static Config from_json(json::value const &v);
    };
    Activation(Context &ctx, Config const &cfg) : Operator(ctx), config_(cfg) {}
    char const *operator_type() const override { return "Activation"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
    Config const &config() const { return config_; }
private:
    Config config_;
};

/// src/ops/softmax.cpp:39-44,189-222
class DLPRIM_API Softmax : public Operator {
public:
    struct Config {
        bool log = false;
        static Config from_json(json::value const &v);
    };
    Softmax(Context &ctx, Config const &cfg) : Operator(ctx), config_(cfg) {}
    char const *operator_type() const override { return "Softmax"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
private:
    Config config_;
};

/// Inference form only (running statistics): src/ops/batch_normalization.cpp:25-57,192-228.
/// Parameters in order: mean, variance, then gamma, beta when affine.
class DLPRIM_API BatchNorm : public Operator {
public:
    struct Config {
        int features = -1;
        float eps = 1e-5f;
        float momentum = 0.1f;
        bool affine = true;
        bool use_global_stats = false;
        static Config from_json(json::value const &v);
    };
    BatchNorm(Context &ctx, Config const &cfg) : Operator(ctx), config_(cfg) {}
    char const *operator_type() const override { return "BatchNorm"; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                 ExecutionContext const &ctx) override;
    Config const &config() const { return config_; }
private:
    Config config_;
};

/// Alias generators: the output shares the input's memory, no kernel runs
/// (include/dlprim/ops/reshape.hpp:17-105).
class DLPRIM_API ReshapeBase : public Operator {
public:
    ReshapeBase(Context &ctx) : Operator(ctx) {}
    bool alias_generator() override { return true; }
    void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &workspace) override;
    void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) override;
    void forward(std::vector<Tensor> &, std::vector<Tensor> &, std::vector<Tensor> &, Tensor &, ExecutionContext const &) override {}
    virtual Shape new_shape(Shape const &in) = 0;
};
class DLPRIM_API Flatten : public ReshapeBase {
public:
    Flatten(Context &ctx) : ReshapeBase(ctx) {}
    char const *operator_type() const override { return "Flatten"; }
    Shape new_shape(Shape const &in) override { return Shape(in[0], in.size_no_batch()); }
};
class DLPRIM_API Squeeze : public ReshapeBase {
public:
    Squeeze(Context &ctx) : ReshapeBase(ctx) {}
    char const *operator_type() const override { return "Squeeze"; }
    Shape new_shape(Shape const &in) override { return in.squeeze(); }
};
class DLPRIM_API Reshape : public ReshapeBase {
public:
    Reshape(Context &ctx, std::vector<int> const &dims) : ReshapeBase(ctx), dims_(dims) {}
    char const *operator_type() const override { return "Reshape"; }
    Shape new_shape(Shape const &in) override;
private:
    std::vector<int> dims_;
};

} // namespace dlprim
