// Operators of the inference path and the operator factory.
#include <dlprim/ops/conv2d.hpp>
#include <dlprim/ops/inner_product.hpp>
#include <dlprim/ops/glue.hpp>
#include <dlprim/json.hpp>
#include "host_util.hpp"

#include <functional>
#include <map>

namespace dlprim {
using host::status_check;

static StandardActivations activation_from_json(json::value const &v)
{
    return activation_from_name(v.get("activation", "identity"));
}
static TensorSpecs same_type(Shape const &s, TensorSpecs const &like) { return TensorSpecs(s, like.dtype()); }

// ================================================================================ Convolution2D
Convolution2DConfig Convolution2DConfig::from_json(json::value const &v)
{
    Convolution2DConfig cfg;
    cfg.channels_in = v.get("channels_in", cfg.channels_in);
    cfg.channels_out = v.get<int>("channels_out");
    utils::get_1dNd_from_json(v, "kernel", cfg.kernel, true);
    utils::get_1dNd_from_json(v, "stride", cfg.stride);
    utils::get_1dNd_from_json(v, "dilate", cfg.dilate);
    utils::get_1dNd_from_json(v, "pad", cfg.pad);
    cfg.groups = v.get("groups", cfg.groups);
    cfg.bias = v.get("bias", cfg.bias);
    cfg.activation = activation_from_json(v);
    cfg.fwd_algo = v.get("fwd_algo", cfg.fwd_algo);
    return cfg;
}

Convolution2D::Convolution2D(Context &ctx, Convolution2DConfig const &cfg) : Operator(ctx), config_(cfg)
{
    DLPRIM_CHECK(config_.channels_out > 0);
    DLPRIM_CHECK(config_.groups > 0);
    for(int i = 0; i < 2; i++) {
        DLPRIM_CHECK(config_.kernel[i] > 0);
        DLPRIM_CHECK(config_.stride[i] > 0);
        DLPRIM_CHECK(config_.dilate[i] > 0);
        DLPRIM_CHECK(config_.pad[i] >= 0);
    }
}
Convolution2D::~Convolution2D() {}

Shape Convolution2D::get_output_shape(Shape const &in) { return core::Conv2DBase::get_output_shape(config_, in); }

void Convolution2D::setup_algo(Shape const &in)
{
    core::Conv2DSettings cfg(config_, in, dtype_);
    conv_ = core::Conv2DForward::create(ctx_, cfg, config_.bias, config_.activation, config_.fwd_algo);
    in_shape_ = in;
    ws_size_ = conv_->workspace();
    packed_valid_ = false;
    size_t packed = conv_->packed_weights_size();
    packed_ = packed > 0 ? Tensor(ctx_, Shape(packed), uint8_data) : Tensor();
}

void Convolution2D::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &params, size_t &workspace)
{
    DLPRIM_CHECK(in.size() == 1);
    Shape in_shape = in[0].shape();
    DLPRIM_CHECK(in_shape.size() == 4);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 convolution is implemented");
    if(config_.channels_in == -1) config_.channels_in = int(in_shape[1]);
    DLPRIM_CHECK(config_.channels_in % config_.groups == 0);
    DLPRIM_CHECK(config_.channels_out % config_.groups == 0);
    Shape output_shape = get_output_shape(in_shape);
    out.assign({TensorSpecs(output_shape, dtype_)});
    params.clear();
    params.push_back(TensorSpecs(Shape(config_.channels_out, config_.channels_in / config_.groups, config_.kernel[0], config_.kernel[1]), dtype_));
    if(config_.bias) params.push_back(TensorSpecs(Shape(config_.channels_out), dtype_));
    setup_algo(in_shape);
    workspace = ws_size_;
}

void Convolution2D::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    out.assign({get_output_shape(in[0])});
    // the plan survives a smaller batch at the same height and width (src/ops/conv2d.cpp:200-209)
    if(!conv_ || in[0][0] > in_shape_[0] || in[0][2] != in_shape_[2] || in[0][3] != in_shape_[3]) setup_algo(in[0]);
    ws = ws_size_;
}

void Convolution2D::ensure_packed(Tensor &w, ExecutionContext const &e)
{
    if(packed_valid_ && packed_source_ == w.device_ptr()) return;
    conv_->pack_weights(w, packed_, e);
    packed_valid_ = true;
    packed_source_ = w.device_ptr();
}

void Convolution2D::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &parameters, Tensor &ws,
                            ExecutionContext const &ectx)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(out[0].shape() == get_output_shape(in[0].shape()));
    DLPRIM_CHECK(parameters.size() == (1u + unsigned(config_.bias)));
    DLPRIM_CHECK(parameters[0].shape() == Shape(config_.channels_out, config_.channels_in / config_.groups, config_.kernel[0], config_.kernel[1]));
    Tensor *bias = nullptr;
    if(config_.bias) {
        DLPRIM_CHECK(parameters[1].shape() == Shape(config_.channels_out));
        bias = &parameters[1];
    }
    DLPRIM_CHECK(conv_);
    if(cache_packed_ && conv_->packed_weights_size() > 0) {
        ensure_packed(parameters[0], ectx);
        conv_->enqueue_packed(in[0], packed_, bias, out[0], nullptr, 0.0f, StandardActivations::identity, &ws, ectx);
    }
    else
        conv_->enqueue(in[0], parameters[0], bias, out[0], ws, 0.0f, ectx);
}

void Convolution2D::forward_fused(Tensor &x, Tensor &y, std::vector<Tensor> &parameters, Tensor &ws, Tensor &residual, float residual_scale,
                                  StandardActivations post_activation, ExecutionContext const &ectx)
{
    DLPRIM_CHECK(conv_);
    DLPRIM_CHECK(y.shape() == get_output_shape(x.shape()));
    DLPRIM_CHECK(parameters.size() == (1u + unsigned(config_.bias)));
    Tensor *bias = config_.bias ? &parameters[1] : nullptr;
    if(conv_->packed_weights_size() > 0) {
        ensure_packed(parameters[0], ectx);
        conv_->enqueue_packed(x, packed_, bias, y, &residual, residual_scale, post_activation, &ws, ectx);
    }
    else
        conv_->enqueue_packed(x, parameters[0], bias, y, &residual, residual_scale, post_activation, &ws, ectx);
}

// ================================================================================ InnerProduct
InnerProductConfig InnerProductConfig::from_json(json::value const &v)
{
    InnerProductConfig cfg;
    cfg.inputs = v.get("inputs", cfg.inputs);
    cfg.outputs = v.get<int>("outputs");
    cfg.bias = v.get("bias", cfg.bias);
    cfg.activation = activation_from_json(v);
    return cfg;
}
InnerProduct::InnerProduct(Context &ctx, InnerProductConfig const &cfg) : Operator(ctx), config_(cfg)
{
    DLPRIM_CHECK(config_.outputs > 0);
}
InnerProduct::~InnerProduct() {}

void InnerProduct::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].shape().size() >= 2);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 inner product is implemented");
    if(config_.inputs == -1) config_.inputs = int(in[0].shape().size_no_batch());
    else DLPRIM_CHECK(config_.inputs == int(in[0].shape().size_no_batch()));
    out.assign({TensorSpecs(Shape(in[0].shape()[0], config_.outputs), dtype_)});
    parameters.clear();
    parameters.push_back(TensorSpecs(Shape(config_.outputs, config_.inputs), dtype_));
    if(config_.bias) parameters.push_back(TensorSpecs(Shape(config_.outputs), dtype_));
    core::IPSettings cfg;
    cfg.inputs = config_.inputs;
    cfg.outputs = config_.outputs;
    cfg.optimal_batch_size = int(in[0].shape()[0]);
    ip_ = core::IPForward::create(ctx_, cfg, config_.bias, config_.activation);
    size_t packed = ip_->packed_weights_size();
    packed_ = packed > 0 ? Tensor(ctx_, Shape(packed), uint8_data) : Tensor();
    packed_valid_ = false;
    ws = 0;
}
void InnerProduct::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].size() >= 2);
    DLPRIM_CHECK(int(in[0].size_no_batch()) == config_.inputs);
    out.assign({Shape(in[0][0], config_.outputs)});
    ws = 0;
}
void InnerProduct::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &parameters, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(in[0].shape().size() >= 2);
    DLPRIM_CHECK(int(in[0].shape().size_no_batch()) == config_.inputs);
    DLPRIM_CHECK(out[0].shape() == Shape(in[0].shape()[0], config_.outputs));
    DLPRIM_CHECK(parameters.size() == (1u + unsigned(config_.bias)));
    DLPRIM_CHECK(parameters[0].shape() == Shape(config_.outputs, config_.inputs));
    Tensor *bias = nullptr;
    if(config_.bias) {
        DLPRIM_CHECK(parameters[1].shape() == Shape(config_.outputs));
        bias = &parameters[1];
    }
    DLPRIM_CHECK(ip_);
    if(cache_packed_ && ip_->packed_weights_size() > 0) {
        if(!packed_valid_ || packed_source_ != parameters[0].device_ptr()) {
            ip_->pack_weights(parameters[0], packed_, e);
            packed_valid_ = true;
            packed_source_ = parameters[0].device_ptr();
        }
        ip_->enqueue_packed(in[0], packed_, bias, out[0], e);
    }
    else
        ip_->enqueue(in[0], parameters[0], bias, out[0], e);
}

// ================================================================================ Pooling2D
Pooling2D::Config Pooling2D::Config::from_json(json::value const &v)
{
    Config cfg;
    std::string mode = v.get("mode", "max");
    if(mode == "max") cfg.mode = max;
    else if(mode == "avg") cfg.mode = avg;
    else throw ValidationError("Invalid pooling mode " + mode);
    utils::get_1dNd_from_json(v, "kernel", cfg.kernel, true);
    utils::get_1dNd_from_json(v, "stride", cfg.stride);
    utils::get_1dNd_from_json(v, "pad", cfg.pad);
    cfg.ceil_mode = v.get("ceil_mode", cfg.ceil_mode);
    cfg.count_include_pad = v.get("count_include_pad", cfg.count_include_pad);
    return cfg;
}
Shape Pooling2D::calc_shape(Shape const &in) const
{
    DLPRIM_CHECK(in.size() == 4);
    int oh = 0, ow = 0;
    status_check(dlp_pooling2d_output_shape(int(in[2]), int(in[3]), config_.kernel, config_.stride, config_.pad, config_.ceil_mode, &oh, &ow));
    return Shape(in[0], in[1], oh, ow);
}
void Pooling2D::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 pooling is implemented");
    out.assign({same_type(calc_shape(in[0].shape()), in[0])});
    p.clear();
    ws = 0;
}
void Pooling2D::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    out.assign({calc_shape(in[0])});
    ws = 0;
}
void Pooling2D::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(out[0].shape() == calc_shape(in[0].shape()));
    Shape s = in[0].shape();
    status_check(dlp_pooling2d_fwd(in[0].device_data<float>(), out[0].device_data<float>(), int(s[0] * s[1]), int(s[2]), int(s[3]),
                                   config_.kernel, config_.stride, config_.pad, config_.ceil_mode, int(config_.mode),
                                   config_.count_include_pad, e.stream_handle()));
}

// ================================================================================ GlobalPooling
GlobalPooling::Config GlobalPooling::Config::from_json(json::value const &v)
{
    Config cfg;
    std::string mode = v.get("mode", "max");
    if(mode == "max") cfg.mode = max;
    else if(mode == "avg") cfg.mode = avg;
    else throw ValidationError("Invalid pooling mode " + mode);
    return cfg;
}
void GlobalPooling::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].shape().size() == 4);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 pooling is implemented");
    out.assign({same_type(Shape(in[0].shape()[0], in[0].shape()[1], 1, 1), in[0])});
    p.clear();
    ws = 0;
}
void GlobalPooling::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].size() == 4);
    out.assign({Shape(in[0][0], in[0][1], 1, 1)});
    ws = 0;
}
void GlobalPooling::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    Shape s = in[0].shape();
    DLPRIM_CHECK(s.size() == 4);
    DLPRIM_CHECK(out[0].shape() == Shape(s[0], s[1], 1, 1));
    status_check(dlp_global_pooling_fwd(in[0].device_data<float>(), out[0].device_data<float>(), int(s[0] * s[1]), int(s[2] * s[3]),
                                        int(config_.mode), e.stream_handle()));
}

// ================================================================================ Elementwise
Elementwise::Config Elementwise::Config::from_json(json::value const &v)
{
    Config cfg;
    std::string op = v.get("operation", "sum");
    if(op == "sum") cfg.op = elementwise_sum;
    else if(op == "prod") cfg.op = elementwise_prod;
    else if(op == "max") cfg.op = elementwise_max;
    else throw ValidationError("Unsupported Elementwise operation " + op);
    cfg.coeff[0] = v.get("coef1", 1.0f);
    cfg.coeff[1] = v.get("coef2", 1.0f);
    cfg.activation = activation_from_json(v);
    return cfg;
}
void Elementwise::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 2);
    DLPRIM_CHECK(in[0].dtype() == in[1].dtype());
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 elementwise is implemented");
    if(in[0].shape() != in[1].shape()) throw NotImplementedError("Elementwise with broadcasting is outside the inference hot path");
    out.assign({in[0]});
    p.clear();
    ws = 0;
}
void Elementwise::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 2);
    if(in[0] != in[1]) throw NotImplementedError("Elementwise with broadcasting is outside the inference hot path");
    out.assign({in[0]});
    ws = 0;
}
void Elementwise::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 2);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(in[0].shape() == in[1].shape());
    DLPRIM_CHECK(out[0].shape() == in[0].shape());
    status_check(dlp_elementwise_fwd(in[0].device_data<float>(), in[1].device_data<float>(), out[0].device_data<float>(),
                                     in[0].shape().total_size(), int(config_.op), config_.coeff[0], config_.coeff[1],
                                     int(config_.activation), e.stream_handle()));
}

// ================================================================================ Activation
Activation::Config Activation::Config::from_json(json::value const &v)
{
    Config cfg;
    cfg.activation = activation_from_json(v);
    return cfg;
}
void Activation::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 activation is implemented");
    out.assign({in[0]});
    p.clear();
    ws = 0;
}
void Activation::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    out.assign({in[0]});
    ws = 0;
}
void Activation::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(in[0].shape() == out[0].shape());
    status_check(dlp_activation_fwd(in[0].device_data<float>(), out[0].device_data<float>(), in[0].shape().total_size(),
                                    int(config_.activation), e.stream_handle()));
}

// ================================================================================ Softmax
Softmax::Config Softmax::Config::from_json(json::value const &v)
{
    Config cfg;
    cfg.log = v.get("log", false);
    return cfg;
}
void Softmax::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].shape().size() >= 2);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 softmax is implemented");
    out.assign({in[0]});
    p.clear();
    ws = 0;
}
void Softmax::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].size() >= 2);
    out.assign({in[0]});
    ws = 0;
}
void Softmax::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(in[0].shape() == out[0].shape());
    Shape s = in[0].shape();
    size_t inner = 1;
    for(int i = 2; i < s.size(); i++) inner *= s[i];
    status_check(dlp_softmax_fwd(in[0].device_data<float>(), out[0].device_data<float>(), int(s[0]), int(s[1]), int(inner), config_.log,
                                 e.stream_handle()));
}

// ================================================================================ BatchNorm
BatchNorm::Config BatchNorm::Config::from_json(json::value const &v)
{
    Config cfg;
    cfg.features = v.get("features", cfg.features);
    cfg.eps = v.get("eps", cfg.eps);
    cfg.momentum = v.get("momentum", cfg.momentum);
    cfg.affine = v.get("affine", cfg.affine);
    cfg.use_global_stats = v.get("use_global_stats", cfg.use_global_stats);
    return cfg;
}
void BatchNorm::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].shape().size() >= 2);
    if(in[0].dtype() != float_data) throw NotImplementedError("Only float32 batch normalisation is implemented");
    if(config_.features == -1) config_.features = int(in[0].shape()[1]);
    DLPRIM_CHECK(config_.features == int(in[0].shape()[1]));
    if(mode_ == CalculationsMode::train) throw NotImplementedError("BatchNorm runs in inference form only on this path");
    out.assign({in[0]});
    p.clear();
    p.push_back(TensorSpecs(Shape(config_.features), float_data, false));
    p.push_back(TensorSpecs(Shape(config_.features), float_data, false));
    if(config_.affine) {
        p.push_back(TensorSpecs(Shape(config_.features), float_data));
        p.push_back(TensorSpecs(Shape(config_.features), float_data));
    }
    ws = 0;
}
void BatchNorm::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(in[0].size() >= 2);
    DLPRIM_CHECK(int(in[0][1]) == config_.features);
    out.assign({in[0]});
    ws = 0;
}
void BatchNorm::forward(std::vector<Tensor> &in, std::vector<Tensor> &out, std::vector<Tensor> &p, Tensor &, ExecutionContext const &e)
{
    DLPRIM_CHECK(in.size() == 1);
    DLPRIM_CHECK(out.size() == 1);
    DLPRIM_CHECK(in[0].shape() == out[0].shape());
    DLPRIM_CHECK(p.size() == (config_.affine ? 4u : 2u));
    Shape s = in[0].shape();
    size_t plane = 1;
    for(int i = 2; i < s.size(); i++) plane *= s[i];
    status_check(dlp_batchnorm_inference_fwd(in[0].device_data<float>(), out[0].device_data<float>(), int(s[0]), config_.features, int(plane),
                                             config_.eps, p[0].device_data<float>(), p[1].device_data<float>(),
                                             config_.affine ? p[2].device_data<float>() : nullptr,
                                             config_.affine ? p[3].device_data<float>() : nullptr, e.stream_handle()));
}

// ================================================================================ alias generators
void ReshapeBase::setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &p, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    out.assign({same_type(new_shape(in[0].shape()), in[0])});
    p.clear();
    ws = 0;
}
void ReshapeBase::reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &ws)
{
    DLPRIM_CHECK(in.size() == 1);
    out.assign({new_shape(in[0])});
    ws = 0;
}
Shape Reshape::new_shape(Shape const &in)
{
    // 0 keeps the input's dimension, a single -1 takes what is left
    std::vector<size_t> dims;
    size_t known = 1;
    int unknown = -1;
    for(size_t i = 0; i < dims_.size(); i++) {
        if(dims_[i] == 0) {
            DLPRIM_CHECK(int(i) < in.size());
            dims.push_back(in[int(i)]);
        }
        else if(dims_[i] == -1) {
            DLPRIM_CHECK(unknown == -1);
            unknown = int(i);
            dims.push_back(1);
            continue;
        }
        else {
            DLPRIM_CHECK(dims_[i] > 0);
            dims.push_back(size_t(dims_[i]));
        }
        known *= dims.back();
    }
    if(unknown >= 0) {
        DLPRIM_CHECK(known > 0 && in.total_size() % known == 0);
        dims[unknown] = in.total_size() / known;
    }
    Shape r = Shape::from_range(dims.begin(), dims.end());
    DLPRIM_CHECK(r.total_size() == in.total_size());
    return r;
}

// ================================================================================ factory
std::unique_ptr<Operator> create_by_name(Context &ctx, std::string const &name, json::value const &p)
{
    typedef std::function<Operator *(Context &, json::value const &)> Maker;
    static const std::map<std::string, Maker> makers = {
        {"Convolution2D", [](Context &c, json::value const &v) -> Operator * { return new Convolution2D(c, Convolution2DConfig::from_json(v)); }},
        {"InnerProduct", [](Context &c, json::value const &v) -> Operator * { return new InnerProduct(c, InnerProductConfig::from_json(v)); }},
        {"Pooling2D", [](Context &c, json::value const &v) -> Operator * { return new Pooling2D(c, Pooling2D::Config::from_json(v)); }},
        {"GlobalPooling", [](Context &c, json::value const &v) -> Operator * { return new GlobalPooling(c, GlobalPooling::Config::from_json(v)); }},
        {"Elementwise", [](Context &c, json::value const &v) -> Operator * { return new Elementwise(c, Elementwise::Config::from_json(v)); }},
        {"Activation", [](Context &c, json::value const &v) -> Operator * { return new Activation(c, Activation::Config::from_json(v)); }},
        {"Softmax", [](Context &c, json::value const &v) -> Operator * { return new Softmax(c, Softmax::Config::from_json(v)); }},
        {"BatchNorm", [](Context &c, json::value const &v) -> Operator * { return new BatchNorm(c, BatchNorm::Config::from_json(v)); }},
        {"Flatten", [](Context &c, json::value const &) -> Operator * { return new Flatten(c); }},
        {"Squeeze", [](Context &c, json::value const &) -> Operator * { return new Squeeze(c); }},
        {"Reshape", [](Context &c, json::value const &v) -> Operator * { return new Reshape(c, v.get<std::vector<int> >("dims")); }},
    };
    auto it = makers.find(name);
    if(it == makers.end()) throw ValidationError("Unknown operator " + name);
    return std::unique_ptr<Operator>(it->second(ctx, p));
}

} // namespace dlprim
