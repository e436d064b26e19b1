// dlprim::core convolution primitives: settings, algorithm selection, enqueue.
// Drop-in for the forward half of the reference's include/dlprim/core/conv.hpp:17-58.
#pragma once
#include <dlprim/tensor.hpp>
#include <dlprim/context.hpp>
#include <memory>
#include <string>

namespace dlprim {
namespace core {

    struct Conv2DSettings : public Convolution2DConfigBase {
        Conv2DSettings(Conv2DSettings const &) = default;
        Conv2DSettings(Convolution2DConfigBase const &v, Shape s, DataType dt) : Convolution2DConfigBase(v), shape(s), dtype(dt) {}
        Shape shape;                    ///< input shape; the batch is a hint rather than a requirement
        DataType dtype = float_data;
    };

    class DLPRIM_API Conv2DBase {
    public:
        virtual ~Conv2DBase() {}
        /// "gemm", "winograd" or "depthwise_separable"
        virtual char const *algo() const = 0;
        /// bytes of scratch that enqueue() needs
        virtual size_t workspace() { return 0; }
        static Shape get_output_shape(Convolution2DConfigBase const &config, Shape const &in);
    };

    class DLPRIM_API Conv2DForward : public Conv2DBase {
    public:
        virtual ~Conv2DForward() {}
        ///  y = factor * y + act(conv(x, w) + bias);  y is not read when factor == 0.
        virtual void enqueue(Tensor &x, Tensor &w, Tensor *bias, Tensor &y, Tensor &ws, float factor, ExecutionContext const &e) = 0;

        /// Extension for inference: pack the weights once, then run with an optional fused residual,
        ///  y = post_act( act(conv(x, w) + bias) + residual_scale * residual ).
        virtual size_t packed_weights_size() const = 0;
        virtual void pack_weights(Tensor &w, Tensor &packed, ExecutionContext const &e) = 0;
        ///  ws: optional scratch of workspace() bytes; with it a problem of few output tiles is cut along K
        ///  so that it still uses the whole GPU (null: no cut).
        virtual void enqueue_packed(Tensor &x, Tensor &packed, Tensor *bias, Tensor &y, Tensor *residual, float residual_scale,
                                    StandardActivations post_activation, Tensor *ws, ExecutionContext const &e) = 0;
        /// name of the kernel variant behind this object
        virtual char const *kernel_name() const = 0;

        static std::unique_ptr<Conv2DForward> create(Context &ctx, Conv2DSettings const &config, bool bias,
                                                     StandardActivations activation = StandardActivations::identity,
                                                     std::string const &algo = std::string());
    };

} // namespace core
} // namespace dlprim
