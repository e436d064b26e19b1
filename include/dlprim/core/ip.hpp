// dlprim::core inner-product primitive; drop-in for the forward half of the reference's
// include/dlprim/core/ip.hpp:19-45.
#pragma once
#include <dlprim/tensor.hpp>
#include <dlprim/context.hpp>
#include <memory>

namespace dlprim {
namespace core {

    struct IPSettings {
        int inputs = -1;              ///< number of input features
        int outputs = -1;             ///< number of output features
        int optimal_batch_size = -1;  ///< batch size the network is expected to run with
        DataType dtype = float_data;
    };

    class DLPRIM_API IPForward {
    public:
        virtual ~IPForward() {}
        ///  y[batch, outputs] = act(x[batch, inputs] * w[outputs, inputs]^T + bias)
        virtual void enqueue(Tensor &x, Tensor &w, Tensor *bias, Tensor &y, ExecutionContext const &e) = 0;
        /// Extension for inference: pack the weights once.
        virtual size_t packed_weights_size() const = 0;
        virtual void pack_weights(Tensor &w, Tensor &packed, ExecutionContext const &e) = 0;
        virtual void enqueue_packed(Tensor &x, Tensor &packed, Tensor *bias, Tensor &y, ExecutionContext const &e) = 0;
        virtual char const *kernel_name() const = 0;
        static std::unique_ptr<IPForward> create(Context &ctx, IPSettings const &config, bool bias,
                                                 StandardActivations activation = StandardActivations::identity);
    };

} // namespace core
} // namespace dlprim
