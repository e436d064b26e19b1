// Operator: the layer interface Net drives -- setup / reshape / forward, as in the reference's
// include/dlprim/operator.hpp:22-178 (inference subset: there is no backward on this path).
#pragma once
#include <dlprim/definitions.hpp>
#include <dlprim/tensor.hpp>
#include <dlprim/context.hpp>
#include <memory>
#include <string>
#include <vector>

namespace dlprim {
namespace json { class value; }

class DLPRIM_API Operator {
public:
    Operator(Context const &ctx) : ctx_(ctx), mode_(CalculationsMode::predict) {}
    virtual ~Operator() {}
    Operator(Operator const &) = delete;
    void operator=(Operator const &) = delete;

    virtual char const *operator_type() const = 0;
    virtual void mode(CalculationsMode mode) { mode_ = mode; }
    virtual CalculationsMode mode() { return mode_; }
    /// true for operators whose output shares the input's memory (Flatten/Reshape/Squeeze)
    virtual bool alias_generator() { return false; }

    /// Fix shapes: fills the output specs, the parameter specs and the workspace size in bytes.
    virtual void setup(std::vector<TensorSpecs> const &in, std::vector<TensorSpecs> &out, std::vector<TensorSpecs> &parameters,
                       size_t &workspace) = 0;
    /// New input shapes: fills the output shapes and the workspace size.
    virtual void reshape(std::vector<Shape> const &in, std::vector<Shape> &out, size_t &workspace) = 0;
    virtual void forward(std::vector<Tensor> &input, std::vector<Tensor> &output, std::vector<Tensor> &parameters, Tensor &workspace,
                         ExecutionContext const &ctx) = 0;

    /// Inference extension: the parameter tensors changed on the device (called by Net after an
    /// upload); operators that keep a packed copy of their weights rebuild it on the next forward.
    virtual void parameters_changed() {}
    /// Inference extension: keep packed weights between calls (Net turns this on in predict mode).
    virtual void cache_packed_parameters(bool) {}
protected:
    Context ctx_;
    CalculationsMode mode_;
};

DLPRIM_API std::unique_ptr<Operator> create_by_name(Context &ctx, std::string const &name, json::value const &parameters);

} // namespace dlprim
