// Checker-side C binding over the reference library's own CPU context.
//
// Test infrastructure only.  It links against oracle/_ref/libdlprim_ref.so
// (the unmodified reference sources built with a null OpenCL header) and lets
// Python drive the reference's operators and Net on Context("cpu") through
// ctypes, so that the restatement in oracle.c and the CUDA path can both be
// compared with what the reference itself computes.  Nothing shipped links it.
#include <dlprim/context.hpp>
#include <dlprim/tensor.hpp>
#include <dlprim/operator.hpp>
#include <dlprim/net.hpp>
#include <dlprim/json.hpp>

#include <chrono>
#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

namespace {
    thread_local std::string g_err;

    struct RefOp {
        dlprim::Context ctx{"cpu"};
        std::unique_ptr<dlprim::Operator> op;
        std::vector<dlprim::TensorSpecs> in_specs, out_specs, par_specs;
        std::vector<dlprim::Tensor> in, out, par;
        dlprim::Tensor ws;
        size_t ws_size = 0;
    };
    struct RefNet {
        dlprim::Context ctx{"cpu"};
        std::unique_ptr<dlprim::Net> net;
    };

    dlprim::json::value parse_json(char const *text)
    {
        dlprim::json::value v;
        std::istringstream ss(text);
        int line = 0;
        if(!v.load(ss, true, &line))
            throw dlprim::ValidationError("JSON syntax error at line " + std::to_string(line));
        return v;
    }
    int write_shape(dlprim::Shape const &s, int *dims)
    {
        for(int i = 0; i < s.size(); i++)
            dims[i] = int(s[i]);
        return s.size();
    }
}

#define REF_GUARD_BEGIN try {
#define REF_GUARD_END(fail) } catch(std::exception const &e) { g_err = e.what(); return fail; }

extern "C" {

char const *ref_last_error() { return g_err.c_str(); }

/// Create one operator by its factory name (e.g. "Convolution2D") with JSON options and
/// run setup() for the given input shapes.  dims holds the shapes back to back.
void *ref_op_create(char const *type, char const *options_json, int n_in, int const *ranks, int const *dims)
{
    REF_GUARD_BEGIN
    std::unique_ptr<RefOp> h(new RefOp());
    dlprim::json::value opts = parse_json(options_json);
    h->op = dlprim::create_by_name(h->ctx, type, opts);
    int pos = 0;
    for(int i = 0; i < n_in; i++) {
        dlprim::Shape s = dlprim::Shape::from_range(dims + pos, dims + pos + ranks[i]);
        pos += ranks[i];
        h->in_specs.push_back(dlprim::TensorSpecs(s, dlprim::float_data));
    }
    h->op->setup(h->in_specs, h->out_specs, h->par_specs, h->ws_size);
    for(auto const &s : h->in_specs)  h->in.push_back(dlprim::Tensor(h->ctx, s.shape(), s.dtype()));
    for(auto const &s : h->out_specs) h->out.push_back(dlprim::Tensor(h->ctx, s.shape(), s.dtype()));
    for(auto const &s : h->par_specs) h->par.push_back(dlprim::Tensor(h->ctx, s.shape(), s.dtype()));
    if(h->ws_size > 0)
        h->ws = dlprim::Tensor(h->ctx, dlprim::Shape(h->ws_size), dlprim::uint8_data);
    return h.release();
    REF_GUARD_END(nullptr)
}
void ref_op_destroy(void *p) { delete static_cast<RefOp *>(p); }
int ref_op_num_outputs(void *p) { return int(static_cast<RefOp *>(p)->out_specs.size()); }
int ref_op_num_params(void *p) { return int(static_cast<RefOp *>(p)->par_specs.size()); }
int ref_op_output_shape(void *p, int i, int *dims) { return write_shape(static_cast<RefOp *>(p)->out_specs.at(i).shape(), dims); }
int ref_op_param_shape(void *p, int i, int *dims) { return write_shape(static_cast<RefOp *>(p)->par_specs.at(i).shape(), dims); }
unsigned long long ref_op_workspace(void *p) { return static_cast<RefOp *>(p)->ws_size; }

/// Copy inputs and parameters in, run Operator::forward on the CPU context, copy outputs out.
/// Returns the wall-clock seconds of forward() alone, or a negative value on error.
double ref_op_forward(void *p, float const *const *inputs, float const *const *params, float *const *outputs)
{
    REF_GUARD_BEGIN
    RefOp *h = static_cast<RefOp *>(p);
    for(size_t i = 0; i < h->in.size(); i++)
        memcpy(h->in[i].host_data(), inputs[i], h->in[i].memory_size());
    for(size_t i = 0; i < h->par.size(); i++)
        memcpy(h->par[i].host_data(), params[i], h->par[i].memory_size());
    dlprim::ExecutionContext e;
    auto t0 = std::chrono::steady_clock::now();
    h->op->forward(h->in, h->out, h->par, h->ws, e);
    auto t1 = std::chrono::steady_clock::now();
    for(size_t i = 0; i < h->out.size(); i++)
        memcpy(outputs[i], h->out[i].host_data(), h->out[i].memory_size());
    return std::chrono::duration<double>(t1 - t0).count();
    REF_GUARD_END(-1.0)
}

/// Build a Net on the CPU context from a JSON description; predict mode, setup() and reshape() done.
void *ref_net_create(char const *net_json)
{
    REF_GUARD_BEGIN
    std::unique_ptr<RefNet> h(new RefNet());
    h->net.reset(new dlprim::Net(h->ctx));
    h->net->mode(dlprim::CalculationsMode::predict);
    dlprim::json::value v = parse_json(net_json);
    h->net->load_from_json(v);
    h->net->setup();
    h->net->reshape();
    return h.release();
    REF_GUARD_END(nullptr)
}
void ref_net_destroy(void *p) { delete static_cast<RefNet *>(p); }
void ref_net_keep_intermediate(void *p, int keep) { static_cast<RefNet *>(p)->net->keep_intermediate_tensors(keep != 0); }

int ref_net_num_params(void *p) { return int(static_cast<RefNet *>(p)->net->params().size()); }
/// Name of the i-th parameter in map order; the buffer must hold n bytes.
int ref_net_param_name(void *p, int i, char *buf, int n)
{
    REF_GUARD_BEGIN
    auto &m = static_cast<RefNet *>(p)->net->params();
    auto it = m.begin();
    std::advance(it, i);
    snprintf(buf, n, "%s", it->first.c_str());
    return 0;
    REF_GUARD_END(-1)
}
int ref_net_param_shape(void *p, char const *name, int *dims)
{
    REF_GUARD_BEGIN
    return write_shape(static_cast<RefNet *>(p)->net->param(name).shape(), dims);
    REF_GUARD_END(-1)
}
int ref_net_set_param(void *p, char const *name, float const *data, unsigned long long count)
{
    REF_GUARD_BEGIN
    dlprim::Tensor &t = static_cast<RefNet *>(p)->net->param(name);
    if(t.shape().total_size() != count)
        throw dlprim::ValidationError(std::string("size mismatch for parameter ") + name);
    memcpy(t.host_data(), data, t.memory_size());
    return 0;
    REF_GUARD_END(-1)
}
int ref_net_tensor_shape(void *p, char const *name, int *dims)
{
    REF_GUARD_BEGIN
    return write_shape(static_cast<RefNet *>(p)->net->tensor(name).shape(), dims);
    REF_GUARD_END(-1)
}
int ref_net_set_tensor(void *p, char const *name, float const *data, unsigned long long count)
{
    REF_GUARD_BEGIN
    dlprim::Tensor &t = static_cast<RefNet *>(p)->net->tensor(name);
    if(t.shape().total_size() != count)
        throw dlprim::ValidationError(std::string("size mismatch for tensor ") + name);
    memcpy(t.host_data(), data, t.memory_size());
    return 0;
    REF_GUARD_END(-1)
}
int ref_net_get_tensor(void *p, char const *name, float *data, unsigned long long count)
{
    REF_GUARD_BEGIN
    dlprim::Tensor &t = static_cast<RefNet *>(p)->net->tensor(name);
    if(t.shape().total_size() != count)
        throw dlprim::ValidationError(std::string("size mismatch for tensor ") + name);
    memcpy(data, t.host_data(), t.memory_size());
    return 0;
    REF_GUARD_END(-1)
}
int ref_net_get_param(void *p, char const *name, float *data, unsigned long long count)
{
    REF_GUARD_BEGIN
    dlprim::Tensor &t = static_cast<RefNet *>(p)->net->param(name);
    if(t.shape().total_size() != count)
        throw dlprim::ValidationError(std::string("size mismatch for parameter ") + name);
    memcpy(data, t.host_data(), t.memory_size());
    return 0;
    REF_GUARD_END(-1)
}
/// Net::save_parameters / Net::load_parameters: the reference's own DLPW writer and reader (src/net.cpp:63-101, :227-305).
int ref_net_save_params(void *p, char const *path)
{
    REF_GUARD_BEGIN
    static_cast<RefNet *>(p)->net->save_parameters(path);
    return 0;
    REF_GUARD_END(-1)
}
int ref_net_load_params(void *p, char const *path)
{
    REF_GUARD_BEGIN
    static_cast<RefNet *>(p)->net->load_parameters(std::string(path), false);
    return 0;
    REF_GUARD_END(-1)
}
/// Net::forward on the CPU context; returns wall-clock seconds or a negative value on error.
double ref_net_forward(void *p)
{
    REF_GUARD_BEGIN
    dlprim::ExecutionContext e;
    auto t0 = std::chrono::steady_clock::now();
    static_cast<RefNet *>(p)->net->forward(e, false);
    auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double>(t1 - t0).count();
    REF_GUARD_END(-1.0)
}

} // extern "C"
