// Plain-C face of the host library (include/dlp_host.h): catches the C++ exceptions at the
// boundary and keeps the message for the calling thread.
#include <dlp_host.h>
#include <dlprim/net.hpp>
#include <dlprim/json.hpp>
#include <dlprim/ops/conv2d.hpp>
#include <dlprim/ops/inner_product.hpp>
#include <dlprim/gpu/gemm.hpp>

#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <typeinfo>

using namespace dlprim;

namespace {
thread_local std::string t_err;

char const *class_of(std::exception const &e)
{
    if(dynamic_cast<NotImplementedError const *>(&e)) return "NotImplementedError";
    if(dynamic_cast<ValidationError const *>(&e)) return "ValidationError";
    if(dynamic_cast<DeviceError const *>(&e)) return "DeviceError";
    if(dynamic_cast<Error const *>(&e)) return "Error";
    return "exception";
}
int write_shape(Shape const &s, int *dims)
{
    for(int i = 0; i < s.size(); i++) dims[i] = int(s[i]);
    return s.size();
}
std::vector<Shape> read_shapes(int n, int const *ranks, int const *dims)
{
    std::vector<Shape> r;
    int pos = 0;
    for(int i = 0; i < n; i++) {
        r.push_back(Shape::from_range(dims + pos, dims + pos + ranks[i]));
        pos += ranks[i];
    }
    return r;
}
} // namespace

#define GUARD_BEGIN try {
#define GUARD_END(fail) } catch(std::exception const &e) { t_err = std::string(class_of(e)) + ": " + e.what(); return fail; }

struct dlp_op {
    Context ctx;
    std::unique_ptr<Operator> op;
    std::vector<TensorSpecs> in_specs, out_specs, par_specs;
    size_t ws = 0;
    std::string kernel;
    dlp_op(int device) : ctx(Context::cuda, 0, device) {}
    void describe()
    {
        kernel.clear();
        if(Convolution2D *c = dynamic_cast<Convolution2D *>(op.get())) kernel = std::string(c->algo()) + " " + c->kernel_name();
        else if(InnerProduct *p = dynamic_cast<InnerProduct *>(op.get())) kernel = p->kernel_name();
    }
};

struct dlp_net {
    Context ctx;
    Net net;
    std::vector<std::string> plan;
    dlp_net(int device) : ctx(Context::cuda, 0, device), net(ctx) {}
};

extern "C" {

const char *dlp_host_last_error(void) { return t_err.c_str(); }

int dlp_op_create(const char *type, const char *options_json, int device, int n_inputs, const int *ranks, const int *dims, dlp_op **out)
{
    GUARD_BEGIN
    std::unique_ptr<dlp_op> h(new dlp_op(device));
    json::value opts = json::parse(options_json);
    h->op = create_by_name(h->ctx, type, opts);
    for(Shape const &s : read_shapes(n_inputs, ranks, dims)) h->in_specs.push_back(TensorSpecs(s, float_data));
    h->op->setup(h->in_specs, h->out_specs, h->par_specs, h->ws);
    h->describe();
    *out = h.release();
    return 0;
    GUARD_END(1)
}
void dlp_op_destroy(dlp_op *op) { delete op; }
int dlp_op_num_outputs(const dlp_op *op) { return int(op->out_specs.size()); }
int dlp_op_num_params(const dlp_op *op) { return int(op->par_specs.size()); }
int dlp_op_output_shape(const dlp_op *op, int i, int *dims) { return write_shape(op->out_specs.at(i).shape(), dims); }
int dlp_op_param_shape(const dlp_op *op, int i, int *dims) { return write_shape(op->par_specs.at(i).shape(), dims); }
size_t dlp_op_workspace(const dlp_op *op) { return op->ws; }
const char *dlp_op_kernel(const dlp_op *op) { return op->kernel.c_str(); }

int dlp_op_reshape(dlp_op *op, int n_inputs, const int *ranks, const int *dims)
{
    GUARD_BEGIN
    std::vector<Shape> in = read_shapes(n_inputs, ranks, dims), out;
    op->op->reshape(in, out, op->ws);
    for(size_t i = 0; i < in.size(); i++) op->in_specs.at(i) = TensorSpecs(in[i], op->in_specs[i].dtype());
    for(size_t i = 0; i < out.size(); i++) op->out_specs.at(i) = TensorSpecs(out[i], op->out_specs[i].dtype());
    op->describe();
    return 0;
    GUARD_END(1)
}

int dlp_op_forward(dlp_op *op, void *const *in_ptrs, void *const *par_ptrs, void *const *out_ptrs, void *ws_ptr, void *stream)
{
    GUARD_BEGIN
    std::vector<Tensor> in, out, par;
    for(size_t i = 0; i < op->in_specs.size(); i++) in.push_back(Tensor(in_ptrs[i], 0, op->in_specs[i].shape(), op->in_specs[i].dtype()));
    for(size_t i = 0; i < op->out_specs.size(); i++) out.push_back(Tensor(out_ptrs[i], 0, op->out_specs[i].shape(), op->out_specs[i].dtype()));
    for(size_t i = 0; i < op->par_specs.size(); i++) par.push_back(Tensor(par_ptrs[i], 0, op->par_specs[i].shape(), op->par_specs[i].dtype()));
    Tensor ws = op->ws > 0 ? Tensor(ws_ptr, 0, Shape(op->ws), uint8_data) : Tensor();
    ExecutionContext e(static_cast<cudaStream_t>(stream));
    op->op->forward(in, out, par, ws, e);
    return 0;
    GUARD_END(1)
}

int dlp_net_create(const char *net_json, int device, int flags, dlp_net **out)
{
    GUARD_BEGIN
    std::unique_ptr<dlp_net> h(new dlp_net(device));
    h->net.mode(CalculationsMode::predict);
    h->net.keep_intermediate_tensors((flags & 1) != 0);
    h->net.fuse_operators((flags & 2) == 0);
    h->net.use_cuda_graph((flags & 4) == 0);
    h->net.concurrent_branches((flags & 16) != 0);
    json::value description = json::parse(net_json);
    if(flags & 8) Net::merge_activations(description);
    h->net.load_from_json(description);
    h->net.setup();
    h->plan = h->net.describe_plan();
    *out = h.release();
    return 0;
    GUARD_END(1)
}
void dlp_net_destroy(dlp_net *net) { delete net; }
int dlp_net_num_params(const dlp_net *net) { return int(const_cast<dlp_net *>(net)->net.params().size()); }
int dlp_net_param_name(const dlp_net *net, int index, char *buf, int n)
{
    GUARD_BEGIN
    auto &m = const_cast<dlp_net *>(net)->net.params();
    if(index < 0 || size_t(index) >= m.size()) throw ValidationError("parameter index out of range");
    auto it = m.begin();
    std::advance(it, index);
    snprintf(buf, n, "%s", it->first.c_str());
    return 0;
    GUARD_END(1)
}
int dlp_net_param_shape(dlp_net *net, const char *name, int *dims)
{
    GUARD_BEGIN
    return write_shape(net->net.param(name).shape(), dims);
    GUARD_END(-1)
}
int dlp_net_tensor_shape(dlp_net *net, const char *name, int *dims)
{
    GUARD_BEGIN
    return write_shape(net->net.tensor(name).shape(), dims);
    GUARD_END(-1)
}
int dlp_net_set_param(dlp_net *net, const char *name, const float *data, size_t count)
{
    GUARD_BEGIN
    Tensor &t = net->net.param(name);
    if(t.shape().total_size() != count) throw ValidationError(std::string("size mismatch for parameter ") + name);
    memcpy(t.host_data(), data, t.memory_size());
    return 0;
    GUARD_END(1)
}
int dlp_net_upload_params(dlp_net *net)
{
    GUARD_BEGIN
    net->net.copy_parameters_to_device();
    return 0;
    GUARD_END(1)
}
int dlp_net_load_params_file(dlp_net *net, const char *path)
{
    GUARD_BEGIN
    net->net.load_parameters(std::string(path));
    return 0;
    GUARD_END(1)
}
int dlp_net_save_params_file(dlp_net *net, const char *path)
{
    GUARD_BEGIN
    net->net.save_parameters(path);
    return 0;
    GUARD_END(1)
}
int dlp_net_set_tensor(dlp_net *net, const char *name, const float *data, size_t count, void *stream)
{
    GUARD_BEGIN
    Tensor &t = net->net.tensor(name);
    if(t.shape().total_size() != count) throw ValidationError(std::string("size mismatch for tensor ") + name);
    t.to_device(ExecutionContext(static_cast<cudaStream_t>(stream)), const_cast<float *>(data), false);
    return 0;
    GUARD_END(1)
}
int dlp_net_get_tensor(dlp_net *net, const char *name, float *data, size_t count, void *stream)
{
    GUARD_BEGIN
    Tensor &t = net->net.tensor(name);
    if(t.shape().total_size() != count) throw ValidationError(std::string("size mismatch for tensor ") + name);
    t.to_host(ExecutionContext(static_cast<cudaStream_t>(stream)), data, false);
    return 0;
    GUARD_END(1)
}
void *dlp_net_tensor_device_ptr(dlp_net *net, const char *name)
{
    GUARD_BEGIN
    return net->net.tensor(name).device_ptr();
    GUARD_END(nullptr)
}
int dlp_net_reshape_input(dlp_net *net, const char *name, int rank, const int *dims)
{
    GUARD_BEGIN
    net->net.reshape_input(name, Shape::from_range(dims, dims + rank));
    return 0;
    GUARD_END(1)
}
int dlp_net_reshape(dlp_net *net)
{
    GUARD_BEGIN
    net->net.reshape();
    net->plan = net->net.describe_plan();
    return 0;
    GUARD_END(1)
}
int dlp_net_forward(dlp_net *net, void *stream, int sync)
{
    GUARD_BEGIN
    net->net.forward(ExecutionContext(static_cast<cudaStream_t>(stream)), sync != 0);
    return 0;
    GUARD_END(1)
}
int dlp_net_forward_timed(dlp_net *net, void *stream, float *step_ms, int capacity)
{
    GUARD_BEGIN
    ExecutionContext e(static_cast<cudaStream_t>(stream));
    std::shared_ptr<TimingData> timing(new TimingData());
    e.enable_timing(timing);
    net->net.forward(e, true);
    timing->resolve();
    int n = 0;
    for(auto const &sec : timing->sections()) {
        if(sec.parent != -1) continue;
        if(n >= capacity) throw ValidationError("step_ms is too small");
        step_ms[n++] = float(sec.time_ms);
    }
    if(n != int(net->plan.size())) throw ValidationError("timed sections do not match the plan");
    return 0;
    GUARD_END(1)
}
int dlp_net_copy_tensor_to_device(dlp_net *net, const char *name, void *dst, size_t count, void *stream)
{
    GUARD_BEGIN
    Tensor &t = net->net.tensor(name);
    if(t.shape().total_size() != count) throw ValidationError(std::string("size mismatch for tensor ") + name);
    if(cudaMemcpyAsync(dst, t.device_ptr(), t.memory_size(), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)) != cudaSuccess)
        throw DeviceError("cudaMemcpyAsync device to device failed");
    return 0;
    GUARD_END(1)
}
int dlp_net_copy_tensor_from_device(dlp_net *net, const char *name, const void *src, size_t count, void *stream)
{
    GUARD_BEGIN
    Tensor &t = net->net.tensor(name);
    if(t.shape().total_size() != count) throw ValidationError(std::string("size mismatch for tensor ") + name);
    if(cudaMemcpyAsync(t.device_ptr(), src, t.memory_size(), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)) != cudaSuccess)
        throw DeviceError("cudaMemcpyAsync device to device failed");
    return 0;
    GUARD_END(1)
}
int dlp_net_num_steps(const dlp_net *net) { return int(net->plan.size()); }
int dlp_net_step_description(const dlp_net *net, int index, char *buf, int n)
{
    if(index < 0 || size_t(index) >= net->plan.size()) return 1;
    snprintf(buf, n, "%s", net->plan[index].c_str());
    return 0;
}
size_t dlp_net_activation_bytes(const dlp_net *net, int without_reuse)
{
    return without_reuse ? net->net.activation_memory_without_reuse() : net->net.activation_memory();
}

int dlp_host_merge_activations(const char *net_json, char *out, size_t capacity)
{
    GUARD_BEGIN
    json::value v = json::parse(net_json);
    int merged = Net::merge_activations(v);
    std::string text = v.save(json::compact);
    if(text.size() + 1 > capacity) throw ValidationError("output buffer too small for the merged description");
    memcpy(out, text.c_str(), text.size() + 1);
    return merged;
    GUARD_END(-1)
}

int dlp_host_gemm(int device, int trans_a, int trans_b, int plan_m, int plan_n, int plan_k, int M, int N, int K, int bias_mode, int activation,
                  void *a, int lda, void *b, int ldb, void *c, int ldc, void *bias, float beta, void *stream)
{
    GUARD_BEGIN
    Context ctx(Context::cuda, 0, device);
    ExecutionContext e(static_cast<cudaStream_t>(stream));
    std::unique_ptr<gpu::GEMM> g = gpu::GEMM::get_optimal_gemm(ctx, float_data, trans_a != 0, trans_b != 0, plan_m, plan_n, plan_k, bias_mode,
                                                               StandardActivations(activation));
    g->gemm(M, N, K, a, 0, lda, b, 0, ldb, c, 0, ldc, bias, 0, beta, M * N, e);
    e.finish();        // the object's scratch goes away with it
    return 0;
    GUARD_END(1)
}

int dlp_host_batch_sgemm(int device, int trans_a, int trans_b, int batch, int M, int N, int K, void *a, int stride_a, int lda, void *b,
                         int stride_b, int ldb, void *c, int stride_c, int ldc, float beta, void *stream)
{
    GUARD_BEGIN
    Context ctx(Context::cuda, 0, device);
    ctx.activate();
    ExecutionContext e(static_cast<cudaStream_t>(stream));
    gpu::GEMM::batch_sgemm(float_data, trans_a != 0, trans_b != 0, batch, M, N, K, a, 0, stride_a, lda, b, 0, stride_b, ldb, c, 0, stride_c,
                           ldc, beta, e);
    return 0;
    GUARD_END(1)
}

int dlp_host_conv_gemm(int device, const int geometry[14], int channels_out_per_group, int batch, int with_bias, int activation, void *filters,
                       void *x, void *y, void *bias, float factor, void *stream)
{
    GUARD_BEGIN
    Context ctx(Context::cuda, 0, device);
    ExecutionContext e(static_cast<cudaStream_t>(stream));
    int kernel[2] = { geometry[0], geometry[1] }, dilate[2] = { geometry[2], geometry[3] }, pad[2] = { geometry[4], geometry[5] },
        stride[2] = { geometry[6], geometry[7] };
    const int groups = geometry[8], src_channels = geometry[9], src_rows = geometry[10], src_cols = geometry[11], tgt_rows = geometry[12],
              tgt_cols = geometry[13];
    const int M = channels_out_per_group, N = tgt_rows * tgt_cols * batch, K = src_channels * kernel[0] * kernel[1];
    std::unique_ptr<gpu::GEMM> g = gpu::GEMM::get_optimal_conv_gemm(ctx, float_data, GemmOpMode::forward, false, true, M, N, K, kernel, dilate, pad,
                                                                    stride, groups, src_channels, src_rows, src_cols, tgt_rows, tgt_cols,
                                                                    with_bias ? gpu::GEMM::bias_M : gpu::GEMM::no_bias,
                                                                    StandardActivations(activation), tgt_rows * tgt_cols);
    g->gemm(M, N, K, filters, 0, K, x, 0, K, y, 0, tgt_rows * tgt_cols, with_bias ? bias : nullptr, 0, factor, M * groups * N, e);
    e.finish();
    return 0;
    GUARD_END(1)
}

} // extern "C"
