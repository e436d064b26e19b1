// C ABI of the library: argument checking, algorithm selection, plans and launches.
// The declarations and their reference counterparts are in include/dlp_cuda.h.
#include "contraction.cuh"
#include "depthwise.cuh"

#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

namespace dlp {

// ---------------------------------------------------------------------------------------------- state
static thread_local std::string t_error;
std::atomic<uint64_t> g_launches{0};
__device__ int g_status_word = 0;

void set_error(const std::string &msg) { t_error = msg; }
dlp_status fail(dlp_status st, const std::string &msg)
{
    t_error = msg;
    return st;
}
dlp_status check_cuda(cudaError_t e, const char *what)
{
    if(e == cudaSuccess) return DLP_OK;
    t_error = std::string(what) + ": " + cudaGetErrorString(e);
    return DLP_CUDA_ERROR;
}

static std::mutex g_dev_mutex;
static std::map<int, int> g_sm_count;
static std::map<int, int *> g_status_ptr;

int sm_count()
{
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    auto it = g_sm_count.find(dev);
    if(it != g_sm_count.end()) return it->second;
    int n = 0;
    if(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
    return n;
}
int *device_status_word()
{
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    auto it = g_status_ptr.find(dev);
    if(it != g_status_ptr.end()) return it->second;
    int *ptr = nullptr;
    if(cudaGetSymbolAddress((void **)&ptr, g_status_word) != cudaSuccess) ptr = nullptr;
    g_status_ptr[dev] = ptr;
    return ptr;
}

static bool valid_act(int a) { return a >= DLP_ACT_IDENTITY && a <= DLP_ACT_RELU6; }

} // namespace dlp

using namespace dlp;

#include "plans.cuh"

static dlp_status conv_out_shape(const dlp_conv2d_desc &d, int in_h, int in_w, int *oh, int *ow)
{
    // src/core/conv.cpp:17-29
    const int ihw[2] = { in_h, in_w };
    int o[2];
    for(int i = 0; i < 2; i++) o[i] = (ihw[i] + 2 * d.pad[i] - d.dilate[i] * (d.kernel[i] - 1) - 1) / d.stride[i] + 1;
    DLP_REQUIRE(o[0] > 0, "output height is not positive");
    DLP_REQUIRE(o[1] > 0, "output width is not positive");
    *oh = o[0];
    *ow = o[1];
    return DLP_OK;
}

static dlp_status validate_conv_desc(const dlp_conv2d_desc *d)
{
    DLP_REQUIRE(d != nullptr, "null descriptor");
    DLP_REQUIRE(d->channels_in > 0 && d->channels_out > 0, "channels must be positive");
    DLP_REQUIRE(d->groups > 0 && d->channels_in % d->groups == 0 && d->channels_out % d->groups == 0, "groups must divide the channels");
    for(int i = 0; i < 2; i++) {
        DLP_REQUIRE(d->kernel[i] > 0 && d->stride[i] > 0 && d->dilate[i] > 0 && d->pad[i] >= 0, "bad kernel/stride/dilate/pad");
        DLP_REQUIRE(d->kernel[i] * d->dilate[i] < 32767, "kernel extent too large");
    }
    DLP_REQUIRE(d->height > 0 && d->width > 0 && d->batch >= 0, "bad input shape");
    DLP_REQUIRE(valid_act(d->activation), "unknown activation");
    DLP_REQUIRE(d->math_mode >= DLP_MATH_AUTO && d->math_mode <= DLP_MATH_TF32X3, "unknown math mode");
    DLP_REQUIRE((long long)d->channels_in * d->height * d->width < (1ll << 31), "one image must have fewer than 2^31 elements");
    return DLP_OK;
}

extern "C" {

const char *dlp_last_error(void) { return t_error.c_str(); }
const char *dlp_version(void) { return "dlprim-b200 0.1 (sm_100a)"; }
uint64_t dlp_launch_count(void) { return g_launches.load(); }

dlp_status dlp_device_status(void *stream, int *code)
{
    DLP_REQUIRE(code != nullptr, "null code pointer");
    DLP_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
    int *ptr = device_status_word();
    if(!ptr) return fail(DLP_CUDA_ERROR, "cannot resolve the device status word");
    int v = 0;
    DLP_CUDA_OK(cudaMemcpy(&v, ptr, sizeof(int), cudaMemcpyDeviceToHost));
    *code = v;
    if(v != 0) {
        int zero = 0;
        DLP_CUDA_OK(cudaMemcpy(ptr, &zero, sizeof(int), cudaMemcpyHostToDevice));
        return fail(DLP_TIMEOUT, "a bounded device-side wait gave up, code " + std::to_string(v));
    }
    return DLP_OK;
}

// Workspace layout of the calls that pack their weights themselves: packed operand first, then (256-byte
// aligned) the scratch that lets the tensor-core launcher split K.  The *_packed calls use their whole
// workspace as that scratch.
static size_t align256(size_t n) { return (n + 255) & ~size_t(255); }
static void scratch_after(void *ws, size_t ws_bytes, size_t first_bytes, void *&scratch, size_t &scratch_bytes)
{
    const size_t off = align256(first_bytes);
    scratch = ws && ws_bytes > off ? static_cast<char *>(ws) + off : nullptr;
    scratch_bytes = scratch ? ws_bytes - off : 0;
}

// ---------------------------------------------------------------------------------------------- convolution
dlp_status dlp_conv2d_output_shape(const dlp_conv2d_desc *desc, int in_h, int in_w, int *out_h, int *out_w)
{
    dlp_status st = validate_conv_desc(desc);
    if(st != DLP_OK) return st;
    DLP_REQUIRE(out_h && out_w, "null output pointer");
    return conv_out_shape(*desc, in_h, in_w, out_h, out_w);
}

dlp_status dlp_conv2d_fwd_create(const dlp_conv2d_desc *desc, dlp_conv2d_plan **out)
{
    dlp_status st = validate_conv_desc(desc);
    if(st != DLP_OK) return st;
    DLP_REQUIRE(out != nullptr, "null plan pointer");
    const dlp_conv2d_desc &d = *desc;
    const std::string algo = d.algo ? d.algo : "";
    DLP_REQUIRE(algo == "" || algo == "auto" || algo == "gemm" || algo == "winograd" || algo == "depthwise_separable",
                "unknown algorithm name " + algo);

    std::unique_ptr<dlp_conv2d_plan> plan(new dlp_conv2d_plan());
    plan->d = d;
    plan->d.algo = nullptr;
    st = conv_out_shape(d, d.height, d.width, &plan->out_h, &plan->out_w);
    if(st != DLP_OK) return st;
    plan->k = d.channels_in / d.groups * d.kernel[0] * d.kernel[1];
    DLP_CUDA_OK(cudaGetDevice(&plan->device));

    // Eligibility as in the reference (src/core/conv.cpp:672-702); the stride-2 depthwise case,
    // which the reference sends to its grouped GEMM, has a native kernel here.
    const bool square = d.kernel[0] == d.kernel[1] && d.pad[0] == d.pad[1] && d.dilate[0] == d.dilate[1] && d.stride[0] == d.stride[1];
    const bool dsc_ref = square && d.groups == d.channels_in && d.channels_in > 1 && d.dilate[0] == 1 && d.stride[0] == 1
                         && d.kernel[0] % 2 == 1 && d.kernel[0] / 2 == d.pad[0];
    const bool dsc_native = d.groups == d.channels_in && d.channels_in > 1 && d.channels_out == d.channels_in
                            && depthwise_supported(d.kernel[0], d.kernel[1], d.stride[0], d.stride[1], d.pad[0], d.pad[1],
                                                   d.dilate[0], d.dilate[1], d.width);
    const bool auto_algo = algo == "" || algo == "auto";

    if(dsc_native && ((algo == "depthwise_separable" && dsc_ref) || auto_algo)) {
        plan->algo = "depthwise_separable";
        plan->kind = CK_DEPTHWISE;
        plan->kernel = "depthwise_k" + std::to_string(d.kernel[0]) + "_s" + std::to_string(d.stride[0]);
    }
    else if(algo == "winograd" && square && d.groups == 1 && d.dilate[0] == 1 && d.stride[0] == 1 && d.kernel[0] == 3 && d.pad[0] == 1) {
        // Only on request.  The reference also takes Winograd under "auto" (src/core/conv.cpp:713-720); here
        // the 3xTF32 tensor-core implicit GEMM is the faster kernel for every eligible shape, so "auto" keeps it.
        // The sixteen products run on the tensor cores unless plain fp32 FMA arithmetic was asked for.
        plan->algo = "winograd";
        plan->kind = CK_WINOGRAD;
        plan->winograd_tc = d.math_mode != DLP_MATH_FP32_FFMA;
        plan->kernel = plan->winograd_tc ? "winograd_f23_tf32x3" : "winograd_f23_ffma";
    }
    else {
        // an incompatible "winograd" or "depthwise_separable" request gets the GEMM algorithm, as in the
        // reference (src/core/conv.cpp:719-727)
        plan->algo = "gemm";
        // the tensor-core loaders keep one validity bit per kernel row and per kernel column in 32-bit words
        // (bit 31 stands for "never")
        // Grouped convolutions run group by group (a launch each) when a group is wide enough to be worth a tile
        // and there are few of them; the rest stay on the grouped FFMA kernel.
        const bool groups_ok = d.groups == 1 || (d.groups <= 16 && d.channels_in / d.groups >= 8 && d.channels_out / d.groups >= 16);
        const bool tc_ok = groups_ok && d.math_mode != DLP_MATH_FP32_FFMA && d.kernel[0] <= MAX_KERNEL_SIDE && d.kernel[1] <= MAX_KERNEL_SIDE;
        if(d.math_mode == DLP_MATH_TF32X3 && !tc_ok)
            return fail(DLP_NOT_IMPLEMENTED, "the tensor-core kernel handles at most 16 groups of at least 8 x 16 channels and kernels of at most 30 x 30");
        plan->kind = tc_ok ? CK_TC : CK_FFMA;
    }
    plan->strided_a = d.kernel[0] == 1 && d.kernel[1] == 1 && d.stride[0] == 1 && d.stride[1] == 1 && d.pad[0] == 0 && d.pad[1] == 0;

    plan->tapblock = plan->kind == CK_TC && !plan->strided_a && (d.channels_in / d.groups) % 32 == 0;
    // Wide kernels over channel counts that do not come in blocks of 32 (a 7x7 stem over 3 channels): kernel columns padded
    // to 8 make a k-block four whole kernel rows, which the loaders address row by row instead of element by element.
    const int row_groups = d.channels_in / d.groups * d.kernel[0];
    plan->rowtaps = plan->kind == CK_TC && !plan->strided_a && !plan->tapblock && d.dilate[0] == 1 && d.dilate[1] == 1 &&
                    d.kernel[1] >= 5 && d.kernel[1] <= ROWTAPS_WIDTH && row_groups <= 1024;
    if(plan->kind != CK_DEPTHWISE && plan->kind != CK_WINOGRAD) {
        plan->packed = tc_packed_layout(d.channels_out / d.groups, plan->rowtaps ? row_groups * ROWTAPS_WIDTH : plan->k);
        if(plan->kind == CK_TC)
            plan->kernel = std::string("igemm_tf32x3_bn") + std::to_string(plan->packed.bn) +
                           (plan->strided_a ? "_1x1" : (plan->tapblock ? "_taps" : (plan->rowtaps ? "_rowtaps" : "_gather")));
        else
            plan->kernel = std::string("igemm_ffma_64x64") + (plan->strided_a ? "_1x1" : "_gather");
        if(!plan->strided_a) {
            // tap table: k -> (c, ky, kx) in the weight tensor's own order [Cin/g][KH][KW]
            const int k_pad = plan->packed.k_pad;
            std::vector<KTap> tab(k_pad);
            plan->num_taps = d.kernel[0] * d.kernel[1];
            std::vector<int> taps(plan->num_taps);
            const int cin_g = d.channels_in / d.groups;
            int idx = 0;
            for(int c = 0; c < cin_g; c++)
                for(int ky = 0; ky < d.kernel[0]; ky++)
                    for(int kx = 0; kx < d.kernel[1]; kx++, idx++) {
                        const int dy = ky * d.dilate[0], dx = kx * d.dilate[1];
                        tab[idx].offset = (c * d.height + dy) * d.width + dx;
                        tab[idx].tap = plan->kind == CK_TC ? (ky << 8) | kx : std::min(ky * d.kernel[1] + kx, plan->num_taps - 1);
                        taps[ky * d.kernel[1] + kx] = (dy << 16) | dx;
                    }
            for(; idx < k_pad; idx++) { tab[idx].offset = 0; tab[idx].tap = TAP_PADDING; }
            if(plan->rowtaps) {
                // one entry per (channel, kernel row); the groups beyond K name a kernel row that never exists
                for(int g = 0; g < k_pad / ROWTAPS_WIDTH; g++) {
                    const int c = g / d.kernel[0], ky = g % d.kernel[0];
                    tab[g].offset = g < row_groups ? (c * d.height + ky) * d.width : 0;
                    tab[g].tap = g < row_groups ? ky : ROW_PADDING;
                }
            }
            DLP_CUDA_OK(cudaMalloc((void **)&plan->ktab, sizeof(KTap) * k_pad));
            cudaError_t e = cudaMalloc((void **)&plan->tap_dydx, sizeof(int) * taps.size());
            if(e == cudaSuccess) e = cudaMemcpy(plan->ktab, tab.data(), sizeof(KTap) * k_pad, cudaMemcpyHostToDevice);
            if(e == cudaSuccess) e = cudaMemcpy(plan->tap_dydx, taps.data(), sizeof(int) * taps.size(), cudaMemcpyHostToDevice);
            if(e != cudaSuccess) {
                cudaFree(plan->ktab);
                if(plan->tap_dydx) cudaFree(plan->tap_dydx);
                return check_cuda(e, "upload of the tap tables");
            }
        }
    }
    *out = plan.release();
    return DLP_OK;
}

void dlp_conv2d_fwd_destroy(dlp_conv2d_plan *plan)
{
    if(!plan) return;
    if(plan->ktab) cudaFree(plan->ktab);
    if(plan->tap_dydx) cudaFree(plan->tap_dydx);
    delete plan;
}
const char *dlp_conv2d_fwd_algo(const dlp_conv2d_plan *plan) { return plan ? plan->algo.c_str() : ""; }
const char *dlp_conv2d_fwd_kernel(const dlp_conv2d_plan *plan) { return plan ? plan->kernel.c_str() : ""; }
size_t dlp_conv2d_fwd_packed_bytes(const dlp_conv2d_plan *plan)
{
    if(!plan) return 0;
    if(plan->kind == CK_WINOGRAD)
        return plan->winograd_tc ? winograd_tc_packed_bytes(plan->d.channels_in, plan->d.channels_out)
                                 : winograd_packed_bytes(plan->d.channels_in, plan->d.channels_out);
    return plan->kind == CK_TC ? plan->packed.bytes() * size_t(plan->d.groups) : 0;     // one packed operand per group
}
size_t dlp_conv2d_fwd_workspace(const dlp_conv2d_plan *plan)
{
    const size_t packed = dlp_conv2d_fwd_packed_bytes(plan);
    if(plan && plan->kind == CK_WINOGRAD && plan->winograd_tc)
        return align256(packed) + winograd_tc_workspace_bytes(std::max(plan->d.batch, 1), plan->d.channels_in, plan->d.channels_out,
                                                              plan->d.height, plan->d.width);
    if(!plan || plan->kind != CK_TC) return packed;
    const size_t split = tc_split_scratch_bytes((long long)plan->d.batch * plan->out_h * plan->out_w, plan->packed);
    return split ? align256(packed) + split : packed;
}

dlp_status dlp_conv2d_fwd_prepack(const dlp_conv2d_plan *plan, const float *w, void *packed, void *stream)
{
    DLP_REQUIRE(plan && w, "null argument");
    if(plan->kind == CK_WINOGRAD) {
        DLP_REQUIRE(packed != nullptr, "null packed buffer");
        if(plan->winograd_tc)
            return winograd_tc_filter_transform(w, static_cast<float *>(packed), plan->d.channels_in, plan->d.channels_out, (cudaStream_t)stream);
        return winograd_filter_transform(w, static_cast<float *>(packed), plan->d.channels_in, plan->d.channels_out, (cudaStream_t)stream);
    }
    if(plan->kind != CK_TC) return DLP_OK;
    DLP_REQUIRE(packed != nullptr, "null packed buffer");
    const int cout_g = plan->d.channels_out / plan->d.groups;
    for(int g = 0; g < plan->d.groups; g++) {
        dlp_status st = tc_prepack(plan->packed, w + (long long)g * cout_g * plan->k, plan->k, 1, cout_g, plan->k,
                                   static_cast<float *>(packed) + g * (plan->packed.bytes() / sizeof(float)),
                                   plan->tapblock ? plan->num_taps : 0, (cudaStream_t)stream, 1, 0, plan->rowtaps ? plan->d.kernel[1] : 0);
        if(st != DLP_OK) return st;
    }
    return DLP_OK;
}

static dlp_status conv_enqueue(const dlp_conv2d_plan *plan, const float *x, const float *w_raw, const float *packed, const float *bias,
                               float *y, float factor, const float *residual, float residual_scale, int post_act, int batch,
                               int in_h, int in_w, cudaStream_t stream, void *scratch, size_t scratch_bytes)
{
    const dlp_conv2d_desc &d = plan->d;
    DLP_REQUIRE(x && y, "null tensor");
    DLP_REQUIRE(batch >= 0, "negative batch");
    DLP_REQUIRE(in_h == d.height && in_w == d.width, "input height/width differ from the plan; create a new plan");
    DLP_REQUIRE(!d.bias == !bias, "bias pointer does not match the plan's bias setting");
    DLP_REQUIRE(valid_act(post_act), "unknown post activation");
    DLP_REQUIRE(!(residual && factor != 0.0f), "factor must be 0 when a residual is fused");
    if(batch == 0) return DLP_OK;

    if(plan->kind == CK_DEPTHWISE) {
        DLP_REQUIRE(w_raw != nullptr, "null weights");
        DLP_REQUIRE(residual == nullptr, "the depthwise kernel has no fused residual");
        return launch_depthwise(x, w_raw, bias, y, batch, d.channels_in, d.height, d.width, d.kernel[0], d.stride[0], d.pad[0],
                                d.activation, factor, stream);
    }

    if(plan->kind == CK_WINOGRAD) {
        DLP_REQUIRE(packed != nullptr, "null transformed filters");
        if(plan->winograd_tc)
            return launch_winograd_tc(x, packed, bias, y, scratch, scratch_bytes, batch, d.channels_in, d.channels_out, d.height, d.width,
                                      d.activation, factor, residual, residual_scale, post_act, stream);
        return launch_winograd_f23(x, packed, bias, y, batch, d.channels_in, d.channels_out, d.height, d.width, d.activation, factor,
                                   residual, residual_scale, post_act, stream);
    }

    const int cin_g = d.channels_in / d.groups, cout_g = d.channels_out / d.groups;
    Contraction p;
    memset(&p, 0, sizeof(p));
    p.rows = (long long)batch * plan->out_h * plan->out_w;
    p.cols = cout_g;
    p.k = plan->k;
    p.a = x;
    p.plane = plan->out_h * plan->out_w;
    p.out_w = plan->out_w;
    p.in_h = d.height; p.in_w = d.width;
    p.stride_h = d.stride[0]; p.stride_w = d.stride[1];
    p.pad_h = d.pad[0]; p.pad_w = d.pad[1];
    p.a_batch_stride = (long long)d.channels_in * d.height * d.width;
    if(plan->strided_a) {
        p.a_mode = A_STRIDED;
        p.a_k_stride = (long long)d.height * d.width;
    }
    else {
        p.a_mode = plan->tapblock ? A_TAPBLOCK : (plan->rowtaps ? A_ROWTAPS : A_GATHER);
        p.a_k_stride = (long long)d.height * d.width;
        p.ktab = plan->ktab;
        p.tap_dydx = plan->tap_dydx;
        p.num_taps = plan->num_taps;
        p.kh = d.kernel[0]; p.kw = d.kernel[1];
        p.dil_h = d.dilate[0]; p.dil_w = d.dilate[1];
    }
    p.b = w_raw;
    p.b_col_stride = plan->k;
    p.b_k_stride = 1;
    p.y = y;
    p.out_mode = OUT_NCHW;
    p.out_channels_total = d.channels_out;
    p.bias = bias;
    p.bias_mode = bias ? DLP_GEMM_BIAS_N : DLP_GEMM_NO_BIAS;
    p.act = d.activation;
    p.beta = factor;
    p.residual = residual;
    p.residual_scale = residual_scale;
    p.post_act = post_act;

    if(plan->kind == CK_TC) {
        DLP_REQUIRE(packed != nullptr, "null packed weights");
        // group g: input channels [g*cin_g, ...), its own packed operand, output channels [g*cout_g, ...)
        for(int g = 0; g < d.groups; g++) {
            Contraction q = p;
            q.a = x + (long long)g * cin_g * d.height * d.width;
            const long long out_off = (long long)g * cout_g * plan->out_h * plan->out_w;
            q.y = y + out_off;
            if(bias) q.bias = bias + g * cout_g;
            if(residual) q.residual = residual + out_off;
            dlp_status st = launch_contraction_tc(q, plan->packed, packed + g * (plan->packed.bytes() / sizeof(float)), stream, scratch,
                                                  scratch_bytes);
            if(st != DLP_OK) return st;
        }
        return DLP_OK;
    }
    DLP_REQUIRE(w_raw != nullptr, "null weights");
    return launch_contraction_ffma(p, d.groups, (long long)cin_g * d.height * d.width, (long long)cout_g * plan->k, cout_g, stream);
}

dlp_status dlp_conv2d_fwd_enqueue(const dlp_conv2d_plan *plan, const float *x, const float *w, const float *bias, float *y, void *ws,
                                  size_t ws_bytes, float factor, int batch, int in_h, int in_w, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    DLP_REQUIRE(batch >= 0, "negative batch");
    if(batch == 0) return DLP_OK;      // an empty batch is valid and launches nothing
    DLP_REQUIRE(w != nullptr, "null weights");
    const float *packed = nullptr;
    if(plan->kind == CK_TC || plan->kind == CK_WINOGRAD) {
        // the weights are packed (split into TF32 hi/lo stages, or Winograd-transformed) in the caller's
        // workspace on every call, as the reference redoes its Winograd filter transform on every call
        DLP_REQUIRE(ws != nullptr && ws_bytes >= dlp_conv2d_fwd_packed_bytes(plan), "workspace smaller than dlp_conv2d_fwd_workspace()");
        dlp_status st = dlp_conv2d_fwd_prepack(plan, w, ws, stream);
        if(st != DLP_OK) return st;
        packed = static_cast<const float *>(ws);
    }
    void *scratch;
    size_t scratch_bytes;
    scratch_after(ws, ws_bytes, dlp_conv2d_fwd_packed_bytes(plan), scratch, scratch_bytes);
    return conv_enqueue(plan, x, w, packed, bias, y, factor, nullptr, 0.0f, DLP_ACT_IDENTITY, batch, in_h, in_w, (cudaStream_t)stream,
                        scratch, scratch_bytes);
}

dlp_status dlp_conv2d_fwd_enqueue_packed(const dlp_conv2d_plan *plan, const float *x, const void *packed, const float *bias, float *y,
                                         void *ws, size_t ws_bytes, float factor, const float *residual, float residual_scale,
                                         int post_activation, int batch, int in_h, int in_w, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    DLP_REQUIRE(batch >= 0, "negative batch");
    if(batch == 0) return DLP_OK;
    DLP_REQUIRE(packed != nullptr, "null weights");
    // plans whose kernel reads raw weights take them through the same argument
    const bool takes_packed = plan->kind == CK_TC || plan->kind == CK_WINOGRAD;
    const float *raw = takes_packed ? nullptr : static_cast<const float *>(packed);
    const float *pk = takes_packed ? static_cast<const float *>(packed) : nullptr;
    if(residual && plan->kind == CK_DEPTHWISE) return fail(DLP_NOT_IMPLEMENTED, "the depthwise kernel has no fused residual");
    return conv_enqueue(plan, x, raw, pk, bias, y, factor, residual, residual_scale, post_activation, batch, in_h, in_w,
                        (cudaStream_t)stream, ws, ws_bytes);
}

// ---------------------------------------------------------------------------------------------- GEMM
static dlp_status gemm_problem(const dlp_gemm_desc &d, int m, int n, int k, const float *a, int lda, const float *b, int ldb, float *c,
                               int ldc, const float *bias, float beta, Contraction &p)
{
    DLP_REQUIRE(m >= 0 && n >= 0 && k >= 0, "negative GEMM size");
    DLP_REQUIRE(a && b && c, "null matrix");
    DLP_REQUIRE(lda >= (d.trans_a ? m : k) && ldb >= (d.trans_b ? k : n) && ldc >= n, "leading dimension too small");
    DLP_REQUIRE((d.bias_mode == DLP_GEMM_NO_BIAS) == (bias == nullptr), "bias pointer does not match the plan's bias mode");
    memset(&p, 0, sizeof(p));
    p.rows = m; p.cols = n; p.k = k;
    p.a = a;
    p.a_mode = A_STRIDED;
    p.a_row_stride = d.trans_a ? 1 : lda;
    p.a_k_stride = d.trans_a ? lda : 1;
    p.b = b;
    p.b_col_stride = d.trans_b ? ldb : 1;
    p.b_k_stride = d.trans_b ? 1 : ldb;
    p.y = c;
    p.out_mode = OUT_ROW_MAJOR;
    p.ldc = ldc;
    p.bias = bias;
    p.bias_mode = d.bias_mode;
    p.act = d.activation;
    p.beta = beta;
    return DLP_OK;
}

dlp_status dlp_gemm_create(const dlp_gemm_desc *desc, dlp_gemm_plan **out)
{
    DLP_REQUIRE(desc && out, "null argument");
    DLP_REQUIRE(desc->m >= 0 && desc->n >= 0 && desc->k >= 0, "negative GEMM size");
    DLP_REQUIRE(desc->bias_mode >= DLP_GEMM_NO_BIAS && desc->bias_mode <= DLP_GEMM_BIAS_N, "unknown bias mode");
    DLP_REQUIRE(valid_act(desc->activation), "unknown activation");
    DLP_REQUIRE(desc->math_mode >= DLP_MATH_AUTO && desc->math_mode <= DLP_MATH_TF32X3, "unknown math mode");
    dlp_gemm_plan *plan = new dlp_gemm_plan();
    plan->d = *desc;
    // tiny products are not worth packing B for
    const bool small = (long long)desc->m * desc->n * desc->k < (1ll << 18);
    plan->use_tc = desc->math_mode == DLP_MATH_TF32X3 || (desc->math_mode == DLP_MATH_AUTO && !small);
    plan->kernel = plan->use_tc ? "gemm_tf32x3" : "gemm_ffma_64x64";
    *out = plan;
    return DLP_OK;
}
void dlp_gemm_destroy(dlp_gemm_plan *plan) { delete plan; }
const char *dlp_gemm_kernel(const dlp_gemm_plan *plan) { return plan ? plan->kernel.c_str() : ""; }
size_t dlp_gemm_workspace(const dlp_gemm_plan *plan)
{
    if(!plan || !plan->use_tc) return 0;
    const TcPacked L = tc_packed_layout(std::max(plan->d.n, 1), std::max(plan->d.k, 1));
    const size_t split = tc_split_scratch_bytes(std::max(plan->d.m, 1), L);
    return split ? align256(L.bytes()) + split : L.bytes();
}

dlp_status dlp_gemm_enqueue(const dlp_gemm_plan *plan, int m, int n, int k, const float *a, int lda, const float *b, int ldb, float *c,
                            int ldc, const float *bias, float beta, void *ws, size_t ws_bytes, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    Contraction p;
    dlp_status st = gemm_problem(plan->d, m, n, k, a, lda, b, ldb, c, ldc, bias, beta, p);
    if(st != DLP_OK) return st;
    if(m == 0 || n == 0) return DLP_OK;
    if(plan->use_tc && k > 0) {
        const TcPacked L = tc_packed_layout(n, k);
        DLP_REQUIRE(ws != nullptr && ws_bytes >= L.bytes(), "workspace smaller than the packed B operand needs");
        st = tc_prepack(L, b, p.b_col_stride, p.b_k_stride, n, k, static_cast<float *>(ws), 0, (cudaStream_t)stream);
        if(st != DLP_OK) return st;
        void *scratch;
        size_t scratch_bytes;
        scratch_after(ws, ws_bytes, L.bytes(), scratch, scratch_bytes);
        return launch_contraction_tc(p, L, static_cast<const float *>(ws), (cudaStream_t)stream, scratch, scratch_bytes);
    }
    return launch_contraction_ffma(p, 1, 0, 0, n, (cudaStream_t)stream);
}

size_t dlp_gemm_batched_workspace(const dlp_gemm_plan *plan, int batch)
{
    if(!plan || !plan->use_tc || batch <= 0) return 0;
    return tc_packed_layout(std::max(plan->d.n, 1), std::max(plan->d.k, 1)).bytes() * size_t(batch);
}

// One launch for the whole batch (src/gemm.cpp:603-638, :348-426 in the reference): the matrices are an outer index of
// the grid.  Tensor-core plans pack every B of the batch into the workspace first (one launch as well).
dlp_status dlp_gemm_batched_enqueue(const dlp_gemm_plan *plan, int batch, int m, int n, int k, const float *a, long long stride_a, int lda,
                                    const float *b, long long stride_b, int ldb, float *c, long long stride_c, int ldc, float beta,
                                    void *ws, size_t ws_bytes, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    DLP_REQUIRE(batch >= 0, "negative batch");
    DLP_REQUIRE(plan->d.bias_mode == DLP_GEMM_NO_BIAS, "the batched product takes no bias, as in the reference");
    if(batch == 0) return DLP_OK;
    DLP_REQUIRE(batch <= 65535, "at most 65535 matrices per call");
    Contraction p;
    dlp_status st = gemm_problem(plan->d, m, n, k, a, lda, b, ldb, c, ldc, nullptr, beta, p);
    if(st != DLP_OK) return st;
    if(m == 0 || n == 0) return DLP_OK;
    if(plan->use_tc && k > 0) {
        const TcPacked L = tc_packed_layout(n, k);
        DLP_REQUIRE(ws != nullptr && ws_bytes >= L.bytes() * size_t(batch), "workspace smaller than dlp_gemm_batched_workspace()");
        st = tc_prepack(L, b, p.b_col_stride, p.b_k_stride, n, k, static_cast<float *>(ws), 0, (cudaStream_t)stream, batch, stride_b);
        if(st != DLP_OK) return st;
        TcBatch bt;
        bt.count = batch;
        bt.a_stride = stride_a;
        bt.y_stride = stride_c;
        return launch_contraction_tc(p, L, static_cast<const float *>(ws), (cudaStream_t)stream, nullptr, 0, bt);
    }
    return launch_contraction_ffma(p, batch, stride_a, stride_b, 0, (cudaStream_t)stream, stride_c);
}

// ---------------------------------------------------------------------------------------------- InnerProduct
dlp_status dlp_ip_fwd_create(const dlp_ip_desc *desc, dlp_ip_plan **out)
{
    DLP_REQUIRE(desc && out, "null argument");
    DLP_REQUIRE(desc->inputs > 0 && desc->outputs > 0, "inputs and outputs must be positive");
    DLP_REQUIRE(valid_act(desc->activation), "unknown activation");
    DLP_REQUIRE(desc->math_mode >= DLP_MATH_AUTO && desc->math_mode <= DLP_MATH_TF32X3, "unknown math mode");
    dlp_ip_plan *plan = new dlp_ip_plan();
    plan->d = *desc;
    plan->use_tc = desc->math_mode != DLP_MATH_FP32_FFMA;
    plan->packed = tc_packed_layout(desc->outputs, desc->inputs);
    plan->kernel = plan->use_tc ? "ip_tf32x3_bn" + std::to_string(plan->packed.bn) : std::string("ip_ffma_64x64");
    *out = plan;
    return DLP_OK;
}
void dlp_ip_fwd_destroy(dlp_ip_plan *plan) { delete plan; }
const char *dlp_ip_fwd_kernel(const dlp_ip_plan *plan) { return plan ? plan->kernel.c_str() : ""; }
size_t dlp_ip_fwd_packed_bytes(const dlp_ip_plan *plan) { return plan && plan->use_tc ? plan->packed.bytes() : 0; }
size_t dlp_ip_fwd_workspace(const dlp_ip_plan *plan)
{
    const size_t packed = dlp_ip_fwd_packed_bytes(plan);
    if(!plan || !plan->use_tc) return packed;
    const size_t split = tc_split_scratch_bytes(std::max(plan->d.optimal_batch_size, 1), plan->packed);
    return split ? align256(packed) + split : packed;
}

dlp_status dlp_ip_fwd_prepack(const dlp_ip_plan *plan, const float *w, void *packed, void *stream)
{
    DLP_REQUIRE(plan && w, "null argument");
    if(!plan->use_tc) return DLP_OK;
    DLP_REQUIRE(packed != nullptr, "null packed buffer");
    return tc_prepack(plan->packed, w, plan->d.inputs, 1, plan->d.outputs, plan->d.inputs, static_cast<float *>(packed), 0, (cudaStream_t)stream);
}

static dlp_status ip_enqueue(const dlp_ip_plan *plan, const float *x, const float *w_raw, const float *packed, const float *bias, float *y,
                             int batch, cudaStream_t stream, void *scratch, size_t scratch_bytes)
{
    DLP_REQUIRE(batch >= 0, "negative batch");
    if(batch == 0) return DLP_OK;
    DLP_REQUIRE(x && y, "null tensor");
    DLP_REQUIRE(!plan->d.bias == !bias, "bias pointer does not match the plan's bias setting");
    if(batch == 0) return DLP_OK;
    dlp_gemm_desc g;
    memset(&g, 0, sizeof(g));
    g.trans_a = 0; g.trans_b = 1;
    g.bias_mode = bias ? DLP_GEMM_BIAS_N : DLP_GEMM_NO_BIAS;
    g.activation = plan->d.activation;
    Contraction p;
    const float *b_any = w_raw ? w_raw : packed;
    dlp_status st = gemm_problem(g, batch, plan->d.outputs, plan->d.inputs, x, plan->d.inputs, b_any, plan->d.inputs, y, plan->d.outputs,
                                 bias, 0.0f, p);
    if(st != DLP_OK) return st;
    if(plan->use_tc) return launch_contraction_tc(p, plan->packed, packed, stream, scratch, scratch_bytes);
    return launch_contraction_ffma(p, 1, 0, 0, plan->d.outputs, stream);
}

dlp_status dlp_ip_fwd_enqueue(const dlp_ip_plan *plan, const float *x, const float *w, const float *bias, float *y, void *ws,
                              size_t ws_bytes, int batch, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    DLP_REQUIRE(w != nullptr, "null weights");
    const float *packed = nullptr;
    if(plan->use_tc) {
        DLP_REQUIRE(ws != nullptr && ws_bytes >= plan->packed.bytes(), "workspace smaller than dlp_ip_fwd_workspace()");
        dlp_status st = dlp_ip_fwd_prepack(plan, w, ws, stream);
        if(st != DLP_OK) return st;
        packed = static_cast<const float *>(ws);
    }
    void *scratch;
    size_t scratch_bytes;
    scratch_after(ws, ws_bytes, dlp_ip_fwd_packed_bytes(plan), scratch, scratch_bytes);
    return ip_enqueue(plan, x, w, packed, bias, y, batch, (cudaStream_t)stream, scratch, scratch_bytes);
}

dlp_status dlp_ip_fwd_enqueue_packed(const dlp_ip_plan *plan, const float *x, const void *packed, const float *bias, float *y, void *ws,
                                     size_t ws_bytes, int batch, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    DLP_REQUIRE(packed != nullptr, "null weights");
    const float *pk = static_cast<const float *>(packed);
    return ip_enqueue(plan, x, plan->use_tc ? nullptr : pk, plan->use_tc ? pk : nullptr, bias, y, batch, (cudaStream_t)stream, ws, ws_bytes);
}

} // extern "C"
