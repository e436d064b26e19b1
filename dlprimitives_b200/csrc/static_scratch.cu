// InnerProduct forward for callers that must not allocate device memory.
//
// The regular entry point, dlp_ip_fwd_enqueue, needs a caller-supplied workspace for the packed form
// of the weights.  Some callers cannot provide one: code that runs after the process has handed all
// of its device memory to a pool it does not control, a plugin called from inside another
// framework's allocator callbacks, or a driver-level harness where cudaMalloc is simply not
// permitted.  For them the scratch lives in a fixed array in the library's own device image: it is
// part of the module, so every GPU that has loaded the module holds DLP_IP_STATIC_SCRATCH_BYTES of it
// until the process exits, and no allocation routine is ever called.  (With lazy module loading the
// module is loaded, and the array's memory reserved, by the first address look-up on a device: the
// first call per device belongs at start-up, while memory is still available.)
#include "plans.cuh"
#include <mutex>

using namespace dlp;

namespace {

// The scratch itself.  In host code this name is only a stand-in for the symbol: it is not a device
// address and must never be handed to a kernel.  The address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) unsigned char g_ip_scratch[DLP_IP_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_mutex;
float *g_scratch_ptr[MAX_DEVICES] = {};   // per-device address of g_ip_scratch, resolved on first use

dlp_status scratch_for_current_device(float **out)
{
    int dev = 0;
    DLP_CUDA_OK(cudaGetDevice(&dev));
    if(dev < 0 || dev >= MAX_DEVICES) return fail(DLP_INVALID_ARGUMENT, "device ordinal out of range for the static scratch table");
    std::lock_guard<std::mutex> lock(g_mutex);
    if(!g_scratch_ptr[dev]) {
        void *ptr = nullptr;
        DLP_CUDA_OK(cudaGetSymbolAddress(&ptr, g_ip_scratch));
        if(!ptr) return fail(DLP_CUDA_ERROR, "cudaGetSymbolAddress returned a null address for the static scratch");
        g_scratch_ptr[dev] = static_cast<float *>(ptr);
    }
    *out = g_scratch_ptr[dev];
    return DLP_OK;
}

} // namespace

extern "C" dlp_status dlp_ip_fwd_enqueue_static(const dlp_ip_plan *plan, const float *x, const float *w, const float *bias, float *y,
                                               int batch, void *stream)
{
    DLP_REQUIRE(plan != nullptr, "null plan");
    DLP_REQUIRE(batch >= 0, "negative batch");
    if(batch == 0) return DLP_OK;
    DLP_REQUIRE(x && w && y, "null tensor");
    DLP_REQUIRE(!plan->d.bias == !bias, "bias pointer does not match the plan's bias setting");

    Contraction p = {};
    p.rows = batch;
    p.cols = plan->d.outputs;
    p.k = plan->d.inputs;
    p.a = x;
    p.a_mode = A_STRIDED;
    p.a_row_stride = plan->d.inputs;
    p.a_k_stride = 1;
    p.b = w;
    p.b_col_stride = plan->d.inputs;
    p.b_k_stride = 1;
    p.y = y;
    p.out_mode = OUT_ROW_MAJOR;
    p.ldc = plan->d.outputs;
    p.bias = bias;
    p.bias_mode = bias ? DLP_GEMM_BIAS_N : DLP_GEMM_NO_BIAS;
    p.act = plan->d.activation;

    if(!plan->use_tc)   // the plain-FMA kernel reads the raw weights and needs no scratch at all
        return launch_contraction_ffma(p, 1, 0, 0, plan->d.outputs, (cudaStream_t)stream);

    const size_t need = plan->packed.bytes();
    if(need > size_t(DLP_IP_STATIC_SCRATCH_BYTES))
        return fail(DLP_INVALID_ARGUMENT, "the packed weights need " + std::to_string(need) + " bytes but the static scratch holds "
                                              + std::to_string(size_t(DLP_IP_STATIC_SCRATCH_BYTES))
                                              + "; use dlp_ip_fwd_enqueue with a workspace for this size");
    float *scratch = nullptr;
    dlp_status st = scratch_for_current_device(&scratch);
    if(st != DLP_OK) return st;
    // The pack kernel writes every element of the padded plane, the zero padding included, so nothing
    // left in the array by an earlier call can leak into this one.
    st = tc_prepack(plan->packed, w, plan->d.inputs, 1, plan->d.outputs, plan->d.inputs, scratch, 0, (cudaStream_t)stream);
    if(st != DLP_OK) return st;
    return launch_contraction_tc(p, plan->packed, scratch, (cudaStream_t)stream);
}
