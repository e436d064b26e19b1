// Shared host/device helpers of the CUDA library: status handling, activation functions, launch counting.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>
#include <atomic>

#include "../../include/dlp_cuda.h"

namespace dlp {

// ---- host side: per-thread error message, launch counter --------------------------------------
void set_error(const std::string &msg);
dlp_status fail(dlp_status st, const std::string &msg);
dlp_status check_cuda(cudaError_t e, const char *what);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(uint64_t(n), std::memory_order_relaxed); }
int sm_count();

#define DLP_REQUIRE(cond, msg)                                                             \
    do {                                                                                   \
        if(!(cond)) return ::dlp::fail(DLP_INVALID_ARGUMENT, std::string("Failed " #cond ": ") + (msg)); \
    } while(0)

#define DLP_CUDA_OK(expr)                                                                  \
    do {                                                                                   \
        dlp_status st__ = ::dlp::check_cuda((expr), #expr);                                \
        if(st__ != DLP_OK) return st__;                                                    \
    } while(0)

#define DLP_LAUNCH_OK(name)                                                                \
    do {                                                                                   \
        ::dlp::count_launch();                                                             \
        dlp_status st__ = ::dlp::check_cuda(cudaPeekAtLastError(), name);                  \
        if(st__ != DLP_OK) return st__;                                                    \
    } while(0)

// ---- device side ---------------------------------------------------------------------------------
// Activation definitions shared by every epilogue; they follow the reference's device macros
// (src/kernels/defs.h:27-49) and its CPU versions (include/dlprim/cpu/cpu_ops.hpp:16-53).
// tanhf/expf are the accurate library forms, not the .approx instructions.
__device__ __forceinline__ float apply_act(float v, int act)
{
    switch(act) {
    case DLP_ACT_RELU: return fmaxf(v, 0.0f);
    case DLP_ACT_TANH: return tanhf(v);
    case DLP_ACT_SIGMOID: return 1.0f / (1.0f + expf(-v));
    case DLP_ACT_RELU6: return fminf(fmaxf(v, 0.0f), 6.0f);
    default: return v;
    }
}

template<typename T> __host__ __device__ inline T ceil_div(T a, T b) { return (a + b - 1) / b; }
template<typename T> __host__ __device__ inline T round_up(T a, T b) { return ceil_div(a, b) * b; }

// Device address of the per-device status word written by kernels whose bounded waits gave up
// (0 = healthy).  Resolved once per device; never allocates.
int *device_status_word();

} // namespace dlp
