/*
 * dlp_cuda.h -- C ABI of the B200 (sm_100a) convolution / GEMM forward kernels.
 *
 * This is the whole boundary between host code and CUDA: plain C, plain
 * pointers and sizes, no C++ or framework types.  All pointers named x, w,
 * bias, y, ws, a, b, c are DEVICE pointers to dense fp32 data; every call
 * enqueues work on the CUDA stream it is given (passed as void* = cudaStream_t)
 * and returns without synchronising.  Nothing is allocated inside an enqueue
 * call unless its comment says otherwise; scratch memory is sized by the
 * *_workspace() queries and supplied by the caller.
 *
 * Each entry point names the interface of the reference library
 * (artyom-beilis/dlprimitives, paths relative to that project) it stands in for.
 *
 * Every function returns a dlp_status; on failure dlp_last_error() gives a
 * message for the calling thread.
 */
#ifndef DLP_CUDA_H
#define DLP_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DLP_API __attribute__((visibility("default")))
#else
#define DLP_API
#endif

typedef enum dlp_status {
    DLP_OK = 0,
    DLP_INVALID_ARGUMENT = 1, /* the reference throws ValidationError (include/dlprim/definitions.hpp:50-53,74-75) */
    DLP_NOT_IMPLEMENTED = 2,  /* the reference throws NotImplementedError (definitions.hpp:45-48) */
    DLP_CUDA_ERROR = 3,       /* the reference surfaces cl::Error */
    DLP_TIMEOUT = 4           /* a bounded device-side wait gave up; see dlp_device_status() */
} dlp_status;

/* Activation codes: StandardActivations, include/dlprim/definitions.hpp:278-284. */
enum { DLP_ACT_IDENTITY = 0, DLP_ACT_RELU = 1, DLP_ACT_TANH = 2, DLP_ACT_SIGMOID = 3, DLP_ACT_RELU6 = 4 };

/* Arithmetic used by the dense contraction kernels. */
enum {
    DLP_MATH_AUTO = 0,      /* tensor cores where the shape allows, FFMA otherwise */
    DLP_MATH_FP32_FFMA = 1, /* plain fp32 FMA on the CUDA cores */
    DLP_MATH_TF32X3 = 2     /* tcgen05 kind::tf32, three products per term (hi*hi + lo*hi + hi*lo), fp32 accumulate */
};

DLP_API const char *dlp_last_error(void);
DLP_API const char *dlp_version(void);

/* Number of kernels this library has launched from the calling process so far (all threads). */
DLP_API uint64_t dlp_launch_count(void);

/* The tensor-core kernels poll mbarriers with an iteration limit.  When a limit is hit the kernel
 * records a code in a per-device word, drains its copies, frees its tensor memory and returns.
 * This call synchronises `stream`, then reads and clears that word: 0 means no wait ever gave up. */
DLP_API dlp_status dlp_device_status(void *stream, int *code);
/* Self-test of the bounded waits (no counterpart in the reference; its OpenCL kernels have no device-side waits).  Launches a
 * one-CTA kernel whose first warp waits on a barrier nothing arrives at, so that it runs into the time limit (0.4 s), and whose
 * second warp waits on another such barrier and is released by the abort flag the first one raises.  Synchronises the stream.
 * observed[] = { warp 0's wait succeeded (0 expected), milliseconds it waited, the same two for warp 1 }.  Afterwards
 * dlp_device_status() returns DLP_TIMEOUT with code DLP_SELFTEST_WAIT_CODE, and the device is as usable as before. */
#define DLP_SELFTEST_WAIT_CODE 900
DLP_API dlp_status dlp_selftest_wait_expiry(int observed[4], void *stream);
/* The tensor pipe's own dense TF32 rate on the current device, in TFLOP/s (no counterpart in the reference): every SM issues
 * tcgen05.mma.kind::tf32 (M 128, N 128, K 8) back to back with nothing loaded or stored, timed with events on the stream
 * (about 2 ms; synchronises).  The 3xTF32 kernels can reach a third of it.  It is what roofline fractions are put beside. */
DLP_API dlp_status dlp_tf32_mma_rate(double *tflops, void *stream);
/* What an MMA issuing scheme costs, in clock cycles per k-block of twelve tcgen05.mma.kind::tf32 (M 128, N n = 64 or 128, K 8;
 * no counterpart in the reference).  MMA-only like the rate above, with every barrier the loop waits on already complete, so the
 * time is the issuing thread's own: the tensor core's queue is short, and what the thread executes between k-blocks is time the
 * tensor core idles.  scheme 0: one thread, no waits; 1: lanes 0..2 of the warp each wait on one barrier, then a vote; 2: every
 * lane tests the same barriers (uniform instructions; the pointwise kernel's loop with resident weights); 3: two issuer warps taking pairs of
 * k-blocks in turn (what the contraction and staged kernels do).  Synchronises the stream. */
DLP_API dlp_status dlp_tf32_issue_probe(int scheme, int n, double *cycles_per_kblock, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Convolution forward.
 * Stands in for dlprim::core::Conv2DSettings / Conv2DForward::create / workspace / algo / enqueue
 * (include/dlprim/core/conv.hpp:17-58, src/core/conv.cpp:45-111,223-297,457-510,672-729).
 * ---------------------------------------------------------------------------------------------- */
typedef struct dlp_conv2d_desc {
    int channels_in;   /* Convolution2DConfigBase, include/dlprim/definitions.hpp:313-321 */
    int channels_out;
    int kernel[2];
    int stride[2];
    int dilate[2];
    int pad[2];
    int groups;
    int batch;         /* Conv2DSettings::shape: batch is a hint (largest batch expected), H and W of the input */
    int height;
    int width;
    int bias;          /* 0 or 1: whether enqueue receives a bias vector */
    int activation;    /* DLP_ACT_* */
    const char *algo;  /* NULL, "", "auto", "gemm", "winograd" or "depthwise_separable" (src/ops/conv2d.cpp:39-41) */
    int math_mode;     /* DLP_MATH_* */
} dlp_conv2d_desc;

typedef struct dlp_conv2d_plan dlp_conv2d_plan;

/* Output shape rule of Conv2DBase::get_output_shape (src/core/conv.cpp:17-29). */
DLP_API dlp_status dlp_conv2d_output_shape(const dlp_conv2d_desc *desc, int in_h, int in_w, int *out_h, int *out_w);

/* Conv2DForward::create: picks the algorithm with the reference's eligibility rules and builds the
 * launch plan (device-side index tables are allocated here, once). */
DLP_API dlp_status dlp_conv2d_fwd_create(const dlp_conv2d_desc *desc, dlp_conv2d_plan **plan);
DLP_API void dlp_conv2d_fwd_destroy(dlp_conv2d_plan *plan);
/* Conv2DBase::algo(): "gemm", "winograd" or "depthwise_separable". */
DLP_API const char *dlp_conv2d_fwd_algo(const dlp_conv2d_plan *plan);
/* Name of the kernel variant behind the plan, e.g. "igemm_tf32x3_bn128". */
DLP_API const char *dlp_conv2d_fwd_kernel(const dlp_conv2d_plan *plan);
/* Conv2DBase::workspace(): bytes of scratch enqueue needs for the planned batch: the packed weights, plus,
 * for problems with too few output tiles to fill the GPU, room for partial sums over parts of K (the
 * results are added in a fixed order, so they do not depend on timing).  enqueue_packed uses a workspace
 * only for the latter; a short or missing one just turns the split off. */
DLP_API size_t dlp_conv2d_fwd_workspace(const dlp_conv2d_plan *plan);
/* Bytes of the pre-packed form of the weights (0 when the kernel reads raw weights). */
DLP_API size_t dlp_conv2d_fwd_packed_bytes(const dlp_conv2d_plan *plan);
/* Pack the weights once (TF32 hi/lo split into padded K-major tiles, or the Winograd filter
 * transform).  The reference redoes its filter transform on every call (src/core/conv.cpp:262-269);
 * inference weights are constant, so callers that own them can pack once and use enqueue_packed. */
DLP_API dlp_status dlp_conv2d_fwd_prepack(const dlp_conv2d_plan *plan, const float *w, void *packed, void *stream);

/* Conv2DForward::enqueue(x, w, bias, y, ws, factor, e):  y = factor * y + act(conv(x, w) + bias).
 * y is not read when factor == 0.  batch/in_h/in_w are the actual sizes of x (the reference re-reads
 * them from the tensors, src/core/conv.cpp:59-62); batch may be smaller than planned, and H/W must
 * match the plan.  ws must hold dlp_conv2d_fwd_workspace() bytes (may be NULL when that is 0). */
DLP_API dlp_status dlp_conv2d_fwd_enqueue(const dlp_conv2d_plan *plan, const float *x, const float *w, const float *bias,
                                          float *y, void *ws, size_t ws_bytes, float factor, int batch, int in_h, int in_w,
                                          void *stream);

/* Same contract with weights already packed by dlp_conv2d_fwd_prepack, plus an optional fused
 * residual: when `residual` is not NULL the result is
 *     y = post_act( act(conv + bias) * 1 + residual_scale * residual )
 * which is the reference's Convolution2D followed by Elementwise("sum", coef2 = residual_scale,
 * activation = post_act) (src/ops/elementwise.cpp:517-559) without the extra pass over memory.
 * residual has the shape of y and may alias it.  factor must be 0 when a residual is given. */
DLP_API dlp_status dlp_conv2d_fwd_enqueue_packed(const dlp_conv2d_plan *plan, const float *x, const void *packed,
                                                 const float *bias, float *y, void *ws, size_t ws_bytes, float factor,
                                                 const float *residual, float residual_scale, int post_activation,
                                                 int batch, int in_h, int in_w, void *stream);

/* ------------------------------------------------------------------------------------------------
 * GEMM.  Stands in for dlprim::gpu::GEMM::get_optimal_gemm / gemm / batch_sgemm
 * (include/dlprim/gpu/gemm.hpp:15-82, src/gemm.cpp:240-426,567-579):
 *     C[M,N] = beta * C + act(op(A) * op(B) + bias),   row-major, offsets folded into the pointers.
 * Transposition, bias mode and activation are fixed at creation, as in the reference.
 * ---------------------------------------------------------------------------------------------- */
enum { DLP_GEMM_NO_BIAS = 0, DLP_GEMM_BIAS_M = 1, DLP_GEMM_BIAS_N = 2 };

typedef struct dlp_gemm_desc {
    int trans_a, trans_b;
    int m, n, k;       /* planning hint; the call-time sizes may be smaller or equal */
    int bias_mode;     /* DLP_GEMM_* */
    int activation;    /* DLP_ACT_* */
    int math_mode;     /* DLP_MATH_* */
} dlp_gemm_desc;

typedef struct dlp_gemm_plan dlp_gemm_plan;

DLP_API dlp_status dlp_gemm_create(const dlp_gemm_desc *desc, dlp_gemm_plan **plan);
DLP_API void dlp_gemm_destroy(dlp_gemm_plan *plan);
DLP_API const char *dlp_gemm_kernel(const dlp_gemm_plan *plan);
DLP_API size_t dlp_gemm_workspace(const dlp_gemm_plan *plan);
DLP_API dlp_status dlp_gemm_enqueue(const dlp_gemm_plan *plan, int m, int n, int k, const float *a, int lda, const float *b,
                                    int ldb, float *c, int ldc, const float *bias, float beta, void *ws, size_t ws_bytes,
                                    void *stream);
/* GEMM::batch_sgemm (src/gemm.cpp:603-638): `batch` independent products with element strides between matrices, in one
 * launch (plus one launch that packs every B for tensor-core plans).  ws: dlp_gemm_batched_workspace(plan, batch) bytes. */
DLP_API size_t dlp_gemm_batched_workspace(const dlp_gemm_plan *plan, int batch);
DLP_API dlp_status dlp_gemm_batched_enqueue(const dlp_gemm_plan *plan, int batch, int m, int n, int k, const float *a,
                                            long long stride_a, int lda, const float *b, long long stride_b, int ldb, float *c,
                                            long long stride_c, int ldc, float beta, void *ws, size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------------------------------------
 * InnerProduct forward.  Stands in for dlprim::core::IPSettings / IPForward::create / enqueue
 * (include/dlprim/core/ip.hpp:19-45, src/core/ip.cpp:15-50):
 *     y[batch, outputs] = act(x[batch, inputs] * w[outputs, inputs]^T + bias[outputs]).
 * ---------------------------------------------------------------------------------------------- */
typedef struct dlp_ip_desc {
    int inputs, outputs;
    int optimal_batch_size;
    int bias;
    int activation;
    int math_mode;
} dlp_ip_desc;

typedef struct dlp_ip_plan dlp_ip_plan;

DLP_API dlp_status dlp_ip_fwd_create(const dlp_ip_desc *desc, dlp_ip_plan **plan);
DLP_API void dlp_ip_fwd_destroy(dlp_ip_plan *plan);
DLP_API const char *dlp_ip_fwd_kernel(const dlp_ip_plan *plan);
DLP_API size_t dlp_ip_fwd_workspace(const dlp_ip_plan *plan);
DLP_API size_t dlp_ip_fwd_packed_bytes(const dlp_ip_plan *plan);
DLP_API dlp_status dlp_ip_fwd_prepack(const dlp_ip_plan *plan, const float *w, void *packed, void *stream);
DLP_API dlp_status dlp_ip_fwd_enqueue(const dlp_ip_plan *plan, const float *x, const float *w, const float *bias, float *y,
                                      void *ws, size_t ws_bytes, int batch, void *stream);
/* ws: optional scratch (dlp_ip_fwd_workspace() bytes at most are used) that lets a small batch use the whole GPU. */
DLP_API dlp_status dlp_ip_fwd_enqueue_packed(const dlp_ip_plan *plan, const float *x, const void *packed, const float *bias,
                                             float *y, void *ws, size_t ws_bytes, int batch, void *stream);

/* InnerProduct forward without any device allocation and without a caller workspace.
 * It has no counterpart in the reference library.  It exists for callers that are not allowed to
 * allocate device memory at the point where they need the result -- a plugin running inside another
 * framework's memory pool, code called from an allocator callback, a harness where cudaMalloc is
 * forbidden -- and therefore cannot hand dlp_ip_fwd_enqueue the workspace it asks for.  The scratch
 * for the packed weights is a fixed array of DLP_IP_STATIC_SCRATCH_BYTES inside the library's device
 * image; every GPU on which the entry point has been called holds that much memory until the process exits.
 *   - Same arguments and result as dlp_ip_fwd_enqueue minus the workspace.
 *   - Plans whose packed weights exceed DLP_IP_STATIC_SCRATCH_BYTES are refused with
 *     DLP_INVALID_ARGUMENT and a message giving both sizes.  Packed weights take
 *     2 * round_up(outputs, 128) * round_up(inputs, 32) * 4 bytes, so a 2048 -> 1000 layer needs exactly
 *     16 MiB and sits on the limit: 2049 inputs, or 1025 outputs at 2048 inputs, are refused.
 *   - The first call on each device looks up the array's device address.  With the CUDA runtime's lazy
 *     module loading that look-up is also the moment the array's memory is reserved on that device, so it
 *     can fail with an out-of-memory error if everything has been given away by then: make the first call
 *     on each device at start-up, while memory is still available, and before starting any stream capture.
 *     From then on the array stays resident until the process exits.
 *   - All calls on a device share the one array, which still holds the previous call's data when the
 *     next one starts (each call overwrites all of it).  Two calls whose kernels may run at the same
 *     time -- different streams without ordering, or several host threads -- race on it: order them.
 *   - Neither this call nor anything it calls uses cudaMalloc, cudaFree or another allocating routine. */
#define DLP_IP_STATIC_SCRATCH_BYTES (16u << 20)
DLP_API dlp_status dlp_ip_fwd_enqueue_static(const dlp_ip_plan *plan, const float *x, const float *w, const float *bias, float *y,
                                             int batch, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Bandwidth-bound operators the inference graph needs between convolutions.
 * ---------------------------------------------------------------------------------------------- */
/* Pooling2D forward (src/ops/pooling.cpp:282-329, include/dlprim/core/pool.hpp:17-27).  mode 0 max, 1 avg. */
DLP_API dlp_status dlp_pooling2d_output_shape(int in_h, int in_w, const int kernel[2], const int stride[2], const int pad[2],
                                              int ceil_mode, int *out_h, int *out_w);
DLP_API dlp_status dlp_pooling2d_fwd(const float *x, float *y, int planes, int in_h, int in_w, const int kernel[2],
                                     const int stride[2], const int pad[2], int ceil_mode, int mode, int count_include_pad,
                                     void *stream);
/* GlobalPooling forward (src/ops/pooling.cpp:427-450): [planes, plane_size] -> [planes].  mode 0 max, 1 avg. */
DLP_API dlp_status dlp_global_pooling_fwd(const float *x, float *y, int planes, int plane_size, int mode, void *stream);
/* Elementwise forward, same-shape operands (src/ops/elementwise.cpp:517-559).  op 0 sum, 1 prod, 2 max. */
DLP_API dlp_status dlp_elementwise_fwd(const float *a, const float *b, float *c, size_t count, int op, float coef1, float coef2,
                                       int activation, void *stream);
/* Activation forward, in place allowed (src/ops/activation.cpp:53-110). */
DLP_API dlp_status dlp_activation_fwd(const float *x, float *y, size_t count, int activation, void *stream);
/* Softmax / log-softmax over dim 1 of [rows, classes, inner] (src/ops/softmax.cpp:189-222). */
DLP_API dlp_status dlp_softmax_fwd(const float *x, float *y, int rows, int classes, int inner, int log_mode, void *stream);
/* BatchNorm in inference, y = A*x + B per channel with A, B from running statistics
 * (src/ops/batch_normalization.cpp:192-228).  gamma/beta may be NULL (affine = false). */
DLP_API dlp_status dlp_batchnorm_inference_fwd(const float *x, float *y, int batch, int features, int plane, float eps,
                                               const float *mean, const float *var, const float *gamma, const float *beta,
                                               void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DLP_CUDA_H */
