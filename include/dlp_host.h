/*
 * dlp_host.h -- plain-C face of the C++ host library (libdlprim_b200.so).
 *
 * The host API proper is C++ (include/dlprim/: Context, Tensor, core::Conv2DForward, gpu::GEMM,
 * the operators and Net, with the reference's own names).  These entry points let a language
 * without a C++ binding -- the Python tests and the benchmark here -- drive the same objects:
 * an operator made by the factory (what the reference's test driver does,
 * tests/test_from_template.cpp:219-448) and a whole Net (tools/benchmark.cpp:71-259).
 *
 * Tensors passed as "device" pointers are device memory; "host" pointers are host memory.
 * Every function that can fail returns 0 on success and non-zero on failure, after which
 * dlp_host_last_error() describes the exception that was caught (its class name first).
 */
#ifndef DLP_HOST_H
#define DLP_HOST_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

#define DLP_HOST_API __attribute__((visibility("default")))

DLP_HOST_API const char *dlp_host_last_error(void);

/* ---- one operator: create_by_name + setup (include/dlprim/operator.hpp) ---- */
typedef struct dlp_op dlp_op;
DLP_HOST_API int dlp_op_create(const char *type, const char *options_json, int device, int n_inputs, const int *ranks,
                               const int *dims, dlp_op **out);
DLP_HOST_API void dlp_op_destroy(dlp_op *op);
DLP_HOST_API int dlp_op_num_outputs(const dlp_op *op);
DLP_HOST_API int dlp_op_num_params(const dlp_op *op);
DLP_HOST_API int dlp_op_output_shape(const dlp_op *op, int index, int *dims);   /* returns the rank */
DLP_HOST_API int dlp_op_param_shape(const dlp_op *op, int index, int *dims);
DLP_HOST_API size_t dlp_op_workspace(const dlp_op *op);
/* "<algo> <kernel>" for Convolution2D, "<kernel>" for InnerProduct, "" otherwise */
DLP_HOST_API const char *dlp_op_kernel(const dlp_op *op);
/* Operator::reshape with new input shapes */
DLP_HOST_API int dlp_op_reshape(dlp_op *op, int n_inputs, const int *ranks, const int *dims);
/* Operator::forward on device buffers laid out as the current shapes say; ws holds dlp_op_workspace() bytes */
DLP_HOST_API int dlp_op_forward(dlp_op *op, void *const *device_inputs, void *const *device_params, void *const *device_outputs,
                                void *device_ws, void *stream);

/* ---- a whole network (include/dlprim/net.hpp) ---- */
typedef struct dlp_net dlp_net;
/* flags: bit 0 keep intermediate tensors, bit 1 no operator fusion, bit 2 no CUDA graph, bit 3 run Net::merge_activations on
 * the description first, bit 4 concurrent branches (Net::concurrent_branches: projection shortcuts on a second stream) */
DLP_HOST_API int dlp_net_create(const char *net_json, int device, int flags, dlp_net **out);
DLP_HOST_API void dlp_net_destroy(dlp_net *net);
DLP_HOST_API int dlp_net_num_params(const dlp_net *net);
DLP_HOST_API int dlp_net_param_name(const dlp_net *net, int index, char *buf, int buf_size);
DLP_HOST_API int dlp_net_param_shape(dlp_net *net, const char *name, int *dims);     /* rank, or -1 */
DLP_HOST_API int dlp_net_tensor_shape(dlp_net *net, const char *name, int *dims);    /* rank, or -1 */
/* copy into the parameter's host mirror; dlp_net_upload_params() sends all mirrors to the device */
DLP_HOST_API int dlp_net_set_param(dlp_net *net, const char *name, const float *host_data, size_t count);
DLP_HOST_API int dlp_net_upload_params(dlp_net *net);
DLP_HOST_API int dlp_net_load_params_file(dlp_net *net, const char *path);
DLP_HOST_API int dlp_net_save_params_file(dlp_net *net, const char *path);
/* Tensor::to_device / to_host for a named tensor, asynchronous on the stream (host memory should be pinned) */
DLP_HOST_API int dlp_net_set_tensor(dlp_net *net, const char *name, const float *host_data, size_t count, void *stream);
DLP_HOST_API int dlp_net_get_tensor(dlp_net *net, const char *name, float *host_data, size_t count, void *stream);
DLP_HOST_API void *dlp_net_tensor_device_ptr(dlp_net *net, const char *name);
DLP_HOST_API int dlp_net_reshape_input(dlp_net *net, const char *name, int rank, const int *dims);
DLP_HOST_API int dlp_net_reshape(dlp_net *net);
DLP_HOST_API int dlp_net_forward(dlp_net *net, void *stream, int sync);
/* One forward pass run operator by operator with a CUDA-event pair around every step of the plan
 * (ExecutionContext timing, include/dlprim/context.hpp); step_ms receives dlp_net_num_steps() values.
 * Synchronises the stream. */
DLP_HOST_API int dlp_net_forward_timed(dlp_net *net, void *stream, float *step_ms, int capacity);
/* device-to-device copies between a named tensor and caller-owned device memory, asynchronous on the stream */
DLP_HOST_API int dlp_net_copy_tensor_to_device(dlp_net *net, const char *name, void *device_dst, size_t count, void *stream);
DLP_HOST_API int dlp_net_copy_tensor_from_device(dlp_net *net, const char *name, const void *device_src, size_t count, void *stream);
DLP_HOST_API int dlp_net_num_steps(const dlp_net *net);
DLP_HOST_API int dlp_net_step_description(const dlp_net *net, int index, char *buf, int buf_size);
DLP_HOST_API size_t dlp_net_activation_bytes(const dlp_net *net, int without_reuse);

/* Net::merge_activations on a network description given as JSON text (no device involved): writes the resulting description
 * into out (capacity bytes, NUL-terminated) and returns the number of Activation operators merged, or -1 on failure. */
DLP_HOST_API int dlp_host_merge_activations(const char *net_json, char *out, size_t capacity);

/* ---- gpu::GEMM (include/dlprim/gpu/gemm.hpp), on device buffers; each call makes the object, runs it and lets it go ---- */
/* GEMM::get_optimal_gemm(...)->gemm(...): C[M,N] = beta*C + act(op(A)*op(B) + bias); the object is made for (plan_m, plan_n,
 * plan_k) and called with (M, N, K), which may be larger */
DLP_HOST_API int dlp_host_gemm(int device, int trans_a, int trans_b, int plan_m, int plan_n, int plan_k, int M, int N, int K, int bias_mode,
                               int activation, void *a, int lda, void *b, int ldb, void *c, int ldc, void *bias, float beta, void *stream);
/* GEMM::batch_sgemm: asynchronous on the stream */
DLP_HOST_API int dlp_host_batch_sgemm(int device, int trans_a, int trans_b, int batch, int M, int N, int K, void *a, int stride_a, int lda,
                                      void *b, int stride_b, int ldb, void *c, int stride_c, int ldc, float beta, void *stream);
/* GEMM::get_optimal_conv_gemm(forward)->gemm(...) called the way the reference's Conv2DForwardGEMM calls it: geometry[] =
 * kernel h,w, dilate h,w, pad h,w, stride h,w, groups, src_channels (per group), src_rows, src_cols, tgt_rows, tgt_cols */
DLP_HOST_API int dlp_host_conv_gemm(int device, const int geometry[14], int channels_out_per_group, int batch, int with_bias, int activation,
                                    void *filters, void *x, void *y, void *bias, float factor, void *stream);

#ifdef __cplusplus
}
#endif
#endif
