// dlprim::gpu::GEMM -- row-major  C[M,N] = beta*C + act(op(A)*op(B) + bias).
// Drop-in for the reference's include/dlprim/gpu/gemm.hpp:15-82 with cl::Buffer& replaced by a
// device pointer; offsets stay in elements.  Transposition, bias mode and activation are fixed when
// the object is created, sizes, pointers, leading dimensions and beta at call time.
#pragma once
#include <dlprim/context.hpp>
#include <dlprim/definitions.hpp>
#include <memory>

namespace dlprim {
namespace gpu {

    typedef void *DeviceBuffer;      ///< base address of a device allocation (stands in for cl::Buffer)
    typedef unsigned long long offset_type;

    class DLPRIM_API GEMM {
    public:
        virtual ~GEMM() {}
        static constexpr int no_bias = 0;
        static constexpr int bias_M = 1;
        static constexpr int bias_N = 2;

        virtual void gemm(int M, int N, int K,
                          DeviceBuffer a, offset_type offset_a, int lda,
                          DeviceBuffer b, offset_type offset_b, int ldb,
                          DeviceBuffer c, offset_type offset_c, int ldc,
                          DeviceBuffer bias, offset_type bias_offset,
                          float beta, int size_of_c, ExecutionContext const &e) = 0;

        static void batch_sgemm(DataType dt, bool trans_a, bool trans_b, int Batch, int M, int N, int K,
                                DeviceBuffer a, offset_type offset_a, int batch_stride_a, int lda,
                                DeviceBuffer b, offset_type offset_b, int batch_stride_b, int ldb,
                                DeviceBuffer c, offset_type offset_c, int batch_stride_c, int ldc,
                                float beta, ExecutionContext const &e);

        static std::unique_ptr<GEMM> get_optimal_gemm(Context &ctx, DataType dtype, bool trans_a, bool trans_b, int M, int N, int K,
                                                      int bias = 0, StandardActivations act = StandardActivations::identity,
                                                      int im2col_chan = 0);

        /// The convolution as a GEMM with implicit im2col (include/dlprim/gpu/gemm.hpp:70-80, src/gemm.cpp:581-601 in the
        /// reference).  gemm() is then called the way Conv2DForwardGEMM calls it (src/core/conv.cpp:51-80): a = the
        /// filters [M = Cout/groups, K], b = the NCHW input, c = the NCHW output with N = batch * tgt_rows * tgt_cols
        /// columns, bias per M, beta = the output's factor.  Only GemmOpMode::forward is implemented.
        static std::unique_ptr<GEMM> get_optimal_conv_gemm(Context &ctx, DataType dtype, GemmOpMode op_mode, bool trans_a, bool trans_b,
                                                           int M, int N, int K, int kernel[2], int dilate[2], int padding[2],
                                                           int stride[2], int groups, int src_channels, int src_rows, int src_cols,
                                                           int tgt_rows, int tgt_cols, int bias = 0,
                                                           StandardActivations act = StandardActivations::identity, int im2col_chan = 0);
    };

} // namespace gpu
} // namespace dlprim
