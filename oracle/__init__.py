"""CPU checker for the convolution / GEMM forward path.  Test infrastructure only."""
