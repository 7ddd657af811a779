// CUDA-core fp32 GEMM with arbitrary element strides (gemm_simt.cuh):
//   C[m,n] (+)= sum_k A(m,k) * B(n,k) (+ bias[n]).
// It serves the shapes the TMA/tcgen05 kernel cannot express (row pitches that
// are not multiples of 16 bytes, e.g. a 10-unit output layer), and it is the
// in-tree fp32 check for the tensor-core kernel.
#include "gemm_simt.cuh"

namespace dlb {

__global__ void __launch_bounds__(256)
    gemm_simt_kernel(SimtOperands o, float *__restrict__ C, long long ldc, int M, int N, int K,
                     const float *__restrict__ bias, int accumulate) {
  pdl_enter();
  __shared__ float shared[SIMT_SMEM_FLOATS];
  gemm_simt_body(o, C, ldc, M, N, K, bias, accumulate, shared, blockIdx.x, gridDim.x);
}

dlb_status gemm_simt(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                     long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  const int grid = ceil_div(N, ST_N) * ceil_div(M, ST_M);
  DLB_LAUNCH_KERNEL(ctx, gemm_simt_kernel, grid, 256, 0, SimtOperands{A.ptr, A.stride_mn, A.stride_k, B.ptr, B.stride_mn, B.stride_k}, C, ldc, M, N, K, ep.bias, ep.accumulate);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // namespace dlb
