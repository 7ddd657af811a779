// CUDA-core fp32 GEMM with arbitrary element strides:
//   C[m,n] (+)= sum_k A(m,k) * B(n,k) (+ bias[n]).
// It serves the shapes the TMA/tcgen05 kernel cannot express (row pitches that
// are not multiples of 16 bytes, e.g. a 10-unit output layer), and it is the
// in-tree fp32 check for the tensor-core kernel.  64x64 tile, 16-deep k slab,
// 256 threads with a 4x4 micro-tile each; sums run sequentially in k like the
// reference's inner loops.
#include "common.cuh"

namespace dlb {

constexpr int ST_M = 64, ST_N = 64, ST_K = 16;

__global__ void __launch_bounds__(256)
    gemm_simt_kernel(const float *__restrict__ A, long long a_sm, long long a_sk,
                     const float *__restrict__ B, long long b_sn, long long b_sk,
                     float *__restrict__ C, long long ldc, int M, int N, int K,
                     const float *__restrict__ bias, int accumulate) {
  __shared__ float As[ST_K][ST_M + 4];
  __shared__ float Bs[ST_K][ST_N + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * ST_M, n0 = blockIdx.x * ST_N;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  // Loader mapping: put the contiguous global direction on consecutive threads.
  const bool a_k_contig = (a_sk == 1), b_k_contig = (b_sk == 1);
  for (int k0 = 0; k0 < K; k0 += ST_K) {
    for (int i = tid; i < ST_M * ST_K; i += 256) {
      int mm, kk;
      if (a_k_contig) { kk = i % ST_K; mm = i / ST_K; } else { mm = i % ST_M; kk = i / ST_M; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? A[(long long)gm * a_sm + (long long)gk * a_sk] : 0.f;
    }
    for (int i = tid; i < ST_N * ST_K; i += 256) {
      int nn, kk;
      if (b_k_contig) { kk = i % ST_K; nn = i / ST_K; } else { nn = i % ST_N; kk = i / ST_N; }
      const int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < N && gk < K) ? B[(long long)gn * b_sn + (long long)gk * b_sk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < ST_K; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      float *c = C + (long long)gm * ldc + gn;
      *c = accumulate ? *c + v : v;
    }
  }
}

dlb_status gemm_simt(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                     long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  dim3 grid(ceil_div(N, ST_N), ceil_div(M, ST_M));
  gemm_simt_kernel<<<grid, 256, 0, ctx->stream>>>(A.ptr, A.stride_mn, A.stride_k, B.ptr,
                                                  B.stride_mn, B.stride_k, C, ldc, M, N, K,
                                                  ep.bias, ep.accumulate);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // namespace dlb
