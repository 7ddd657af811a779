// CUDA-core fp32 product C[m,n] (+)= sum_k A(m,k) B(n,k) (+ bias[n]) with
// arbitrary element strides, as a device function: the body of gemm_simt_kernel
// and the path the tensor-core kernels take themselves when the range guard has
// flagged one of their operands (no second launch is needed for the guard).
// 64 x 64 tile, 16-deep k slab, 256 working threads with a 4 x 4 micro-tile each;
// sums run sequentially in k like the reference's inner loops.  Blocks walk the
// tiles grid-stride; threads beyond the first 256 of a block only keep the
// barriers.
#pragma once

#include "common.cuh"
#include "epilogue.cuh"

namespace dlb {

constexpr int ST_M = 64, ST_N = 64, ST_K = 16;
constexpr int SIMT_SMEM_FLOATS = 2 * ST_K * (ST_M + 4);

struct SimtOperands {
  const float *A;
  long long a_sm, a_sk;
  const float *B;
  long long b_sn, b_sk;
};

// `shared` holds SIMT_SMEM_FLOATS floats.  first_tile / tile_stride: the block's
// share of the tiles.  fe: the fused epilogue of the launch, or null.
__device__ __forceinline__ void gemm_simt_body(const SimtOperands &o, float *__restrict__ C, long long ldc, int M,
                                               int N, int K, const float *__restrict__ bias, int accumulate,
                                               float *shared, int first_tile, int tile_stride,
                                               const FusedEpilogue *fe = nullptr) {
  const bool fused = fe && fe->mode != EPI_PLAIN;
  const float plane_scale = fused && fe->sink.hi ? sink_scale(fe->sink) : 1.f;
  float(*As)[ST_M + 4] = reinterpret_cast<float(*)[ST_M + 4]>(shared);
  float(*Bs)[ST_N + 4] = reinterpret_cast<float(*)[ST_N + 4]>(shared + ST_K * (ST_M + 4));
  const int tid = threadIdx.x;
  const bool worker = tid < 256;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  const bool a_k_contig = (o.a_sk == 1), b_k_contig = (o.b_sk == 1);
  const int tiles_n = (N + ST_N - 1) / ST_N, tiles = tiles_n * ((M + ST_M - 1) / ST_M);
  for (int tile = first_tile; tile < tiles; tile += tile_stride) {
    const int m0 = (tile / tiles_n) * ST_M, n0 = (tile % tiles_n) * ST_N;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += ST_K) {
      if (worker) {
        // Loader mapping: the contiguous global direction on consecutive threads.
        for (int i = tid; i < ST_M * ST_K; i += 256) {
          int mm, kk;
          if (a_k_contig) { kk = i % ST_K; mm = i / ST_K; } else { mm = i % ST_M; kk = i / ST_M; }
          const int gm = m0 + mm, gk = k0 + kk;
          As[kk][mm] = (gm < M && gk < K) ? o.A[(long long)gm * o.a_sm + (long long)gk * o.a_sk] : 0.f;
        }
        for (int i = tid; i < ST_N * ST_K; i += 256) {
          int nn, kk;
          if (b_k_contig) { kk = i % ST_K; nn = i / ST_K; } else { nn = i % ST_N; kk = i / ST_N; }
          const int gn = n0 + nn, gk = k0 + kk;
          Bs[kk][nn] = (gn < N && gk < K) ? o.B[(long long)gn * o.b_sn + (long long)gk * o.b_sk] : 0.f;
        }
      }
      __syncthreads();
      if (worker) {
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
      }
      __syncthreads();
    }
    if (worker) {
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
          if (fused) epilogue_element(*fe, c, gm, gn, N, v, plane_scale);
          else *c = accumulate ? *c + v : v;
        }
      }
    }
  }
}

// The same as a call of its own, so that the registers of this rarely taken
// path are not part of the allocation of the tensor-core kernels' main path.
static __device__ __noinline__ void gemm_simt_guard_path(SimtOperands o, float *C, long long ldc, int M, int N,
                                                         int K, const float *bias, int accumulate, float *shared,
                                                         const FusedEpilogue *fe = nullptr) {
  gemm_simt_body(o, C, ldc, M, N, K, bias, accumulate, shared, blockIdx.x, gridDim.x, fe);
}

}  // namespace dlb
