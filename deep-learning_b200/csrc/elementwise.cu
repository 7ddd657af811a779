// HBM-bound kernels of the fully-connected step: batch-renormalization sums,
// finalize, normalise + activation + dropout, their backward passes, softmax,
// output error, and the TF32 residual split.  All are streaming kernels with
// 128-bit accesses; per-unit (column) reductions go through partials in the
// context scratch arena and are finished in double in a fixed order, so results
// do not depend on block scheduling.
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "math.cuh"
#include "planes.cuh"
#include "ring.cuh"

namespace dlb {

// ---------------------------------------------------------------------------
// Column reductions over a row-major [rows, n] tensor.
//
// Grid (column blocks, row chunks).  A block of 256 threads covers 128 columns
// (32 lanes x float4) and 8 row lanes; each thread walks its rows with stride
// 8 accumulating NSUM float4 in registers, the 8 row lanes are folded through
// shared memory in double, and the block writes NSUM x 128 doubles to
// partials[chunk][s][col].  reduce_partials then sums the chunks in order.
// ---------------------------------------------------------------------------
// 32 x 8 threads: 64 x 4 (1 KB of a row per block) was measured within 3 % either
// way on every kernel of the family.
constexpr int CR_LANES_X = 32;
constexpr int CR_LANES_Y = 8;
constexpr int CR_COLS = CR_LANES_X * 4;
// Most blocks per SM a plan counts on.  Capping the kernels' registers so that
// every one of them reaches it was measured and is slower (the backward
// reduction: 74 us at 64 registers with spills against 55 us at 71 registers
// and three blocks per SM).
constexpr int CR_MAX_PER_SM = 4;

// Shared memory of a reduction block: the copy ring while it walks the rows,
// then the fold of the 8 row lanes.
template <int NSUM, class Op>
constexpr size_t column_reduce_shared_bytes() {
  const size_t ring = ring_bytes(Op::NIN, Op::DEPTH > 0 ? Op::DEPTH : 0, CR_LANES_X * CR_LANES_Y);
  const size_t fold = sizeof(double) * CR_LANES_Y * NSUM * (CR_COLS + 1);
  return ring > fold ? ring : fold;
}

template <int NSUM, class Op>
__global__ void __launch_bounds__(CR_LANES_X *CR_LANES_Y, Op::MIN_BLOCKS)
    column_reduce_kernel(Op op, int rows, int n, int rows_per_chunk, double *partials) {
  pdl_enter();
  extern __shared__ float4 cr_shared[];
  const int tx = threadIdx.x % CR_LANES_X, ty = threadIdx.x / CR_LANES_X;
  const int col = blockIdx.x * CR_COLS + tx * 4;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  float acc[NSUM][4];
#pragma unroll
  for (int s = 0; s < NSUM; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[s][j] = 0.f;

  if (col < n) {
    if ((n & 3) == 0) {
      typename Op::Cols4 c;
      op.load_cols4(col, c);
      // The rows come through the thread's copy ring (Op::DEPTH - 1 rows of
      // Op::NIN tensors under way); the sums take them in ascending order.
      const float *in[Op::NIN];
      op.inputs(in);
      if constexpr (Op::DEPTH > 0) {
        ring_walk<Op::NIN, Op::DEPTH, CR_LANES_X * CR_LANES_Y>(cr_shared, in, (size_t)n, col, r0 + ty, r1, CR_LANES_Y,
                                      [&](int r, const float4(&x)[Op::NIN]) { op.use4(r, col, c, x, acc); });
      } else {
        // Read-only kernels with registers to spare: Op::IN_FLIGHT rows per
        // iteration by plain loads, all of them sent before the first is used.
        constexpr int U = Op::IN_FLIGHT;
        for (int r = r0 + ty; r < r1; r += U * CR_LANES_Y) {
          float4 x[U][Op::NIN];
#pragma unroll
          for (int k = 0; k < U; ++k)
            if (r + k * CR_LANES_Y < r1) {
#pragma unroll
              for (int i = 0; i < Op::NIN; ++i)
                x[k][i] = __ldg(reinterpret_cast<const float4 *>(in[i] + (size_t)(r + k * CR_LANES_Y) * n + col));
            }
#pragma unroll
          for (int k = 0; k < U; ++k)
            if (r + k * CR_LANES_Y < r1) op.use4(r + k * CR_LANES_Y, col, c, x[k], acc);
        }
      }
    } else {
      for (int j = 0; j < 4 && col + j < n; ++j) {
        typename Op::Cols1 c;
        op.load_cols1(col + j, c);
        float a1[NSUM];
#pragma unroll
        for (int s = 0; s < NSUM; ++s) a1[s] = 0.f;
        for (int r = r0 + ty; r < r1; r += CR_LANES_Y) op.row1(r, col + j, c, a1);
#pragma unroll
        for (int s = 0; s < NSUM; ++s) acc[s][j] = a1[s];
      }
    }
  }
  ring_drain();
  double(*red)[NSUM][CR_COLS + 1] = reinterpret_cast<double(*)[NSUM][CR_COLS + 1]>(cr_shared);
#pragma unroll
  for (int s = 0; s < NSUM; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) red[ty][s][tx * 4 + j] = (double)acc[s][j];
  __syncthreads();
  // 256 threads fold NSUM*128 columns.
  for (int i = threadIdx.x; i < NSUM * CR_COLS; i += CR_LANES_X * CR_LANES_Y) {
    const int s = i / CR_COLS, c = i % CR_COLS;
    const int gc = blockIdx.x * CR_COLS + c;
    if (gc < n) {
      double t = 0.0;
#pragma unroll
      for (int y = 0; y < CR_LANES_Y; ++y) t += red[y][s][c];
      partials[((size_t)blockIdx.y * NSUM + s) * n + gc] = t;
    }
  }
}

__global__ void reduce_partials_kernel(const double *partials, int chunks, int total, double *out) {
  pdl_enter();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  double t = 0.0;
  for (int c = 0; c < chunks; ++c) t += partials[(size_t)c * total + i];
  out[i] = t;
}

// Chunking of the rows: one wave of blocks over the SMs, CR_MAX_PER_SM blocks on
// each or as many as `resident` (what an SM holds of the kernel) allows if that
// is fewer; a grid larger than what is resident at once leaves a partial second
// wave that costs a whole one.  Chunks of at least 64 rows.
static void column_reduce_plan(int sm_count, int rows, int n, int resident, int *chunks, int *rows_per_chunk) {
  const int col_blocks = ceil_div(n, CR_COLS);
  const int target = max(1, min(resident, CR_MAX_PER_SM));
  int c = ceil_div(sm_count * target, col_blocks);
  if ((long long)c * col_blocks > (long long)sm_count * resident) c = max(1, sm_count * target / col_blocks);
  c = max(1, min(c, ceil_div(rows, 64)));
  *rows_per_chunk = ceil_div(ceil_div(rows, c), CR_LANES_Y) * CR_LANES_Y;
  *chunks = ceil_div(rows, *rows_per_chunk);
}

// Room for the partials of any kernel of the family (callers place their final
// sums behind them in the same scratch request).
static size_t column_reduce_partial_bytes(dlb_ctx *ctx, int nsum, int rows, int n) {
  int chunks, rpc;
  column_reduce_plan(ctx->sm_count, rows, n, 1 << 20, &chunks, &rpc);  // the most chunks any kernel's plan makes
  return align_up((size_t)chunks * nsum * n * sizeof(double), 256);
}

// Lets `Kernel` take `bytes` of dynamic shared memory on the current device
// (needed above 48 KB); once per kernel and device.
template <auto Kernel>
static void kernel_shared_limit(size_t bytes) {
  static bool done[MAX_DEVICES] = {};
  int dev = 0;
  if (bytes <= 48 * 1024 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || done[dev]) return;
  if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess)
    done[dev] = true;
  else
    cudaGetLastError();
}

// Blocks of one reduction kernel an SM of the current device holds.  The query
// allocates nothing.
template <int NSUM, class Op>
static int column_reduce_per_sm() {
  int blocks = CR_MAX_PER_SM;
  kernel_shared_limit<column_reduce_kernel<NSUM, Op>>(column_reduce_shared_bytes<NSUM, Op>());
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, column_reduce_kernel<NSUM, Op>, CR_LANES_X * CR_LANES_Y,
                                                    column_reduce_shared_bytes<NSUM, Op>()) != cudaSuccess) {
    cudaGetLastError();
    blocks = CR_MAX_PER_SM;
  }
  return max(1, blocks);
}

template <int NSUM, class Op>
static dlb_status column_reduce(dlb_ctx *ctx, Op op, int rows, int n, double *out) {
  const int col_blocks = ceil_div(n, CR_COLS);
  static int per_sm_of[MAX_DEVICES] = {};  // 0: not asked yet on that device
  int &per_sm = per_sm_of[ctx->device];
  if (per_sm == 0) per_sm = column_reduce_per_sm<NSUM, Op>();
  int chunks, rows_per_chunk;
  column_reduce_plan(ctx->sm_count, rows, n, per_sm, &chunks, &rows_per_chunk);
  void *scr = nullptr;
  DLB_TRY(scratch(ctx, column_reduce_partial_bytes(ctx, NSUM, rows, n), &scr));
  double *partials = static_cast<double *>(scr);
  DLB_LAUNCH_KERNEL(ctx, (column_reduce_kernel<NSUM, Op>), dim3(col_blocks, chunks), CR_LANES_X * CR_LANES_Y, (column_reduce_shared_bytes<NSUM, Op>()), op, rows, n, rows_per_chunk, partials);
  DLB_LAUNCHED(ctx);
  const int total = NSUM * n;
  DLB_LAUNCH_KERNEL(ctx, reduce_partials_kernel, ceil_div(total, 256), 256, 0, partials, chunks, total, out);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// --- sum(z), sum(z^2) --------------------------------------------------------
// The two read-only reductions use plain loads, four rows per thread in flight:
// six or eight in flight, or the copy ring, leave the 64 MiB pass where it is
// (15.1 - 15.7 us with its second launch; 10 us of it is the transfer).
struct SumSqOp {
  const float *Z;
  int n;
  struct Cols4 {};
  struct Cols1 {};
  __device__ void load_cols4(int, Cols4 &) const {}
  __device__ void load_cols1(int, Cols1 &) const {}
  static constexpr int NIN = 1, DEPTH = 0, IN_FLIGHT = 4, MIN_BLOCKS = 1;
  __device__ void inputs(const float *(&in)[1]) const { in[0] = Z; }
  __device__ void use4(int, int, const Cols4 &, const float4 (&x)[1], float (&acc)[2][4]) const {
    const float4 z = x[0];
    acc[0][0] += z.x; acc[0][1] += z.y; acc[0][2] += z.z; acc[0][3] += z.w;
    acc[1][0] += z.x * z.x; acc[1][1] += z.y * z.y; acc[1][2] += z.z * z.z; acc[1][3] += z.w * z.w;
  }
  __device__ void row1(int r, int col, const Cols1 &, float (&acc)[2]) const {
    const float z = Z[(size_t)r * n + col];
    acc[0] += z;
    acc[1] += z * z;
  }
};

// --- sum(x) only (bias gradient) ----------------------------------------------
struct SumOp {
  const float *X;
  int n;
  struct Cols4 {};
  struct Cols1 {};
  __device__ void load_cols4(int, Cols4 &) const {}
  __device__ void load_cols1(int, Cols1 &) const {}
  static constexpr int NIN = 1, DEPTH = 0, IN_FLIGHT = 4, MIN_BLOCKS = 1;
  __device__ void inputs(const float *(&in)[1]) const { in[0] = X; }
  __device__ void use4(int, int, const Cols4 &, const float4 (&x)[1], float (&acc)[1][4]) const {
    const float4 z = x[0];
    acc[0][0] += z.x; acc[0][1] += z.y; acc[0][2] += z.z; acc[0][3] += z.w;
  }
  __device__ void row1(int r, int col, const Cols1 &, float (&acc)[1]) const {
    acc[0] += X[(size_t)r * n + col];
  }
};

// Per-column constants of a batch-renormalised unit.
struct BrnCol {
  float mean, sigma, r, d, gamma, beta;
  float r_over_sigma;  // formed once per unit; every kernel normalises through it
};
struct BrnPtrs {
  const float *mean, *sigma, *r, *d, *gamma, *beta;
  __device__ BrnCol at(int c) const {
    const float s = sigma[c], rr = r[c];
    return BrnCol{mean[c], s, rr, d[c], gamma[c], beta[c], rr / s};
  }
};
static BrnPtrs brn_ptrs(const dlb_brn_unit_arrays *u) {
  return BrnPtrs{u->mean, u->sigma, u->r, u->d, u->gamma, u->beta};
}

// value_hat = (z - mean) / sigma * r + d      (fwp_mp.cpp L:4732), with the
// per-unit quotient r / sigma formed once instead of a division per element (a
// difference of one rounding; forward and backward both come through here, so
// they agree bit for bit on which side of a derivative jump a value lies).
__device__ __forceinline__ float brn_hat(float z, const BrnCol &c) {
  return __fmaf_rn(z - c.mean, c.r_over_sigma, c.d);
}
// value_normalize = gamma * value_hat + beta  (fwp_mp.cpp L:4736)
__device__ __forceinline__ float brn_norm(float xh, const BrnCol &c) {
  return __fmaf_rn(c.gamma, xh, c.beta);
}

// --- activation backward (+ BRN backward sums) --------------------------------
// AF: the activation function when the caller knows it at compile time (the
// switch then folds away), or -1 to read it from `af`.
template <bool NORM, int AF = -1>
struct ActBackwardOp {
  float *dA;
  const float *Z, *A;
  BrnPtrs u;
  int af, n;
  // Per-unit constants plus the two quotients of bwp_mp.cpp L:1571-1574,
  // -r / sigma and -r / (sigma * sigma), formed once per unit as the reference
  // forms them once per element with the same operands.
  struct Col {
    BrnCol c;
    float q_mean, q_sigma;
  };
  struct Cols4 { Col k[4]; };
  struct Cols1 { Col k; };
  __device__ Col make(int col) const {
    Col k;
    k.c = u.at(col);
    const float neg_r = -k.c.r;
    k.q_mean = neg_r / k.c.sigma;
    k.q_sigma = neg_r / (k.c.sigma * k.c.sigma);
    return k;
  }
  __device__ void load_cols4(int col, Cols4 &k) const {
    if (NORM)
      for (int j = 0; j < 4; ++j) k.k[j] = make(col + j);
  }
  __device__ void load_cols1(int col, Cols1 &k) const {
    if (NORM) k.k = make(col);
  }
  __device__ __forceinline__ float one(float da, float z, float a, const Col &k, float *s0,
                                       float *s1, float *s2, float *s3) const {
    float y = z, xh = 0.f;
    if (NORM) {
      xh = brn_hat(z, k.c);
      y = brn_norm(xh, k.c);
    }
    const float e = da * af_derive(AF >= 0 ? AF : af, y, a);
    if (NORM) {
      // bwp_mp.cpp L:1559-1574
      *s0 += e * xh;
      *s1 += e;
      const float eh = e * k.c.gamma;
      *s2 += eh * k.q_mean;
      *s3 += eh * (z - k.c.mean) * k.q_sigma;
    }
    return e;
  }
  static constexpr int NIN = 3, DEPTH = 4, IN_FLIGHT = 0, MIN_BLOCKS = 3;
  __device__ void inputs(const float *(&in)[3]) const { in[0] = dA; in[1] = Z; in[2] = A; }
  __device__ void use4(int r, int col, const Cols4 &k, const float4 (&x)[3], float (&acc)[4][4]) const {
    const size_t o = (size_t)r * n + col;
    float4 da = x[0];
    const float4 z = x[1], a = x[2];
    da.x = one(da.x, z.x, a.x, k.k[0], &acc[0][0], &acc[1][0], &acc[2][0], &acc[3][0]);
    da.y = one(da.y, z.y, a.y, k.k[1], &acc[0][1], &acc[1][1], &acc[2][1], &acc[3][1]);
    da.z = one(da.z, z.z, a.z, k.k[2], &acc[0][2], &acc[1][2], &acc[2][2], &acc[3][2]);
    da.w = one(da.w, z.w, a.w, k.k[3], &acc[0][3], &acc[1][3], &acc[2][3], &acc[3][3]);
    *reinterpret_cast<float4 *>(dA + o) = da;
  }
  __device__ void row1(int r, int col, const Cols1 &k, float (&acc)[4]) const {
    const size_t o = (size_t)r * n + col;
    dA[o] = one(dA[o], Z[o], A[o], k.k, &acc[0], &acc[1], &acc[2], &acc[3]);
  }
};

// ---------------------------------------------------------------------------
// Plain streaming kernels: grid-stride over float4 with a scalar tail path when
// the row length is not a multiple of 4.
// ---------------------------------------------------------------------------
static inline int stream_grid(dlb_ctx *ctx, size_t work_items, int block) {
  size_t blocks = (work_items + block - 1) / block;
  size_t cap = (size_t)ctx->sm_count * 16;
  return (int)max((size_t)1, min(blocks, cap));
}

// Row chunking of the row-loop kernels: one wave of four blocks of 256 threads
// per SM (what their shared memory and registers are sized for), chunks a
// multiple of the 8 row lanes.
static void rows_plan(dlb_ctx *ctx, int rows, int n, int *chunks, int *rows_per_chunk) {
  const int col_blocks = ceil_div(n, CR_COLS);
  int c = max(1, ctx->sm_count * 4 / col_blocks);
  c = max(1, min(c, ceil_div(rows, CR_LANES_Y)));
  *rows_per_chunk = ceil_div(ceil_div(rows, c), CR_LANES_Y) * CR_LANES_Y;
  *chunks = ceil_div(rows, *rows_per_chunk);
}

__global__ void split_tf32_kernel(const float *__restrict__ x, float *__restrict__ lo, size_t n) {
  pdl_enter();
  const size_t n4 = n / 4;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
    float4 o;
    o.x = tf32_lo(v.x); o.y = tf32_lo(v.y); o.z = tf32_lo(v.z); o.w = tf32_lo(v.w);
    reinterpret_cast<float4 *>(lo)[i] = o;
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    lo[i] = tf32_lo(x[i]);
}

struct DropoutDev {
  int type;
  float scale;  // inverted Bernoulli: 1 / keep
  const uint8_t *mask;
  const float *noise;
};

__device__ __forceinline__ float apply_dropout(float a, const DropoutDev &dp, int col, size_t idx) {
  switch (dp.type) {
    case DLB_DROPOUT_BERNOULLI: return dp.mask[col] ? a : 0.f;                  // fwp_mp.cpp L:4842-4868
    case DLB_DROPOUT_BERNOULLI_INVERTED: return dp.mask[col] ? a * dp.scale : 0.f;  // L:4809-4840
    case DLB_DROPOUT_UOUT: return a + a * dp.noise[idx];                         // L:4959-4985
    case DROPOUT_INFERENCE_SCALE: return a * dp.scale;                           // L:4870-4892
    default: return a;
  }
}

template <bool NORM, bool VEC4>
__global__ void activation_forward_kernel(const float *__restrict__ Z, BrnPtrs u, int af,
                                          DropoutDev dp, float *__restrict__ A,
                                          float *__restrict__ A_lo, int rows, int n, unsigned *amax) {
  pdl_enter();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned mx = 0;
  if (VEC4) {
    const int n4 = n / 4;
    const size_t total = (size_t)rows * n4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int col = (int)(i % n4) * 4;
      const float4 z = __ldg(reinterpret_cast<const float4 *>(Z) + i);
      float zz[4] = {z.x, z.y, z.z, z.w}, out[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float y = zz[j];
        if (NORM) {
          const BrnCol c = u.at(col + j);
          y = brn_norm(brn_hat(y, c), c);
        }
        out[j] = apply_dropout(af_fire(af, y), dp, col + j, i * 4 + j);
        lo[j] = tf32_lo(out[j]);
        mx = max(mx, abs_bits(out[j]));
      }
      reinterpret_cast<float4 *>(A)[i] = make_float4(out[0], out[1], out[2], out[3]);
      if (A_lo) reinterpret_cast<float4 *>(A_lo)[i] = make_float4(lo[0], lo[1], lo[2], lo[3]);
    }
  } else {
    const size_t total = (size_t)rows * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int col = (int)(i % n);
      float y = Z[i];
      if (NORM) {
        const BrnCol c = u.at(col);
        y = brn_norm(brn_hat(y, c), c);
      }
      const float a = apply_dropout(af_fire(af, y), dp, col, i);
      A[i] = a;
      mx = max(mx, abs_bits(a));
      if (A_lo) A_lo[i] = tf32_lo(a);
    }
  }
  amax_commit(amax, mx);
}

// One warp per row.  ref: fwp_mp.cpp L:4772-4807 (max, exp(x-max), * 1/sum).
__global__ void softmax_forward_kernel(const float *__restrict__ Z, float *__restrict__ Q, int rows,
                                       int n) {
  pdl_enter();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
  if (warp >= rows) return;
  const float *z = Z + (size_t)warp * n;
  float *q = Q + (size_t)warp * n;
  float mx = -3.402823466e+38f;
  for (int i = lane; i < n; i += 32) mx = fmaxf(mx, z[i]);
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int i = lane; i < n; i += 32) {
    const float e = expf(z[i] - mx);
    q[i] = e;
    sum += e;
  }
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  for (int i = lane; i < n; i += 32) q[i] *= inv;
}

template <bool VEC4>
__global__ void brn_backward_apply_kernel(float *__restrict__ delta, float *__restrict__ delta_lo,
                                          const float *__restrict__ Z, BrnPtrs u,
                                          const double *__restrict__ sums, float inv_rows,
                                          float rows_f, int rows, int n, unsigned *amax) {
  pdl_enter();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned mx = 0;
  const double *d_mean = sums + 2 * (size_t)n, *d_sigma = sums + 3 * (size_t)n;
  auto one = [&](float e, float z, int col) {
    const BrnCol c = u.at(col);
    // bwp_mp.cpp L:1565 (dX_h = dY * scale) then L:1608-1621.
    float t = e * c.gamma;
    t *= c.r / c.sigma;
    t += (float)d_sigma[col] * ((z - c.mean) / (rows_f * c.sigma));
    t += (float)d_mean[col] * inv_rows;
    return t;
  };
  if (VEC4) {
    const int n4 = n / 4;
    const size_t total = (size_t)rows * n4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int col = (int)(i % n4) * 4;
      float4 e = reinterpret_cast<const float4 *>(delta)[i];
      const float4 z = __ldg(reinterpret_cast<const float4 *>(Z) + i);
      e.x = one(e.x, z.x, col); e.y = one(e.y, z.y, col + 1);
      e.z = one(e.z, z.z, col + 2); e.w = one(e.w, z.w, col + 3);
      mx = max(max(mx, abs_bits(e.x)), max(abs_bits(e.y), max(abs_bits(e.z), abs_bits(e.w))));
      reinterpret_cast<float4 *>(delta)[i] = e;
      if (delta_lo)
        reinterpret_cast<float4 *>(delta_lo)[i] =
            make_float4(tf32_lo(e.x), tf32_lo(e.y), tf32_lo(e.z), tf32_lo(e.w));
    }
  } else {
    const size_t total = (size_t)rows * n;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const float t = one(delta[i], Z[i], (int)(i % n));
      delta[i] = t;
      mx = max(mx, abs_bits(t));
      if (delta_lo) delta_lo[i] = tf32_lo(t);
    }
  }
  amax_commit(amax, mx);
}

template <bool VEC4>
__global__ void activation_backward_plain_kernel(float *__restrict__ dA, const float *__restrict__ Z,
                                                 const float *__restrict__ A, int af,
                                                 size_t total) {
  pdl_enter();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  if (VEC4) {
    const size_t t4 = total / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < t4; i += stride) {
      float4 e = reinterpret_cast<const float4 *>(dA)[i];
      const float4 z = __ldg(reinterpret_cast<const float4 *>(Z) + i);
      const float4 a = __ldg(reinterpret_cast<const float4 *>(A) + i);
      e.x *= af_derive(af, z.x, a.x); e.y *= af_derive(af, z.y, a.y);
      e.z *= af_derive(af, z.z, a.z); e.w *= af_derive(af, z.w, a.w);
      reinterpret_cast<float4 *>(dA)[i] = e;
    }
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
      dA[i] *= af_derive(af, Z[i], A[i]);
  }
}

// ---------------------------------------------------------------------------
// Row-loop forms of the two normalised [rows, units] kernels (units % 4 == 0).
// Grid (column blocks, row chunks) like the column reductions: a thread keeps
// one float4 column group, loads its per-unit constants once and walks rows
// with stride 8, so the inner loop is one 16-byte load per input tensor and
// one 16-byte store per output tensor, each warp touching 512 contiguous bytes.
// ---------------------------------------------------------------------------
// Calls f with the activation function as a compile-time constant, so that the
// per-element switch of af_fire / af_derive folds away in the hot kernels.
template <class F>
static dlb_status with_af(int af, F f) {
  switch (af) {
    case DLB_AF_RELU: return f(std::integral_constant<int, DLB_AF_RELU>{});
    case DLB_AF_LEAKY_RELU: return f(std::integral_constant<int, DLB_AF_LEAKY_RELU>{});
    case DLB_AF_ELU: return f(std::integral_constant<int, DLB_AF_ELU>{});
    case DLB_AF_SELU: return f(std::integral_constant<int, DLB_AF_SELU>{});
    case DLB_AF_ISRLU: return f(std::integral_constant<int, DLB_AF_ISRLU>{});
    default: return f(std::integral_constant<int, DLB_AF_LINEAR>{});  // what af_fire does with any other value
  }
}

// The rows come through a thread-private copy ring in shared memory: AF_DEPTH - 1
// rows of 16 bytes per thread under way, 44 KB per block, where plain loads held
// four (a register quadruple each, at the 64 registers four blocks per SM allow).
constexpr int AF_DEPTH = 12;     // one input tensor
constexpr int APPLY_DEPTH = 6;   // two input tensors
constexpr int ROWS_PER_SM = 4;   // blocks per SM both kernels are built for

// PLANES: the kernel also writes the fp16 planes of A (with the scale predicted
// from the buffer's previous split) and the row / column maxima of the range
// guard; otherwise it leaves max |A| in the sink's slot for the split pass that
// follows.
template <bool PLANES, int AF>
__global__ void __launch_bounds__(CR_LANES_X *CR_LANES_Y, ROWS_PER_SM)
    activation_forward_rows_kernel(const float *__restrict__ Z, BrnPtrs u, DropoutDev dp,
                                   float *__restrict__ A, float *__restrict__ A_lo, int rows, int n,
                                   int rows_per_chunk, PlaneSink sink) {
  pdl_enter();
  extern __shared__ float4 row_ring[];
  const int tx = threadIdx.x % CR_LANES_X, ty = threadIdx.x / CR_LANES_X;
  const int col = blockIdx.x * CR_COLS + tx * 4;
  const bool live_col = col < n;
  if (!PLANES && !live_col) return;
  const int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
  LineTracker track;
  const float plane_scale = PLANES ? sink_scale(sink) : 1.f;
  if (live_col) {
    BrnCol c[4];
    // Bernoulli dropout has one flag per unit: a factor per owned column, 0 for a
    // dropped unit, 1 (plain: kept units pass unchanged, as the reference leaves
    // them; a * 1 is a) or 1 / keep probability (inverted) for a kept one.
    float keep[4];
    const bool bern = dp.type == DLB_DROPOUT_BERNOULLI || dp.type == DLB_DROPOUT_BERNOULLI_INVERTED;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      c[j] = u.at(col + j);
      keep[j] = bern ? (dp.mask[col + j] ? (dp.type == DLB_DROPOUT_BERNOULLI_INVERTED ? dp.scale : 1.f) : 0.f) : 1.f;
    }
    const float *in[1] = {Z};
    ring_walk<1, AF_DEPTH, CR_LANES_X * CR_LANES_Y>(row_ring, in, (size_t)n, col, r0 + ty, r1, CR_LANES_Y, [&](int r, const float4(&x)[1]) {
      const size_t o = (size_t)r * n + col;
      const float zz[4] = {x[0].x, x[0].y, x[0].z, x[0].w};
      float out[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) out[j] = af_fire(AF, brn_norm(brn_hat(zz[j], c[j]), c[j]));
      if (bern || dp.type == DLB_DROPOUT_NONE) {
        // A dropped unit is 0 whatever the activation came to (a select, not a product).
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = keep[j] == 0.f ? 0.f : out[j] * keep[j];
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = apply_dropout(out[j], dp, col + j, o + j);
      }
      *reinterpret_cast<float4 *>(A + o) = make_float4(out[0], out[1], out[2], out[3]);
      if (PLANES) {
        sink_store4(sink, o, out, plane_scale);
        track.row(sink, r, out);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) track.all = max(track.all, abs_bits(out[j]));
        if (A_lo)
          *reinterpret_cast<float4 *>(A_lo + o) =
              make_float4(tf32_lo(out[0]), tf32_lo(out[1]), tf32_lo(out[2]), tf32_lo(out[3]));
      }
    });
  }
  if (PLANES) {
    ring_drain();
    track.finish(sink, reinterpret_cast<unsigned *>(row_ring), tx, ty, CR_LANES_Y, blockIdx.x * CR_COLS, n, live_col, CR_LANES_X);
  } else if (sink.slot) {
    amax_commit(reinterpret_cast<unsigned *>(sink.slot) + SLOT_AMAX, track.all);
  }
}

template <bool PLANES>
__global__ void __launch_bounds__(CR_LANES_X *CR_LANES_Y, ROWS_PER_SM)
    brn_backward_apply_rows_kernel(float *__restrict__ delta, float *__restrict__ delta_lo,
                                   const float *__restrict__ Z, BrnPtrs u,
                                   const double *__restrict__ sums, float inv_rows, float rows_f,
                                   int rows, int n, int rows_per_chunk, PlaneSink sink) {
  pdl_enter();
  extern __shared__ float4 row_ring[];
  const int tx = threadIdx.x % CR_LANES_X, ty = threadIdx.x / CR_LANES_X;
  const int col = blockIdx.x * CR_COLS + tx * 4;
  const bool live_col = col < n;
  if (!PLANES && !live_col) return;
  const int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
  LineTracker track;
  const float plane_scale = PLANES ? sink_scale(sink) : 1.f;
  if (live_col) {
    // Per-unit factors in the reference's grouping (bwp_mp.cpp L:1608-1621):
    // r / sigma, d_sigma / (N * sigma), d_mean / N.  The reference divides
    // (z - mean) by N * sigma per element; the quotient d_sigma / (N sigma) is
    // formed once per unit here (a division is a dozen instructions, and this
    // kernel is bound by instruction issue), a difference of one rounding in a
    // term that is summed.
    float gamma[4], mean[4], r_over_sigma[4], d_sigma_n[4], d_mean_n[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const BrnCol c = u.at(col + j);
      gamma[j] = c.gamma;
      mean[j] = c.mean;
      r_over_sigma[j] = c.r / c.sigma;
      d_sigma_n[j] = (float)sums[3 * (size_t)n + col + j] / (rows_f * c.sigma);
      d_mean_n[j] = (float)sums[2 * (size_t)n + col + j] * inv_rows;
    }
    const float *in[2] = {delta, Z};
    ring_walk<2, APPLY_DEPTH, CR_LANES_X * CR_LANES_Y>(row_ring, in, (size_t)n, col, r0 + ty, r1, CR_LANES_Y, [&](int r, const float4(&x)[2]) {
      const size_t o = (size_t)r * n + col;
      const float e[4] = {x[0].x, x[0].y, x[0].z, x[0].w}, z[4] = {x[1].x, x[1].y, x[1].z, x[1].w};
      float t[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = e[j] * gamma[j];
        v *= r_over_sigma[j];
        v += d_sigma_n[j] * (z[j] - mean[j]);
        v += d_mean_n[j];
        t[j] = v;
      }
      *reinterpret_cast<float4 *>(delta + o) = make_float4(t[0], t[1], t[2], t[3]);
      if (PLANES) {
        sink_store4(sink, o, t, plane_scale);
        track.row(sink, r, t);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) track.all = max(track.all, abs_bits(t[j]));
        if (delta_lo)
          *reinterpret_cast<float4 *>(delta_lo + o) =
              make_float4(tf32_lo(t[0]), tf32_lo(t[1]), tf32_lo(t[2]), tf32_lo(t[3]));
      }
    });
  }
  if (PLANES) {
    ring_drain();
    track.finish(sink, reinterpret_cast<unsigned *>(row_ring), tx, ty, CR_LANES_Y, blockIdx.x * CR_COLS, n, live_col, CR_LANES_X);
  } else if (sink.slot) {
    amax_commit(reinterpret_cast<unsigned *>(sink.slot) + SLOT_AMAX, track.all);
  }
}

__global__ void brn_finalize_kernel(const double *__restrict__ sums, int n, float batch_scale,
                                    float momentum, float eps, float r_max, float d_max,
                                    dlb_brn_unit_arrays u) {
  pdl_enter();
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= n) return;
  // fwp_mp.cpp L:4688-4717, in the reference's order: the running averages
  // move first and r, d are taken from the moved averages.
  const float mean = (float)sums[h] * batch_scale;
  float mavg = u.mean_average[h];
  mavg += momentum * (mean - mavg);
  const float sigma = sqrtf((float)sums[n + h] * batch_scale - mean * mean + eps);
  float savg = u.sigma_average[h];
  savg += momentum * (sigma - savg);
  u.mean[h] = mean;
  u.sigma[h] = sigma;
  u.mean_average[h] = mavg;
  u.sigma_average[h] = savg;
  u.r[h] = clipf(sigma / savg, 1.f / r_max, r_max);
  u.d[h] = clipf((mean - mavg) / savg, -d_max, d_max);
}

__global__ void sums_to_grads_kernel(const double *__restrict__ sums, int n, float *d_gamma,
                                     float *d_beta, int accumulate) {
  pdl_enter();
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= n) return;
  const float g = (float)sums[h], b = (float)sums[n + h];
  if (accumulate) {
    d_gamma[h] += g;
    d_beta[h] += b;
  } else {
    d_gamma[h] = g;
    d_beta[h] = b;
  }
}

__global__ void sums_to_bias_grad_kernel(const double *__restrict__ sums, int n, float *dbias,
                                         int accumulate) {
  pdl_enter();
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= n) return;
  if (accumulate) dbias[h] += (float)sums[h];
  else dbias[h] = (float)sums[h];
}

// MSE (or any non-softmax output): delta = f'(x,q) * 2 (q - y) / (N * n_out).
__global__ void loss_delta_mse_kernel(const float *__restrict__ pre, const float *__restrict__ q,
                                      const float *__restrict__ y, float *__restrict__ delta,
                                      float *__restrict__ delta_lo, int af, size_t total,
                                      float denom, double *loss_sum, unsigned *amax) {
  pdl_enter();
  __shared__ double red[8];
  double local = 0.0;
  unsigned mx = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const float qq = q[i], yy = y[i];
    const float diff = qq - yy;
    local += (double)(diff * diff);  // loss_fn: pow(q - y, 2) in float, summed in double
    float dl = 2.f * diff;
    dl /= denom;
    const float e = af_derive(af, pre[i], qq) * dl;
    delta[i] = e;
    mx = max(mx, abs_bits(e));
    if (delta_lo) delta_lo[i] = tf32_lo(e);
  }
  amax_commit(amax, mx);
  for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x / 32); ++w) t += red[w];
    atomicAdd(loss_sum, t);
  }
}

// Softmax + cross-entropy, one warp per row.
// delta_j = sum_k (q_j [j == k] - q_k q_j) L'_k with L'_k = 0 unless y_k == 1
// (compute_error_mp.cpp L:84-107): the warp first lists the classes with
// y_k == 1 in ascending order (one for a one-hot target), then every j adds the
// terms of those classes only, in the reference's order and with its
// expressions; the terms left out are the ones the reference adds as zeros.
// A row with more than SOFTMAX_LIST such classes takes the full double loop.
constexpr int SOFTMAX_LIST = 32;
__global__ void loss_delta_softmax_ce_kernel(const float *__restrict__ q, const float *__restrict__ y,
                                             float *__restrict__ delta, float *__restrict__ delta_lo,
                                             int rows, int n, float rows_global, double *loss_sum,
                                             unsigned *amax) {
  pdl_enter();
  __shared__ int list_k[8][SOFTMAX_LIST];
  __shared__ float list_q[8][SOFTMAX_LIST], list_dl[8][SOFTMAX_LIST];
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32, w = threadIdx.x / 32;
  double local = 0.0;
  unsigned mx = 0;
  if (warp < rows) {
    const float *qr = q + (size_t)warp * n, *yr = y + (size_t)warp * n;
    const float EPS = 1e-7f;
    int count = 0;
    for (int k0 = 0; k0 < n; k0 += 32) {
      const int k = k0 + lane;
      const bool hit = k < n && yr[k] == 1.f;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int at = count + __popc(m & ((1u << lane) - 1u));
        if (at < SOFTMAX_LIST) {
          const float qk = qr[k];
          float dl = -1.f / clipf(qk, EPS, 1.f - EPS);
          dl /= rows_global;
          list_k[w][at] = k;
          list_q[w][at] = qk;
          list_dl[w][at] = dl;
        }
      }
      count += __popc(m);
    }
    __syncwarp();
    for (int j = lane; j < n; j += 32) {
      const float qj = qr[j];
      float e = 0.f;
      if (count <= SOFTMAX_LIST) {
        for (int i = 0; i < count; ++i) {
          const float qk = list_q[w][i];
          e += (qj * (j == list_k[w][i] ? 1.f : 0.f) - qk * qj) * list_dl[w][i];
        }
      } else {
        for (int k = 0; k < n; ++k) {
          if (yr[k] == 1.f) {
            const float qk = qr[k];
            float dl = -1.f / clipf(qk, EPS, 1.f - EPS);
            dl /= rows_global;
            e += (qj * (j == k ? 1.f : 0.f) - qk * qj) * dl;
          }
        }
      }
      delta[(size_t)warp * n + j] = e;
      mx = max(mx, abs_bits(e));
      if (delta_lo) delta_lo[(size_t)warp * n + j] = tf32_lo(e);
      if (yr[j] == 1.f) local += (double)(-(yr[j] * logf(clipf(qj, EPS, 1.f - EPS))));
    }
  }
  amax_commit(amax, mx);
  for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if (lane == 0 && local != 0.0) atomicAdd(loss_sum, local);
}

}  // namespace dlb

using namespace dlb;

extern "C" {

dlb_status dlb_split_tf32(dlb_ctx *ctx, const float *x, float *x_lo, size_t n) {
  DLB_REQUIRE(ctx && x && x_lo, "dlb_split_tf32: null");
  if (n == 0) return DLB_OK;
  DLB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(x_lo) & 15) == 0,
              "dlb_split_tf32: pointers must be 16-byte aligned");
  DLB_LAUNCH_KERNEL(ctx, split_tf32_kernel, stream_grid(ctx, n / 4 + 1, 256), 256, 0, x, x_lo, n);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_brn_forward_sums(dlb_ctx *ctx, const float *Z, int rows, int n_units,
                                double *sums) {
  DLB_REQUIRE(ctx && Z && sums && rows > 0 && n_units > 0, "dlb_brn_forward_sums");
  DLB_REQUIRE((n_units & 3) || (reinterpret_cast<uintptr_t>(Z) & 15) == 0,
              "dlb_brn_forward_sums: Z must be 16-byte aligned");
  return column_reduce<2>(ctx, SumSqOp{Z, n_units}, rows, n_units, sums);
}

dlb_status dlb_brn_forward_finalize(dlb_ctx *ctx, const double *sums, int global_rows,
                                    int n_units, float momentum, float epsilon, float r_max,
                                    float d_max, const dlb_brn_unit_arrays *u) {
  DLB_REQUIRE(ctx && sums && u && global_rows > 0 && n_units > 0, "dlb_brn_forward_finalize");
  DLB_REQUIRE(u->mean && u->sigma && u->mean_average && u->sigma_average && u->r && u->d,
              "dlb_brn_forward_finalize: null unit array");
  DLB_LAUNCH_KERNEL(ctx, brn_finalize_kernel, ceil_div(n_units, 256), 256, 0, sums, n_units, 1.f / (float)global_rows, momentum, epsilon, r_max, d_max, *u);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// Shapes for which the row kernels run: they are the ones that can write the
// fp16 planes themselves.
static bool rows_kernel_applies(const void *a, const void *b, const void *c, int n_units) {
  return (n_units % 4 == 0) &&
         ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

dlb_status activation_forward_impl(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                                  int af, const dlb_dropout_desc *dropout, float *A,
                                  float *A_lo, int rows, int n_units, const PlaneSink &sink) {
  unsigned *amax = sink.slot ? reinterpret_cast<unsigned *>(sink.slot) + SLOT_AMAX : nullptr;
  DLB_REQUIRE(ctx && Z && A && rows > 0 && n_units > 0, "dlb_activation_forward");
  DropoutDev dp{DLB_DROPOUT_NONE, 1.f, nullptr, nullptr};
  if (dropout && dropout->type != DLB_DROPOUT_NONE) {
    dp.type = dropout->type;
    dp.mask = dropout->mask;
    dp.noise = dropout->noise;
    if (dp.type == DLB_DROPOUT_BERNOULLI || dp.type == DLB_DROPOUT_BERNOULLI_INVERTED) {
      DLB_REQUIRE(dp.mask, "dlb_activation_forward: Bernoulli dropout needs a mask");
      if (dp.type == DLB_DROPOUT_BERNOULLI_INVERTED) {
        DLB_REQUIRE(dropout->value > 0.f, "dlb_activation_forward: keep probability");
        dp.scale = 1.f / dropout->value;
      }
    } else if (dp.type == DROPOUT_INFERENCE_SCALE) {
      dp.scale = dropout->value;
    } else if (dp.type == DLB_DROPOUT_UOUT) {
      DLB_REQUIRE(dp.noise, "dlb_activation_forward: UOut needs noise");
    } else {
      set_error("dlb_activation_forward: dropout type %d is not applied here", dp.type);
      return DLB_ERR_UNSUPPORTED;
    }
  }
  BrnPtrs p{};
  if (u) p = brn_ptrs(u);
  const bool vec4 = (n_units % 4 == 0) && ((reinterpret_cast<uintptr_t>(Z) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(A) & 15) == 0) &&
                    (!A_lo || (reinterpret_cast<uintptr_t>(A_lo) & 15) == 0);
  if (u && vec4) {
    int chunks, rpc;
    rows_plan(ctx, rows, n_units, &chunks, &rpc);
    const dim3 grid(ceil_div(n_units, CR_COLS), chunks);
    constexpr size_t shared = ring_bytes(1, AF_DEPTH, CR_LANES_X * CR_LANES_Y);
    return with_af(af, [&](auto AF) {
      constexpr int F = decltype(AF)::value;
      if (sink.hi)
        DLB_LAUNCH_KERNEL(ctx, (activation_forward_rows_kernel<true, F>), grid, CR_LANES_X * CR_LANES_Y, shared, Z, p, dp, A, A_lo, rows, n_units, rpc, sink);
      else
        DLB_LAUNCH_KERNEL(ctx, (activation_forward_rows_kernel<false, F>), grid, CR_LANES_X * CR_LANES_Y, shared, Z, p, dp, A, A_lo, rows, n_units, rpc, sink);
      DLB_LAUNCHED(ctx);
      return DLB_OK;
    });
  }
  DLB_REQUIRE(!sink.hi, "dlb_activation_forward: planes from a kernel that cannot write them");
  const size_t items = vec4 ? (size_t)rows * (n_units / 4) : (size_t)rows * n_units;
  const int grid = stream_grid(ctx, items, 256);
#define LAUNCH(NORM, V)                                                                 \
  DLB_LAUNCH_KERNEL(ctx, (activation_forward_kernel<NORM, V>), grid, 256, 0, Z, p, af, dp, A, A_lo, rows, n_units, amax)
  if (u) { if (vec4) LAUNCH(true, true); else LAUNCH(true, false); }
  else   { if (vec4) LAUNCH(false, true); else LAUNCH(false, false); }
#undef LAUNCH
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_softmax_forward(dlb_ctx *ctx, const float *Z, float *Q, int rows, int n_units) {
  DLB_REQUIRE(ctx && Z && Q && rows > 0 && n_units > 0, "dlb_softmax_forward");
  DLB_LAUNCH_KERNEL(ctx, softmax_forward_kernel, ceil_div(rows, 8), 256, 0, Z, Q, rows, n_units);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_activation_backward(dlb_ctx *ctx, float *dA, const float *Z, const float *A,
                                   const dlb_brn_unit_arrays *u, int af, int rows, int n_units,
                                   double *sums) {
  DLB_REQUIRE(ctx && dA && Z && A && rows > 0 && n_units > 0, "dlb_activation_backward");
  if (u) {
    DLB_REQUIRE(sums, "dlb_activation_backward: sums required with batch renormalization");
    DLB_REQUIRE((n_units & 3) || ((reinterpret_cast<uintptr_t>(dA) | reinterpret_cast<uintptr_t>(Z) |
                                   reinterpret_cast<uintptr_t>(A)) & 15) == 0,
                "dlb_activation_backward: tensors must be 16-byte aligned");
    return with_af(af, [&](auto AF) {
      return column_reduce<4>(ctx, ActBackwardOp<true, decltype(AF)::value>{dA, Z, A, brn_ptrs(u), af, n_units}, rows,
                              n_units, sums);
    });
  }
  const size_t total = (size_t)rows * n_units;
  const bool vec4 = (total % 4 == 0) && ((reinterpret_cast<uintptr_t>(dA) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(Z) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
  const int grid = stream_grid(ctx, vec4 ? total / 4 : total, 256);
  if (vec4)
    DLB_LAUNCH_KERNEL(ctx, activation_backward_plain_kernel<true>, grid, 256, 0, dA, Z, A, af, total);
  else
    DLB_LAUNCH_KERNEL(ctx, activation_backward_plain_kernel<false>, grid, 256, 0, dA, Z, A, af, total);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status brn_backward_apply_impl(dlb_ctx *ctx, float *delta, float *delta_lo, const float *Z,
                                  const dlb_brn_unit_arrays *u, const double *sums,
                                  int global_rows, int rows, int n_units, const PlaneSink &sink) {
  unsigned *amax = sink.slot ? reinterpret_cast<unsigned *>(sink.slot) + SLOT_AMAX : nullptr;
  DLB_REQUIRE(ctx && delta && Z && u && sums && rows > 0 && n_units > 0 && global_rows > 0,
              "dlb_brn_backward_apply");
  const bool vec4 = (n_units % 4 == 0) && ((reinterpret_cast<uintptr_t>(Z) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(delta) & 15) == 0) &&
                    (!delta_lo || (reinterpret_cast<uintptr_t>(delta_lo) & 15) == 0);
  const size_t items = vec4 ? (size_t)rows * (n_units / 4) : (size_t)rows * n_units;
  const int grid = stream_grid(ctx, items, 256);
  const float nf = (float)global_rows;
  if (vec4) {
    int chunks, rpc;
    rows_plan(ctx, rows, n_units, &chunks, &rpc);
    const dim3 rgrid(ceil_div(n_units, CR_COLS), chunks);
    constexpr size_t shared = ring_bytes(2, APPLY_DEPTH, CR_LANES_X * CR_LANES_Y);
    if (sink.hi)
      DLB_LAUNCH_KERNEL(ctx, brn_backward_apply_rows_kernel<true>, rgrid, CR_LANES_X * CR_LANES_Y, shared, delta, delta_lo, Z, brn_ptrs(u), sums, 1.f / nf, nf, rows, n_units, rpc, sink);
    else
      DLB_LAUNCH_KERNEL(ctx, brn_backward_apply_rows_kernel<false>, rgrid, CR_LANES_X * CR_LANES_Y, shared, delta, delta_lo, Z, brn_ptrs(u), sums, 1.f / nf, nf, rows, n_units, rpc, sink);
  } else {
    DLB_REQUIRE(!sink.hi, "dlb_brn_backward_apply: planes from a kernel that cannot write them");
    DLB_LAUNCH_KERNEL(ctx, brn_backward_apply_kernel<false>, grid, 256, 0, delta, delta_lo, Z, brn_ptrs(u), sums, 1.f / nf, nf, rows, n_units, amax);
  }
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_brn_backward_param_grads(dlb_ctx *ctx, const double *sums, int n_units,
                                        float *d_gamma, float *d_beta, int accumulate) {
  DLB_REQUIRE(ctx && sums && d_gamma && d_beta && n_units > 0, "dlb_brn_backward_param_grads");
  DLB_LAUNCH_KERNEL(ctx, sums_to_grads_kernel, ceil_div(n_units, 256), 256, 0, sums, n_units, d_gamma, d_beta, accumulate);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status loss_delta_impl(dlb_ctx *ctx, int loss, int af, const float *pre, const float *q,
                          const float *y, float *delta, float *delta_lo, int rows, int n_out,
                          int global_rows, double *loss_sum, unsigned *amax) {
  DLB_REQUIRE(ctx && q && y && delta && loss_sum && rows > 0 && n_out > 0 && global_rows > 0,
              "dlb_loss_delta");
  if (loss == DLB_LOSS_MSE && af != DLB_AF_SOFTMAX) {
    DLB_REQUIRE(pre, "dlb_loss_delta: pre-activation values required");
    const size_t total = (size_t)rows * n_out;
    // loss_fn_derivative divides by static_cast<real>(bs * n_out).
    const float denom = (float)((size_t)global_rows * (size_t)n_out);
    DLB_LAUNCH_KERNEL(ctx, loss_delta_mse_kernel, stream_grid(ctx, total, 256), 256, 0, pre, q, y, delta, delta_lo, af, total, denom, loss_sum, amax);
    DLB_LAUNCHED(ctx);
    return DLB_OK;
  }
  if (loss == DLB_LOSS_CROSS_ENTROPY && af == DLB_AF_SOFTMAX) {
    DLB_LAUNCH_KERNEL(ctx, loss_delta_softmax_ce_kernel, ceil_div(rows, 8), 256, 0, q, y, delta, delta_lo, rows, n_out, (float)global_rows, loss_sum, amax);
    DLB_LAUNCHED(ctx);
    return DLB_OK;
  }
  set_error("dlb_loss_delta: loss %d with activation %d is outside the supported path", loss, af);
  return DLB_ERR_UNSUPPORTED;
}

}  // extern "C"

namespace dlb {
// Column sum of delta into the bias gradient (used by dlb_fc_weight_gradient).
dlb_status bias_gradient(dlb_ctx *ctx, const float *delta, int rows, int n, float *dbias,
                         int accumulate) {
  void *scr = nullptr;
  const size_t partial_bytes = column_reduce_partial_bytes(ctx, 1, rows, n);
  DLB_TRY(scratch(ctx, partial_bytes + (size_t)n * sizeof(double), &scr));
  double *out = reinterpret_cast<double *>(static_cast<char *>(scr) + partial_bytes);
  DLB_TRY(column_reduce<1>(ctx, SumOp{delta, n}, rows, n, out));
  DLB_LAUNCH_KERNEL(ctx, sums_to_bias_grad_kernel, ceil_div(n, 256), 256, 0, out, n, dbias, accumulate);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}
}  // namespace dlb

// ---------------------------------------------------------------------------
// Residual block: ShakeDrop and the shortcut sum.
// ---------------------------------------------------------------------------
namespace dlb {

// block[b,:] *= noise[b,:] on flagged rows (in place, as the reference perturbs
// the block's output buffer), out = x + block, plus the residual plane of out.
__global__ void residual_forward_kernel(const float *__restrict__ x, float *__restrict__ block,
                                        const uint8_t *__restrict__ row_mask,
                                        const float *__restrict__ noise, float *__restrict__ out,
                                        float *__restrict__ out_lo, int rows, int width, int vec,
                                        unsigned *amax) {
  pdl_enter();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned mx = 0;
  if (vec) {
    const int w4 = width / 4;
    const size_t total = (size_t)rows * w4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int r = (int)(i / w4);
      float4 o = reinterpret_cast<float4 *>(block)[i];
      if (row_mask && row_mask[r]) {
        const float4 k = __ldg(reinterpret_cast<const float4 *>(noise) + i);
        o.x *= k.x; o.y *= k.y; o.z *= k.z; o.w *= k.w;
        reinterpret_cast<float4 *>(block)[i] = o;
      }
      const float4 s = __ldg(reinterpret_cast<const float4 *>(x) + i);
      const float4 v = make_float4(s.x + o.x, s.y + o.y, s.z + o.z, s.w + o.w);
      mx = max(max(mx, abs_bits(v.x)), max(abs_bits(v.y), max(abs_bits(v.z), abs_bits(v.w))));
      reinterpret_cast<float4 *>(out)[i] = v;
      if (out_lo)
        reinterpret_cast<float4 *>(out_lo)[i] =
            make_float4(tf32_lo(v.x), tf32_lo(v.y), tf32_lo(v.z), tf32_lo(v.w));
    }
  } else {
    const size_t total = (size_t)rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int r = (int)(i / width);
      float o = block[i];
      if (row_mask && row_mask[r]) {
        o *= noise[i];
        block[i] = o;
      }
      const float v = x[i] + o;
      out[i] = v;
      mx = max(mx, abs_bits(v));
      if (out_lo) out_lo[i] = tf32_lo(v);
    }
  }
  amax_commit(amax, mx);
}

// delta = d * noise on flagged rows, d elsewhere, plus its residual plane.
// d has rows of ld_d floats of which `width` are read from column `first` on
// (the block's window of the residual layer's error when the widths differ).
__global__ void shakedrop_backward_kernel(const float *__restrict__ d, int ld_d, int first,
                                          const uint8_t *__restrict__ row_mask,
                                          const float *__restrict__ noise, float *__restrict__ delta,
                                          float *__restrict__ delta_lo, int rows, int width,
                                          unsigned *amax) {
  pdl_enter();
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t total = (size_t)rows * width;
  unsigned mx = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = (int)(i / width);
    float v = d[(size_t)r * ld_d + first + (i - (size_t)r * width)];
    if (row_mask && row_mask[r]) v *= noise[i];
    delta[i] = v;
    mx = max(mx, abs_bits(v));
    if (delta_lo) delta_lo[i] = tf32_lo(v);
  }
  amax_commit(amax, mx);
}

// The shortcut sum for unequal widths: the output is as wide as the wider of x
// (width wx) and block (width wb); the narrower one enters from column `pad`
// on (Forward_Pass__Zero_Padded_Identity__OpenMP, fwp_mp.cpp L:5058-5123).
// ShakeDrop perturbs the block in place as in the equal-width kernel.
__global__ void residual_forward_padded_kernel(const float *__restrict__ x, int wx, float *__restrict__ block,
                                               int wb, int pad, const uint8_t *__restrict__ row_mask,
                                               const float *__restrict__ noise, float *__restrict__ out,
                                               float *__restrict__ out_lo, int rows, unsigned *amax) {
  pdl_enter();
  const int W = max(wx, wb);
  const int off_x = wx < W ? pad : 0, off_b = wb < W ? pad : 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t total = (size_t)rows * W;
  unsigned mx = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = (int)(i / W), c = (int)(i % W);
    float v = 0.f;
    const int cb = c - off_b;
    if (cb >= 0 && cb < wb) {
      const size_t j = (size_t)r * wb + cb;
      float o = block[j];
      if (row_mask && row_mask[r]) {
        o *= noise[j];
        block[j] = o;
      }
      v = o;
    }
    const int cx = c - off_x;
    if (cx >= 0 && cx < wx) v += x[(size_t)r * wx + cx];
    out[i] = v;
    mx = max(mx, abs_bits(v));
    if (out_lo) out_lo[i] = tf32_lo(v);
  }
  amax_commit(amax, mx);
}

}  // namespace dlb

static dlb_status residual_forward_impl(dlb_ctx *ctx, const float *x, float *block,
                                           const uint8_t *row_mask, const float *noise, float *out,
                                           float *out_lo, int rows, int width, unsigned *amax) {
  DLB_REQUIRE(ctx && x && block && out && rows > 0 && width > 0, "dlb_residual_forward");
  DLB_REQUIRE(!row_mask || noise, "dlb_residual_forward: row flags need the noise draws");
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(block) |
                       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(out_lo) |
                       reinterpret_cast<uintptr_t>(noise);
  const int vec = (width % 4 == 0) && (al & 15) == 0;
  const size_t items = vec ? (size_t)rows * (width / 4) : (size_t)rows * width;
  DLB_LAUNCH_KERNEL(ctx, residual_forward_kernel, stream_grid(ctx, items, 256), 256, 0, x, block, row_mask, noise, out, out_lo, rows, width, vec, amax);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

static dlb_status residual_forward_padded_impl(dlb_ctx *ctx, const float *x, int wx, float *block, int wb,
                                               const uint8_t *row_mask, const float *noise, float *out,
                                               float *out_lo, int rows, unsigned *amax) {
  DLB_REQUIRE(ctx && x && block && out && rows > 0 && wx > 0 && wb > 0, "dlb_residual_forward_padded");
  DLB_REQUIRE(!row_mask || noise, "dlb_residual_forward_padded: row flags need the noise draws");
  const int W = wx > wb ? wx : wb;
  const int pad = ((wx > wb ? wx - wb : wb - wx) + 1) / 2;  // v1/learner/compile.cpp L:344-352
  DLB_LAUNCH_KERNEL(ctx, residual_forward_padded_kernel, stream_grid(ctx, (size_t)rows * W, 256), 256, 0, x, wx, block, wb, pad, row_mask, noise, out, out_lo, rows, amax);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

static dlb_status shakedrop_backward_impl(dlb_ctx *ctx, const float *d, int ld_d, int first,
                                          const uint8_t *row_mask, const float *noise, float *delta,
                                          float *delta_lo, int rows, int width, unsigned *amax) {
  DLB_REQUIRE(ctx && d && delta && rows > 0 && width > 0 && first >= 0 && first + width <= ld_d,
              "dlb_shakedrop_backward");
  DLB_REQUIRE(!row_mask || noise, "dlb_shakedrop_backward: row flags need the noise draws");
  DLB_LAUNCH_KERNEL(ctx, shakedrop_backward_kernel, stream_grid(ctx, (size_t)rows * width, 256), 256, 0, d, ld_d, first, row_mask, noise, delta, delta_lo, rows, width, amax);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// ---------------------------------------------------------------------------
// Batch-renormalization sums without any allocation.
//
// The partial sums live in an array that is part of the library's device image
// (every GPU that loads the library holds it until the process exits), so the
// entry point below never calls cudaMalloc / cudaFree, directly or through the
// context's scratch arena.  In host code the array's name is only a stand-in
// for the symbol, not a device address: the address is looked up once per
// device with cudaGetSymbolAddress and that pointer is what the kernels get.
// ---------------------------------------------------------------------------
namespace dlb {

static __device__ __align__(256) double g_noalloc_partials[DLB_NOALLOC_SCRATCH_DOUBLES];

struct NoallocDevice {
  std::once_flag once;
  dlb_status status = DLB_ERR_INVALID;
  double *partials = nullptr;  // device address of g_noalloc_partials on this device
  int sm_count = 0;
  int per_sm = 0;              // resident blocks of the sums kernel per SM
};
static NoallocDevice g_noalloc_devices[MAX_DEVICES];

static dlb_status noalloc_setup(NoallocDevice *d, int dev) {
  double *ptr = nullptr;
  DLB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_noalloc_partials));
  int sms = 0;
  DLB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  DLB_REQUIRE(ptr && sms > 0, "dlb_brn_forward_sums_noalloc: device set-up");
  d->per_sm = column_reduce_per_sm<2, SumSqOp>();
  d->sm_count = sms;
  d->partials = ptr;
  return DLB_OK;
}

// Set-up for the current device, once per device whichever host thread comes
// first: address of the array, SM count, resident blocks per SM.  None of the
// three calls allocates.
static dlb_status noalloc_device(NoallocDevice **out) {
  int dev = -1;
  DLB_CUDA(cudaGetDevice(&dev));
  DLB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "dlb_brn_forward_sums_noalloc: device index");
  NoallocDevice &d = g_noalloc_devices[dev];
  std::call_once(d.once, [&] { d.status = noalloc_setup(&d, dev); });
  DLB_REQUIRE(d.status == DLB_OK, "dlb_brn_forward_sums_noalloc: the set-up of this device failed");
  *out = &d;
  return DLB_OK;
}

}  // namespace dlb

extern "C" dlb_status dlb_brn_forward_sums_noalloc(const float *Z, int rows, int n_units,
                                                   double *sums, void *stream) {
  DLB_REQUIRE(Z && sums && rows > 0 && n_units > 0, "dlb_brn_forward_sums_noalloc");
  DLB_REQUIRE((n_units & 3) || (reinterpret_cast<uintptr_t>(Z) & 15) == 0,
              "dlb_brn_forward_sums_noalloc: Z must be 16-byte aligned");
  NoallocDevice *dev = nullptr;
  DLB_TRY(noalloc_device(&dev));
  // Z and sums must be memory of the current device (the array used below is).
  cudaPointerAttributes attr;
  DLB_CUDA(cudaPointerGetAttributes(&attr, Z));
  int cur = -1;
  DLB_CUDA(cudaGetDevice(&cur));
  DLB_REQUIRE(attr.type == cudaMemoryTypeDevice && attr.device == cur,
              "dlb_brn_forward_sums_noalloc: Z is not memory of the current device");
  // The chunking of the allocating entry point (same plan function, same
  // occupancy figure), so both add the same partial sums in the same order.
  const int col_blocks = ceil_div(n_units, CR_COLS);
  int chunks, rows_per_chunk;
  column_reduce_plan(dev->sm_count, rows, n_units, dev->per_sm, &chunks, &rows_per_chunk);
  const size_t need = (size_t)chunks * 2 * (size_t)n_units;
  if (need > (size_t)DLB_NOALLOC_SCRATCH_DOUBLES) {
    set_error("dlb_brn_forward_sums_noalloc: %d rows x %d units need %zu partial sums, the built-in "
              "scratch holds %u; use dlb_brn_forward_sums or fewer units per call",
              rows, n_units, need, (unsigned)DLB_NOALLOC_SCRATCH_DOUBLES);
    return DLB_ERR_INVALID;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  column_reduce_kernel<2, SumSqOp><<<dim3(col_blocks, chunks), CR_LANES_X * CR_LANES_Y,
                                     column_reduce_shared_bytes<2, SumSqOp>(), s>>>(
      SumSqOp{Z, n_units}, rows, n_units, rows_per_chunk, dev->partials);
  DLB_CUDA(cudaGetLastError());
  const int total = 2 * n_units;
  reduce_partials_kernel<<<ceil_div(total, 256), 256, 0, s>>>(dev->partials, chunks, total, sums);
  DLB_CUDA(cudaGetLastError());
  return DLB_OK;
}

// ---------------------------------------------------------------------------
// Entry points that produce a GEMM operand together with its plane buffer.
// Under the TF32 form the kernel writes the residual plane itself; under the
// fp16 form the planes need the tensor's maximum first, so the kernel runs
// without the plane output and dlb_split_planes follows.
// ---------------------------------------------------------------------------
namespace {
struct PlaneOutput {
  float *kernel_arg = nullptr;  // TF32 form: the residual plane the producing kernel writes
  PlaneJob job;                 // fp16 form
  // can_fuse: the kernel that will run writes planes and range statistics itself
  // when handed a full sink.
  dlb_status begin(dlb_ctx *ctx, const float *x, float *planes, int rows, int cols, bool can_fuse) {
    if (!ctx || !planes) return DLB_OK;
    if (ctx->gemm_kind != DLB_GEMM_F16X3) {
      kernel_arg = planes;
      return DLB_OK;
    }
    if (rows <= 0 || cols <= 0) return DLB_OK;  // the kernel's own argument check reports it
    return planes_open(ctx, x, planes, (size_t)rows * cols, rows, cols, can_fuse, &job);
  }
  const PlaneSink &sink() const { return job.sink; }
  unsigned *amax() const {
    return job.sink.slot ? reinterpret_cast<unsigned *>(job.sink.slot) + SLOT_AMAX : nullptr;
  }
  dlb_status finish(dlb_ctx *ctx, dlb_status st) const {
    if (st != DLB_OK) return st;
    return planes_close(ctx, job);
  }
};
}  // namespace

extern "C" {

dlb_status dlb_activation_forward(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u, int af,
                                  const dlb_dropout_desc *dropout, float *A, float *A_lo, int rows,
                                  int n_units) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, A, A_lo, rows, n_units, u != nullptr && rows_kernel_applies(Z, A, nullptr, n_units)));
  return p.finish(ctx, activation_forward_impl(ctx, Z, u, af, dropout, A, p.kernel_arg, rows, n_units, p.sink()));
}

dlb_status dlb_brn_backward_apply(dlb_ctx *ctx, float *delta, float *delta_lo, const float *Z,
                                  const dlb_brn_unit_arrays *u, const double *sums, int global_rows,
                                  int rows, int n_units) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, delta, delta_lo, rows, n_units, rows_kernel_applies(Z, delta, nullptr, n_units)));
  return p.finish(ctx, brn_backward_apply_impl(ctx, delta, p.kernel_arg, Z, u, sums, global_rows, rows, n_units,
                                               p.sink()));
}

dlb_status dlb_loss_delta(dlb_ctx *ctx, int loss, int af, const float *pre, const float *q, const float *y,
                          float *delta, float *delta_lo, int rows, int n_out, int global_rows,
                          double *loss_sum) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, delta, delta_lo, rows, n_out, false));
  return p.finish(ctx, loss_delta_impl(ctx, loss, af, pre, q, y, delta, p.kernel_arg, rows, n_out, global_rows,
                                       loss_sum, p.amax()));
}

dlb_status dlb_residual_forward(dlb_ctx *ctx, const float *x, float *block, const uint8_t *row_mask,
                                const float *noise, float *out, float *out_lo, int rows, int width) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, out, out_lo, rows, width, false));
  return p.finish(ctx, residual_forward_impl(ctx, x, block, row_mask, noise, out, p.kernel_arg, rows, width, p.amax()));
}

dlb_status dlb_shakedrop_backward(dlb_ctx *ctx, const float *d, const uint8_t *row_mask, const float *noise,
                                  float *delta, float *delta_lo, int rows, int width) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, delta, delta_lo, rows, width, false));
  return p.finish(ctx, shakedrop_backward_impl(ctx, d, width, 0, row_mask, noise, delta, p.kernel_arg, rows, width,
                                               p.amax()));
}

dlb_status dlb_residual_forward_padded(dlb_ctx *ctx, const float *x, int width_x, float *block, int width_block,
                                       const uint8_t *row_mask, const float *noise, float *out, float *out_lo,
                                       int rows) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, out, out_lo, rows, width_x > width_block ? width_x : width_block, false));
  return p.finish(ctx, residual_forward_padded_impl(ctx, x, width_x, block, width_block, row_mask, noise, out,
                                                    p.kernel_arg, rows, p.amax()));
}

dlb_status dlb_shakedrop_backward_window(dlb_ctx *ctx, const float *d, int width_d, int first,
                                         const uint8_t *row_mask, const float *noise, float *delta,
                                         float *delta_lo, int rows, int width) {
  PlaneOutput p;
  DLB_TRY(p.begin(ctx, delta, delta_lo, rows, width, false));
  return p.finish(ctx, shakedrop_backward_impl(ctx, d, width_d, first, row_mask, noise, delta, p.kernel_arg, rows,
                                               width, p.amax()));
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Evaluation: loss and accuracy counter of the outputs of a forward pass, no
// error.  One warp per row.
// ref: compute_loss_fwp_mp (v1/learner/compute_loss_mp.cpp L:28-113), loss_fn
// (v1/learner/compute_loss.cpp L:55-99).
// ---------------------------------------------------------------------------
namespace dlb {
__global__ void loss_eval_kernel(int loss, int accu_fn, float accu_var, const float *__restrict__ q,
                                 const float *__restrict__ y, int rows, int n, double *loss_sum,
                                 double *accu_sum) {
  pdl_enter();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) / 32, lane = threadIdx.x % 32;
  double local = 0.0, hits = 0.0;
  if (warp < rows) {
    const float *qr = q + (size_t)warp * n, *yr = y + (size_t)warp * n;
    const float EPS = 1e-7f;
    // Largest output (the last of equal maxima, as `q >= q_max` keeps it) and
    // the last target flag, for the cross-entropy accuracy.
    float best = -3.402823466e+38f;
    int predict = 0, target = n;
    for (int j = lane; j < n; j += 32) {
      const float qj = qr[j], yj = yr[j];
      if (loss == DLB_LOSS_CROSS_ENTROPY) {
        if (yj == 1.f) local += (double)(-(yj * logf(clipf(qj, EPS, 1.f - EPS))));
      } else {
        const float d = qj - yj;
        local += (double)(d * d);
      }
      if (accu_fn == DLB_ACCU_DISTANCE) {
        if (fabsf(qj - yj) <= accu_var) hits += 1.0;
      } else {
        if (qj >= best) { best = qj; predict = j; }
        if (yj == 1.f) target = j;
      }
    }
    if (accu_fn == DLB_ACCU_CROSS_ENTROPY) {
      for (int o = 16; o; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int op = __shfl_xor_sync(0xffffffffu, predict, o);
        int ot = __shfl_xor_sync(0xffffffffu, target, o);
        if (ob > best || (ob == best && op > predict)) { best = ob; predict = op; }
        // the last flagged index wins; n means none
        if (ot != n && (target == n || ot > target)) target = ot;
      }
      if (lane == 0 && predict == target) hits = 1.0;
    }
  }
  for (int o = 16; o; o >>= 1) {
    local += __shfl_xor_sync(0xffffffffu, local, o);
    if (accu_fn == DLB_ACCU_DISTANCE) hits += __shfl_xor_sync(0xffffffffu, hits, o);
  }
  if (lane == 0) {
    if (loss_sum && local != 0.0) atomicAdd(loss_sum, local);
    if (hits != 0.0) atomicAdd(accu_sum, hits);
  }
}
}  // namespace dlb

extern "C" dlb_status dlb_loss_eval(dlb_ctx *ctx, int loss, int accu_fn, float accu_var, const float *q,
                                    const float *y, int rows, int n_out, double *loss_sum,
                                    double *accu_sum) {
  DLB_REQUIRE(ctx && q && y && accu_sum && rows > 0 && n_out > 0, "dlb_loss_eval");
  if ((loss != DLB_LOSS_MSE && loss != DLB_LOSS_CROSS_ENTROPY) ||
      (accu_fn != DLB_ACCU_DISTANCE && accu_fn != DLB_ACCU_CROSS_ENTROPY)) {
    set_error("dlb_loss_eval: loss %d / accuracy function %d outside the supported set", loss, accu_fn);
    return DLB_ERR_UNSUPPORTED;
  }
  DLB_LAUNCH_KERNEL(ctx, loss_eval_kernel, ceil_div(rows, 8), 256, 0, loss, accu_fn, accu_var, q, y, rows, n_out, loss_sum, accu_sum);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}
