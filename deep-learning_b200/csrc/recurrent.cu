// Time-batched kernels of the recurrent (IndRNN) step.  Tensors are
// [T, rows, n] row-major: time step t, example b, unit h at ((t * rows) + b) * n
// + h, the reference's own order (v1/learner/fwp_rec_mp.cpp L:774-775).  Batch
// renormalization keeps statistics of its own per time step, stored [T, n]
// (v1/learner/allocate.cpp L:1348-1356), so one launch covers all T steps
// instead of T launches over [rows, n] slices.
//
//   time_major        [rows, T*n] (one example per row, as the caller holds it)
//                     -> [T, rows, n] plus the TF32 residual plane
//   time_reduce       per (t, unit) sums over the rows: statistics forward,
//                     the four batch-renormalization sums and du backward
//   time_forward      normalise, add u * h_{t-1}, activate: a thread owns
//                     (b, 4 units) and walks t = 0..T-1 with h in registers
//   time_backward     the reverse walk: dAF_t = dA_t f'_t + u f'_t dAF_{t+1}
//   time_apply        batch-renormalization backward apply for all t
//
// All are HBM-bound streaming kernels with 128-bit accesses when n % 4 == 0.
#include "common.cuh"
#include "math.cuh"
#include "planes.cuh"
#include "ring.cuh"

namespace dlb {

namespace {

constexpr int TR_LANES_X = 32;
constexpr int TR_LANES_Y = 8;
constexpr int TR_RING_DEPTH = 4;

template <int W>
struct Vec {
  float v[W];
};
template <int W>
__device__ __forceinline__ Vec<W> ldv(const float *p) {
  Vec<W> r;
  if constexpr (W == 4) {
    const float4 q = *reinterpret_cast<const float4 *>(p);
    r.v[0] = q.x; r.v[1] = q.y; r.v[2] = q.z; r.v[3] = q.w;
  } else {
    r.v[0] = *p;
  }
  return r;
}
template <int W>
__device__ __forceinline__ void stv(float *p, const Vec<W> &x) {
  if constexpr (W == 4) *reinterpret_cast<float4 *>(p) = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
  else *p = x.v[0];
}

// Per-(t, unit) constants of batch renormalization.
struct TimeBrn {
  const float *mean, *sigma, *r, *d;  // [T, n]
  const float *gamma, *beta;          // [n]
  const float *rs;                    // [T, n]: r / sigma, formed once per (t, unit) for the walks
};
static TimeBrn time_brn(const dlb_brn_unit_arrays *u) {
  return TimeBrn{u->mean, u->sigma, u->r, u->d, u->gamma, u->beta, nullptr};
}

// value_hat of v1/learner/fwp_mp.cpp L:4732, (z - mean) / sigma * r + d, through
// the per-(t, unit) quotient r / sigma: every time kernel normalises through
// this one expression, so all of them see the same bits on either side of a
// derivative jump.
__device__ __forceinline__ float hat(float z, float mean, float r_over_sigma, float d) {
  return __fmaf_rn(z - mean, r_over_sigma, d);
}

__global__ void time_quotient_kernel(const float *__restrict__ r, const float *__restrict__ sigma,
                                     float *__restrict__ rs, size_t total) {
  pdl_enter();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) rs[i] = r[i] / sigma[i];
}

// pre_t = y_t + u * h_{t-1}; the forward and the backward walk use this one
// expression so that both see the same bits on either side of a derivative kink.
__device__ __forceinline__ float recur(float y, float u, float h_prev) { return __fmaf_rn(u, h_prev, y); }

// ---------------------------------------------------------------------------
template <int W>
__global__ void time_major_kernel(const float *__restrict__ x, float *__restrict__ out,
                                  float *__restrict__ out_lo, int rows, int T, int n, unsigned *amax) {
  pdl_enter();
  const int nw = n / W;
  const size_t total = (size_t)T * rows * nw;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  unsigned mx = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int c = (int)(i % nw) * W;
    const size_t tb = i / nw;
    const int b = (int)(tb % rows), t = (int)(tb / rows);
    const Vec<W> v = ldv<W>(x + ((size_t)b * T + t) * n + c);
    stv<W>(out + i * W, v);
#pragma unroll
    for (int j = 0; j < W; ++j) mx = max(mx, abs_bits(v.v[j]));
    if (out_lo) {
      Vec<W> lo;
#pragma unroll
      for (int j = 0; j < W; ++j) lo.v[j] = tf32_lo(v.v[j]);
      stv<W>(out_lo + i * W, lo);
    }
  }
  amax_commit(amax, mx);
}

// ---------------------------------------------------------------------------
// Reductions over the rows for every (t, unit).  Grid (column blocks, T); a
// block of 32 x 8 threads covers 32*W units, each thread walks rows b = ty,
// ty+8, ... in float, the 8 row lanes fold in double in a fixed order.
// sums[(s * T + t) * n + h].
// ---------------------------------------------------------------------------
template <int NSUM, int W, class Op>
__global__ void __launch_bounds__(TR_LANES_X *TR_LANES_Y)
    time_reduce_kernel(Op op, int T, int rows, int n, double *__restrict__ sums) {
  pdl_enter();
  __shared__ double red[TR_LANES_Y][NSUM][TR_LANES_X * W + 1];
  const int tx = threadIdx.x % TR_LANES_X, ty = threadIdx.x / TR_LANES_X;
  const int col = (blockIdx.x * TR_LANES_X + tx) * W;
  const int t = blockIdx.y;
  float acc[NSUM][W];
#pragma unroll
  for (int s = 0; s < NSUM; ++s)
#pragma unroll
    for (int j = 0; j < W; ++j) acc[s][j] = 0.f;
  if (col < n) {
    typename Op::template Cols<W> k;
    op.template load<W>(t, col, n, k);
    if constexpr (W == 4 && Op::RING_NIN > 0) {
      // The rows through the thread's copy ring (ring.cuh): TR_RING_DEPTH - 1
      // rows of every input under way while one is added up.
      extern __shared__ float4 reduce_ring[];
      const float *in[Op::RING_NIN];
      op.ring_inputs(t, (size_t)rows * n, in);
      ring_walk<Op::RING_NIN, TR_RING_DEPTH, TR_LANES_X * TR_LANES_Y>(
          reduce_ring, in, (size_t)n, col, t * rows + ty, (t + 1) * rows, TR_LANES_Y,
          [&](int, const float4(&x)[Op::RING_NIN]) { op.use4(t, k, x, acc); });
    } else {
      for (int b = ty; b < rows; b += TR_LANES_Y)
        op.template row<W>(t, ((size_t)t * rows + b) * n + col, (size_t)rows * n, k, acc);
    }
  }
#pragma unroll
  for (int s = 0; s < NSUM; ++s)
#pragma unroll
    for (int j = 0; j < W; ++j) red[ty][s][tx * W + j] = (double)acc[s][j];
  __syncthreads();
  for (int i = threadIdx.x; i < NSUM * TR_LANES_X * W; i += TR_LANES_X * TR_LANES_Y) {
    const int s = i / (TR_LANES_X * W), c = i % (TR_LANES_X * W);
    const int gc = blockIdx.x * TR_LANES_X * W + c;
    if (gc < n) {
      double v = 0.0;
#pragma unroll
      for (int y = 0; y < TR_LANES_Y; ++y) v += red[y][s][c];
      sums[((size_t)s * T + t) * n + gc] = v;
    }
  }
}

struct TimeSumSqOp {
  const float *Z;
  static constexpr int RING_NIN = 0;  // plain loads: 6.3 TB/s as it is
  template <int W> struct Cols {};
  template <int W> __device__ void load(int, int, int, Cols<W> &) const {}
  template <int W>
  __device__ void row(int, size_t o, size_t, const Cols<W> &, float (&acc)[2][W]) const {
    const Vec<W> z = ldv<W>(Z + o);
#pragma unroll
    for (int j = 0; j < W; ++j) {
      acc[0][j] += z.v[j];
      acc[1][j] += z.v[j] * z.v[j];
    }
  }
};

// Backward sums over dAF (the error w.r.t. the normalised value):
//   NORM: s0 = sum e x_hat, s1 = sum e, s2 = sum e gamma (-r / sigma),
//         s3 = sum e gamma (z - mean) (-r / sigma^2)   (bwp_mp.cpp L:1559-1574)
//   REC:  last sum = sum h_{t-1} e for t >= 1   (update_derivative_rec_mp.cpp L:460-487)
template <bool NORM, bool REC>
struct TimeBackwardOp {
  const float *E, *Z, *A;
  TimeBrn u;
  static constexpr int NS = (NORM ? 4 : 0) + (REC ? 1 : 0);
  // Through the ring: the error, the sums (NORM) and the output of the step
  // before (REC).  At t = 0 that stream reads the step's own output, which is
  // valid memory, and the values are not used.
  static constexpr int RING_NIN = 1 + (NORM ? 1 : 0) + (REC ? 1 : 0);
  __device__ void ring_inputs(int t, size_t step, const float *(&in)[RING_NIN]) const {
    int i = 0;
    in[i++] = E;
    if (NORM) in[i++] = Z;
    if (REC) in[i++] = t > 0 ? A - step : A;
  }
  template <class K>
  __device__ void use4(int t, const K &k, const float4 (&x)[RING_NIN], float (&acc)[NS][4]) const {
    const float e[4] = {x[0].x, x[0].y, x[0].z, x[0].w};
    if (NORM) {
      const float z[4] = {x[1].x, x[1].y, x[1].z, x[1].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float xh = hat(z[j], k.mean[j], k.rs[j], k.d[j]);
        acc[0][j] += e[j] * xh;
        acc[1][j] += e[j];
        const float eh = e[j] * k.gamma[j];
        acc[2][j] += eh * k.q_mean[j];
        acc[3][j] += eh * (z[j] - k.mean[j]) * k.q_sigma[j];
      }
    }
    if (REC && t > 0) {
      const float4 q = x[RING_NIN - 1];
      const float hp[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[NS - 1][j] += hp[j] * e[j];
    }
  }
  template <int W>
  struct Cols {
    float mean[W], sigma[W], r[W], rs[W], d[W], gamma[W], q_mean[W], q_sigma[W];
  };
  template <int W>
  __device__ void load(int t, int col, int n, Cols<W> &k) const {
    if constexpr (NORM) {
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const size_t i = (size_t)t * n + col + j;
      k.mean[j] = u.mean[i];
      k.sigma[j] = u.sigma[i];
      k.r[j] = u.r[i];
      k.rs[j] = k.r[j] / k.sigma[j];
      k.d[j] = u.d[i];
      k.gamma[j] = u.gamma[col + j];
      const float neg_r = -k.r[j];
      k.q_mean[j] = neg_r / k.sigma[j];
      k.q_sigma[j] = neg_r / (k.sigma[j] * k.sigma[j]);
    }
    }
  }
  template <int W>
  __device__ void row(int t, size_t o, size_t step, const Cols<W> &k, float (&acc)[NS][W]) const {
    const Vec<W> e = ldv<W>(E + o);
    if (NORM) {
      const Vec<W> z = ldv<W>(Z + o);
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const float xh = hat(z.v[j], k.mean[j], k.rs[j], k.d[j]);
        acc[0][j] += e.v[j] * xh;
        acc[1][j] += e.v[j];
        const float eh = e.v[j] * k.gamma[j];
        acc[2][j] += eh * k.q_mean[j];
        acc[3][j] += eh * (z.v[j] - k.mean[j]) * k.q_sigma[j];
      }
    }
    if (REC && t > 0) {
      const Vec<W> hp = ldv<W>(A + o - step);
#pragma unroll
      for (int j = 0; j < W; ++j) acc[NS - 1][j] += hp.v[j] * e.v[j];
    }
  }
};

// mean, sigma, running averages, r and d for every (t, unit), in the order of
// v1/learner/fwp_mp.cpp L:4688-4717 (the averages move first).
__global__ void time_finalize_kernel(const double *__restrict__ sums, int T, int n, float batch_scale,
                                     float momentum, float eps, float r_max, float d_max,
                                     dlb_brn_unit_arrays u) {
  pdl_enter();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)T * n;
  if (i >= total) return;
  const float mean = (float)sums[i] * batch_scale;
  float mavg = u.mean_average[i];
  mavg += momentum * (mean - mavg);
  const float sigma = sqrtf((float)sums[total + i] * batch_scale - mean * mean + eps);
  float savg = u.sigma_average[i];
  savg += momentum * (sigma - savg);
  u.mean[i] = mean;
  u.sigma[i] = sigma;
  u.mean_average[i] = mavg;
  u.sigma_average[i] = savg;
  u.r[i] = clipf(sigma / savg, 1.f / r_max, r_max);
  u.d[i] = clipf((mean - mavg) / savg, -d_max, d_max);
}

// out[h] (+)= sum over t (from T-1 down, the backward order) of sums[t, h].
__global__ void time_fold_kernel(const double *__restrict__ sums, int T, int n, float *out) {
  pdl_enter();
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= n) return;
  double v = 0.0;
  for (int t = T - 1; t >= 0; --t) v += sums[(size_t)t * n + h];
  out[h] += (float)v;
}

// y_t = gamma * x_hat + beta for the units a thread owns, statistics of step t.
template <int W>
__device__ __forceinline__ Vec<W> normalised(const Vec<W> &z, const TimeBrn &u, size_t stat,
                                             const float (&gamma)[W], const float (&beta)[W]) {
  const Vec<W> mean = ldv<W>(u.mean + stat), rs = ldv<W>(u.rs + stat), d = ldv<W>(u.d + stat);
  Vec<W> y;
#pragma unroll
  for (int j = 0; j < W; ++j) y.v[j] = __fmaf_rn(gamma[j], hat(z.v[j], mean.v[j], rs.v[j], d.v[j]), beta[j]);
  return y;
}

// Forward walk over time.  One thread per (example, W units); h stays in
// registers from one step to the next, and the loads of step t + 1 do not
// depend on step t, so the compiler can issue them ahead of the dependent math.
// ref: Forward_Pass__FC_Ind_RNN__OpenMP (v1/learner/fwp_rec_mp.cpp L:762-800)
// followed by the activation (L:335-348).
// DROP: Bernoulli dropout of time step t, flags mask[t * n + unit], applied to
// the stored output, so that the recurrence of step t + 1 reads the masked
// value (fwp_mp.cpp L:1228-1262, L:4842-4868); kept units are multiplied by
// keep_scale (1, or 1 / p for the inverted form); without a mask every unit is
// (the inference form, fwp_rec_mp.cpp L:299-312).
template <int W, bool NORM, bool REC, bool DROP>
__global__ void __launch_bounds__(256)
    time_forward_kernel(const float *__restrict__ Z, TimeBrn u, const float *__restrict__ rec, int af,
                        const uint8_t *__restrict__ mask, float keep_scale, const float *__restrict__ noise,
                        float *__restrict__ A, float *__restrict__ A_lo, int T, int rows, int n,
                        unsigned *amax) {
  pdl_enter();
  const int nw = n / W;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nw) return;
  unsigned mx = 0;
  const int col = (int)(i % nw) * W;
  const size_t step = (size_t)rows * n;
  size_t o = (i / nw) * n + col;
  float gamma[W], beta[W], w[W], h[W];
#pragma unroll
  for (int j = 0; j < W; ++j) {
    gamma[j] = NORM ? u.gamma[col + j] : 1.f;
    beta[j] = NORM ? u.beta[col + j] : 0.f;
    w[j] = REC ? rec[col + j] : 0.f;
    h[j] = 0.f;
  }
#pragma unroll 4
  for (int t = 0; t < T; ++t, o += step) {
    Vec<W> y = ldv<W>(Z + o);
    if (NORM) y = normalised<W>(y, u, (size_t)t * n + col, gamma, beta);
    Vec<W> out, lo;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float pre = (REC && t > 0) ? recur(y.v[j], w[j], h[j]) : y.v[j];
      h[j] = af_fire(af, pre);
      if (DROP) {
        // UOut: h += h * U(-beta, beta), a draw per element (fwp_mp.cpp L:4959-4985).
        if (noise) h[j] = h[j] + h[j] * noise[o + j];
        const float f = mask ? (mask[(size_t)t * n + col + j] ? keep_scale : 0.f) : keep_scale;
        h[j] = f == 0.f ? 0.f : (f == 1.f ? h[j] : h[j] * f);
      }
      out.v[j] = h[j];
      lo.v[j] = tf32_lo(h[j]);
      mx = max(mx, abs_bits(h[j]));
    }
    stv<W>(A + o, out);
    if (A_lo) stv<W>(A_lo + o, lo);
  }
  amax_commit(amax, mx);
}

// The forward walk with its loads through the thread's copy ring (ring.cuh):
// the sums of WALK_FWD_DEPTH - 1 time steps ahead and their statistics are under
// way while a step is worked on, at no cost in registers.  Same arithmetic,
// element for element, as time_forward_kernel<4, ...>, which stays for widths
// that are not a multiple of four.  Measured at [64, 1024, 2048]: 299 us with
// plain loads (the compiler keeps one step's loads in flight at 56 registers;
// DRAM 41 %, L2 25 %, L1 30 % busy: latency-bound), 202 us through the ring with
// blocks of 128 threads and three slots (eight blocks to an SM; deeper rings
// with fewer threads were slower: 224 us with four slots, 274 with six).
constexpr int WALK_BLOCK = 128;
constexpr int WALK_FWD_DEPTH = 3;
// PLANES: the kernel writes the fp16 planes of A with the scale predicted for
// them and the row / column maxima of the range guard (n a multiple of 128, so
// that the lanes of a warp are on one row).
template <bool NORM, bool REC, bool DROP, bool PLANES>
__global__ void __launch_bounds__(WALK_BLOCK)
    time_forward_ring_kernel(const float *__restrict__ Z, TimeBrn u, const float *__restrict__ rec, int af,
                             const uint8_t *__restrict__ mask, float keep_scale, const float *__restrict__ noise,
                             float *__restrict__ A, float *__restrict__ A_lo, int T, int rows, int n,
                             unsigned *amax, PlaneSink sink) {
  pdl_enter();
  extern __shared__ float4 walk_ring[];
  constexpr int W = 4;
  constexpr int NIN = NORM ? 4 : 1;
  const int nw = n / W;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = i < (size_t)rows * nw;
  unsigned mx = 0;
  const float plane_scale = PLANES ? sink_scale(sink) : 1.f;
  LineTracker track;
  if (live) {
    const int col = (int)(i % nw) * W;
    const size_t step = (size_t)rows * n;
    size_t o = (i / nw) * n + col;
    int row = (int)(i / nw);  // of the [T * rows, n] matrix
    float gamma[W], beta[W], w[W], h[W];
#pragma unroll
    for (int j = 0; j < W; ++j) {
      gamma[j] = NORM ? u.gamma[col + j] : 1.f;
      beta[j] = NORM ? u.beta[col + j] : 0.f;
      w[j] = REC ? rec[col + j] : 0.f;
      h[j] = 0.f;
    }
    const char *src[NIN];
    long long stride[NIN];
    src[0] = reinterpret_cast<const char *>(Z + o);
    stride[0] = (long long)(step * sizeof(float));
    if constexpr (NORM) {
      src[1] = reinterpret_cast<const char *>(u.mean + col);
      src[2] = reinterpret_cast<const char *>(u.rs + col);
      src[3] = reinterpret_cast<const char *>(u.d + col);
      stride[1] = stride[2] = stride[3] = (long long)((size_t)n * sizeof(float));
    }
    int valid[NIN];
#pragma unroll
    for (int k = 0; k < NIN; ++k) valid[k] = T;
    ring_steps<NIN, WALK_FWD_DEPTH, WALK_BLOCK>(walk_ring, src, stride, valid, T, [&](int t, const float4(&x)[NIN]) {
      float y[W] = {x[0].x, x[0].y, x[0].z, x[0].w};
      if constexpr (NORM) {
        const float mean[W] = {x[1].x, x[1].y, x[1].z, x[1].w}, rs[W] = {x[2].x, x[2].y, x[2].z, x[2].w},
                    d[W] = {x[3].x, x[3].y, x[3].z, x[3].w};
#pragma unroll
        for (int j = 0; j < W; ++j) y[j] = __fmaf_rn(gamma[j], hat(y[j], mean[j], rs[j], d[j]), beta[j]);
      }
      Vec<W> out, lo;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const float pre = (REC && t > 0) ? recur(y[j], w[j], h[j]) : y[j];
        h[j] = af_fire(af, pre);
        if (DROP) {
          if (noise) h[j] = h[j] + h[j] * noise[o + j];
          const float f = mask ? (mask[(size_t)t * n + col + j] ? keep_scale : 0.f) : keep_scale;
          h[j] = f == 0.f ? 0.f : (f == 1.f ? h[j] : h[j] * f);
        }
        out.v[j] = h[j];
        lo.v[j] = tf32_lo(h[j]);
        mx = max(mx, abs_bits(h[j]));
      }
      stv<W>(A + o, out);
      if (PLANES) {
        sink_store4(sink, o, out.v, plane_scale);
        track.row(sink, row, out.v);
      } else if (A_lo) {
        stv<W>(A_lo + o, lo);
      }
      o += step;
      row += rows;
    });
    if (PLANES && sink.colmax) {
      // Every thread of the grid owns four columns of one example: a column's
      // maximum is raised by the few threads that exceed what is there.
#pragma unroll
      for (int j = 0; j < W; ++j)
        if (track.cm[j] > __ldcg(sink.colmax + col + j)) atomicMax(sink.colmax + col + j, track.cm[j]);
    }
  }
  if (PLANES) amax_commit(reinterpret_cast<unsigned *>(sink.slot) + SLOT_AMAX, track.all);
  else amax_commit(amax, mx);
}

// Reverse walk: E holds dA on entry and dAF on return.
// ref: Backward_Pass__FC__DF_Ind_RNN__OpenMP (v1/learner/bwp_mp.cpp L:1188-1263).
// pre_t is recomputed from Z, the statistics and h_{t-1} with the forward
// walk's own expressions instead of being stored.
template <int W, bool NORM, bool REC>
__global__ void __launch_bounds__(256)
    time_backward_kernel(float *__restrict__ E, const float *__restrict__ Z,
                         const float *__restrict__ A, TimeBrn u, const float *__restrict__ rec, int af,
                         int T, int rows, int n) {
  pdl_enter();
  const int nw = n / W;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nw) return;
  const int col = (int)(i % nw) * W;
  const size_t step = (size_t)rows * n;
  size_t o = (i / nw) * n + col + (size_t)(T - 1) * step;
  float gamma[W], beta[W], w[W], next[W];
#pragma unroll
  for (int j = 0; j < W; ++j) {
    gamma[j] = NORM ? u.gamma[col + j] : 1.f;
    beta[j] = NORM ? u.beta[col + j] : 0.f;
    w[j] = REC ? rec[col + j] : 0.f;
    next[j] = 0.f;
  }
  Vec<W> h = ldv<W>(A + o);
#pragma unroll 4
  for (int t = T - 1; t >= 0; --t, o -= step) {
    const Vec<W> da = ldv<W>(E + o);
    Vec<W> y = ldv<W>(Z + o);
    if (NORM) y = normalised<W>(y, u, (size_t)t * n + col, gamma, beta);
    Vec<W> hp;
    if (t > 0) hp = ldv<W>(A + o - step);
    Vec<W> e;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float pre = (REC && t > 0) ? recur(y.v[j], w[j], hp.v[j]) : y.v[j];
      const float fp = af_derive(af, pre, h.v[j]);
      const float d = da.v[j] * fp;
      e.v[j] = (REC && t + 1 != T) ? d + w[j] * fp * next[j] : d;
      next[j] = e.v[j];
    }
    stv<W>(E + o, e);
    if (t > 0) h = hp;
  }
}

// The reverse walk through the copy ring: per step the error, the sums and the
// output of the step before (h_{t-1}; the stream ends one step early), and the
// step's statistics.  Same arithmetic as time_backward_kernel<4, ...>.
constexpr int WALK_BWD_DEPTH = 3;
template <bool NORM, bool REC>
__global__ void __launch_bounds__(WALK_BLOCK)
    time_backward_ring_kernel(float *__restrict__ E, const float *__restrict__ Z, const float *__restrict__ A,
                              TimeBrn u, const float *__restrict__ rec, int af, int T, int rows, int n) {
  pdl_enter();
  extern __shared__ float4 walk_ring[];
  constexpr int W = 4;
  constexpr int NIN = NORM ? 6 : 3;
  const int nw = n / W;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * nw) return;
  const int col = (int)(i % nw) * W;
  const size_t step = (size_t)rows * n;
  size_t o = (i / nw) * n + col + (size_t)(T - 1) * step;
  float gamma[W], beta[W], w[W], next[W];
#pragma unroll
  for (int j = 0; j < W; ++j) {
    gamma[j] = NORM ? u.gamma[col + j] : 1.f;
    beta[j] = NORM ? u.beta[col + j] : 0.f;
    w[j] = REC ? rec[col + j] : 0.f;
    next[j] = 0.f;
  }
  Vec<W> h = ldv<W>(A + o);
  const char *src[NIN];
  long long stride[NIN];
  int valid[NIN];
  const long long back = -(long long)(step * sizeof(float));
  src[0] = reinterpret_cast<const char *>(E + o);
  src[1] = reinterpret_cast<const char *>(Z + o);
  src[2] = reinterpret_cast<const char *>(A + o) + back;  // h_{t-1}
  stride[0] = stride[1] = stride[2] = back;
  valid[0] = valid[1] = T;
  valid[2] = T - 1;
  if constexpr (NORM) {
    const size_t s0 = (size_t)(T - 1) * n + col;
    src[3] = reinterpret_cast<const char *>(u.mean + s0);
    src[4] = reinterpret_cast<const char *>(u.rs + s0);
    src[5] = reinterpret_cast<const char *>(u.d + s0);
    stride[3] = stride[4] = stride[5] = -(long long)((size_t)n * sizeof(float));
    valid[3] = valid[4] = valid[5] = T;
  }
  ring_steps<NIN, WALK_BWD_DEPTH, WALK_BLOCK>(walk_ring, src, stride, valid, T, [&](int k, const float4(&x)[NIN]) {
    const int t = T - 1 - k;
    const float da[W] = {x[0].x, x[0].y, x[0].z, x[0].w};
    float y[W] = {x[1].x, x[1].y, x[1].z, x[1].w};
    const float hp[W] = {x[2].x, x[2].y, x[2].z, x[2].w};  // read for t > 0 only
    if constexpr (NORM) {
      const float mean[W] = {x[3].x, x[3].y, x[3].z, x[3].w}, rs[W] = {x[4].x, x[4].y, x[4].z, x[4].w},
                  d[W] = {x[5].x, x[5].y, x[5].z, x[5].w};
#pragma unroll
      for (int j = 0; j < W; ++j) y[j] = __fmaf_rn(gamma[j], hat(y[j], mean[j], rs[j], d[j]), beta[j]);
    }
    Vec<W> e;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float pre = (REC && t > 0) ? recur(y[j], w[j], hp[j]) : y[j];
      const float fp = af_derive(af, pre, h.v[j]);
      const float dd = da[j] * fp;
      e.v[j] = (REC && t + 1 != T) ? dd + w[j] * fp * next[j] : dd;
      next[j] = e.v[j];
    }
    stv<W>(E + o, e);
    if (t > 0) {
#pragma unroll
      for (int j = 0; j < W; ++j) h.v[j] = hp[j];
    }
    o -= step;
  });
}

// Batch-renormalization backward apply for every t (bwp_mp.cpp L:1608-1621).
// Grid (column blocks, T), rows walked with stride 8.
template <int W, bool PLANES = false>
__global__ void __launch_bounds__(TR_LANES_X *TR_LANES_Y)
    time_apply_kernel(float *__restrict__ delta, float *__restrict__ delta_lo,
                      const float *__restrict__ Z, TimeBrn u, const double *__restrict__ sums,
                      float inv_rows, float rows_f, int T, int rows, int n, unsigned *amax, PlaneSink sink) {
  pdl_enter();
  __shared__ unsigned fold[PLANES ? TR_LANES_Y * TR_LANES_X * 4 : 1];
  const int tx = threadIdx.x % TR_LANES_X, ty = threadIdx.x / TR_LANES_X;
  const int col = (blockIdx.x * TR_LANES_X + tx) * W;
  const int t = blockIdx.y;
  const float plane_scale = PLANES ? sink_scale(sink) : 1.f;
  LineTracker track;
  if (PLANES) {
    // W = 4 here; every thread reaches the fold below.
    if (col < n) {
      float gamma[4], mean[4], r_over_sigma[4], n_sigma[4], d_sigma[4], d_mean_n[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const size_t s = (size_t)t * n + col + j;
        const float sigma = u.sigma[s];
        gamma[j] = u.gamma[col + j];
        mean[j] = u.mean[s];
        r_over_sigma[j] = u.r[s] / sigma;
        n_sigma[j] = rows_f * sigma;
        d_mean_n[j] = (float)sums[((size_t)2 * T + t) * n + col + j] * inv_rows;
        d_sigma[j] = (float)sums[((size_t)3 * T + t) * n + col + j];
      }
      // The rows come through the thread's copy ring (ring.cuh).
      extern __shared__ float4 apply_ring[];
      const float *in[2] = {delta, Z};
      ring_walk<2, TR_RING_DEPTH, TR_LANES_X * TR_LANES_Y>(
          apply_ring, in, (size_t)n, col, t * rows + ty, (t + 1) * rows, TR_LANES_Y, [&](int r, const float4(&x)[2]) {
            const size_t o = (size_t)r * n + col;
            const float e[4] = {x[0].x, x[0].y, x[0].z, x[0].w}, z[4] = {x[1].x, x[1].y, x[1].z, x[1].w};
            float out[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float v = e[j] * gamma[j];
              v *= r_over_sigma[j];
              v += d_sigma[j] * ((z[j] - mean[j]) / n_sigma[j]);
              v += d_mean_n[j];
              out[j] = v;
            }
            *reinterpret_cast<float4 *>(delta + o) = make_float4(out[0], out[1], out[2], out[3]);
            sink_store4(sink, o, out, plane_scale);
            track.row(sink, r, out);
          });
    }
    track.finish(sink, fold, tx, ty, TR_LANES_Y, blockIdx.x * TR_LANES_X * 4, n, col < n, TR_LANES_X);
    return;
  }
  if (col >= n) return;
  unsigned mx = 0;
  float gamma[W], mean[W], r_over_sigma[W], n_sigma[W], d_sigma[W], d_mean_n[W];
#pragma unroll
  for (int j = 0; j < W; ++j) {
    const size_t s = (size_t)t * n + col + j;
    const float sigma = u.sigma[s];
    gamma[j] = u.gamma[col + j];
    mean[j] = u.mean[s];
    r_over_sigma[j] = u.r[s] / sigma;
    n_sigma[j] = rows_f * sigma;
    d_mean_n[j] = (float)sums[((size_t)2 * T + t) * n + col + j] * inv_rows;
    d_sigma[j] = (float)sums[((size_t)3 * T + t) * n + col + j];
  }
  for (int b = ty; b < rows; b += TR_LANES_Y) {
    const size_t o = ((size_t)t * rows + b) * n + col;
    const Vec<W> e = ldv<W>(delta + o), z = ldv<W>(Z + o);
    Vec<W> out, lo;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      float v = e.v[j] * gamma[j];
      v *= r_over_sigma[j];
      v += d_sigma[j] * ((z.v[j] - mean[j]) / n_sigma[j]);
      v += d_mean_n[j];
      out.v[j] = v;
      lo.v[j] = tf32_lo(v);
      mx = max(mx, abs_bits(v));
    }
    stv<W>(delta + o, out);
    if (delta_lo) stv<W>(delta_lo + o, lo);
  }
  amax_commit(amax, mx);
}

__global__ void clamp_kernel(float *p, int n, float lo, float hi) {
  pdl_enter();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = clipf(p[i], lo, hi);
}

bool aligned16(std::initializer_list<const void *> ps) {
  for (const void *p : ps)
    if (reinterpret_cast<uintptr_t>(p) & 15) return false;
  return true;
}

int walk_grid(size_t threads) { return (int)((threads + 255) / 256); }

// Lets a walk kernel take `bytes` of dynamic shared memory on the current
// device; once per kernel and device.
template <auto Kernel>
void walk_shared_limit(size_t bytes) {
  static bool done[MAX_DEVICES] = {};
  int dev = 0;
  // (A kernel with static shared memory of its own needs the attribute below 48 KB too.)
  if (bytes == 0 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES || done[dev]) return;
  if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess)
    done[dev] = true;
  else
    cudaGetLastError();
}

// r / sigma for every (t, unit) into context scratch, for the walk that follows.
dlb_status time_quotients(dlb_ctx *ctx, TimeBrn *p, int T, int n) {
  const size_t total = (size_t)T * n;
  void *scr = nullptr;
  DLB_TRY(scratch(ctx, total * sizeof(float), &scr));
  float *rs = static_cast<float *>(scr);
  DLB_LAUNCH_KERNEL(ctx, time_quotient_kernel, (unsigned)((total + 255) / 256), 256, 0, p->r, p->sigma, rs, total);
  DLB_LAUNCHED(ctx);
  p->rs = rs;
  return DLB_OK;
}

}  // namespace
}  // namespace dlb

using namespace dlb;

extern "C" {

dlb_status time_major_impl(dlb_ctx *ctx, const float *x, float *out, float *out_lo, int rows,
                          int seq_w, int n, unsigned *amax) {
  DLB_REQUIRE(ctx && x && out && rows > 0 && seq_w > 0 && n > 0, "dlb_time_major");
  const bool v4 = n % 4 == 0 && aligned16({x, out, out_lo});
  const size_t items = (size_t)seq_w * rows * (v4 ? n / 4 : n);
  const int grid = (int)min((items + 255) / 256, (size_t)ctx->sm_count * 16);
  if (v4) DLB_LAUNCH_KERNEL(ctx, time_major_kernel<4>, grid, 256, 0, x, out, out_lo, rows, seq_w, n, amax);
  else DLB_LAUNCH_KERNEL(ctx, time_major_kernel<1>, grid, 256, 0, x, out, out_lo, rows, seq_w, n, amax);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_brn_time_forward_sums(dlb_ctx *ctx, const float *Z, int seq_w, int rows, int n,
                                     double *sums) {
  DLB_REQUIRE(ctx && Z && sums && seq_w > 0 && rows > 0 && n > 0, "dlb_brn_time_forward_sums");
  const bool v4 = n % 4 == 0 && aligned16({Z});
  const dim3 grid(ceil_div(n, TR_LANES_X * (v4 ? 4 : 1)), seq_w);
  if (v4)
    DLB_LAUNCH_KERNEL(ctx, (time_reduce_kernel<2, 4, TimeSumSqOp>), grid, TR_LANES_X * TR_LANES_Y, 0, TimeSumSqOp{Z}, seq_w, rows, n, sums);
  else
    DLB_LAUNCH_KERNEL(ctx, (time_reduce_kernel<2, 1, TimeSumSqOp>), grid, TR_LANES_X * TR_LANES_Y, 0, TimeSumSqOp{Z}, seq_w, rows, n, sums);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_brn_time_forward_finalize(dlb_ctx *ctx, const double *sums, int global_rows,
                                         int seq_w, int n, float momentum, float epsilon,
                                         float r_max, float d_max, const dlb_brn_unit_arrays *u) {
  DLB_REQUIRE(ctx && sums && u && global_rows > 0 && seq_w > 0 && n > 0, "dlb_brn_time_forward_finalize");
  DLB_REQUIRE(u->mean && u->sigma && u->mean_average && u->sigma_average && u->r && u->d,
              "dlb_brn_time_forward_finalize: null unit array");
  const size_t total = (size_t)seq_w * n;
  DLB_LAUNCH_KERNEL(ctx, time_finalize_kernel, (unsigned)((total + 255) / 256), 256, 0, sums, seq_w, n, 1.f / (float)global_rows, momentum, epsilon, r_max, d_max, *u);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// Whether the forward walk can write the planes of its output itself.
static bool walk_writes_planes(const float *Z, const float *A, const dlb_brn_unit_arrays *u, int n) {
  return n % 128 == 0 && aligned16({Z, A}) && (!u || aligned16({u->mean, u->d}));
}

dlb_status indrnn_forward_impl(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                              const float *recurrent, int af, const uint8_t *mask, float keep_scale,
                              const float *noise, float *A, float *A_lo, int seq_w, int rows, int n,
                              unsigned *amax, const PlaneSink *sink = nullptr) {
  DLB_REQUIRE(ctx && Z && A && seq_w > 0 && rows > 0 && n > 0, "dlb_indrnn_forward");
  TimeBrn p{};
  if (u) {
    p = time_brn(u);
    DLB_TRY(time_quotients(ctx, &p, seq_w, n));
  }
  const bool v4 = n % 4 == 0 && aligned16({Z, A, A_lo, p.mean, p.rs, p.d});
  const int grid = walk_grid((size_t)rows * (v4 ? n / 4 : n));
  const bool drop = mask != nullptr || keep_scale != 1.f || noise != nullptr;
#define LAUNCH(W, NORM, REC)                                                                          \
  do {                                                                                                \
    if (drop)                                                                                         \
      DLB_LAUNCH_KERNEL(ctx, (time_forward_kernel<W, NORM, REC, true>), grid, 256, 0, Z, p, recurrent, af, mask, keep_scale, noise, A, A_lo, seq_w, rows, n, amax);                      \
    else                                                                                              \
      DLB_LAUNCH_KERNEL(ctx, (time_forward_kernel<W, NORM, REC, false>), grid, 256, 0, Z, p, recurrent, af, nullptr, 1.f, nullptr, A, A_lo, seq_w, rows, n, amax);                          \
  } while (0)
#define PICK(W)                                                        \
  do {                                                                 \
    if (u && recurrent) LAUNCH(W, true, true);                         \
    else if (u) LAUNCH(W, true, false);                                \
    else if (recurrent) LAUNCH(W, false, true);                        \
    else LAUNCH(W, false, false);                                      \
  } while (0)
  if (v4) {
    // Through the copy ring; shared memory: DEPTH slots of 1 or 4 float4 per thread.
    const int ring_grid = (int)(((size_t)rows * (n / 4) + WALK_BLOCK - 1) / WALK_BLOCK);
    const PlaneSink none{};
#define RING3(NORM, REC, DROP, PL)                                                                               \
  do {                                                                                                           \
    constexpr size_t bytes = ring_bytes(NORM ? 4 : 1, WALK_FWD_DEPTH, WALK_BLOCK);                               \
    walk_shared_limit<time_forward_ring_kernel<NORM, REC, DROP, PL>>(bytes);                                     \
    DLB_LAUNCH_KERNEL(ctx, (time_forward_ring_kernel<NORM, REC, DROP, PL>), ring_grid, WALK_BLOCK, bytes, Z, p, recurrent, af, DROP ? mask : nullptr, DROP ? keep_scale : 1.f, DROP ? noise : nullptr, A, A_lo, seq_w, rows, n, amax, PL ? *sink : none); \
  } while (0)
#define RING(NORM, REC)                                                                                          \
  do {                                                                                                           \
    if (sink && drop) RING3(NORM, REC, true, true);                                                              \
    else if (sink) RING3(NORM, REC, false, true);                                                                \
    else if (drop) RING3(NORM, REC, true, false);                                                                \
    else RING3(NORM, REC, false, false);                                                                         \
  } while (0)
    if (u && recurrent) RING(true, true);
    else if (u) RING(true, false);
    else if (recurrent) RING(false, true);
    else RING(false, false);
#undef RING
#undef RING3
  } else {
    PICK(1);
  }
#undef LAUNCH
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_indrnn_backward_walk(dlb_ctx *ctx, float *E, const float *Z, const float *A,
                                    const dlb_brn_unit_arrays *u, const float *recurrent, int af,
                                    int seq_w, int rows, int n) {
  DLB_REQUIRE(ctx && E && Z && A && seq_w > 0 && rows > 0 && n > 0, "dlb_indrnn_backward_walk");
  TimeBrn p{};
  if (u) {
    p = time_brn(u);
    DLB_TRY(time_quotients(ctx, &p, seq_w, n));
  }
  const bool v4 = n % 4 == 0 && aligned16({E, Z, A, p.mean, p.rs, p.d});
  const int grid = walk_grid((size_t)rows * (v4 ? n / 4 : n));
#define LAUNCH(W, NORM, REC)                                                                 \
  DLB_LAUNCH_KERNEL(ctx, (time_backward_kernel<W, NORM, REC>), grid, 256, 0, E, Z, A, p, recurrent, af, seq_w, rows, n)
  if (v4) {
    const int ring_grid = (int)(((size_t)rows * (n / 4) + WALK_BLOCK - 1) / WALK_BLOCK);
#define RING(NORM, REC)                                                                       \
  do {                                                                                        \
    constexpr size_t bytes = ring_bytes(NORM ? 6 : 3, WALK_BWD_DEPTH, WALK_BLOCK);            \
    walk_shared_limit<time_backward_ring_kernel<NORM, REC>>(bytes);                           \
    DLB_LAUNCH_KERNEL(ctx, (time_backward_ring_kernel<NORM, REC>), ring_grid, WALK_BLOCK, bytes, E, Z, A, p, recurrent, af, seq_w, rows, n); \
  } while (0)
    if (u && recurrent) RING(true, true);
    else if (u) RING(true, false);
    else if (recurrent) RING(false, true);
    else RING(false, false);
#undef RING
  } else {
    PICK(1);
  }
#undef LAUNCH
#undef PICK
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_indrnn_backward_sums(dlb_ctx *ctx, const float *E, const float *Z, const float *A,
                                    const dlb_brn_unit_arrays *u, int recurrent, int seq_w,
                                    int rows, int n, double *sums) {
  DLB_REQUIRE(ctx && E && sums && seq_w > 0 && rows > 0 && n > 0 && (u || recurrent),
              "dlb_indrnn_backward_sums");
  DLB_REQUIRE((!u || Z) && (!recurrent || A), "dlb_indrnn_backward_sums: missing tensor");
  TimeBrn p{};
  if (u) p = time_brn(u);
  const bool v4 = n % 4 == 0 && aligned16({E, Z, A});
  const dim3 grid(ceil_div(n, TR_LANES_X * (v4 ? 4 : 1)), seq_w);
  const int threads = TR_LANES_X * TR_LANES_Y;
#define LAUNCH(W, NORM, REC)                                                                  \
  do {                                                                                        \
    constexpr size_t bytes = W == 4 ? ring_bytes(TimeBackwardOp<NORM, REC>::RING_NIN, TR_RING_DEPTH, TR_LANES_X * TR_LANES_Y) : 0; \
    walk_shared_limit<time_reduce_kernel<TimeBackwardOp<NORM, REC>::NS, W, TimeBackwardOp<NORM, REC>>>(bytes);   \
    DLB_LAUNCH_KERNEL(ctx, (time_reduce_kernel<TimeBackwardOp<NORM, REC>::NS, W, TimeBackwardOp<NORM, REC>>), grid, \
                      threads, bytes, (TimeBackwardOp<NORM, REC>{E, Z, A, p}), seq_w, rows, n, sums); \
  } while (0)
#define PICK(W)                                           \
  do {                                                    \
    if (u && recurrent) LAUNCH(W, true, true);            \
    else if (u) LAUNCH(W, true, false);                   \
    else LAUNCH(W, false, true);                          \
  } while (0)
  if (v4) PICK(4); else PICK(1);
#undef LAUNCH
#undef PICK
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_time_fold(dlb_ctx *ctx, const double *sums, int seq_w, int n, float *out) {
  DLB_REQUIRE(ctx && sums && out && seq_w > 0 && n > 0, "dlb_time_fold");
  DLB_LAUNCH_KERNEL(ctx, time_fold_kernel, ceil_div(n, 256), 256, 0, sums, seq_w, n, out);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status brn_time_backward_apply_impl(dlb_ctx *ctx, float *delta, float *delta_lo, const float *Z,
                                       const dlb_brn_unit_arrays *u, const double *sums,
                                       int global_rows, int seq_w, int rows, int n, unsigned *amax,
                                       const PlaneSink *sink = nullptr) {
  DLB_REQUIRE(ctx && delta && Z && u && sums && global_rows > 0 && seq_w > 0 && rows > 0 && n > 0,
              "dlb_brn_time_backward_apply");
  const bool v4 = n % 4 == 0 && aligned16({delta, delta_lo, Z});
  const dim3 grid(ceil_div(n, TR_LANES_X * (v4 ? 4 : 1)), seq_w);
  const float nf = (float)global_rows;
  const PlaneSink none{};
  if (v4 && sink) {
    constexpr size_t bytes = ring_bytes(2, TR_RING_DEPTH, TR_LANES_X * TR_LANES_Y);
    walk_shared_limit<time_apply_kernel<4, true>>(bytes);
    DLB_LAUNCH_KERNEL(ctx, (time_apply_kernel<4, true>), grid, TR_LANES_X * TR_LANES_Y, bytes, delta, delta_lo, Z, time_brn(u), sums, 1.f / nf, nf, seq_w, rows, n, amax, *sink);
  } else if (v4)
    DLB_LAUNCH_KERNEL(ctx, (time_apply_kernel<4, false>), grid, TR_LANES_X * TR_LANES_Y, 0, delta, delta_lo, Z, time_brn(u), sums, 1.f / nf, nf, seq_w, rows, n, amax, none);
  else
    DLB_LAUNCH_KERNEL(ctx, (time_apply_kernel<1, false>), grid, TR_LANES_X * TR_LANES_Y, 0, delta, delta_lo, Z, time_brn(u), sums, 1.f / nf, nf, seq_w, rows, n, amax, none);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_indrnn_clamp(dlb_ctx *ctx, float *recurrent, int n, float lo, float hi) {
  DLB_REQUIRE(ctx && recurrent && n > 0 && lo <= hi, "dlb_indrnn_clamp");
  DLB_LAUNCH_KERNEL(ctx, clamp_kernel, ceil_div(n, 256), 256, 0, recurrent, n, lo, hi);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // extern "C"

// Producers of GEMM operands: under the fp16 operand form the producing kernel
// leaves max |x| in the plane buffer's scale slot and the split follows.
namespace {
struct TimePlanes {
  float *kernel_arg = nullptr;
  PlaneJob job;
  unsigned *amax = nullptr;
  // The tensor is [seq_w * rows, n]: its range statistics are per row of that
  // matrix and per unit.
  // can_write: the producing kernel can write the planes itself (it then gets
  // sink()); otherwise it leaves the maximum and the split pass follows.
  dlb_status begin(dlb_ctx *ctx, const float *x, float *planes, size_t rows, int n, bool can_write = false) {
    if (!ctx || !planes) return DLB_OK;
    if (ctx->gemm_kind != DLB_GEMM_F16X3) {
      kernel_arg = planes;
      return DLB_OK;
    }
    if (rows == 0 || n <= 0 || rows > 0x7fffffffu) return DLB_OK;
    DLB_TRY(planes_open(ctx, x, planes, rows * (size_t)n, (int)rows, n, can_write, &job));
    amax = reinterpret_cast<unsigned *>(job.sink.slot) + 2;
    return DLB_OK;
  }
  const PlaneSink *sink() const { return job.active && job.fused ? &job.sink : nullptr; }
  dlb_status finish(dlb_ctx *ctx) const { return planes_close(ctx, job); }
};
}  // namespace

extern "C" {

dlb_status dlb_time_major(dlb_ctx *ctx, const float *x, float *out, float *out_lo, int rows, int seq_w,
                          int n) {
  const size_t total = (size_t)(seq_w > 0 ? seq_w : 0) * (rows > 0 ? rows : 0) * (n > 0 ? n : 0);
  TimePlanes p;
  DLB_TRY(p.begin(ctx, out, out_lo, total / (size_t)(n > 0 ? n : 1), n));
  DLB_TRY(time_major_impl(ctx, x, out, p.kernel_arg, rows, seq_w, n, p.amax));
  return p.finish(ctx);
}

dlb_status dlb_indrnn_forward(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                              const float *recurrent, int af, float *A, float *A_lo, int seq_w, int rows,
                              int n) {
  const size_t total = (size_t)(seq_w > 0 ? seq_w : 0) * (rows > 0 ? rows : 0) * (n > 0 ? n : 0);
  TimePlanes p;
  DLB_TRY(p.begin(ctx, A, A_lo, total / (size_t)(n > 0 ? n : 1), n, walk_writes_planes(Z, A, u, n)));
  DLB_TRY(indrnn_forward_impl(ctx, Z, u, recurrent, af, nullptr, 1.f, nullptr, A, p.kernel_arg, seq_w, rows, n, p.amax, p.sink()));
  return p.finish(ctx);
}

dlb_status dlb_indrnn_forward_dropout(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                                      const float *recurrent, int af, const uint8_t *mask, float keep_scale,
                                      float *A, float *A_lo, int seq_w, int rows, int n) {
  const size_t total = (size_t)(seq_w > 0 ? seq_w : 0) * (rows > 0 ? rows : 0) * (n > 0 ? n : 0);
  TimePlanes p;
  DLB_TRY(p.begin(ctx, A, A_lo, total / (size_t)(n > 0 ? n : 1), n, walk_writes_planes(Z, A, u, n)));
  DLB_TRY(indrnn_forward_impl(ctx, Z, u, recurrent, af, mask, keep_scale, nullptr, A, p.kernel_arg, seq_w, rows, n, p.amax, p.sink()));
  return p.finish(ctx);
}

dlb_status dlb_indrnn_forward_uout(dlb_ctx *ctx, const float *Z, const dlb_brn_unit_arrays *u,
                                   const float *recurrent, int af, const float *noise, float *A, float *A_lo,
                                   int seq_w, int rows, int n) {
  DLB_REQUIRE(noise, "dlb_indrnn_forward_uout: UOut needs its draws");
  const size_t total = (size_t)(seq_w > 0 ? seq_w : 0) * (rows > 0 ? rows : 0) * (n > 0 ? n : 0);
  TimePlanes p;
  DLB_TRY(p.begin(ctx, A, A_lo, total / (size_t)(n > 0 ? n : 1), n, walk_writes_planes(Z, A, u, n)));
  DLB_TRY(indrnn_forward_impl(ctx, Z, u, recurrent, af, nullptr, 1.f, noise, A, p.kernel_arg, seq_w, rows, n, p.amax, p.sink()));
  return p.finish(ctx);
}

dlb_status dlb_brn_time_backward_apply(dlb_ctx *ctx, float *delta, float *delta_lo, const float *Z,
                                       const dlb_brn_unit_arrays *u, const double *sums, int global_rows,
                                       int seq_w, int rows, int n) {
  const size_t total = (size_t)(seq_w > 0 ? seq_w : 0) * (rows > 0 ? rows : 0) * (n > 0 ? n : 0);
  TimePlanes p;
  DLB_TRY(p.begin(ctx, delta, delta_lo, total / (size_t)(n > 0 ? n : 1), n, n % 4 == 0 && aligned16({delta, Z})));
  DLB_TRY(brn_time_backward_apply_impl(ctx, delta, p.kernel_arg, Z, u, sums, global_rows, seq_w, rows, n,
                                       p.amax, p.sink()));
  return p.finish(ctx);
}

}  // extern "C"
