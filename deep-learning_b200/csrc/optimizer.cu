// Adam-family and gradient-descent updates over flat parameter / gradient /
// moment vectors: one
// streaming pass with 128-bit loads and stores, the rule chosen at compile time
// so the inner loop carries no branch on it.  Algorithmic traffic per element:
// read p, g, m, v and write p, m, v, g<-0 = 32 bytes (Adam, AdaBound, NosAdam,
// AdaMax); +8 for the running maximum (AMSGrad, AMSBound); +4 for the
// regularisation mask when weight decay is on.  Gradient descent reads p, g and
// writes p, g<-0 (16 bytes), +8 for the previous delta with momentum.
#include <math.h>

#include <type_traits>

#include "common.cuh"
#include "math.cuh"
#include "planes.cuh"

namespace dlb {

enum Rule { R_ADAM, R_AMSGRAD, R_ADABOUND, R_AMSBOUND, R_ADAMAX, R_GD, R_GD_MOMENTUM, R_GD_NESTEROV };

struct OptState {
  float p, g, m, v, vh;
};

// One element.  The arithmetic follows the reference loops term by term
// (v1/optimizers/adam.cpp L:146-160, amsgrad.cpp, adabound.cpp, amsbound.cpp
// L:100-120, nosadam.cpp L:86-99); NosAdam is Adam with beta2 replaced by the
// time-dependent value, which the host passes in `beta2`.
template <int RULE, bool WD>
__device__ __forceinline__ void update_one(OptState &s, float mask, const dlb_optimizer_scalars &k) {
  const float g = s.g;
  if (RULE == R_GD || RULE == R_GD_MOMENTUM || RULE == R_GD_NESTEROV) {
    // v1/optimizers/gradient_descent.cpp L:57-130, gradient_descent_momentum.cpp
    // L:66-107, nesterov_accelerated_gradient.cpp L:66-109: lr_t is the learning
    // rate, beta1 the momentum, m the previous delta.
    float step = k.lr_t * g;
    if (RULE != R_GD) {
      s.m = step + k.beta1 * s.m;
      step = RULE == R_GD_NESTEROV ? k.beta1 * s.m - step : s.m;
    }
    if (WD) step += mask * k.weight_decay * s.p;
    s.p -= step;
    s.g = 0.f;
    return;
  }
  s.m = k.beta1 * s.m + (1.f - k.beta1) * g;
  if (RULE == R_ADAMAX) {
    s.v = fmaxf(k.beta2 * s.v, fabsf(g));
  } else {
    s.v = k.beta2 * s.v + (1.f - k.beta2) * g * g;
  }
  float step;
  if (RULE == R_ADAM) {
    step = k.lr_t * s.m / (sqrtf(s.v) + k.epsilon);
  } else if (RULE == R_AMSGRAD) {
    s.vh = fmaxf(s.vh, s.v);
    step = k.lr_t * s.m / (sqrtf(s.vh) + k.epsilon);
  } else if (RULE == R_ADABOUND) {
    step = clipf(k.lr_t / (sqrtf(s.v) + k.epsilon), k.lower_bound, k.upper_bound) * s.m;
  } else if (RULE == R_AMSBOUND) {
    s.vh = fmaxf(s.vh, s.v);
    step = clipf(k.lr_t / (sqrtf(s.vh) + k.epsilon), k.lower_bound, k.upper_bound) * s.m;
  } else {  // AdaMax: lr_t = lr / (1 - beta1^t)
    step = k.lr_t * s.m / (s.v + k.epsilon);
  }
  if (WD) step += mask * k.weight_decay * s.p;
  s.p -= step;
  s.g = 0.f;
}

template <int RULE, bool WD>
__global__ void __launch_bounds__(256)
    optimizer_kernel(dlb_optimizer_scalars k, float *__restrict__ p, float *__restrict__ g,
                     float *__restrict__ m, float *__restrict__ v, float *__restrict__ vh,
                     const float *__restrict__ mask, size_t n, unsigned *amax) {
  pdl_enter();
  unsigned mx = 0;  // largest |p| written, for the fp16 split of a weight matrix
  constexpr bool HAT = (RULE == R_AMSGRAD || RULE == R_AMSBOUND);
  constexpr bool FIRST = RULE != R_GD;                                              // m is read and written
  constexpr bool SECOND = !(RULE == R_GD || RULE == R_GD_MOMENTUM || RULE == R_GD_NESTEROV);  // v likewise
  const size_t n4 = n / 4;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 P = reinterpret_cast<float4 *>(p)[i];
    const float4 G = reinterpret_cast<float4 *>(g)[i];
    float4 H = make_float4(0.f, 0.f, 0.f, 0.f), K = H, M = H, V = H;
    if (FIRST) M = reinterpret_cast<float4 *>(m)[i];
    if (SECOND) V = reinterpret_cast<float4 *>(v)[i];
    if (HAT) H = reinterpret_cast<float4 *>(vh)[i];
    if (WD) K = __ldg(reinterpret_cast<const float4 *>(mask) + i);
    OptState s0{P.x, G.x, M.x, V.x, H.x}, s1{P.y, G.y, M.y, V.y, H.y}, s2{P.z, G.z, M.z, V.z, H.z},
        s3{P.w, G.w, M.w, V.w, H.w};
    update_one<RULE, WD>(s0, K.x, k);
    update_one<RULE, WD>(s1, K.y, k);
    update_one<RULE, WD>(s2, K.z, k);
    update_one<RULE, WD>(s3, K.w, k);
    reinterpret_cast<float4 *>(p)[i] = make_float4(s0.p, s1.p, s2.p, s3.p);
    mx = max(max(mx, abs_bits(s0.p)), max(abs_bits(s1.p), max(abs_bits(s2.p), abs_bits(s3.p))));
    if (FIRST) reinterpret_cast<float4 *>(m)[i] = make_float4(s0.m, s1.m, s2.m, s3.m);
    if (SECOND) reinterpret_cast<float4 *>(v)[i] = make_float4(s0.v, s1.v, s2.v, s3.v);
    if (HAT) reinterpret_cast<float4 *>(vh)[i] = make_float4(s0.vh, s1.vh, s2.vh, s3.vh);
    reinterpret_cast<float4 *>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // Tail (n not a multiple of 4).
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    OptState s{p[i], g[i], FIRST ? m[i] : 0.f, SECOND ? v[i] : 0.f, HAT ? vh[i] : 0.f};
    update_one<RULE, WD>(s, WD ? mask[i] : 0.f, k);
    p[i] = s.p; g[i] = 0.f;
    mx = max(mx, abs_bits(s.p));
    if (FIRST) m[i] = s.m;
    if (SECOND) v[i] = s.v;
    if (HAT) vh[i] = s.vh;
  }
  amax_commit(amax, mx);
}

// The same update over a weight matrix [rows, cols] (cols a multiple of 4) that
// also writes the fp16 planes of the new weights, with the scale predicted from
// the matrix's previous split, and the row / column maxima of the range guard:
// the next forward pass finds the planes ready and no split pass reads the
// matrix again.  Grid (column blocks of 128, row chunks); a thread owns four
// columns and walks its rows eight apart.
constexpr int OPT_LANES_Y = 8;
template <int RULE, bool WD>
__global__ void __launch_bounds__(32 * OPT_LANES_Y)
    optimizer_rows_kernel(dlb_optimizer_scalars k, float *__restrict__ p, float *__restrict__ g,
                          float *__restrict__ m, float *__restrict__ v, float *__restrict__ vh,
                          const float *__restrict__ mask, int rows, int cols, int rows_per_chunk, PlaneSink sink) {
  pdl_enter();
  __shared__ unsigned line_shared[OPT_LANES_Y * 128];
  constexpr bool HAT = (RULE == R_AMSGRAD || RULE == R_AMSBOUND);
  constexpr bool FIRST = RULE != R_GD;
  constexpr bool SECOND = !(RULE == R_GD || RULE == R_GD_MOMENTUM || RULE == R_GD_NESTEROV);
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int col = blockIdx.x * 128 + tx * 4;
  const bool live = col < cols;
  const float plane_scale = sink_scale(sink);
  LineTracker track;
  if (live) {
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    for (int r = r0 + ty; r < r1; r += OPT_LANES_Y) {
      const size_t o = (size_t)r * cols + col;
      float4 P = *reinterpret_cast<const float4 *>(p + o);
      const float4 G = *reinterpret_cast<const float4 *>(g + o);
      float4 H = make_float4(0.f, 0.f, 0.f, 0.f), K = H, M = H, V = H;
      if (FIRST) M = *reinterpret_cast<const float4 *>(m + o);
      if (SECOND) V = *reinterpret_cast<const float4 *>(v + o);
      if (HAT) H = *reinterpret_cast<const float4 *>(vh + o);
      if (WD) K = __ldg(reinterpret_cast<const float4 *>(mask + o));
      OptState s0{P.x, G.x, M.x, V.x, H.x}, s1{P.y, G.y, M.y, V.y, H.y}, s2{P.z, G.z, M.z, V.z, H.z},
          s3{P.w, G.w, M.w, V.w, H.w};
      update_one<RULE, WD>(s0, K.x, k);
      update_one<RULE, WD>(s1, K.y, k);
      update_one<RULE, WD>(s2, K.z, k);
      update_one<RULE, WD>(s3, K.w, k);
      const float out[4] = {s0.p, s1.p, s2.p, s3.p};
      *reinterpret_cast<float4 *>(p + o) = make_float4(s0.p, s1.p, s2.p, s3.p);
      if (FIRST) *reinterpret_cast<float4 *>(m + o) = make_float4(s0.m, s1.m, s2.m, s3.m);
      if (SECOND) *reinterpret_cast<float4 *>(v + o) = make_float4(s0.v, s1.v, s2.v, s3.v);
      if (HAT) *reinterpret_cast<float4 *>(vh + o) = make_float4(s0.vh, s1.vh, s2.vh, s3.vh);
      *reinterpret_cast<float4 *>(g + o) = make_float4(0.f, 0.f, 0.f, 0.f);
      sink_store4(sink, o, out, plane_scale);
      track.row(sink, r, out);
    }
  }
  track.finish(sink, line_shared, tx, ty, OPT_LANES_Y, blockIdx.x * 128, cols, live);
}

// Calls f(std::integral_constant<int, R>) with the kernel rule of an optimizer
// code of the C ABI.
template <class F>
static dlb_status with_rule(int rule, const dlb_optimizer_scalars &s, F f) {
  switch (rule) {
    case DLB_OPT_ADAM:
    case DLB_OPT_NOSADAM: return f(std::integral_constant<int, R_ADAM>{});
    case DLB_OPT_AMSGRAD: return f(std::integral_constant<int, R_AMSGRAD>{});
    case DLB_OPT_ADABOUND: return f(std::integral_constant<int, R_ADABOUND>{});
    case DLB_OPT_AMSBOUND: return f(std::integral_constant<int, R_AMSBOUND>{});
    case DLB_OPT_ADAMAX: return f(std::integral_constant<int, R_ADAMAX>{});
    case DLB_OPT_GD:
      // The three forms of Model::Update_Parameter__Gradient_Descent
      // (v1/optimizers/gradient_descent.cpp L:24-55).
      if (s.beta1 == 0.f) return f(std::integral_constant<int, R_GD>{});
      if (s.beta2 != 0.f) return f(std::integral_constant<int, R_GD_NESTEROV>{});
      return f(std::integral_constant<int, R_GD_MOMENTUM>{});
    default:
      set_error("dlb_optimizer_step: optimizer %d is outside the supported path", rule);
      return DLB_ERR_UNSUPPORTED;
  }
}

template <int RULE>
static dlb_status launch_rule_rows(dlb_ctx *ctx, const dlb_optimizer_scalars &k, float *p, float *g, float *m,
                                   float *v, float *vh, const float *mask, int rows, int cols,
                                   const PlaneSink &sink) {
  const int col_blocks = ceil_div(cols, 128);
  int chunks = max(1, min(ceil_div(ctx->sm_count * 8, col_blocks), ceil_div(rows, OPT_LANES_Y)));
  const int rpc = ceil_div(ceil_div(rows, chunks), OPT_LANES_Y) * OPT_LANES_Y;
  chunks = ceil_div(rows, rpc);
  const dim3 grid(col_blocks, chunks);
  if (k.weight_decay != 0.f)
    DLB_LAUNCH_KERNEL(ctx, (optimizer_rows_kernel<RULE, true>), grid, 32 * OPT_LANES_Y, 0, k, p, g, m, v, vh, mask, rows, cols, rpc, sink);
  else
    DLB_LAUNCH_KERNEL(ctx, (optimizer_rows_kernel<RULE, false>), grid, 32 * OPT_LANES_Y, 0, k, p, g, m, v, vh, mask, rows, cols, rpc, sink);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

template <int RULE>
static dlb_status launch_rule(dlb_ctx *ctx, const dlb_optimizer_scalars &k, float *p, float *g,
                              float *m, float *v, float *vh, const float *mask, size_t n,
                              unsigned *amax) {
  // Enough blocks to keep every SM's memory pipeline full; each thread moves
  // 8-10 float4 per iteration.
  const size_t blocks_needed = (n / 4 + 255) / 256 + 1;
  const int grid = (int)min(blocks_needed, (size_t)ctx->sm_count * 8);
  if (k.weight_decay != 0.f)
    DLB_LAUNCH_KERNEL(ctx, (optimizer_kernel<RULE, true>), grid, 256, 0, k, p, g, m, v, vh, mask, n, amax);
  else
    DLB_LAUNCH_KERNEL(ctx, (optimizer_kernel<RULE, false>), grid, 256, 0, k, p, g, m, v, vh, mask, n, amax);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// ---- gradient clipping by the Euclidean norm -------------------------------
// euclidean_norm_mp (v1/ops/constraints/euclidean.cpp L:48-71): the norm of the
// whole vector, and g *= max / norm when norm >= max.  Three launches: block
// partials of the sum of squares (fp64), one block that folds them in a fixed
// order into the factor, and the scaling pass, which returns at once when the
// factor is 1.

constexpr int CLIP_BLOCKS = 1024;

__global__ void __launch_bounds__(256) sumsq_partials_kernel(const float *__restrict__ g, size_t n, double *partials) {
  pdl_enter();
  double acc = 0.0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t n4 = (reinterpret_cast<uintptr_t>(g) & 15) == 0 ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(g) + i);
    acc += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc += (double)g[i] * g[i];
  __shared__ double warp_sums[8];
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (threadIdx.x % 32 == 0) warp_sums[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < 8; ++w) s += warp_sums[w];
    partials[blockIdx.x] = s;
  }
}

__global__ void __launch_bounds__(256) clip_factor_kernel(const double *partials, int blocks, float max_norm, float *factor) {
  pdl_enter();
  __shared__ double part[256];
  double s = 0.0;
  for (int i = threadIdx.x; i < blocks; i += 256) s += partials[i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o; o >>= 1) {
    if ((int)threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float norm = sqrtf((float)part[0]);
    *factor = norm >= max_norm ? max_norm / norm : 1.f;
  }
}

__global__ void __launch_bounds__(256) scale_by_factor_kernel(float *__restrict__ g, size_t n, const float *factor) {
  pdl_enter();
  const float f = *factor;
  if (f == 1.f) return;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t n4 = (reinterpret_cast<uintptr_t>(g) & 15) == 0 ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 v = reinterpret_cast<float4 *>(g)[i];
    v.x *= f, v.y *= f, v.z *= f, v.w *= f;
    reinterpret_cast<float4 *>(g)[i] = v;
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) g[i] *= f;
}

}  // namespace dlb

using namespace dlb;

extern "C" {

dlb_status dlb_optimizer_step(dlb_ctx *ctx, int rule, const dlb_optimizer_scalars *s, float *p,
                              float *g, float *first, float *second, float *second_hat,
                              const float *wd_mask, size_t n) {
  return optimizer_step_amax(ctx, rule, s, p, g, first, second, second_hat, wd_mask, n, nullptr);
}

}  // extern "C"

// The same pass that also leaves the largest |p| it wrote (raw bits) in *amax,
// so that the fp16 split of a weight matrix needs no pass of its own for it.
dlb_status dlb::optimizer_step_amax(dlb_ctx *ctx, int rule, const dlb_optimizer_scalars *s, float *p, float *g,
                                    float *first, float *second, float *second_hat, const float *wd_mask,
                                    size_t n, unsigned *amax) {
  DLB_REQUIRE(ctx && s && p && g, "dlb_optimizer_step: null");
  if (n == 0) return DLB_OK;
  const bool hat = rule == DLB_OPT_AMSGRAD || rule == DLB_OPT_AMSBOUND;
  const bool descent = rule == DLB_OPT_GD;
  DLB_REQUIRE(first || (descent && s->beta1 == 0.f), "dlb_optimizer_step: first required");
  DLB_REQUIRE(second || descent, "dlb_optimizer_step: second required");
  DLB_REQUIRE(!hat || second_hat, "dlb_optimizer_step: second_hat required");
  DLB_REQUIRE(s->weight_decay == 0.f || wd_mask, "dlb_optimizer_step: weight decay needs a mask");
  const uintptr_t al = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       (descent && s->beta1 == 0.f ? 0 : reinterpret_cast<uintptr_t>(first)) |
                       (descent ? 0 : reinterpret_cast<uintptr_t>(second)) |
                       (hat ? reinterpret_cast<uintptr_t>(second_hat) : 0) |
                       (s->weight_decay != 0.f ? reinterpret_cast<uintptr_t>(wd_mask) : 0);
  DLB_REQUIRE((al & 15) == 0, "dlb_optimizer_step: arrays must be 16-byte aligned");
  return with_rule(rule, *s, [&](auto R) {
    return launch_rule<decltype(R)::value>(ctx, *s, p, g, first, second, second_hat, wd_mask, n, amax);
  });
}

// The pass over one weight matrix [rows, cols] that also writes the matrix's
// fp16 planes and range statistics through `sink` (optimizer_rows_kernel).
dlb_status dlb::optimizer_step_sink(dlb_ctx *ctx, int rule, const dlb_optimizer_scalars *s, float *p, float *g,
                                    float *first, float *second, float *second_hat, const float *wd_mask,
                                    int rows, int cols, const PlaneSink &sink) {
  DLB_REQUIRE(ctx && s && p && g && rows > 0 && cols > 0 && (cols & 3) == 0 && sink.hi && sink.slot,
              "optimizer_step_sink");
  return with_rule(rule, *s, [&](auto R) {
    return launch_rule_rows<decltype(R)::value>(ctx, *s, p, g, first, second, second_hat, wd_mask, rows, cols, sink);
  });
}

extern "C" {

dlb_status dlb_clip_gradient(dlb_ctx *ctx, float *g, size_t n, float max_norm) {
  DLB_REQUIRE(ctx && g && max_norm > 0.f, "dlb_clip_gradient");
  if (n == 0) return DLB_OK;
  void *scr = nullptr;
  DLB_TRY(scratch(ctx, (CLIP_BLOCKS + 1) * sizeof(double), &scr));
  double *partials = static_cast<double *>(scr);
  float *factor = reinterpret_cast<float *>(partials + CLIP_BLOCKS);
  const int blocks = (int)min((size_t)CLIP_BLOCKS, (n / 4 + 255) / 256 + 1);
  DLB_LAUNCH_KERNEL(ctx, sumsq_partials_kernel, blocks, 256, 0, g, n, partials);
  DLB_LAUNCHED(ctx);
  DLB_LAUNCH_KERNEL(ctx, clip_factor_kernel, 1, 256, 0, partials, blocks, max_norm, factor);
  DLB_LAUNCHED(ctx);
  DLB_LAUNCH_KERNEL(ctx, scale_by_factor_kernel, blocks, 256, 0, g, n, factor);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_optimizer_prepare(int rule, const float *hyper, float *time_step,
                                 float *nos_previous, dlb_optimizer_scalars *out) {
  DLB_REQUIRE(hyper && time_step && out, "dlb_optimizer_prepare: null");
  const float lr = hyper[0], beta1 = hyper[1], beta2 = hyper[2], eps = hyper[3], gamma = hyper[4],
              final_lr = hyper[5], bound_gamma = hyper[6];
  const bool bias_correction = hyper[7] != 0.f;
  *time_step += 1.f;  // the reference keeps the step count in a float
  const float t = *time_step;
  if (rule == DLB_OPT_GD) {
    // hyper = {learning_rate, learning_momentum, use_nesterov(0/1)}.
    dlb_optimizer_scalars d{};
    d.lr_t = hyper[0];
    d.beta1 = hyper[1];
    d.beta2 = hyper[2] != 0.f ? 1.f : 0.f;
    *out = d;
    return DLB_OK;
  }
  dlb_optimizer_scalars k{};
  k.beta1 = beta1;
  k.beta2 = beta2;
  k.epsilon = eps;
  k.weight_decay = 0.f;
  k.lower_bound = 0.f;
  k.upper_bound = 0.f;
  // lr * sqrt(1 - beta2^t) / (1 - beta1^t), float pow as in adam.cpp L:113-118.
  k.lr_t = bias_correction ? lr * sqrtf(1.f - powf(beta2, t)) / (1.f - powf(beta1, t)) : lr;
  switch (rule) {
    case DLB_OPT_ADAM:
    case DLB_OPT_AMSGRAD:
      break;
    case DLB_OPT_ADABOUND:
    case DLB_OPT_AMSBOUND:
      // adabound.cpp L:52-60 / amsbound.cpp L:52-60
      k.lower_bound = final_lr * (1.f - 1.f / (bound_gamma * t + 1.f));
      k.upper_bound = final_lr * (1.f + 1.f / (bound_gamma * t));
      break;
    case DLB_OPT_NOSADAM: {
      DLB_REQUIRE(nos_previous, "dlb_optimizer_prepare: NosAdam needs its running sum");
      // nosadam.cpp L:50-53, L:70
      const float b = powf(t, -gamma);
      k.beta2 = *nos_previous / (*nos_previous + b);
      *nos_previous += b;
      break;
    }
    case DLB_OPT_ADAMAX:
      k.lr_t = lr / (1.f - powf(beta1, t));
      break;
    default:
      set_error("dlb_optimizer_prepare: optimizer %d is outside the supported path", rule);
      return DLB_ERR_UNSUPPORTED;
  }
  *out = k;
  return DLB_OK;
}

}  // extern "C"
