// Scalar device functions of the fully-connected step: activations, their
// derivatives in the reference's own (not textbook) form, and the TF32 split.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "dlb200.h"

namespace dlb {

// Constants of v1/ops/activations/functions.hpp L:95-99.
#define DLB_SELU_ALPHA 1.6732632423543772848170429916717f
#define DLB_SELU_SCALE 1.0507009873554804934193349852946f
#define DLB_LRELU_ALPHA 0.01f

// e^x for x <= 0, the only range ELU and SELU ask for (anything else, NaN
// included, is discarded by the caller's select).  2^(x log2(e)) with the
// rounding error of the product x * log2(e) carried along and applied as a
// first-order correction, so the result is as good as ex2.approx itself (2^-22
// relative, the class of expf) at a third of expf's instructions: these
// kernels are bound by instruction issue.  Arguments below -88 count as -88
// (the result flushes to 0, as e^x does in fp32 there).
__device__ __forceinline__ float exp_nonpositive(float x) {
  const float L_HI = 1.4426950216293335f, L_LO = 1.925963033500011e-8f, LN2 = 0.69314718055994531f;
  x = fmaxf(x, -88.f);
  const float t = x * L_HI;
  float e = __fmaf_rn(x, L_HI, -t);
  e = __fmaf_rn(x, L_LO, e);
  // volatile: the compiler then evaluates this for every element and selects,
  // instead of branching around it per element (a divergent branch and its
  // reconvergence cost more than the seven instructions they skip).
  float p;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(t));
  return __fmaf_rn(p * LN2, e, p);
}

// f(x).  ref: AF_FIRE, v1/ops/activations/functions.hpp L:86-108, L:124-219.
__device__ __forceinline__ float af_fire(int af, float x) {
  switch (af) {
    case DLB_AF_RELU: return x < 0.f ? 0.f : x;
    case DLB_AF_LEAKY_RELU: return x < 0.f ? DLB_LRELU_ALPHA * x : x;
    case DLB_AF_ELU: {
      const float neg = 1.f * (exp_nonpositive(x) - 1.f);
      return x < 0.f ? neg : x;
    }
    case DLB_AF_SELU: {
      const float neg = DLB_SELU_ALPHA * exp_nonpositive(x) - DLB_SELU_ALPHA;
      return DLB_SELU_SCALE * (x <= 0.f ? neg : x);
    }
    case DLB_AF_ISRLU: return x < 0.f ? x * (1.f / sqrtf(1.f + 1.f * x * x)) : x;
    default: return x;  // LINEAR
  }
}

// f'(x, q) with q the stored (post-dropout) activation.  The ELU and SELU
// forms are the reference's: ELU'(x<0) = q, SELU'(x<=0) = scale*(q+alpha).
// ref: Model::activation_fn_derivative, v1/learner/model.cpp L:2594-2650.
__device__ __forceinline__ float af_derive(int af, float x, float q) {
  switch (af) {
    case DLB_AF_RELU: return x < 0.f ? 0.f : 1.f;
    case DLB_AF_LEAKY_RELU: return x < 0.f ? DLB_LRELU_ALPHA : 1.f;
    case DLB_AF_ELU: return x < 0.f ? 1.f * q : 1.f;
    case DLB_AF_SELU: return DLB_SELU_SCALE * (x <= 0.f ? (q + DLB_SELU_ALPHA) : 1.f);
    case DLB_AF_ISRLU: {
      if (x < 0.f) {
        float t = q / x;
        return t * t * t;
      }
      return 1.f;
    }
    default: return 1.f;  // LINEAR
  }
}

// What a TF32 tensor-core operand keeps of an fp32 word: sign, exponent and
// the top 10 mantissa bits.
__device__ __forceinline__ float tf32_hi(float a) {
  return __uint_as_float(__float_as_uint(a) & 0xFFFFE000u);
}

// Remainder a - hi(a) (exact in fp32), rounded to nearest TF32 so that the
// tensor core's own truncation of it loses nothing more.
__device__ __forceinline__ float tf32_lo(float a) {
  float r = a - tf32_hi(a);
  if (!(fabsf(a) <= 3.402823466e+38f)) r = 0.f;  // inf/nan: no residual
  uint32_t o;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(o) : "f"(r));
  return __uint_as_float(o);
}

// Largest |x| seen by a kernel, as raw bits (monotonic for non-negative
// floats): each thread keeps a running maximum and the lanes still active at
// the end fold theirs into the slot.  Kernels that produce a GEMM operand use
// this so that the fp16 split that follows needs no pass of its own for the
// tensor's maximum.
__device__ __forceinline__ unsigned abs_bits(float v) { return __float_as_uint(v) & 0x7fffffffu; }
__device__ __forceinline__ void amax_commit(unsigned *slot, unsigned m) {
  if (!slot) return;
  const unsigned mask = __activemask();
  m = __reduce_max_sync(mask, m);
  // Most warps find a larger value already there: read before the atomic so
  // that thousands of warps do not queue on one address.
  if ((threadIdx.x & 31u) == (unsigned)(__ffs(mask) - 1) && m > *reinterpret_cast<volatile unsigned *>(slot))
    atomicMax(slot, m);
}

__device__ __forceinline__ float clipf(float v, float lo, float hi) {
  return v < lo ? lo : (v > hi ? hi : v);
}

}  // namespace dlb
