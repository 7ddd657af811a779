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

// f(x).  ref: AF_FIRE, v1/ops/activations/functions.hpp L:86-108, L:124-219.
__device__ __forceinline__ float af_fire(int af, float x) {
  switch (af) {
    case DLB_AF_RELU: return x < 0.f ? 0.f : x;
    case DLB_AF_LEAKY_RELU: return x < 0.f ? DLB_LRELU_ALPHA * x : x;
    case DLB_AF_ELU: return x < 0.f ? 1.f * (expf(x) - 1.f) : x;
    case DLB_AF_SELU:
      return DLB_SELU_SCALE * (x <= 0.f ? DLB_SELU_ALPHA * expf(x) - DLB_SELU_ALPHA : x);
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
