// Device side of FusedEpilogue: what the store of a product does with one
// element besides writing it.
#pragma once

#include "common.cuh"
#include "math.cuh"
#include "planes.cuh"

namespace dlb {

// Factor of unit `col` under the epilogue's dropout: 0 for a dropped unit.
__device__ __forceinline__ float epilogue_keep(const FusedEpilogue &e, int col) {
  if (e.mode != EPI_ACTIVATION) return 1.f;
  return e.mask ? (e.mask[col] ? e.keep_scale : 0.f) : e.keep_scale;
}

// Stores element (row, col) of the product, `val` = sum + bias, and returns the
// value of the produced operand there (the activation, or the error).
__device__ __forceinline__ float epilogue_store(const FusedEpilogue &e, float *dst, size_t at, float val, float keep) {
  if (e.mode == EPI_ACTIVATION) {
    *dst = val;
    float a = af_fire(e.af, val);
    if (e.noise) a = a + a * e.noise[at];       // UOut (fwp_mp.cpp L:4959-4985)
    a = keep == 0.f ? 0.f : a * keep;            // a dropped unit is 0 whatever f came to
    e.out[at] = a;
    return a;
  }
  const float x = val * af_derive(e.af, e.z[at], e.a[at]);
  *dst = x;
  return x;
}

// The two fp16 planes of element `at`.
__device__ __forceinline__ void epilogue_planes(const FusedEpilogue &e, size_t at, float x, float scale) {
  __half h, l;
  plane_halves(x, scale, &h, &l);
  e.sink.hi[at] = *reinterpret_cast<const uint16_t *>(&h);
  e.sink.lo[at] = *reinterpret_cast<const uint16_t *>(&l);
}

// One element at a time, statistics by atomics: the form of the CUDA-core path.
__device__ __forceinline__ void epilogue_element(const FusedEpilogue &e, float *dst, int row, int col, int N, float val,
                                                 float scale) {
  const size_t at = (size_t)row * N + col;
  const float x = epilogue_store(e, dst, at, val, epilogue_keep(e, col));
  if (e.sink.hi) epilogue_planes(e, at, x, scale);
  const unsigned b = abs_bits(x);
  if (b) {
    if (e.sink.rowmax) atomicMax(e.sink.rowmax + row, b);
    if (e.sink.colmax) atomicMax(e.sink.colmax + col, b);
    if (e.sink.slot) atomicMax(reinterpret_cast<unsigned *>(e.sink.slot) + SLOT_AMAX, b);
  }
}

}  // namespace dlb
