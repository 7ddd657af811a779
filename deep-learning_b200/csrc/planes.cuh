// Device side of the fp16 operand planes: the scale slot, the split of a value
// into its two halves, and the statistics a producing kernel leaves for the
// range guard.
//
// Scale slot of a plane buffer (SLOT_WORDS 4-byte words):
//   [SLOT_S]     s, the power of two the planes in the buffer were scaled by
//   [SLOT_INV]   1 / s
//   [SLOT_AMAX]  raw bits of max |x| of the split in progress; zero between splits
//   [SLOT_FLAGS] non-zero: the planes cannot stand for the tensor (see below)
//   [SLOT_NEXT]  the scale predicted for the next split of this buffer
//
// A split with the tensor's own maximum known (two passes over the tensor) puts
// s max|x| in [2^14, 2^15).  A producing kernel that writes the planes itself
// cannot know its maximum beforehand and uses the scale predicted from the
// buffer's previous split, which aims at [2^12, 2^13): the tensor may grow
// eightfold from one step to the next before a value leaves the fp16 range.
//
// Range guard.  hi = fp16(s x), lo = fp16(s x - hi) carry 22 bits of x while
// s |x| >= 2^-3; below that lo falls into the fp16 subnormals and a bit is lost
// per factor of two.  That is harmless for small elements among large ones (the
// error is 2^-39 of the tensor's maximum), but not when every element of a row
// or a column is small: the outputs that row or column feeds are then wrong by
// more than fp32 rounding relative to their own size.  Producers therefore
// leave max |x| per row and per column, and the check that follows the split
// (sink_finalize) flags the tensor when a non-zero row or column maximum is
// below PLANE_TINY / s (18 bits left) or when the tensor's maximum overflowed
// the predicted scale; rows and columns have flags of their own.  A small line
// only hurts where it is a line of the product's output: the lines of an
// operand along its free dimension (a row of a k-contiguous operand, a column
// of an mn-contiguous one).  Along the contraction its terms are added to the
// terms of the large lines, and their error is 2^-39 of those.  The
// tensor-core kernels therefore look at the overflow flag and at the flag of
// the operand's free dimension, and compute a product with an operand flagged
// there on the CUDA cores from the fp32 tensors instead.
// rows_exempt (PlaneSink): the rows of the tensor are examples of a batch and
// the tensor is an error of the backward pass.  Such a row reaches the
// parameters only through sums over the examples; when it is 2^-19 of the
// largest row it is lost in those sums in fp32 as well, so its own relative
// error is not guarded (its absolute error stays 2^-39 of the tensor's
// maximum).  After a few steps on a classifier most rows of the errors are
// that small: the examples the model already gets right.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"
#include "math.cuh"

namespace dlb {

constexpr int SLOT_S = 0, SLOT_INV = 1, SLOT_AMAX = 2, SLOT_FLAGS = 3, SLOT_NEXT = 4;
constexpr int PLANE_EXP_OWN = 14;        // s max in [2^14, 2^15): the scale from the tensor's own maximum
constexpr int PLANE_EXP_PREDICTED = 12;  // s max in [2^12, 2^13): the scale predicted for the next split
constexpr float PLANE_TINY = 0.0078125f; // 2^-7: a line whose largest s |x| is below this has under 18 bits
constexpr float PLANE_HALF_MAX = 65504.f;
// Bits of a slot's flag word (SLOT_FLAGS): the planes overflowed or hold NaN /
// infinity; some row; some column of the tensor is too small for the scale.
constexpr unsigned GUARD_WHOLE = 1u, GUARD_ROWS = 2u, GUARD_COLS = 4u;

// s = 2^(target - E) for max = 1.f * 2^E; 1 for a zero, infinite or NaN maximum.
__host__ __device__ __forceinline__ float plane_scale_from_bits(unsigned bits, int target) {
  const int be = (int)(bits >> 23);  // biased exponent of the maximum
  if (bits == 0 || be == 255) return 1.f;
  int se = target - (be - 127) + 127;  // biased exponent of s
  se = se < 1 ? 1 : (se > 254 ? 254 : se);
  const unsigned u = (unsigned)se << 23;
#ifdef __CUDA_ARCH__
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, sizeof(f));
  return f;
#endif
}

// The scale a kernel writing through `k` uses for this split.
__device__ __forceinline__ float sink_scale(const PlaneSink &k) {
  if (!k.hi) return 1.f;
  return k.predicted ? k.slot[SLOT_NEXT]
                     : plane_scale_from_bits(reinterpret_cast<const unsigned *>(k.slot)[SLOT_AMAX], PLANE_EXP_OWN);
}

__device__ __forceinline__ void plane_halves(float v, float s, __half *h, __half *l) {
  const float t = v * s;
  const __half a = __float2half_rn(t);
  *h = a;
  *l = __float2half_rn(t - __half2float(a));
}

// Four consecutive elements starting at element `off` (a multiple of 4): one
// 8-byte store into each plane.
__device__ __forceinline__ void sink_store4(const PlaneSink &k, size_t off, const float (&v)[4], float s) {
  // Two values per conversion instruction: the same roundings as plane_halves.
  const float t0 = v[0] * s, t1 = v[1] * s, t2 = v[2] * s, t3 = v[3] * s;
  const __half2 h01 = __floats2half2_rn(t0, t1), h23 = __floats2half2_rn(t2, t3);
  const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
  const __half2 l01 = __floats2half2_rn(t0 - f01.x, t1 - f01.y), l23 = __floats2half2_rn(t2 - f23.x, t3 - f23.y);
  uint2 hi, lo;
  hi.x = *reinterpret_cast<const unsigned *>(&h01);
  hi.y = *reinterpret_cast<const unsigned *>(&h23);
  lo.x = *reinterpret_cast<const unsigned *>(&l01);
  lo.y = *reinterpret_cast<const unsigned *>(&l23);
  *reinterpret_cast<uint2 *>(k.hi + off) = hi;
  *reinterpret_cast<uint2 *>(k.lo + off) = lo;
}

// Statistics of a thread that owns four columns and visits whole rows together
// with the other lanes of its warp (every lane of the warp is on the same row
// in the same call): the row's maximum goes out with one atomic per warp and
// row, the column maxima stay in registers until `finish`.
struct LineTracker {
  unsigned cm[4] = {0u, 0u, 0u, 0u};
  unsigned all = 0u;
  __device__ __forceinline__ void row(const PlaneSink &k, int r, const float (&v)[4]) {
    unsigned m = 0u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned b = abs_bits(v[j]);
      cm[j] = max(cm[j], b);
      m = max(m, b);
    }
    all = max(all, m);
    if (k.rowmax) {
      const unsigned mask = __activemask();
      const unsigned w = __reduce_max_sync(mask, m);
      if ((threadIdx.x & 31u) == (unsigned)(__ffs(mask) - 1) && w) atomicMax(k.rowmax + r, w);
    }
  }
  // Called by every thread of the block (threads past the last column with
  // live = false).  The block is lanes_x x lanes_y threads over lanes_x * 4
  // columns; `shared` holds lanes_y * lanes_x * 4 words; tx in [0, lanes_x), ty in
  // [0, lanes_y), col0 the block's first column, n the number of columns.
  __device__ __forceinline__ void finish(const PlaneSink &k, unsigned *shared, int tx, int ty, int lanes_y,
                                         int col0, int n, bool live, int lanes_x = 32) {
    if (k.slot) amax_commit(reinterpret_cast<unsigned *>(k.slot) + SLOT_AMAX, live ? all : 0u);
    if (!k.colmax) return;
    const int cols = lanes_x * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) shared[ty * cols + tx * 4 + j] = live ? cm[j] : 0u;
    __syncthreads();
    for (int t = ty * lanes_x + tx; t < cols; t += lanes_x * lanes_y) {
      if (col0 + t < n) {
        unsigned m = 0u;
        for (int y = 0; y < lanes_y; ++y) m = max(m, shared[y * cols + t]);
        if (m) atomicMax(k.colmax + col0 + t, m);
      }
    }
  }
};

// After a split (planes_finalize_kernel, one block): turns the statistics into
// what the consumers read: the scale and its inverse, the guard flag, the scale
// predicted for the next split; and clears what the next split accumulates into
// (maximum, line maxima).  A launch of its own: letting the last block of the
// writing kernel do it (a fence and a ticket per block) was measured at 13 us per
// 64 MiB tensor, the launch at 6.
__device__ __forceinline__ void sink_finalize(const PlaneSink &k) {
  unsigned *uslot = reinterpret_cast<unsigned *>(k.slot);
  const unsigned amax = __ldcg(uslot + SLOT_AMAX);
  float s = k.predicted ? __ldcg(k.slot + SLOT_NEXT) : plane_scale_from_bits(amax, PLANE_EXP_OWN);
  const bool finite = amax != 0u && (amax >> 23) != 255u;
  // NaN or infinity in the tensor, or growth past the predicted scale.
  bool overflow = !(__uint_as_float(amax) * s < PLANE_HALF_MAX);
  bool resplit = false;
  if (overflow && finite && k.predicted && k.hi && k.x) {
    // The tensor outgrew the scale predicted for it (more than eightfold since
    // its last split): this block writes the planes again with the scale of the
    // tensor's own maximum.  A few milliseconds for a 256 MB tensor, against
    // its products on the CUDA cores.
    s = plane_scale_from_bits(amax, PLANE_EXP_OWN);
    for (size_t o = (size_t)threadIdx.x * 4; o + 3 < k.n; o += (size_t)blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4 *>(k.x + o);
      const float a[4] = {v.x, v.y, v.z, v.w};
      sink_store4(k, o, a, s);
    }
    overflow = false;
    resplit = true;
  }
  // Lines [0, rows) are the rows, the rest the columns.
  int tiny_rows = 0, tiny_cols = 0;
  // Exempt rows were not recorded (rowmax was null for the producer): their
  // words are zero and stay so.
  unsigned *lines = k.lines;
  const int n_rows = k.n_rows;
  for (int i = (k.rows_exempt ? n_rows : 0) + threadIdx.x; i < (lines ? k.n_lines : 0); i += blockDim.x) {
    const unsigned v = __ldcg(lines + i);
    if (v) {
      if (__uint_as_float(v) * s < PLANE_TINY) {
        if (i < n_rows) tiny_rows = 1;
        else tiny_cols = 1;
      }
      lines[i] = 0u;
    }
  }
  tiny_rows = __syncthreads_or(tiny_rows);
  tiny_cols = __syncthreads_or(tiny_cols);
  if (threadIdx.x == 0) {
    const unsigned unsafe = (overflow ? GUARD_WHOLE : 0u) | (tiny_rows ? GUARD_ROWS : 0u) | (tiny_cols ? GUARD_COLS : 0u);
    k.slot[SLOT_S] = s;
    k.slot[SLOT_INV] = 1.f / s;
    uslot[SLOT_FLAGS] = unsafe;
    // The next split is predicted from this one's maximum; an empty or
    // non-finite tensor leaves the prediction where it was.
    k.slot[SLOT_NEXT] = finite ? plane_scale_from_bits(amax, PLANE_EXP_PREDICTED) : s;
    uslot[SLOT_AMAX] = 0u;
    if (unsafe && k.guard) atomicAdd(k.guard, 1ull);
    if (resplit && k.guard) atomicAdd(k.guard + 2, 1ull);
  }
}

}  // namespace dlb
