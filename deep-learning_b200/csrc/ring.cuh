// Thread-private rings of asynchronous 16-byte copies (cp.async) for the
// row-walking HBM-bound kernels.
//
// Those kernels are bound by bytes in flight: with plain loads a thread holds a
// register quadruple per outstanding 16-byte request, and at 64 registers and
// four blocks of 256 threads an SM has 64 KB under way where the memory system
// needs well over 100 KB to stay busy.  Here a thread sends the rows it is
// going to visit into slots of shared memory that only it reads: DEPTH slots of
// NIN float4 per thread, DEPTH - 1 rows under way while one is worked on.  No
// thread reads another's slot, so there is no barrier in the loop, only the
// copy-group wait of the issuing thread.
#pragma once

#include "common.cuh"

namespace dlb {

__device__ __forceinline__ void cp_async16(void *shared_dst, const void *global_src) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(shared_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(global_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// Bytes of shared memory a block of `threads` threads needs for the ring.
constexpr size_t ring_bytes(int nin, int depth, int threads) { return (size_t)nin * depth * threads * sizeof(float4); }

__device__ __forceinline__ void cp_async16_to(unsigned shared_addr, const void *global_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(shared_addr), "l"(global_src) : "memory");
}
__device__ __forceinline__ float4 ring_read(unsigned shared_addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(shared_addr)
               : "memory");
  return v;
}

// Walks rows first, first + step, ... < end of NIN row-major tensors with row
// pitch `pitch` floats, at column `col` (a multiple of 4, 16-byte aligned
// addresses), and calls body(row, x) with x[i] the float4 of tensor i, rows in
// ascending order.  `ring` is the block's ring (THREADS threads); the caller
// must not touch it before ring_drain().  Slot and source addresses advance by
// additions; a row costs about a dozen instructions beside the body.
template <int NIN, int DEPTH, int THREADS, class Body>
__device__ __forceinline__ void ring_walk(float4 *ring, const float *const (&in)[NIN], size_t pitch, int col,
                                          int first, int end, int step, Body body) {
  constexpr unsigned TENSOR_BYTES = THREADS * 16u;       // one tensor's float4 of every thread
  constexpr unsigned SLOT_BYTES = NIN * TENSOR_BYTES;    // one row of all tensors
  const unsigned base = (unsigned)__cvta_generic_to_shared(ring + threadIdx.x);
  const unsigned wrap = base + DEPTH * SLOT_BYTES;
  const char *src[NIN];
#pragma unroll
  for (int i = 0; i < NIN; ++i) src[i] = reinterpret_cast<const char *>(in[i] + (size_t)first * pitch + col);
  const size_t src_step = (size_t)step * pitch * sizeof(float);
  // Row r + (DEPTH - 1) * step is sent while row r is worked on.
  const int last_issue = end - (DEPTH - 1) * step;
  unsigned fill = base;
#pragma unroll
  for (int d = 0; d < DEPTH - 1; ++d) {
    if (first + d * step < end) {
#pragma unroll
      for (int i = 0; i < NIN; ++i) cp_async16_to(fill + i * TENSOR_BYTES, src[i]);
    }
    cp_async_commit();
#pragma unroll
    for (int i = 0; i < NIN; ++i) src[i] += src_step;
    fill += SLOT_BYTES;
  }
  unsigned use = base;
  for (int r = first; r < end; r += step) {
    // The slot filled here was read in the iteration before this one.
    if (r < last_issue) {
#pragma unroll
      for (int i = 0; i < NIN; ++i) cp_async16_to(fill + i * TENSOR_BYTES, src[i]);
    }
    cp_async_commit();
#pragma unroll
    for (int i = 0; i < NIN; ++i) src[i] += src_step;
    fill += SLOT_BYTES;
    if (fill == wrap) fill = base;
    cp_async_wait<DEPTH - 1>();  // all but the newest DEPTH - 1 groups: row r has arrived
    float4 x[NIN];
#pragma unroll
    for (int i = 0; i < NIN; ++i) x[i] = ring_read(use + i * TENSOR_BYTES);
    use += SLOT_BYTES;
    if (use == wrap) use = base;
    body(r, x);
  }
}

// The general form: `count` steps over NIN streams of float4, stream i starting
// at src[i] and moving by stride[i] bytes per step (any sign: a walk back in
// time has negative strides, a per-step vector of statistics a short one).
// body(k, x) sees step k = 0 .. count - 1 in order.
// valid[i]: stream i is only read for steps k < valid[i] (x[i] of later steps is
// whatever the slot held).
template <int NIN, int DEPTH, int THREADS, class Body>
__device__ __forceinline__ void ring_steps(float4 *ring, const char *(&src)[NIN], const long long (&stride)[NIN],
                                           const int (&valid)[NIN], int count, Body body) {
  constexpr unsigned TENSOR_BYTES = THREADS * 16u;
  constexpr unsigned SLOT_BYTES = NIN * TENSOR_BYTES;
  const unsigned base = (unsigned)__cvta_generic_to_shared(ring + threadIdx.x);
  const unsigned wrap = base + DEPTH * SLOT_BYTES;
  unsigned fill = base;
#pragma unroll
  for (int d = 0; d < DEPTH - 1; ++d) {
#pragma unroll
    for (int i = 0; i < NIN; ++i)
      if (d < valid[i]) cp_async16_to(fill + i * TENSOR_BYTES, src[i]);
    cp_async_commit();
#pragma unroll
    for (int i = 0; i < NIN; ++i) src[i] += stride[i];
    fill += SLOT_BYTES;
  }
  unsigned use = base;
  for (int k = 0; k < count; ++k) {
    const int ahead = k + DEPTH - 1;  // the step sent now
#pragma unroll
    for (int i = 0; i < NIN; ++i)
      if (ahead < valid[i]) cp_async16_to(fill + i * TENSOR_BYTES, src[i]);
    cp_async_commit();
#pragma unroll
    for (int i = 0; i < NIN; ++i) src[i] += stride[i];
    fill += SLOT_BYTES;
    if (fill == wrap) fill = base;
    cp_async_wait<DEPTH - 1>();
    float4 x[NIN];
#pragma unroll
    for (int i = 0; i < NIN; ++i) x[i] = ring_read(use + i * TENSOR_BYTES);
    use += SLOT_BYTES;
    if (use == wrap) use = base;
    body(k, x);
  }
}

// After the walk, before the block reuses the ring's memory for something else.
__device__ __forceinline__ void ring_drain() {
  cp_async_wait<0>();
  __syncthreads();
}

}  // namespace dlb
