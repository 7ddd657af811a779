// Operand planes of the tensor-core products.
//
// 3xFP16: a tensor x is used as hi + lo with hi = fp16(s x), lo = fp16(s x - hi),
// s a power of two per tensor chosen from max |x| so that s max lies in
// [2^14, 2^15).  The plane buffer of a tensor (its `_lo` argument in the C ABI)
// has the tensor's byte size and holds the hi plane followed by the lo plane.
// The context remembers, under the buffer's address, which tensor was split
// into it, its element count and the device slot of s; the FC entry points
// look their `_lo` arguments up there.
#include <cuda_fp16.h>

#include "common.cuh"

namespace dlb {

namespace {

// Largest |x| as raw bits (monotonic for non-negative floats).
__global__ void absmax_kernel(const float *__restrict__ x, size_t n, unsigned *slot) {
  unsigned m = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t n4 = n / 4;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (vec) {
#pragma unroll 4
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x) + i);
      m = max(max(m, v.x & 0x7fffffffu), max(v.y & 0x7fffffffu, max(v.z & 0x7fffffffu, v.w & 0x7fffffffu)));
    }
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      m = max(m, __float_as_uint(x[i]) & 0x7fffffffu);
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
      m = max(m, __float_as_uint(x[i]) & 0x7fffffffu);
  }
  for (int o = 16; o; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (threadIdx.x % 32 == 0 && m > *reinterpret_cast<volatile unsigned *>(slot)) atomicMax(slot, m);
}

// s = 2^(14 - E) for max = 1.f * 2^E; 1 for a zero, infinite or NaN maximum.
__device__ __forceinline__ float scale_from_bits(unsigned bits) {
  const int be = (int)(bits >> 23);  // biased exponent of the maximum
  if (bits == 0 || be == 255) return 1.f;
  int se = 14 - (be - 127) + 127;    // biased exponent of s
  se = min(max(se, 1), 254);
  return __uint_as_float((unsigned)se << 23);
}

__global__ void split_f16_kernel(const float *__restrict__ x, size_t n, __half *__restrict__ hi,
                                 __half *__restrict__ lo, float *slot) {
  const float s = scale_from_bits(reinterpret_cast<const unsigned *>(slot)[2]);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    slot[0] = s;
    slot[1] = 1.f / s;
  }
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) | (reinterpret_cast<uintptr_t>(hi) & 7) |
                    (reinterpret_cast<uintptr_t>(lo) & 7)) == 0;
  auto one = [s](float v, __half *h, __half *l) {
    const float t = v * s;
    const __half a = __float2half_rn(t);
    *h = a;
    *l = __float2half_rn(t - __half2float(a));
  };
  const size_t n4 = vec ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
    __half h[4], l[4];
    one(v.x, h, l);
    one(v.y, h + 1, l + 1);
    one(v.z, h + 2, l + 2);
    one(v.w, h + 3, l + 3);
    reinterpret_cast<uint2 *>(hi)[i] = *reinterpret_cast<uint2 *>(h);
    reinterpret_cast<uint2 *>(lo)[i] = *reinterpret_cast<uint2 *>(l);
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    one(x[i], hi + i, lo + i);
}

int stream_blocks(dlb_ctx *ctx, size_t items) {
  const size_t blocks = (items + 255) / 256;
  return (int)max((size_t)1, min(blocks, (size_t)ctx->sm_count * 16));
}

dlb_status scale_slot(dlb_ctx *ctx, float **out) {
  if (!ctx->scale_pool) {
    DLB_CUDA(cudaMalloc(&ctx->scale_pool, (size_t)SCALE_SLOTS * 4 * sizeof(float)));
    ctx->scale_free.reserve(SCALE_SLOTS);
    for (int i = SCALE_SLOTS - 1; i >= 0; --i) ctx->scale_free.push_back(i);
  }
  if (ctx->scale_free.empty()) {
    set_error("dlb_split_planes: more than %d plane buffers are registered", SCALE_SLOTS);
    return DLB_ERR_INVALID;
  }
  *out = ctx->scale_pool + 4 * (size_t)ctx->scale_free.back();
  ctx->scale_free.pop_back();
  return DLB_OK;
}

}  // namespace

dlb_status split_f16(dlb_ctx *ctx, const float *x, size_t n, uint16_t *hi, uint16_t *lo, float *slot) {
  DLB_CUDA(cudaMemsetAsync(slot + 2, 0, sizeof(float), ctx->stream));
  const int grid = stream_blocks(ctx, n / 4 + 1);
  absmax_kernel<<<grid, 256, 0, ctx->stream>>>(x, n, reinterpret_cast<unsigned *>(slot) + 2);
  DLB_LAUNCHED(ctx);
  split_f16_kernel<<<grid, 256, 0, ctx->stream>>>(x, n, reinterpret_cast<__half *>(hi),
                                                  reinterpret_cast<__half *>(lo), slot);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

bool planes_lookup(dlb_ctx *ctx, const float *aux, GemmOperand *o) {
  if (!aux || ctx->planes.empty()) return false;
  const uintptr_t p = reinterpret_cast<uintptr_t>(aux);
  auto it = ctx->planes.upper_bound(p);
  if (it == ctx->planes.begin()) return false;
  --it;
  const dlb_ctx::PlaneEntry &e = it->second;
  if (p >= it->first + e.n * sizeof(float)) return false;
  const size_t off = (p - it->first) / sizeof(float);
  if (e.x + off != o->ptr) return false;  // the buffer belongs to another tensor
  const uint16_t *hi = reinterpret_cast<const uint16_t *>(it->first) + off;
  const uint16_t *lo = hi + e.n;
  if ((reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 15) return false;
  o->h_hi = hi;
  o->h_lo = lo;
  o->scale = e.scale;
  return true;
}

// Registers `planes` as the plane buffer of x[0..n), clears the maximum of its
// scale slot and returns the slot; the caller then lets max |x| (bits) arrive
// in slot[2] and calls planes_finish.
dlb_status planes_begin(dlb_ctx *ctx, const float *x, float *planes, size_t n, float **slot_out) {
  DLB_REQUIRE(x && planes && n > 0 && n < ((size_t)1 << 40), "plane buffer: tensor, buffer and size");
  const uintptr_t key = reinterpret_cast<uintptr_t>(planes);
  // Buffers registered earlier that this one overwrites are stale: those that
  // start inside it, and one that starts before and reaches into it.
  planes_forget(ctx, key + 1, n * sizeof(float) - 1);
  auto before = ctx->planes.lower_bound(key);
  if (before != ctx->planes.begin()) {
    --before;
    if (before->first + before->second.n * sizeof(float) > key) planes_forget(ctx, before->first, 1);
  }
  auto it = ctx->planes.find(key);
  if (it == ctx->planes.end()) {
    float *slot = nullptr;
    DLB_TRY(scale_slot(ctx, &slot));
    it = ctx->planes.emplace(key, dlb_ctx::PlaneEntry{x, n, slot}).first;
  }
  it->second.x = x;
  it->second.n = n;
  DLB_CUDA(cudaMemsetAsync(it->second.scale + 2, 0, sizeof(float), ctx->stream));
  *slot_out = it->second.scale;
  return DLB_OK;
}

dlb_status planes_finish(dlb_ctx *ctx, const float *x, float *planes, size_t n, float *slot) {
  __half *hi = reinterpret_cast<__half *>(planes);
  split_f16_kernel<<<stream_blocks(ctx, n / 4 + 1), 256, 0, ctx->stream>>>(x, n, hi, hi + n, slot);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// Drops the entries whose buffer starts inside [base, base + bytes).
void planes_forget(dlb_ctx *ctx, uintptr_t base, size_t bytes) {
  auto it = ctx->planes.lower_bound(base);
  while (it != ctx->planes.end() && it->first < base + bytes) {
    ctx->scale_free.push_back((int)((it->second.scale - ctx->scale_pool) / 4));
    it = ctx->planes.erase(it);
  }
}

}  // namespace dlb

using namespace dlb;

extern "C" {

dlb_status dlb_ctx_set_gemm_kind(dlb_ctx *ctx, int kind) {
  DLB_REQUIRE(ctx && (kind == DLB_GEMM_TF32X3 || kind == DLB_GEMM_F16X3), "dlb_ctx_set_gemm_kind");
  if (kind == ctx->gemm_kind) return DLB_OK;
  // Plane buffers written under the other form do not hold what this form
  // reads: drop every registration and let the models split their weights
  // again (they compare plane_generation before each forward pass).
  DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  planes_forget(ctx, 0, ~(size_t)0);
  ctx->plane_generation++;
  ctx->gemm_kind = kind;
  return DLB_OK;
}

int dlb_ctx_gemm_kind(dlb_ctx *ctx) { return ctx ? ctx->gemm_kind : -1; }

dlb_status dlb_split_planes(dlb_ctx *ctx, const float *x, float *planes, size_t n) {
  DLB_REQUIRE(ctx && x && planes, "dlb_split_planes: null");
  if (n == 0) return DLB_OK;
  if (ctx->gemm_kind == DLB_GEMM_TF32X3) return dlb_split_tf32(ctx, x, planes, n);
  float *slot = nullptr;
  DLB_TRY(planes_begin(ctx, x, planes, n, &slot));
  absmax_kernel<<<stream_blocks(ctx, n / 4 + 1), 256, 0, ctx->stream>>>(x, n, reinterpret_cast<unsigned *>(slot) + 2);
  DLB_LAUNCHED(ctx);
  return planes_finish(ctx, x, planes, n, slot);
}

}  // extern "C"
