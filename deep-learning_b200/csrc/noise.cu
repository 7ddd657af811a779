// Noise of the step drawn on the device: Bernoulli dropout masks, UOut draws
// and ShakeDrop flags and factors, as an alternative to the arrays that the
// host hands over (the reference draws them from per-thread generators during
// the step: Model::Dropout_Bernoulli, Forward_Pass__Dropout__Uout__OpenMP
// fwp_mp.cpp L:4959-4985, Forward_Pass__Dropout__ShakeDrop__OpenMP L:4922-4957;
// those streams depend on the thread count and cannot be reproduced, so only
// the distributions are the reference's).
//
// The generator is Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random
// numbers: as easy as 1, 2, 3", SC'11): a keyed bijection of a 128-bit counter,
// ten rounds of two 32x32->64 multiplications.  Element i of a draw is word
// i mod 4 of the block with counter (i / 4, stream, step) and key = seed, so a
// draw is a pure function of (seed, stream, step, first + i): ranks that hold
// different rows of a batch draw their slices of the same array, and the union
// does not depend on how the rows are sharded.
#include "common.cuh"

namespace dlb {

namespace {

constexpr uint32_t PHILOX_M0 = 0xD2511F53u, PHILOX_M1 = 0xCD9E8D57u;
constexpr uint32_t PHILOX_W0 = 0x9E3779B9u, PHILOX_W1 = 0xBB67AE85u;

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(PHILOX_M0, c.x), lo0 = PHILOX_M0 * c.x;
    const uint32_t hi1 = __umulhi(PHILOX_M1, c.z), lo1 = PHILOX_M1 * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += PHILOX_W0;
    k.y += PHILOX_W1;
  }
  return c;
}

// 24 random bits -> [0, 1).
__device__ __forceinline__ float unit_float(uint32_t x) { return (float)(x >> 8) * (1.f / 16777216.f); }

struct NoiseKey {
  uint2 key;        // seed
  uint32_t stream;  // which array of the step
  uint32_t step;
  uint64_t first;   // index of out[0] in the whole array
};

__device__ __forceinline__ uint4 block_of(const NoiseKey &k, uint64_t block) {
  return philox4x32_10(make_uint4((uint32_t)block, (uint32_t)(block >> 32), k.stream, k.step), k.key);
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int w) {
  return w == 0 ? v.x : (w == 1 ? v.y : (w == 2 ? v.z : v.w));
}

// One thread per generator block (four consecutive elements of the array).
template <typename Emit>
__device__ __forceinline__ void for_each_word(const NoiseKey &k, size_t n, Emit emit) {
  const uint64_t first_block = k.first / 4, last_block = (k.first + n + 3) / 4;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t b = first_block + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; b < last_block; b += stride) {
    const uint4 v = block_of(k, b);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint64_t i = b * 4 + w;
      if (i >= k.first && i < k.first + n) emit((size_t)(i - k.first), word_of(v, w));
    }
  }
}

__global__ void __launch_bounds__(256) uniform_kernel(float *__restrict__ out, size_t n, float lo, float width, NoiseKey k) {
  pdl_enter();
  // Two roundings (no fused multiply-add), so that a host restatement in fp32
  // gives the same bits.
  for_each_word(k, n, [=](size_t i, uint32_t x) { out[i] = __fadd_rn(__fmul_rn(unit_float(x), width), lo); });
}

__global__ void __launch_bounds__(256) bernoulli_kernel(uint8_t *__restrict__ out, size_t n, float p, NoiseKey k) {
  pdl_enter();
  for_each_word(k, n, [=](size_t i, uint32_t x) { out[i] = unit_float(x) < p ? 1 : 0; });
}

NoiseKey make_key(uint64_t seed, uint32_t stream, uint32_t step, uint64_t first) {
  NoiseKey k;
  k.key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  k.stream = stream;
  k.step = step;
  k.first = first;
  return k;
}

int noise_blocks(dlb_ctx *ctx, size_t n) {
  return (int)std::max<size_t>(1, std::min<size_t>((n / 4 + 256) / 256, (size_t)ctx->sm_count * 16));
}

}  // namespace

}  // namespace dlb

using namespace dlb;

extern "C" {

dlb_status dlb_noise_uniform(dlb_ctx *ctx, float *out, size_t n, float lo, float hi, uint64_t seed,
                             uint32_t stream, uint32_t step, uint64_t first) {
  DLB_REQUIRE(ctx && (out || n == 0) && hi >= lo, "dlb_noise_uniform");
  if (n == 0) return DLB_OK;
  DLB_LAUNCH_KERNEL(ctx, uniform_kernel, noise_blocks(ctx, n), 256, 0, out, n, lo, hi - lo, make_key(seed, stream, step, first));
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_noise_bernoulli(dlb_ctx *ctx, uint8_t *out, size_t n, float p, uint64_t seed, uint32_t stream,
                               uint32_t step, uint64_t first) {
  DLB_REQUIRE(ctx && (out || n == 0) && p >= 0.f && p <= 1.f, "dlb_noise_bernoulli");
  if (n == 0) return DLB_OK;
  DLB_LAUNCH_KERNEL(ctx, bernoulli_kernel, noise_blocks(ctx, n), 256, 0, out, n, p, make_key(seed, stream, step, first));
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // extern "C"
