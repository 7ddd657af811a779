// FC GEMM on Blackwell tensor cores (sm_100a): C[m,n] (+)= sum_k A(m,k) B(n,k).
//
// fp32-faithful product by TF32 splitting ("3xTF32"): every fp32 operand x is
// used as hi(x) + lo(x), where hi(x) is what a kind::tf32 MMA reads of the raw
// fp32 word (sign, exponent, top 10 mantissa bits) and lo(x) = x - hi(x) comes
// from a residual plane in global memory.  Each 8-deep k step issues
//     D += lo(A) hi(B);  D += hi(A) lo(B);  D += hi(A) hi(B)
// into an fp32 accumulator in tensor memory.  The dropped lo*lo term is below
// 2^-20 of the product.
//
// Accumulation.  The tensor core adds into its fp32 accumulator with
// truncation, so a long k loop into one accumulator loses about half an ulp of
// the running sum per MMA, always towards zero: the error grows like k^1.5 and
// at k = 4096 is ten times that of an fp32 FMA loop.  The k loop is therefore
// cut into chunks of CHUNK_KB k-blocks; each chunk starts a fresh accumulator
// in one of two tensor-memory buffers, and while the tensor core works on the
// next chunk the eight drain warps read the finished one (tcgen05.ld) and add
// it into fp32 registers with round-to-nearest.  The truncation then acts on
// short sums only.
//
// One CTA computes a 128 x BN tile.  Warp 0 (one lane) streams operand tiles
// with TMA (cp.async.bulk.tensor, swizzled, no multicast) into a ring of
// shared-memory stages guarded by full/empty mbarriers; warp 1 (one lane)
// issues tcgen05.mma and commits each stage back to the producer and each chunk
// to the drain warps; warps 2-9 drain, and at the end add the bias and write
// rows to global memory through a per-warp shared-memory transpose (in the
// then idle ring) so that each store instruction covers 128 contiguous bytes.
//
// Operand majors.  "K-major": k is the contiguous direction in global memory
// (X and W in the forward product); tiles are rows of BK floats under the 64- or
// 128-byte swizzle.  "MN-major": m (or n) is contiguous (W in the
// input-gradient product, delta and X in the weight-gradient product).  An
// MN-major tile is fetched through a 3-d view {32 floats, k, mn/32} under the
// "128-byte swizzle of 32-byte atoms", the only shared-memory layout a TF32
// MN-major operand may have: 32-float columns, each a stack of 4-row groups.
//
// Every mbarrier wait is bounded by a clock budget; on expiry the kernel writes
// DLB_ERR_TIMEOUT to the status word, waits (bounded) for its TMA loads in
// flight, frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "gemm_simt.cuh"
#include "tc_ptx.cuh"

namespace dlb {

namespace {

using namespace tc;

template <int BN, int BK, int STAGES, int ES>
struct SmemPlan {
  static constexpr int A_BYTES = BM * BK * ES;
  static constexpr int B_BYTES = BN * BK * ES;
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int EPI_OFFSET = RING_BYTES;  // per-warp transpose buffers of the epilogue
  static constexpr int EPI_BYTES = NUM_DRAIN_WARPS * 32 * 33 * 4;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
  static_assert(TOTAL <= 232448, "shared memory of one CTA");
};

// One unit of work: an output tile over a range of k blocks.  Output tiles are
// numbered row-major over (m block, n block); items [0, whole_tiles) are whole
// tiles.  The remaining tiles (those that would form a last, partly filled
// wave over the SMs) are two items each, one per half of the k range, which
// add their partial results into an output the host has zeroed: with exactly
// two addends the sum does not depend on which half arrives first.
struct WorkItem {
  int m0, n0, kb_begin, num_kb, split, k_half;
};
template <int BN, int CHUNK_KB>
__device__ __forceinline__ WorkItem work_item(int item, int tiles_n, int whole_tiles, int total_kb) {
  WorkItem w;
  w.split = item >= whole_tiles;
  const int tile_id = w.split ? whole_tiles + ((item - whole_tiles) >> 1) : item;
  w.k_half = w.split ? ((item - whole_tiles) & 1) : 0;
  w.n0 = (tile_id % tiles_n) * BN;
  w.m0 = (tile_id / tiles_n) * BM;
  const int mid_kb = min(total_kb, (total_kb / 2 + CHUNK_KB - 1) / CHUNK_KB * CHUNK_KB);
  w.kb_begin = (w.split && w.k_half) ? mid_kb : 0;
  w.num_kb = (w.split ? (w.k_half ? total_kb : mid_kb) : total_kb) - w.kb_begin;
  return w;
}

// Barrier slots: [0,S) full, [S,2S) empty, 2S..2S+1 accumulator full,
// 2S+2..2S+3 accumulator empty, then three 8-byte scalars.
// ES = 4: fp32 operands read as TF32 plus their TF32 residual planes.
// ES = 2: fp16 planes hi = fp16(s x), lo = fp16(s x - hi) of every operand,
// s a power of two per tensor; the result is scaled back by 1 / (s_a s_b).
//
// Persistent: the grid is one CTA per SM (or fewer), and CTA c works through
// items c, c + gridDim.x, ...  The stage ring, the two accumulator buffers and
// their barrier phases run on across items, so the producer prefetches the
// next item's operands and the tensor core starts its first chunks while the
// drain warps still write the previous tile.
template <int BN, int BK, int STAGES, int CHUNK_KB, bool A_MN, bool B_MN, int ES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    gemm_x3_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_lo,
                   const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b_lo,
                   float *__restrict__ C, long long ldc, int M, int N, int K,
                   const float *__restrict__ bias, int accumulate, int tiles_n, int whole_tiles,
                   int total_items, const float *__restrict__ scale_a,
                   const float *__restrict__ scale_b, int *status, const unsigned *guard_a,
                   const unsigned *guard_b, unsigned mask_a, unsigned mask_b, SimtOperands fp32, unsigned long long *fallbacks) {
  pdl_enter();
  using P = SmemPlan<BN, BK, STAGES, ES>;
  // Range guard of the fp16 planes: with a flagged operand the product is formed
  // from the fp32 tensors on the CUDA cores by this same launch, every CTA
  // taking its share of the 64 x 64 tiles.
  if ((guard_a && (*guard_a & mask_a)) || (guard_b && (*guard_b & mask_b))) {
    extern __shared__ __align__(16) uint8_t guard_smem[];
    if (fallbacks && blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(fallbacks, 1ull);
    gemm_simt_guard_path(fp32, C, ldc, M, N, K, bias, accumulate, reinterpret_cast<float *>(guard_smem));
    return;
  }
  static_assert(ES == 4 || ES == 2, "fp32 (TF32) or fp16 operands");
  constexpr int MN_W = 128 / ES;  // elements of one 128-byte column of an MN-major tile
  static_assert(BN == 256, "two accumulators of 256 columns; the drain reads 64 columns at a time");
  constexpr int HALF = BN / 2;  // columns per drain warp
  extern __shared__ uint8_t smem_raw[];
  // Swizzled tiles need 1024-byte alignment of each tile base.
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + P::BAR_OFFSET);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * STAGES + 4);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 5);
  unsigned *issued_kb = reinterpret_cast<unsigned *>(bars + 2 * STAGES + 6);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int total_kb = (K + BK - 1) / BK;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES),
                 acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, NUM_DRAIN_WARPS);
    }
    *abort_flag = 0;
    *issued_kb = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // Whole warp allocates two accumulators of BN columns (power of two).
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)),
                 "r"((uint32_t)(2 * BN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = *tmem_holder;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      unsigned it = 0;  // k blocks issued by this CTA so far, over all items
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const WorkItem w = work_item<BN, CHUNK_KB>(item, tiles_n, whole_tiles, total_kb);
        for (int kb = 0; kb < w.num_kb; ++kb, ++it) {
          const unsigned s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, status);
          if (!ok) break;
          const uint32_t fb = full0 + 8 * s;
          const uint32_t st = base + s * P::STAGE_BYTES;
          mbar_expect_tx(fb, P::STAGE_BYTES);
          const int k0 = (w.kb_begin + kb) * BK;
          if (A_MN) {
            tma_load_3d(st, &tm_a, fb, 0, k0, w.m0 / MN_W);
            tma_load_3d(st + P::A_BYTES, &tm_a_lo, fb, 0, k0, w.m0 / MN_W);
          } else {
            tma_load_2d(st, &tm_a, fb, k0, w.m0);
            tma_load_2d(st + P::A_BYTES, &tm_a_lo, fb, k0, w.m0);
          }
          if (B_MN) {
            tma_load_3d(st + 2 * P::A_BYTES, &tm_b, fb, 0, k0, w.n0 / MN_W);
            tma_load_3d(st + 2 * P::A_BYTES + P::B_BYTES, &tm_b_lo, fb, 0, k0, w.n0 / MN_W);
          } else {
            tma_load_2d(st + 2 * P::A_BYTES, &tm_b, fb, k0, w.n0);
            tma_load_2d(st + 2 * P::A_BYTES + P::B_BYTES, &tm_b_lo, fb, k0, w.n0);
          }
          *issued_kb = it + 1;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // Instruction descriptor: fp32 accumulate, operand format, majors, N, M.
      constexpr uint32_t FMT = ES == 4 ? 2u : 0u;  // operand format: TF32 / F16
      const uint32_t idesc = (1u << 4) | (FMT << 7) | (FMT << 10) | ((A_MN ? 1u : 0u) << 15) |
                             ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      // K-major tiles: rows of BK*ES bytes, 8-row groups SBO apart, k step = 32 B
      // inside the swizzled row.  MN-major tiles: 128-byte columns (32 floats or
      // 64 halfs) LBO apart, each a stack of k rows; fp32: 4-row (512 B) groups
      // under the swizzle of 32-byte atoms, fp16: 8-row (1024 B) groups under the
      // plain 128-byte swizzle; k step = the rows of one instruction.
      constexpr int KI = 32 / ES;  // k per instruction: 8 (TF32), 16 (F16)
      constexpr uint32_t K_ROW = BK * ES;
      static_assert(K_ROW == 64 || K_ROW == 128, "k-major rows of 64 or 128 bytes");
      constexpr uint32_t K_LAYOUT = (K_ROW == 128) ? LAYOUT_SW128 : LAYOUT_SW64;
      constexpr uint32_t MN_SBO = ES == 4 ? 512 : 1024;
      constexpr uint32_t MN_LAYOUT = ES == 4 ? LAYOUT_SW128_BASE32B : LAYOUT_SW128;
      constexpr uint32_t A_LBO = A_MN ? BK * 128 : 16, A_SBO = A_MN ? MN_SBO : 8 * K_ROW;
      constexpr uint32_t B_LBO = B_MN ? BK * 128 : 16, B_SBO = B_MN ? MN_SBO : 8 * K_ROW;
      constexpr uint32_t A_LAYOUT = A_MN ? MN_LAYOUT : K_LAYOUT;
      constexpr uint32_t B_LAYOUT = B_MN ? MN_LAYOUT : K_LAYOUT;
      constexpr uint32_t A_KSTEP = A_MN ? KI * 128 : 32, B_KSTEP = B_MN ? KI * 128 : 32;
      bool ok = true;
      unsigned it = 0;  // k blocks consumed so far, over all items
      unsigned cc = 0;  // chunks started so far, over all items
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const WorkItem w = work_item<BN, CHUNK_KB>(item, tiles_n, whole_tiles, total_kb);
        int kb = 0;
        while (kb < w.num_kb && ok) {
          const unsigned buf = cc & 1, use = cc >> 1;
          // The drain warps must have emptied this buffer's previous chunk.
          ok = mbar_wait(acc_empty0 + 8 * buf, (use & 1) ^ 1, abort_flag, status);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_acc + (uint32_t)(buf * BN);
          const int kb_end = min(w.num_kb, kb + CHUNK_KB);
          bool first = true;
          for (; kb < kb_end; ++kb, ++it) {
            const unsigned s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            ok = mbar_wait(full0 + 8 * s, ph, abort_flag, status);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t st = base + s * P::STAGE_BYTES;
            const uint32_t a_hi = st, a_lo = st + P::A_BYTES, b_hi = st + 2 * P::A_BYTES,
                           b_lo = st + 2 * P::A_BYTES + P::B_BYTES;
#pragma unroll
            for (int k8 = 0; k8 < BK / KI; ++k8) {
              const uint64_t da_hi = make_smem_desc(a_hi + k8 * A_KSTEP, A_LBO, A_SBO, A_LAYOUT);
              const uint64_t da_lo = make_smem_desc(a_lo + k8 * A_KSTEP, A_LBO, A_SBO, A_LAYOUT);
              const uint64_t db_hi = make_smem_desc(b_hi + k8 * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
              const uint64_t db_lo = make_smem_desc(b_lo + k8 * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
              if (ES == 4) {
                umma_tf32(d_tmem, da_lo, db_hi, idesc, first ? 0u : 1u);
                umma_tf32(d_tmem, da_hi, db_lo, idesc, 1u);
                umma_tf32(d_tmem, da_hi, db_hi, idesc, 1u);
              } else {
                umma_f16(d_tmem, da_lo, db_hi, idesc, first ? 0u : 1u);
                umma_f16(d_tmem, da_hi, db_lo, idesc, 1u);
                umma_f16(d_tmem, da_hi, db_hi, idesc, 1u);
              }
              first = false;
            }
            umma_commit(empty0 + 8 * s);  // stage reusable once these MMAs retire
          }
          if (ok) umma_commit(acc_full0 + 8 * buf);  // chunk complete
          ++cc;
        }
      }
    }
  } else {
    // ---------------- drain + epilogue: warps 2..9 ----------------
    const int q = warp & 3;          // tensor-memory lane quadrant this warp may read
    const int h = (warp - 2) >> 2;   // which half of the BN columns
    float *tile = reinterpret_cast<float *>(smem + P::EPI_OFFSET) + (warp - 2) * 32 * 33;
    // fp16 planes hold s x: both factors are powers of two, the scaling is exact.
    const float out_a = ES == 2 ? 1.f / __ldg(scale_a) : 1.f, out_b = ES == 2 ? 1.f / __ldg(scale_b) : 1.f;
    float acc[HALF];
    bool ok = true;
    unsigned cc = 0;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const WorkItem w = work_item<BN, CHUNK_KB>(item, tiles_n, whole_tiles, total_kb);
      const int num_chunks = (w.num_kb + CHUNK_KB - 1) / CHUNK_KB;
#pragma unroll
      for (int j = 0; j < HALF; ++j) acc[j] = 0.f;
      for (int c = 0; c < num_chunks; ++c, ++cc) {
        const unsigned buf = cc & 1, use = cc >> 1;
        ok = mbar_wait(acc_full0 + 8 * buf, use & 1, abort_flag, status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + h * HALF);
#pragma unroll
        for (int j = 0; j < HALF / 32; ++j) {
          uint32_t v[32];
          tmem_ld32(taddr + j * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[j * 32 + i] += __uint_as_float(v[i]);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
      }
      if (!ok) break;
      // The tile is complete in registers; the tensor core is already on the
      // next item.  Rows go out through the warp's transpose buffer so that
      // each store instruction covers 128 contiguous bytes.
      const int row_base = w.m0 + q * 32;
#pragma unroll
      for (int j = 0; j < HALF / 32; ++j) {
        const int col0 = w.n0 + h * HALF + j * 32;
        if (col0 < N) {
          // lane owns row (row_base + lane): park its 32 values, then each
          // instruction below stores one row's 32 consecutive floats.
#pragma unroll
          for (int i = 0; i < 32; ++i)
            tile[lane * 33 + i] = ES == 2 ? acc[j * 32 + i] * out_a * out_b : acc[j * 32 + i];
          __syncwarp();
          const int col = col0 + lane;
          if (col < N) {
            const float b = (bias && w.k_half == 0) ? __ldg(bias + col) : 0.f;
            if (w.split) {
#pragma unroll 4
              for (int r = 0; r < 32; ++r) {
                const int row = row_base + r;
                if (row < M) atomicAdd(C + (long long)row * ldc + col, tile[r * 33 + lane] + b);
              }
            } else {
#pragma unroll 4
              for (int r = 0; r < 32; ++r) {
                const int row = row_base + r;
                if (row < M) {
                  float *dst = C + (long long)row * ldc + col;
                  float val = tile[r * 33 + lane] + b;
                  if (accumulate) val += *dst;
                  *dst = val;
                }
              }
            }
          }
          __syncwarp();
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // Let TMA loads that were already issued land before the CTA's shared
    // memory is handed to another block.
    const unsigned issued = *issued_kb;
    const long long t0 = clock64();
    for (unsigned kb = issued > (unsigned)STAGES ? issued - STAGES : 0; kb < issued; ++kb) {
      const unsigned s = kb % STAGES;
      const uint32_t ph = (kb / STAGES) & 1;
      while (!mbar_try_wait(full0 + 8 * s, ph)) {
        if (clock64() - t0 > DRAIN_BUDGET_CLOCKS) break;
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc),
                 "r"((uint32_t)(2 * BN))
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
}  // namespace

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// K-major operand: global [mn, k] with row pitch ld (elements of `es` bytes);
// box {BK, rows}.
bool tmap_k_major(CUtensorMap *m, const void *ptr, int es, uint64_t mn, uint64_t k, uint64_t ld,
                  uint32_t box_k, uint32_t box_mn) {
  const cuuint64_t dims[2] = {k, mn};
  const cuuint64_t strides[1] = {ld * es};
  const cuuint32_t box[2] = {box_k, box_mn};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = box_k * es == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  return encode_tiled()(m, es == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                        const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// MN-major operand: global [k, mn] with row pitch ld, viewed as {w, k, mn/w}
// with w = 128 bytes of elements (32 floats, 64 halfs); box {w, BK, cols/w}
// lands as 128-byte columns.  fp32 needs the swizzle of 32-byte atoms, fp16 the
// plain 128-byte swizzle.
bool tmap_mn_major(CUtensorMap *m, const void *ptr, int es, uint64_t mn, uint64_t k, uint64_t ld,
                   uint32_t box_k, uint32_t box_mn) {
  const uint32_t w = 128 / es;
  const cuuint64_t dims[3] = {w, k, mn / w};
  const cuuint64_t strides[2] = {ld * es, 128};
  const cuuint32_t box[3] = {w, box_k, box_mn / w};
  const cuuint32_t estr[3] = {1, 1, 1};
  return encode_tiled()(m, es == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                        const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        es == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The descriptor of an operand, from the context's cache when the same
// (address, shape, box) was encoded before: a descriptor depends on nothing else.
bool tmap_cached(dlb_ctx *ctx, CUtensorMap *out, bool mn_major, const void *ptr, int es, uint64_t mn,
                 uint64_t k, uint64_t ld, uint32_t box_k, uint32_t box_mn) {
  static_assert(sizeof(CUtensorMap) == sizeof(dlb_ctx::TmapBlob), "descriptor size");
  const dlb_ctx::TmapKey key{reinterpret_cast<uintptr_t>(ptr), mn, k, ld, box_k, box_mn, es, mn_major ? 1 : 0};
  auto it = ctx->tmaps.find(key);
  if (it != ctx->tmaps.end()) {
    memcpy(out, it->second.bytes, sizeof(CUtensorMap));
    return true;
  }
  const bool ok = mn_major ? tmap_mn_major(out, ptr, es, mn, k, ld, box_k, box_mn)
                           : tmap_k_major(out, ptr, es, mn, k, ld, box_k, box_mn);
  if (!ok) return false;
  if (ctx->tmaps.size() >= 4096) ctx->tmaps.clear();
  dlb_ctx::TmapBlob blob;
  memcpy(blob.bytes, out, sizeof(CUtensorMap));
  ctx->tmaps.emplace(key, blob);
  return true;
}

namespace {

// What TMA can address: 16-byte aligned base and row pitch; an MN-major extent
// that is a whole number of 128-byte columns.
bool operand_ok(const void *ptr, int es, long long stride_mn, long long stride_k, int mn, int k) {
  const int per16 = 16 / es, w = 128 / es;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
  if (stride_k == 1) return stride_mn % per16 == 0 && stride_mn >= k;
  if (stride_mn == 1) return stride_k % per16 == 0 && stride_k >= mn && mn % w == 0;
  return false;
}

struct TileConfig {
  int bn, bk, stages, chunk;
};
// Selected by DLB_GEMM_TILE=<bn>x<bk bytes / 4>x<stages>x<chunk k-blocks> for experiments.
TileConfig tile_config() {
  static TileConfig cfg = [] {
    TileConfig c{256, 16, 4, 4};
    if (const char *e = getenv("DLB_GEMM_TILE")) {
      int bn, bk, st, ch;
      if (sscanf(e, "%dx%dx%dx%d", &bn, &bk, &st, &ch) == 4) c = TileConfig{bn, bk, st, ch};
    }
    return c;
  }();
  return cfg;
}

// BKW = k-block in 4-byte words per row (16 -> 64-byte rows): BK = BKW floats or
// 2 * BKW halfs.
template <int BN, int BKW, int STAGES, int CHUNK_KB, bool A_MN, bool B_MN, int ES>
dlb_status launch(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                  long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  constexpr int BK = BKW * 4 / ES;
  using P = SmemPlan<BN, BK, STAGES, ES>;
  const void *a_hi = ES == 4 ? (const void *)A.ptr : (const void *)A.h_hi;
  const void *a_lo = ES == 4 ? (const void *)A.lo : (const void *)A.h_lo;
  const void *b_hi = ES == 4 ? (const void *)B.ptr : (const void *)B.h_hi;
  const void *b_lo = ES == 4 ? (const void *)B.lo : (const void *)B.h_lo;
  CUtensorMap ta, tal, tb, tbl;
  bool ok = true;
  ok &= tmap_cached(ctx, &ta, A_MN, a_hi, ES, M, K, A_MN ? A.stride_k : A.stride_mn, BK, BM);
  ok &= tmap_cached(ctx, &tal, A_MN, a_lo, ES, M, K, A_MN ? A.stride_k : A.stride_mn, BK, BM);
  ok &= tmap_cached(ctx, &tb, B_MN, b_hi, ES, N, K, B_MN ? B.stride_k : B.stride_mn, BK, BN);
  ok &= tmap_cached(ctx, &tbl, B_MN, b_lo, ES, N, K, B_MN ? B.stride_k : B.stride_mn, BK, BN);
  if (!ok) {
    set_error("gemm_tcgen05: cuTensorMapEncodeTiled rejected an operand");
    return DLB_ERR_CUDA;
  }
  auto kernel = gemm_x3_kernel<BN, BK, STAGES, CHUNK_KB, A_MN, B_MN, ES>;
  // The attribute belongs to the (function, device) pair: once per device.
  static bool attr_set[MAX_DEVICES] = {};
  if (!attr_set[ctx->device]) {
    DLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::TOTAL));
    attr_set[ctx->device] = true;
  }
  // One CTA per SM is resident, so the tiles run in waves of sm_count.  When
  // the last wave would fill at most half of the SMs, its tiles are split in
  // two along k: twice as many CTAs of half the length, and the wave takes half
  // the time (4096^3: 512 tiles = 3 waves + 68 tiles -> 3 waves + 136 halves).
  // Not with accumulate (three addends would depend on arrival order) and not
  // for a short k loop.  DLB_GEMM_SPLIT=0 turns it off.
  const int tiles_n = ceil_div(N, BN), tiles = tiles_n * ceil_div(M, BM);
  static const bool split_enabled = [] {
    const char *e = getenv("DLB_GEMM_SPLIT");
    return !(e && e[0] == '0');
  }();
  // CTAs of this launch: one per SM, less the SMs left to a collective while one
  // is in flight on the second stream (the persistent CTAs would otherwise hold
  // every SM until the product ends and the gradient all-reduce could not
  // start).
  const int lanes = max(1, ctx->sm_count - (ctx->comm_pending ? ctx->gemm_reserve_sms : 0));
  int split_tiles = 0;
  const int rest = tiles % lanes;
  if (split_enabled && !ep.accumulate && rest > 0 && 2 * rest <= lanes &&
      ceil_div(K, BK) >= 8 * CHUNK_KB)
    split_tiles = rest;
  const int whole_tiles = tiles - split_tiles;
  if (split_tiles) {
    const int first_row = (whole_tiles / tiles_n) * BM;
    DLB_CUDA(cudaMemset2DAsync(C + (long long)first_row * ldc, (size_t)ldc * sizeof(float), 0,
                               (size_t)N * sizeof(float), (size_t)(M - first_row), ctx->stream));
  }
  const int items = whole_tiles + 2 * split_tiles;
  DLB_LAUNCH_KERNEL(ctx, kernel, min(items, lanes), NUM_THREADS, P::TOTAL, ta, tal, tb, tbl, C, ldc, M, N, K, ep.bias, ep.accumulate, tiles_n, whole_tiles, items, A.scale, B.scale, ctx->d_status, ES == 2 ? A.guard : nullptr, ES == 2 ? B.guard : nullptr, A.guard_mask, B.guard_mask, SimtOperands{A.ptr, A.fp32_stride_mn ? A.fp32_stride_mn : A.stride_mn, A.fp32_stride_k ? A.fp32_stride_k : A.stride_k, B.ptr, B.stride_mn, B.stride_k}, ctx->d_guard ? ctx->d_guard + 1 : nullptr);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

template <bool A_MN, bool B_MN, int ES>
dlb_status launch_tile(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                       long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  const TileConfig t = tile_config();
#define DLB_TILE(TBN, TBK, TST, TCH)                                              \
  if (t.bn == (TBN) && t.bk == (TBK) && t.stages == (TST) && t.chunk == (TCH))   \
    return launch<TBN, TBK, TST, TCH, A_MN, B_MN, ES>(ctx, A, B, C, ldc, M, N, K, ep);
  DLB_TILE(256, 16, 4, 4)
  DLB_TILE(256, 16, 4, 2)
  DLB_TILE(256, 16, 4, 8)
  DLB_TILE(256, 16, 4, 16)
#undef DLB_TILE
  set_error("gemm_tcgen05: tile %dx%dx%dx%d is not compiled in", t.bn, t.bk, t.stages, t.chunk);
  return DLB_ERR_UNSUPPORTED;
}

template <int ES>
dlb_status launch_majors(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                         long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  // A dimension of extent 1 along k makes stride_k ambiguous; treat k-contiguous first.
  const bool a_mn = !(A.stride_k == 1);
  const bool b_mn = !(B.stride_k == 1);
  if (!a_mn && !b_mn) return launch_tile<false, false, ES>(ctx, A, B, C, ldc, M, N, K, ep);
  if (!a_mn && b_mn) return launch_tile<false, true, ES>(ctx, A, B, C, ldc, M, N, K, ep);
  if (a_mn && b_mn) return launch_tile<true, true, ES>(ctx, A, B, C, ldc, M, N, K, ep);
  set_error("gemm_tcgen05: MN-major A with K-major B is not instantiated");
  return DLB_ERR_UNSUPPORTED;
}

bool shape_ok(const GemmOperand &A, const GemmOperand &B, const float *C, long long ldc, int M,
              int N, int K) {
  if (!encode_tiled()) return false;
  if (M < 1 || N < 1 || K < 1) return false;
  if (reinterpret_cast<uintptr_t>(C) & 3) return false;
  if (ldc < N) return false;
  // MN-major A with K-major B never occurs in the FC step.
  if (A.stride_mn == 1 && A.stride_k != 1 && B.stride_k == 1 && B.stride_mn != 1) return false;
  return true;
}

}  // namespace

bool gemm_tcgen05_supported(const GemmOperand &A, const GemmOperand &B, const float *C,
                            long long ldc, int M, int N, int K) {
  return shape_ok(A, B, C, ldc, M, N, K) && operand_ok(A.ptr, 4, A.stride_mn, A.stride_k, M, K) &&
         operand_ok(B.ptr, 4, B.stride_mn, B.stride_k, N, K);
}

// The fp16-plane form: planes have the strides of their tensor, so the test is
// on the strides alone (the planes' own base alignment is checked at launch).
bool gemm_f16_supported(const GemmOperand &A, const GemmOperand &B, const float *C, long long ldc,
                        int M, int N, int K) {
  return shape_ok(A, B, C, ldc, M, N, K) && operand_ok(nullptr, 2, A.stride_mn, A.stride_k, M, K) &&
         operand_ok(nullptr, 2, B.stride_mn, B.stride_k, N, K);
}

dlb_status gemm_tcgen05(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                        long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  if (A.h_hi && A.h_lo && B.h_hi && B.h_lo) {
    const uintptr_t al = reinterpret_cast<uintptr_t>(A.h_hi) | reinterpret_cast<uintptr_t>(A.h_lo) |
                         reinterpret_cast<uintptr_t>(B.h_hi) | reinterpret_cast<uintptr_t>(B.h_lo);
    if (!gemm_f16_supported(A, B, C, ldc, M, N, K) || (al & 15) || !A.scale || !B.scale) {
      set_error("gemm_tcgen05: fp16 planes outside the TMA path");
      return DLB_ERR_UNSUPPORTED;
    }
    if (gemm_pair_enabled() && (long long)M * N >= 256 * 256) return gemm_pair(ctx, A, B, C, ldc, M, N, K, ep);
    if (ep.fused) {
      set_error("gemm_tcgen05: a fused epilogue runs on the 2-CTA kernel only");
      return DLB_ERR_UNSUPPORTED;
    }
    return launch_majors<2>(ctx, A, B, C, ldc, M, N, K, ep);
  }
  if (ep.fused) {
    set_error("gemm_tcgen05: a fused epilogue needs fp16 planes");
    return DLB_ERR_UNSUPPORTED;
  }
  if (!gemm_tcgen05_supported(A, B, C, ldc, M, N, K) || !A.lo || !B.lo) {
    set_error("gemm_tcgen05: operand layout outside the TMA path");
    return DLB_ERR_UNSUPPORTED;
  }
  return launch_majors<4>(ctx, A, B, C, ldc, M, N, K, ep);
}

}  // namespace dlb
