// The fp16-plane FC product on pairs of SMs: C[m,n] (+)= sum_k A(m,k) B(n,k).
//
// gemm_x3_kernel (gemm_tcgen05.cu) is bound by shared-memory bandwidth: per
// k-block of a 128 x 256 tile the tensor core reads 72 KB of operands while TMA
// writes 48 KB, more per clock than one SM's shared memory delivers.  Here two
// CTAs of a cluster share a 256 x 256 tile (tcgen05.mma.cta_group::2): each CTA
// holds its 128 rows of A and one half (128 columns) of B, the tensor cores of
// both SMs read both halves of B, and each SM accumulates its 128 x 256 part
// in its own tensor memory.  Per SM and k-block that is 48 KB read and 32 KB
// written, a third less, and six stages fit where four did.
//
// Roles per CTA as in gemm_x3_kernel: warp 0 loads with TMA, warp 1 issues the
// MMAs (in the even CTA of the pair only), warps 2-9 drain the accumulator
// chunks into registers and store the tile.  Barriers across the pair:
//   full[s]       lives in the even CTA; both CTAs' TMA loads complete on it
//   empty[s]      one per CTA; the MMA lane's commit arrives on both
//   acc_full[b]   one per CTA; the commit of a chunk arrives on both
//   acc_empty[b]  lives in the even CTA; the drain warps of both CTAs arrive
// Persistent over work items, last partial round cut along k, chunked
// accumulation, bounded waits: as in gemm_x3_kernel.
#include <stdlib.h>

#include "common.cuh"
#include "gemm_simt.cuh"
#include "tc_ptx.cuh"

namespace dlb {

namespace {

using namespace tc;

constexpr int PM = 256;  // rows of a pair's tile (2 x BM)
constexpr int PN = 256;  // columns of a pair's tile
constexpr int PBK = 32;  // halfs per k-block (64-byte rows)
constexpr int HALF_N = PN / 2;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of a CTA pair: the completion may be counted on the peer's barrier.
__device__ __forceinline__ void tma_pair_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_pair_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma_pair_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair when all MMAs
// issued so far have completed.
__device__ __forceinline__ void umma_pair_commit(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(both)
      : "memory");
}

template <int STAGES>
struct PairPlan {
  static constexpr int A_BYTES = BM * PBK * 2;       // this CTA's 128 rows of A, one plane
  static constexpr int B_BYTES = HALF_N * PBK * 2;   // this CTA's 128 columns of B, one plane
  static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int EPI_OFFSET = RING_BYTES;
  static constexpr int EPI_BYTES = NUM_DRAIN_WARPS * 32 * 33 * 4;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
  static_assert(TOTAL <= 232448, "shared memory of one CTA");
};

// A work item: a whole tile, or one of the `parts` pieces along k of a tile of
// the last partial round (pieces start on chunk boundaries).
struct PairItem {
  int m0, n0, kb_begin, num_kb, split, piece;
};
__host__ __device__ __forceinline__ int piece_start(int piece, int parts, int total_kb, int chunk_kb) {
  const int at = (int)(((long long)piece * total_kb / parts + chunk_kb - 1) / chunk_kb * chunk_kb);
  return at < total_kb ? at : total_kb;
}
// Order of the tiles.  band = 0: row by row.  band > 0: the tile rows are taken
// in bands of `band`; inside a band the tiles run down a column of the band,
// then the next column, so that the pairs working at the same time cover a
// near-square patch of the output (74 pairs: 8 rows x 9 columns, 17 operand
// blocks instead of the 21 of 4.6 rows x 16 columns) and the band's rows of A
// stay in L2 while the columns of B stream past.
__host__ __device__ __forceinline__ void tile_coords(int tile_id, int tiles_m, int tiles_n, int band, int *tm,
                                                     int *tn) {
  if (band <= 0) {
    *tm = tile_id / tiles_n;
    *tn = tile_id % tiles_n;
    return;
  }
  const int per_band = band * tiles_n;
  const int b = tile_id / per_band, in_band = tile_id - b * per_band;
  const int rows = min(band, tiles_m - b * band);  // the last band may be lower
  *tn = in_band / rows;
  *tm = b * band + in_band % rows;
}

template <int CHUNK_KB>
__device__ __forceinline__ PairItem pair_item(int item, int tiles_m, int tiles_n, int band, int whole_tiles,
                                              int parts, int total_kb) {
  PairItem w;
  w.split = item >= whole_tiles;
  const int tile_id = w.split ? whole_tiles + (item - whole_tiles) / parts : item;
  w.piece = w.split ? (item - whole_tiles) % parts : 0;
  int tm, tn;
  tile_coords(tile_id, tiles_m, tiles_n, band, &tm, &tn);
  w.n0 = tn * PN;
  w.m0 = tm * PM;
  w.kb_begin = w.split ? piece_start(w.piece, parts, total_kb, CHUNK_KB) : 0;
  w.num_kb = (w.split ? piece_start(w.piece + 1, parts, total_kb, CHUNK_KB) : total_kb) - w.kb_begin;
  return w;
}

template <int STAGES, int CHUNK_KB, bool A_MN, bool B_MN, bool FUSED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    gemm_x3_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a_lo,
                        const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_b_lo,
                        float *__restrict__ C, long long ldc, int M, int N, int K,
                        const float *__restrict__ bias, int accumulate, int tiles_n, int band, int whole_tiles,
                        int parts, int total_items, const float *__restrict__ scale_a,
                        const float *__restrict__ scale_b, int *status, const unsigned *guard_a,
                        const unsigned *guard_b, unsigned mask_a, unsigned mask_b,
                        const float *__restrict__ line_inv_a, SimtOperands fp32, unsigned long long *fallbacks,
                        const FusedEpilogue fe) {
  pdl_enter();
  using P = PairPlan<STAGES>;
  // Range guard: the planes of a flagged operand do not stand for its tensor.
  // The product is then formed from the fp32 tensors on the CUDA cores, every
  // CTA taking its share of the 64 x 64 tiles (a rare and slow path that keeps
  // the result right; the counter tells the host that it was taken).  Both
  // CTAs of a pair read the same words and take the same branch.
  if ((guard_a && (*guard_a & mask_a)) || (guard_b && (*guard_b & mask_b))) {
    extern __shared__ __align__(16) uint8_t guard_smem[];
    if (fallbacks && blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(fallbacks, 1ull);
    gemm_simt_guard_path(fp32, C, ldc, M, N, K, bias, accumulate, reinterpret_cast<float *>(guard_smem),
                         FUSED ? &fe : nullptr);
    return;
  }
  constexpr int MN_W = 64;  // halfs of one 128-byte column of an MN-major tile
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t *smem = smem_raw + (base - raw);
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + P::BAR_OFFSET);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * STAGES + 4);
  uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 5);
  unsigned *issued_kb = reinterpret_cast<unsigned *>(bars + 2 * STAGES + 6);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_rank();  // 0: the CTA that issues the MMAs
  const int pair = blockIdx.x / 2, pairs = gridDim.x / 2;
  const int total_kb = (K + PBK - 1) / PBK;
  const int tiles_m = (M + PM - 1) / PM;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES),
                 acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);   // the even CTA's producer; bytes of both CTAs' loads
      mbar_init(empty0 + 8 * s, 1);  // one commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 2 * NUM_DRAIN_WARPS);  // drain warps of both CTAs
    }
    *abort_flag = 0;
    *issued_kb = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // Two accumulators of 256 columns in the tensor memory of both SMs.
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)),
                 "r"((uint32_t)(2 * PN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them
  tcgen05_fence_after();
  const uint32_t tmem_acc = *tmem_holder;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      const uint32_t lead_full0 = map_to_cta(full0, 0);
      unsigned it = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += pairs) {
        const PairItem w = pair_item<CHUNK_KB>(item, tiles_m, tiles_n, band, whole_tiles, parts, total_kb);
        const int am0 = w.m0 + (int)rank * BM, bn0 = w.n0 + (int)rank * HALF_N;
        for (int kb = 0; kb < w.num_kb; ++kb, ++it) {
          const unsigned s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, abort_flag, status);
          if (!ok) break;
          const uint32_t fb = lead_full0 + 8 * s;
          const uint32_t st = base + s * P::STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * P::STAGE_BYTES);
          const int k0 = (w.kb_begin + kb) * PBK;
          if (A_MN) {
            tma_pair_3d(st, &tm_a, fb, 0, k0, am0 / MN_W);
            tma_pair_3d(st + P::A_BYTES, &tm_a_lo, fb, 0, k0, am0 / MN_W);
          } else {
            tma_pair_2d(st, &tm_a, fb, k0, am0);
            tma_pair_2d(st + P::A_BYTES, &tm_a_lo, fb, k0, am0);
          }
          if (B_MN) {
            tma_pair_3d(st + 2 * P::A_BYTES, &tm_b, fb, 0, k0, bn0 / MN_W);
            tma_pair_3d(st + 2 * P::A_BYTES + P::B_BYTES, &tm_b_lo, fb, 0, k0, bn0 / MN_W);
          } else {
            tma_pair_2d(st + 2 * P::A_BYTES, &tm_b, fb, k0, bn0);
            tma_pair_2d(st + 2 * P::A_BYTES + P::B_BYTES, &tm_b_lo, fb, k0, bn0);
          }
          *issued_kb = it + 1;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      // fp32 accumulate, F16 operands, majors, N = 256, M = 256 over the pair.
      const uint32_t idesc = (1u << 4) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                             ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(PM >> 4) << 24);
      constexpr int KI = 16;
      constexpr uint32_t K_ROW = PBK * 2;  // 64-byte rows, 64-byte swizzle
      constexpr uint32_t A_LBO = A_MN ? PBK * 128 : 16, A_SBO = A_MN ? 1024 : 8 * K_ROW;
      constexpr uint32_t B_LBO = B_MN ? PBK * 128 : 16, B_SBO = B_MN ? 1024 : 8 * K_ROW;
      constexpr uint32_t A_LAYOUT = A_MN ? LAYOUT_SW128 : LAYOUT_SW64;
      constexpr uint32_t B_LAYOUT = B_MN ? LAYOUT_SW128 : LAYOUT_SW64;
      constexpr uint32_t A_KSTEP = A_MN ? KI * 128 : 32, B_KSTEP = B_MN ? KI * 128 : 32;
      bool ok = true;
      unsigned it = 0, cc = 0;
      for (int item = pair; item < total_items && ok; item += pairs) {
        const PairItem w = pair_item<CHUNK_KB>(item, tiles_m, tiles_n, band, whole_tiles, parts, total_kb);
        int kb = 0;
        while (kb < w.num_kb && ok) {
          const unsigned buf = cc & 1, use = cc >> 1;
          ok = mbar_wait(acc_empty0 + 8 * buf, (use & 1) ^ 1, abort_flag, status);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_acc + (uint32_t)(buf * PN);
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
            for (int k8 = 0; k8 < PBK / KI; ++k8) {
              const uint64_t da_hi = make_smem_desc(a_hi + k8 * A_KSTEP, A_LBO, A_SBO, A_LAYOUT);
              const uint64_t da_lo = make_smem_desc(a_lo + k8 * A_KSTEP, A_LBO, A_SBO, A_LAYOUT);
              const uint64_t db_hi = make_smem_desc(b_hi + k8 * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
              const uint64_t db_lo = make_smem_desc(b_lo + k8 * B_KSTEP, B_LBO, B_SBO, B_LAYOUT);
              umma_pair_f16(d_tmem, da_lo, db_hi, idesc, first ? 0u : 1u);
              umma_pair_f16(d_tmem, da_hi, db_lo, idesc, 1u);
              umma_pair_f16(d_tmem, da_hi, db_hi, idesc, 1u);
              first = false;
            }
            umma_pair_commit(empty0 + 8 * s);
          }
          if (ok) umma_pair_commit(acc_full0 + 8 * buf);
          ++cc;
        }
      }
    }
  } else {
    // ---------------- drain + epilogue: warps 2..9 of both CTAs ----------------
    const int q = warp & 3;
    const int h = (warp - 2) >> 2;
    constexpr int HALF = PN / 2;
    float *tile = reinterpret_cast<float *>(smem + P::EPI_OFFSET) + (warp - 2) * 32 * 33;
    const float out_b = 1.f / __ldg(scale_b);
    const float tensor_out_a = line_inv_a ? 1.f : 1.f / __ldg(scale_a);
    const float plane_scale = FUSED && fe.sink.hi ? sink_scale(fe.sink) : 1.f;
    const uint32_t lead_acc_empty0 = map_to_cta(acc_empty0, 0);
    float acc[HALF];
    bool ok = true;
    unsigned cc = 0;
    for (int item = pair; item < total_items && ok; item += pairs) {
      const PairItem w = pair_item<CHUNK_KB>(item, tiles_m, tiles_n, band, whole_tiles, parts, total_kb);
      const int num_chunks = (w.num_kb + CHUNK_KB - 1) / CHUNK_KB;
#pragma unroll
      for (int j = 0; j < HALF; ++j) acc[j] = 0.f;
      for (int c = 0; c < num_chunks; ++c, ++cc) {
        const unsigned buf = cc & 1, use = cc >> 1;
        ok = mbar_wait(acc_full0 + 8 * buf, use & 1, abort_flag, status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t taddr = tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * PN + h * HALF);
#pragma unroll
        for (int j = 0; j < HALF / 32; ++j) {
          uint32_t v[32];
          tmem_ld32(taddr + j * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[j * 32 + i] += __uint_as_float(v[i]);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(lead_acc_empty0 + 8 * buf);
      }
      if (!ok) break;
      const int row_base = w.m0 + (int)rank * BM + q * 32;
      // This thread holds row row_base + lane; planes with a scale per line bring 1 / scale per row.
      const float out_a = line_inv_a ? __ldg(line_inv_a + min(row_base + lane, M - 1)) : tensor_out_a;
#pragma unroll
      for (int j = 0; j < HALF / 32; ++j) {
        const int col0 = w.n0 + h * HALF + j * 32;
        if (col0 < N) {
#pragma unroll
          for (int i = 0; i < 32; ++i) tile[lane * 33 + i] = acc[j * 32 + i] * out_a * out_b;
          __syncwarp();
          const int col = col0 + lane;
          if (col < N) {
            const float b = (bias && w.piece == 0) ? __ldg(bias + col) : 0.f;
            if (FUSED) {
              // Launches with a fused epilogue have no split tiles and do not
              // accumulate.  The lanes of the warp that are here hold 32
              // consecutive columns of one row at a time.
              const float keep = epilogue_keep(fe, col);
              unsigned col_max = 0u;
#pragma unroll 2
              for (int r = 0; r < 32; ++r) {
                const int row = row_base + r;
                if (row < M) {
                  const size_t at = (size_t)row * N + col;
                  const float x = epilogue_store(fe, C + (long long)row * ldc + col, at, tile[r * 33 + lane] + b, keep);
                  if (fe.sink.hi) epilogue_planes(fe, at, x, plane_scale);
                  const unsigned bits = abs_bits(x);
                  col_max = max(col_max, bits);
                  if (fe.sink.rowmax) {
                    const unsigned row_max = __reduce_max_sync(__activemask(), bits);
                    if (lane == 0 && row_max) atomicMax(fe.sink.rowmax + row, row_max);
                  }
                }
              }
              if (fe.sink.colmax && col_max) atomicMax(fe.sink.colmax + col, col_max);
              if (fe.sink.slot) amax_commit(reinterpret_cast<unsigned *>(fe.sink.slot) + SLOT_AMAX, col_max);
            } else if (w.split) {
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
  if (*abort_flag && threadIdx.x == 0 && rank == 0) {
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
  cluster_sync_all();  // neither CTA leaves while the other may still signal it or read its tiles
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc),
                 "r"((uint32_t)(2 * PN))
                 : "memory");
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {

template <int STAGES, int CHUNK_KB, bool A_MN, bool B_MN, bool FUSED = false>
dlb_status launch_pair(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C, long long ldc,
                       int M, int N, int K, const GemmEpilogue &ep) {
  using P = PairPlan<STAGES>;
  CUtensorMap ta, tal, tb, tbl;
  bool ok = true;
  ok &= tmap_cached(ctx, &ta, A_MN, A.h_hi, 2, M, K, A_MN ? A.stride_k : A.stride_mn, PBK, BM);
  ok &= tmap_cached(ctx, &tal, A_MN, A.h_lo, 2, M, K, A_MN ? A.stride_k : A.stride_mn, PBK, BM);
  ok &= tmap_cached(ctx, &tb, B_MN, B.h_hi, 2, N, K, B_MN ? B.stride_k : B.stride_mn, PBK, HALF_N);
  ok &= tmap_cached(ctx, &tbl, B_MN, B.h_lo, 2, N, K, B_MN ? B.stride_k : B.stride_mn, PBK, HALF_N);
  if (!ok) {
    set_error("gemm_pair: cuTensorMapEncodeTiled rejected an operand");
    return DLB_ERR_CUDA;
  }
  auto kernel = gemm_x3_pair_kernel<STAGES, CHUNK_KB, A_MN, B_MN, FUSED>;
  static bool attr_set[MAX_DEVICES] = {};  // the attribute belongs to the (function, device) pair
  if (!attr_set[ctx->device]) {
    DLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P::TOTAL));
    attr_set[ctx->device] = true;
  }
  // Pairs of SMs work through the 256 x 256 tiles in rounds.  The tiles of the
  // last partial round are cut along k into pieces that add into a zeroed
  // output when that shortens the round: with `rest` tiles on `lanes` pairs it
  // then lasts ceil(rest * parts / lanes) / parts of a full round.  Two pieces
  // add in either order to the same bits.  Three pieces measured slower than
  // no cut (the atomic adds of 46 tiles x 3 cost more than the third of a
  // round they save) and would not be reproducible, so MAX_PARTS is 2.
  // SMs are left free only while an all-reduce is in flight on the second
  // stream.
  const int tiles_n = ceil_div(N, PN), tiles = tiles_n * ceil_div(M, PM);
  const int sms = max(2, ctx->sm_count - (ctx->comm_pending ? ctx->gemm_reserve_sms : 0));
  const int lanes = sms / 2;
  const int total_kb = ceil_div(K, PBK);
  const int rest = tiles % lanes;
  int parts = 1;
  if (!ep.accumulate && rest > 0 && !FUSED) {  // a fused epilogue needs the whole sum of an element in one place
    // Twelfths of a round; a cut must save at least a twelfth per extra piece.
    int best = 12;
    constexpr int MAX_PARTS = 2;
    for (int p = 2; p <= MAX_PARTS; ++p) {
      if (total_kb < p * 4 * CHUNK_KB) break;  // a piece runs at least four chunks
      const int cost = ceil_div(rest * p, lanes) * 12 / p + (p - 1);
      if (cost < best) {
        best = cost;
        parts = p;
      }
    }
  }
  const int split_tiles = parts > 1 ? rest : 0;
  const int whole_tiles = tiles - split_tiles;
  static const int band = getenv("DLB_GEMM_BAND") ? atoi(getenv("DLB_GEMM_BAND")) : 8;
  const int tiles_m = ceil_div(M, PM);
  if (split_tiles) {
    // The cut tiles are the last of the order: a rectangle that holds them all
    // is cleared (whole tiles inside it store over the zeros).
    int tm, tn;
    tile_coords(whole_tiles, tiles_m, tiles_n, band, &tm, &tn);
    int first_row, first_col;
    if (band <= 0) {
      first_row = tm * PM;
      first_col = 0;
    } else {
      first_row = (tm / band) * band * PM;  // the band the first cut tile lies in
      // Cut tiles that reach into the bands below start those at column 0.
      first_col = (tm / band + 1) * band >= tiles_m ? tn * PN : 0;
    }
    DLB_CUDA(cudaMemset2DAsync(C + (long long)first_row * ldc + first_col, (size_t)ldc * sizeof(float), 0,
                               (size_t)(N - first_col) * sizeof(float), (size_t)(M - first_row), ctx->stream));
  }
  const int items = whole_tiles + parts * split_tiles;
  DLB_LAUNCH_KERNEL(ctx, kernel, 2 * min(items, lanes), NUM_THREADS, P::TOTAL, ta, tal, tb, tbl, C, ldc, M, N, K, ep.bias, ep.accumulate, tiles_n, band, whole_tiles, parts, items, A.scale, B.scale, ctx->d_status, A.guard, B.guard, A.guard_mask, B.guard_mask, A.line_inv, SimtOperands{A.ptr, A.fp32_stride_mn ? A.fp32_stride_mn : A.stride_mn, A.fp32_stride_k ? A.fp32_stride_k : A.stride_k, B.ptr, B.stride_mn, B.stride_k}, ctx->d_guard ? ctx->d_guard + 1 : nullptr, FUSED ? *ep.fused : FusedEpilogue{});
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // namespace

// On unless DLB_GEMM_PAIR=0.
bool gemm_pair_enabled() {
  static const bool on = [] {
    const char *e = getenv("DLB_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Chunk of k-blocks per accumulator drain: 8 unless DLB_GEMM_PAIR_CHUNK says 4 or 16.
int gemm_pair_chunk() {
  static const int chunk = [] {
    const char *e = getenv("DLB_GEMM_PAIR_CHUNK");
    return e ? atoi(e) : 8;
  }();
  return chunk;
}

dlb_status gemm_pair(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C, long long ldc,
                     int M, int N, int K, const GemmEpilogue &ep) {
  const bool a_mn = !(A.stride_k == 1);
  const bool b_mn = !(B.stride_k == 1);
  const int chunk = gemm_pair_chunk();
  if (ep.fused && ep.fused->mode != EPI_PLAIN) {
    // Instantiated for the two layouts that carry one (forward: both operands
    // K-major; input gradient: weights MN-major) at the default chunk.
    if (chunk == 8 && !ep.accumulate && !a_mn)
      return b_mn ? launch_pair<6, 8, false, true, true>(ctx, A, B, C, ldc, M, N, K, ep)
                  : launch_pair<6, 8, false, false, true>(ctx, A, B, C, ldc, M, N, K, ep);
    set_error("gemm_pair: no fused epilogue for this layout");
    return DLB_ERR_UNSUPPORTED;
  }
#define DLB_PAIR(CH)                                                                                  \
  if (chunk == (CH)) {                                                                                \
    if (!a_mn && !b_mn) return launch_pair<6, CH, false, false>(ctx, A, B, C, ldc, M, N, K, ep);      \
    if (!a_mn && b_mn) return launch_pair<6, CH, false, true>(ctx, A, B, C, ldc, M, N, K, ep);        \
    if (a_mn && b_mn) return launch_pair<6, CH, true, true>(ctx, A, B, C, ldc, M, N, K, ep);          \
  }
  DLB_PAIR(4)
  DLB_PAIR(8)
  DLB_PAIR(16)
#undef DLB_PAIR
  set_error("gemm_pair: MN-major A with K-major B is not instantiated");
  return DLB_ERR_UNSUPPORTED;
}

}  // namespace dlb
