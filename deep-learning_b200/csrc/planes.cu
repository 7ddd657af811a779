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
#include <string.h>

#include "common.cuh"
#include "planes.cuh"

namespace dlb {

namespace {

// Largest |x| as raw bits (monotonic for non-negative floats).
__global__ void absmax_kernel(const float *__restrict__ x, size_t n, unsigned *slot) {
  pdl_enter();
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

// Flat split of a tensor without a shape (or one whose rows are not a whole
// number of float4): planes only, no line statistics.
__global__ void split_flat_kernel(const float *__restrict__ x, size_t n, PlaneSink k) {
  pdl_enter();
  const float s = sink_scale(k);
  __half *hi = reinterpret_cast<__half *>(k.hi), *lo = reinterpret_cast<__half *>(k.lo);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) | (reinterpret_cast<uintptr_t>(hi) & 7) |
                    (reinterpret_cast<uintptr_t>(lo) & 7)) == 0;
  const size_t n4 = vec ? n / 4 : 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + i);
    const float a[4] = {v.x, v.y, v.z, v.w};
    sink_store4(k, i * 4, a, s);
  }
  for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    plane_halves(x[i], s, hi + i, lo + i);
}

// Split of a [rows, cols] tensor (cols a multiple of 4) with the row and column
// maxima: grid (column blocks of 128, row chunks), a thread owns four columns
// and walks its rows eight apart, as the other row kernels of the step do.
constexpr int SPLIT_LANES_Y = 8;
__global__ void __launch_bounds__(32 * SPLIT_LANES_Y)
    split_rows_kernel(const float *__restrict__ x, int rows, int cols, int rows_per_chunk, PlaneSink k) {
  pdl_enter();
  __shared__ unsigned shared[SPLIT_LANES_Y * 128];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int col = blockIdx.x * 128 + tx * 4;
  const bool live = col < cols;
  const float s = sink_scale(k);
  LineTracker track;
  if (live) {
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    for (int r = r0 + ty; r < r1; r += 2 * SPLIT_LANES_Y) {
      const int r2 = r + SPLIT_LANES_Y;
      const size_t o = (size_t)r * cols + col, o2 = (size_t)r2 * cols + col;
      const float4 v = __ldg(reinterpret_cast<const float4 *>(x + o));
      float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r2 < r1) w = __ldg(reinterpret_cast<const float4 *>(x + o2));
      const float a[4] = {v.x, v.y, v.z, v.w};
      sink_store4(k, o, a, s);
      track.row(k, r, a);
      if (r2 < r1) {
        const float b[4] = {w.x, w.y, w.z, w.w};
        sink_store4(k, o2, b, s);
        track.row(k, r2, b);
      }
    }
  }
  // Under a predicted scale the tensor's maximum is found here as well; where it
  // was known before (it gave s) the atomic maximum changes nothing.
  track.finish(k, shared, tx, ty, SPLIT_LANES_Y, blockIdx.x * 128, cols, live);
}

// Largest |x| of every column of x [K, M]: blocks of 32 columns x 8 row lanes
// over a slab of rows, one atomic per column and block.
__global__ void column_absmax_kernel(const float *__restrict__ x, long long pitch, int K, int M, int rows_per_block,
                                     unsigned *__restrict__ cmax) {
  pdl_enter();
  __shared__ unsigned fold[8][32];
  const int m = blockIdx.x * 32 + threadIdx.x;
  const int k0 = blockIdx.y * rows_per_block, k1 = min(K, k0 + rows_per_block);
  unsigned v = 0u;
  if (m < M)
    for (int k = k0 + threadIdx.y; k < k1; k += 8) v = max(v, abs_bits(x[(long long)k * pitch + m]));
  fold[threadIdx.y][threadIdx.x] = v;
  __syncthreads();
  if (threadIdx.y == 0 && m < M) {
#pragma unroll
    for (int y = 1; y < 8; ++y) v = max(v, fold[y][threadIdx.x]);
    if (v) atomicMax(cmax + m, v);
  }
}

// planes_t[m, k] = halves of s_m x[k, m], s_m from the column's maximum: 32 x 32
// tiles through shared memory.
__global__ void transpose_split_kernel(const float *__restrict__ x, long long pitch, int K, int M,
                                       const unsigned *__restrict__ cmax, uint16_t *__restrict__ hi_t,
                                       uint16_t *__restrict__ lo_t, long long kp, float *__restrict__ line_inv) {
  pdl_enter();
  __shared__ float tile[32][33];
  const int m0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  for (int y = threadIdx.y; y < 32; y += 8) {
    const int k = k0 + y, m = m0 + threadIdx.x;
    tile[y][threadIdx.x] = (k < K && m < M) ? x[(long long)k * pitch + m] : 0.f;
  }
  __syncthreads();
  for (int y = threadIdx.y; y < 32; y += 8) {
    const int m = m0 + y, k = k0 + threadIdx.x;
    if (m < M && k < kp) {
      const float s = plane_scale_from_bits(cmax[m], PLANE_EXP_OWN);
      __half h, l;
      plane_halves(tile[threadIdx.x][y], s, &h, &l);
      hi_t[(long long)m * kp + k] = *reinterpret_cast<const uint16_t *>(&h);
      lo_t[(long long)m * kp + k] = *reinterpret_cast<const uint16_t *>(&l);
      if (k == 0) line_inv[m] = 1.f / s;
    }
  }
}

__global__ void __launch_bounds__(1024) planes_finalize_kernel(PlaneSink k) {
  pdl_enter(); sink_finalize(k); }

int stream_blocks(dlb_ctx *ctx, size_t items) {
  const size_t blocks = (items + 255) / 256;
  return (int)max((size_t)1, min(blocks, (size_t)ctx->sm_count * 16));
}

dlb_status scale_slot(dlb_ctx *ctx, float **out) {
  if (!ctx->scale_pool) {
    DLB_CUDA(cudaMalloc(&ctx->scale_pool, (size_t)SCALE_SLOTS * SLOT_WORDS * sizeof(float)));
    ctx->scale_free.reserve(SCALE_SLOTS);
    for (int i = SCALE_SLOTS - 1; i >= 0; --i) ctx->scale_free.push_back(i);
  }
  if (ctx->scale_free.empty()) {
    set_error("dlb_split_planes: more than %d plane buffers are registered", SCALE_SLOTS);
    return DLB_ERR_INVALID;
  }
  *out = ctx->scale_pool + (size_t)SLOT_WORDS * ctx->scale_free.back();
  ctx->scale_free.pop_back();
  return DLB_OK;
}

dlb_status guard_counters(dlb_ctx *ctx) {
  if (ctx->d_guard) return DLB_OK;
  DLB_CUDA(cudaMalloc(&ctx->d_guard, 4 * sizeof(unsigned long long)));
  DLB_CUDA(cudaMemsetAsync(ctx->d_guard, 0, 4 * sizeof(unsigned long long), ctx->stream));
  return DLB_OK;
}

void release_entry(dlb_ctx *ctx, dlb_ctx::PlaneEntry &e) {
  ctx->scale_free.push_back((int)((e.scale - ctx->scale_pool) / SLOT_WORDS));
  if (e.lines) {
    cudaStreamSynchronize(ctx->stream);  // a check kernel may still read the array
    cudaFree(e.lines);
    e.lines = nullptr;
  }
}

// The split pass of a tensor whose maximum is in its slot (or whose predicted
// scale is to be used): by rows with statistics where the shape allows.
dlb_status launch_split(dlb_ctx *ctx, const float *x, size_t n, int rows, int cols, const PlaneSink &k) {
  const bool by_rows = rows > 0 && cols > 0 && (cols & 3) == 0 && (size_t)rows * cols == n &&
                       ((reinterpret_cast<uintptr_t>(x) & 15) | (reinterpret_cast<uintptr_t>(k.hi) & 7) |
                        (reinterpret_cast<uintptr_t>(k.lo) & 7)) == 0;
  if (by_rows) {
    const int col_blocks = ceil_div(cols, 128);
    int chunks = max(1, min(ceil_div(ctx->sm_count * 8, col_blocks), ceil_div(rows, 2 * SPLIT_LANES_Y)));
    const int rpc = ceil_div(ceil_div(rows, chunks), 2 * SPLIT_LANES_Y) * 2 * SPLIT_LANES_Y;
    chunks = ceil_div(rows, rpc);
    DLB_LAUNCH_KERNEL(ctx, split_rows_kernel, dim3(col_blocks, chunks), 32 * SPLIT_LANES_Y, 0, x, rows, cols, rpc, k);
  } else {
    PlaneSink flat = k;
    flat.rowmax = flat.colmax = flat.lines = nullptr;
    flat.n_lines = flat.n_rows = 0;
    DLB_LAUNCH_KERNEL(ctx, split_flat_kernel, stream_blocks(ctx, n / 4 + 1), 256, 0, x, n, flat);
  }
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // namespace

dlb_status planes_transpose_scaled(dlb_ctx *ctx, const float *x, long long pitch, int K, int M, uint16_t *hi_t,
                                   uint16_t *lo_t, long long kp, unsigned *cmax, float *line_inv) {
  DLB_CUDA(cudaMemsetAsync(cmax, 0, (size_t)M * sizeof(unsigned), ctx->stream));
  const int slabs = max(1, min(ceil_div(K, 64), ceil_div(ctx->sm_count * 8, ceil_div(M, 32))));
  const int rows_per_block = ceil_div(K, slabs);
  DLB_LAUNCH_KERNEL(ctx, column_absmax_kernel, dim3(ceil_div(M, 32), ceil_div(K, rows_per_block)), dim3(32, 8), 0, x, pitch, K, M, rows_per_block, cmax);
  DLB_LAUNCHED(ctx);
  DLB_LAUNCH_KERNEL(ctx, transpose_split_kernel, dim3(ceil_div(M, 32), ceil_div((int)kp, 32)), dim3(32, 8), 0, x, pitch, K, M, cmax, hi_t, lo_t, kp, line_inv);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

void planes_rows_exempt(dlb_ctx *ctx, const float *planes, size_t bytes, bool on) {
  if (!planes) return;
  const uintptr_t key = reinterpret_cast<uintptr_t>(planes);
  if (on && !ctx->guard_strict) ctx->rows_exempt[key] = bytes;
  else ctx->rows_exempt.erase(key);
}

// Whether a plane buffer starting at `key` lies inside a marked one.
static bool rows_exempt_at(const dlb_ctx *ctx, uintptr_t key) {
  auto it = ctx->rows_exempt.upper_bound(key);
  if (it == ctx->rows_exempt.begin()) return false;
  --it;
  return key < it->first + it->second;
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
  o->guard = reinterpret_cast<const unsigned *>(e.scale) + SLOT_FLAGS;
  o->guard_mask = guard_mask_of(*o);
  return true;
}

// Points a sink at the line statistics of a [rows, cols] tensor; the rows of an
// exempt tensor are not recorded at all.
static void sink_lines(PlaneSink &k, unsigned *lines, int rows, int cols, bool exempt) {
  k.lines = lines;
  k.n_rows = lines ? rows : 0;
  k.n_lines = lines ? rows + cols : 0;
  k.rowmax = lines && !exempt ? lines : nullptr;
  k.colmax = lines ? lines + rows : nullptr;
  k.rows_exempt = exempt ? 1 : 0;
}

// Registers `planes` as the plane buffer of x[0..n) with the given shape (0, 0:
// none) and fills the job.  A registration of the same tensor, size and shape
// is kept, with its predicted scale; anything else this buffer overlaps is
// stale and dropped.
dlb_status planes_open(dlb_ctx *ctx, const float *x, float *planes, size_t n, int rows, int cols,
                       bool kernel_can_fuse, PlaneJob *job) {
  DLB_REQUIRE(x && planes && n > 0 && n < ((size_t)1 << 40), "plane buffer: tensor, buffer and size");
  if ((size_t)rows * (size_t)cols != n) rows = cols = 0;
  const uintptr_t key = reinterpret_cast<uintptr_t>(planes);
  planes_forget(ctx, key + 1, n * sizeof(float) - 1);
  auto before = ctx->planes.lower_bound(key);
  if (before != ctx->planes.begin()) {
    --before;
    if (before->first + before->second.n * sizeof(float) > key) planes_forget(ctx, before->first, 1);
  }
  auto it = ctx->planes.find(key);
  if (it != ctx->planes.end() &&
      (it->second.x != x || it->second.n != n || it->second.rows != rows || it->second.cols != cols)) {
    planes_forget(ctx, key, 1);
    it = ctx->planes.end();
  }
  if (it == ctx->planes.end()) {
    dlb_ctx::PlaneEntry e;
    e.x = x;
    e.n = n;
    e.rows = rows;
    e.cols = cols;
    DLB_TRY(scale_slot(ctx, &e.scale));
    DLB_CUDA(cudaMemsetAsync(e.scale, 0, SLOT_WORDS * sizeof(float), ctx->stream));
    if (rows > 0) {
      DLB_CUDA(cudaMalloc(&e.lines, (size_t)(rows + cols) * sizeof(unsigned)));
      DLB_CUDA(cudaMemsetAsync(e.lines, 0, (size_t)(rows + cols) * sizeof(unsigned), ctx->stream));
    }
    it = ctx->planes.emplace(key, e).first;
  }
  dlb_ctx::PlaneEntry &e = it->second;
  static const bool fuse_enabled = [] {
    const char *v = getenv("DLB_PLANES_FUSED");
    return !(v && v[0] == '0');
  }();
  job->x = x;
  job->planes = planes;
  job->n = n;
  job->rows = rows;
  job->cols = cols;
  job->active = true;
  job->fused = kernel_can_fuse && e.seen && fuse_enabled && rows > 0 && (cols & 3) == 0 &&
               (reinterpret_cast<uintptr_t>(planes) & 7) == 0 && ((n * 2) & 7) == 0;
  DLB_TRY(guard_counters(ctx));
  job->sink = PlaneSink{};
  job->sink.slot = e.scale;
  job->sink.guard = ctx->d_guard;
  job->sink.rows_exempt = rows_exempt_at(ctx, key) ? 1 : 0;
  if (job->fused) {
    sink_lines(job->sink, e.lines, rows, cols, job->sink.rows_exempt != 0);
    job->sink.hi = reinterpret_cast<uint16_t *>(planes);
    job->sink.lo = job->sink.hi + n;
    job->sink.predicted = 1;
    job->sink.x = x;
    job->sink.n = n;
  }
  return DLB_OK;
}

dlb_status planes_close(dlb_ctx *ctx, const PlaneJob &job) {
  if (!job.active) return DLB_OK;
  auto it = ctx->planes.find(reinterpret_cast<uintptr_t>(job.planes));
  DLB_REQUIRE(it != ctx->planes.end(), "plane buffer: closed without a registration");
  dlb_ctx::PlaneEntry &e = it->second;
  if (!job.fused) {
    // The producing kernel left the tensor's maximum in the slot: the split pass.
    PlaneSink k;
    k.hi = reinterpret_cast<uint16_t *>(job.planes);
    k.lo = k.hi + job.n;
    k.slot = e.scale;
    sink_lines(k, e.lines, e.rows, e.cols, job.sink.rows_exempt != 0);
    k.predicted = 0;
    k.guard = ctx->d_guard;
    DLB_TRY(launch_split(ctx, job.x, job.n, e.rows, e.cols, k));
  }
  PlaneSink k = job.sink;
  sink_lines(k, e.lines, e.rows, e.cols, job.sink.rows_exempt != 0);
  k.predicted = job.fused ? 1 : 0;
  DLB_LAUNCH_KERNEL(ctx, planes_finalize_kernel, 1, 1024, 0, k);
  DLB_LAUNCHED(ctx);
  e.seen = true;
  return DLB_OK;
}

dlb_status planes_absmax(dlb_ctx *ctx, const float *x, size_t n, float *slot) {
  DLB_LAUNCH_KERNEL(ctx, absmax_kernel, stream_blocks(ctx, n / 4 + 1), 256, 0, x, n, reinterpret_cast<unsigned *>(slot) + SLOT_AMAX);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status planes_split_adhoc(dlb_ctx *ctx, const float *x, size_t n, int rows, int cols, uint16_t *hi,
                              uint16_t *lo, float *slot, unsigned *lines) {
  if ((size_t)rows * (size_t)cols != n) rows = cols = 0;
  DLB_CUDA(cudaMemsetAsync(slot, 0, SLOT_WORDS * sizeof(float), ctx->stream));
  if (rows > 0 && lines) DLB_CUDA(cudaMemsetAsync(lines, 0, (size_t)(rows + cols) * sizeof(unsigned), ctx->stream));
  DLB_TRY(planes_absmax(ctx, x, n, slot));
  DLB_TRY(guard_counters(ctx));
  PlaneSink k;
  k.hi = hi;
  k.lo = lo;
  k.slot = slot;
  sink_lines(k, rows > 0 ? lines : nullptr, rows, cols, false);
  k.guard = ctx->d_guard;
  DLB_TRY(launch_split(ctx, x, n, rows, cols, k));
  DLB_LAUNCH_KERNEL(ctx, planes_finalize_kernel, 1, 1024, 0, k);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

// Drops the entries whose buffer starts inside [base, base + bytes).
void planes_forget(dlb_ctx *ctx, uintptr_t base, size_t bytes) {
  auto it = ctx->planes.lower_bound(base);
  while (it != ctx->planes.end() && it->first < base + bytes) {
    release_entry(ctx, it->second);
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

dlb_status dlb_split_planes_2d(dlb_ctx *ctx, const float *x, float *planes, int rows, int cols) {
  DLB_REQUIRE(ctx && x && planes && rows >= 0 && cols >= 0, "dlb_split_planes_2d");
  const size_t n = (size_t)rows * (size_t)cols;
  if (n == 0) return DLB_OK;
  if (ctx->gemm_kind == DLB_GEMM_TF32X3) return dlb_split_tf32(ctx, x, planes, n);
  PlaneJob job;
  DLB_TRY(planes_open(ctx, x, planes, n, rows, cols, true, &job));
  // With a scale predicted from this buffer's previous split one pass does; the
  // first split takes the tensor's maximum first.
  if (job.fused) DLB_TRY(launch_split(ctx, x, n, rows, cols, job.sink));
  else DLB_TRY(planes_absmax(ctx, x, n, job.sink.slot));
  return planes_close(ctx, job);
}

dlb_status dlb_split_planes(dlb_ctx *ctx, const float *x, float *planes, size_t n) {
  DLB_REQUIRE(ctx && x && planes, "dlb_split_planes: null");
  if (n == 0) return DLB_OK;
  if (ctx->gemm_kind == DLB_GEMM_TF32X3) return dlb_split_tf32(ctx, x, planes, n);
  PlaneJob job;
  DLB_TRY(planes_open(ctx, x, planes, n, 0, 0, false, &job));
  DLB_TRY(planes_absmax(ctx, x, n, job.sink.slot));
  return planes_close(ctx, job);
}

dlb_status dlb_ctx_set_guard_strict(dlb_ctx *ctx, int strict) {
  DLB_REQUIRE(ctx, "dlb_ctx_set_guard_strict: null");
  ctx->guard_strict = strict != 0;
  if (ctx->guard_strict) ctx->rows_exempt.clear();
  return DLB_OK;
}

dlb_status dlb_ctx_guard_resplits(dlb_ctx *ctx, uint64_t *tensors_resplit) {
  DLB_REQUIRE(ctx && tensors_resplit, "dlb_ctx_guard_resplits: null");
  unsigned long long host = 0;
  if (ctx->d_guard) {
    DLB_CUDA(cudaMemcpyAsync(&host, ctx->d_guard + 2, sizeof(host), cudaMemcpyDeviceToHost, ctx->stream));
    DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  *tensors_resplit = host;
  return DLB_OK;
}

dlb_status dlb_ctx_guard_counters(dlb_ctx *ctx, uint64_t *tensors_flagged, uint64_t *products_on_fallback) {
  DLB_REQUIRE(ctx && tensors_flagged && products_on_fallback, "dlb_ctx_guard_counters: null");
  unsigned long long host[2] = {0, 0};
  if (ctx->d_guard) {
    DLB_CUDA(cudaMemcpyAsync(host, ctx->d_guard, sizeof(host), cudaMemcpyDeviceToHost, ctx->stream));
    DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  *tensors_flagged = host[0];
  *products_on_fallback = host[1];
  return DLB_OK;
}

}  // extern "C"
