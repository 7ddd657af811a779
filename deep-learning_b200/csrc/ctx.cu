// Context, device memory helpers, the GEMM dispatcher behind the three FC entry
// points, and the NCCL exchange of libdlb200.
#include <dlfcn.h>
#include <nccl.h>
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace dlb {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

dlb_status scratch(dlb_ctx *ctx, size_t bytes, void **out) {
  if (bytes > ctx->scratch_bytes) {
    // Growing invalidates earlier scratch pointers, so wait for their users.
    DLB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) DLB_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    const size_t want = align_up(bytes + bytes / 4, (size_t)1 << 20);
    DLB_CUDA(cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
  }
  *out = ctx->scratch;
  return DLB_OK;
}

bool gemm_tcgen05_supported(const GemmOperand &, const GemmOperand &, const float *, long long, int,
                            int, int);
dlb_status bias_gradient(dlb_ctx *ctx, const float *delta, int rows, int n, float *dbias,
                         int accumulate);

// Number of elements spanned by an operand stored densely in global memory.
static size_t operand_elems(const GemmOperand &o, int mn, int k) {
  if (o.stride_k == 1) return (size_t)(mn - 1) * o.stride_mn + k;
  return (size_t)(k - 1) * o.stride_k + mn;
}

// A pair of events around one piece of work while per-launch profiling is on.
struct ProfileSpan {
  dlb_ctx *ctx;
  dlb_ctx::GemmRecord rec;
  bool on = false;
  dlb_status begin(dlb_ctx *c, int kind, double flops) {
    ctx = c;
    if (!c->gemm_profile) return DLB_OK;
    cudaEvent_t *ev[2] = {&rec.start, &rec.stop};
    for (cudaEvent_t *e : ev) {
      if (!c->event_pool.empty()) {
        *e = c->event_pool.back();
        c->event_pool.pop_back();
      } else {
        DLB_CUDA(cudaEventCreate(e));
      }
    }
    rec.flops = flops;
    rec.kind = kind;
    DLB_CUDA(cudaEventRecord(rec.start, c->stream));
    on = true;
    return DLB_OK;
  }
  dlb_status end() {
    if (!on) return DLB_OK;
    DLB_CUDA(cudaEventRecord(rec.stop, ctx->stream));
    ctx->gemm_records.push_back(rec);
    return DLB_OK;
  }
};

// Runs the tensor-core kernel, bracketed by a pair of events when per-launch
// profiling is on.
static dlb_status gemm_tensor_core(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                                   long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  ProfileSpan span;
  DLB_TRY(span.begin(ctx, 0, 2.0 * M * N * K));
  const dlb_status st = gemm_tcgen05(ctx, A, B, C, ldc, M, N, K, ep);
  DLB_TRY(span.end());
  return st;
}

// The fused epilogue exists in the 2-CTA fp16-plane kernel at its default
// chunk, for K-major A, with both operands' planes kept by the caller and a
// dense output.
bool gemm_fused_supported(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, const float *C, long long ldc,
                          int M, int N, int K) {
  const bool big = (long long)M * N >= 256 * 256 && K >= 32;
  if (!(ctx->use_tensor_core && ctx->tensor_core_ok && big && ctx->gemm_kind == DLB_GEMM_F16X3)) return false;
  if (!gemm_pair_enabled() || gemm_pair_chunk() != 8 || A.stride_k != 1 || ldc != N) return false;
  if (!gemm_f16_supported(A, B, C, ldc, M, N, K)) return false;
  GemmOperand a = A, b = B;
  return (a.h_hi || planes_lookup(ctx, a.lo, &a)) && (b.h_hi || planes_lookup(ctx, b.lo, &b));
}

dlb_status gemm(dlb_ctx *ctx, const GemmOperand &A_in, const GemmOperand &B_in, float *C,
                long long ldc, int M, int N, int K, const GemmEpilogue &ep) {
  GemmOperand A = A_in, B = B_in;
  if (ep.fused && !gemm_fused_supported(ctx, A, B, C, ldc, M, N, K)) {
    set_error("gemm: fused epilogue asked for a product outside gemm_fused_supported");
    return DLB_ERR_UNSUPPORTED;
  }
  // The tensor-core tile is 128 x 256; below that the CUDA-core kernel is
  // used, as it is for layouts TMA cannot address.
  const bool big = (long long)M * N >= 128 * 64 && K >= 32;
  if (!(ctx->use_tensor_core && ctx->tensor_core_ok && big)) return gemm_simt(ctx, A, B, C, ldc, M, N, K, ep);

  // A weight-gradient product (both operands mn-contiguous) whose A TMA cannot
  // tile as it lies (output rows not a multiple of 64, e.g. 1000 classes), or
  // whose caller asked for a scale per output row (the classes of a softmax
  // error differ by many orders of magnitude: the ones nobody is wrong about
  // have errors 2^-20 and less of the others', and one scale for the tensor
  // would leave their gradient rows with few bits).  A's planes are made for
  // this product in scratch: k contiguous, every line with the scale of its own
  // maximum (two passes over the fp32 tensor, 12 bytes per element), and the
  // product runs on the 2-CTA kernel in the k-contiguous x mn-contiguous form,
  // each output row multiplied by its line's 1 / scale.  Nothing of A is left
  // for the range guard to flag.
  if (ctx->gemm_kind == DLB_GEMM_F16X3 && A.stride_mn == 1 && A.stride_k != 1 && B.stride_mn == 1 &&
      B.stride_k != 1 && gemm_pair_enabled() && (long long)M * N >= 256 * 256 && !ep.fused &&
      (A.rescale_lines || !gemm_f16_supported(A, B, C, ldc, M, N, K))) {
    GemmOperand a = A, b = B;
    const bool have_b = b.h_hi || planes_lookup(ctx, b.lo, &b);
    const long long kp = (long long)align_up((size_t)K, 8);
    if (have_b && a.stride_k >= M) {
      const size_t plane = align_up((size_t)M * kp, 64);
      void *scr = nullptr;
      DLB_TRY(scratch(ctx, 2 * plane * sizeof(uint16_t) + 2 * (size_t)M * sizeof(float), &scr));
      uint16_t *hi_t = static_cast<uint16_t *>(scr), *lo_t = hi_t + plane;
      unsigned *cmax = reinterpret_cast<unsigned *>(lo_t + plane);
      float *line_inv = reinterpret_cast<float *>(cmax + M);
      a.fp32_stride_mn = a.stride_mn;
      a.fp32_stride_k = a.stride_k;
      a.h_hi = hi_t;
      a.h_lo = lo_t;
      a.stride_mn = kp;
      a.stride_k = 1;
      a.scale = line_inv;  // not read
      a.line_inv = line_inv;
      a.guard = nullptr;
      if (gemm_f16_supported(a, b, C, ldc, M, N, K)) {
        DLB_TRY(planes_transpose_scaled(ctx, A.ptr, A.stride_k, K, M, hi_t, lo_t, kp, cmax, line_inv));
        A = a;
        B = b;
      }
    }
  }

  if (ctx->gemm_kind == DLB_GEMM_F16X3 && gemm_f16_supported(A, B, C, ldc, M, N, K)) {
    // fp16 planes: the caller's registered plane buffers, or planes derived
    // into scratch for this call.
    const bool a_have = A.h_hi || planes_lookup(ctx, A.lo, &A);
    const bool b_have = B.h_hi || planes_lookup(ctx, B.lo, &B);
    const size_t a_n = a_have ? 0 : align_up(operand_elems(A, M, K), 64);
    const size_t b_n = b_have ? 0 : align_up(operand_elems(B, N, K), 64);
    if (a_n + b_n) {
      // Behind the planes: two scale slots, then the line maxima of the dense
      // operands ([M + K] and [N + K] words).
      const size_t line_words = align_up((size_t)M + K, 4) + align_up((size_t)N + K, 4);
      void *scr = nullptr;
      DLB_TRY(scratch(ctx, (a_n + b_n) * 2 * sizeof(uint16_t) + (2 * SLOT_WORDS + line_words) * 4 + 64, &scr));
      uint16_t *h = static_cast<uint16_t *>(scr);
      float *slots = reinterpret_cast<float *>(h + 2 * (a_n + b_n));
      unsigned *lines = reinterpret_cast<unsigned *>(slots + 2 * SLOT_WORDS);
      // A dense operand is a [mn, k] (k contiguous) or [k, mn] (mn contiguous) matrix.
      auto shape = [](const GemmOperand &o, int mn, int k, int *rows, int *cols) {
        *rows = *cols = 0;
        if (o.stride_k == 1 && o.stride_mn == k) { *rows = mn; *cols = k; }
        else if (o.stride_mn == 1 && o.stride_k == mn) { *rows = k; *cols = mn; }
      };
      if (!a_have) {
        int r, c;
        shape(A, M, K, &r, &c);
        DLB_TRY(planes_split_adhoc(ctx, A.ptr, operand_elems(A, M, K), r, c, h, h + a_n, slots, lines));
        A.h_hi = h;
        A.h_lo = h + a_n;
        A.scale = slots;
        A.guard = reinterpret_cast<const unsigned *>(slots) + 3;
        A.guard_mask = guard_mask_of(A);
      }
      if (!b_have) {
        uint16_t *hb = h + 2 * a_n;
        int r, c;
        shape(B, N, K, &r, &c);
        DLB_TRY(planes_split_adhoc(ctx, B.ptr, operand_elems(B, N, K), r, c, hb, hb + b_n, slots + SLOT_WORDS,
                                   lines + align_up((size_t)M + K, 4)));
        B.h_hi = hb;
        B.h_lo = hb + b_n;
        B.scale = slots + SLOT_WORDS;
        B.guard = reinterpret_cast<const unsigned *>(slots + SLOT_WORDS) + 3;
        B.guard_mask = guard_mask_of(B);
      }
    }
    // A product with an operand the range guard flagged is computed by the
    // same launch on the CUDA cores, from the fp32 tensors.
    return gemm_tensor_core(ctx, A, B, C, ldc, M, N, K, ep);
  }

  if (gemm_tcgen05_supported(A, B, C, ldc, M, N, K)) {
    // TF32 residual planes the caller did not keep are derived into scratch.
    // Under the fp16 form a caller's plane buffer does not hold them.
    A.h_hi = A.h_lo = B.h_hi = B.h_lo = nullptr;
    if (ctx->gemm_kind != DLB_GEMM_TF32X3) A.lo = B.lo = nullptr;
    const size_t a_n = A.lo ? 0 : align_up(operand_elems(A, M, K), 64);
    const size_t b_n = B.lo ? 0 : align_up(operand_elems(B, N, K), 64);
    if (a_n + b_n) {
      void *scr = nullptr;
      DLB_TRY(scratch(ctx, (a_n + b_n) * sizeof(float), &scr));
      float *s = static_cast<float *>(scr);
      if (!A.lo) {
        DLB_TRY(dlb_split_tf32(ctx, A.ptr, s, operand_elems(A, M, K)));
        A.lo = s;
      }
      if (!B.lo) {
        DLB_TRY(dlb_split_tf32(ctx, B.ptr, s + a_n, operand_elems(B, N, K)));
        B.lo = s + a_n;
      }
    }
    return gemm_tensor_core(ctx, A, B, C, ldc, M, N, K, ep);
  }
  return gemm_simt(ctx, A, B, C, ldc, M, N, K, ep);
}

// ---- NCCL through dlopen: the library is only needed by multi-GPU runs ------
struct Nccl {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                                cudaStream_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static Nccl *nccl() {
  static Nccl n;
  static bool tried = false;
  if (!tried) {
    tried = true;
    n.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!n.handle) n.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (n.handle) {
      n.GetUniqueId = (decltype(n.GetUniqueId))dlsym(n.handle, "ncclGetUniqueId");
      n.CommInitRank = (decltype(n.CommInitRank))dlsym(n.handle, "ncclCommInitRank");
      n.CommDestroy = (decltype(n.CommDestroy))dlsym(n.handle, "ncclCommDestroy");
      n.AllReduce = (decltype(n.AllReduce))dlsym(n.handle, "ncclAllReduce");
      n.AllGather = (decltype(n.AllGather))dlsym(n.handle, "ncclAllGather");
      n.ReduceScatter = (decltype(n.ReduceScatter))dlsym(n.handle, "ncclReduceScatter");
      n.GetErrorString = (decltype(n.GetErrorString))dlsym(n.handle, "ncclGetErrorString");
    }
  }
  if (!n.handle || !n.GetUniqueId || !n.CommInitRank || !n.AllReduce) return nullptr;
  return &n;
}

#define DLB_NCCL(call)                                                              \
  do {                                                                              \
    ncclResult_t r__ = (call);                                                      \
    if (r__ != ncclSuccess) {                                                       \
      dlb::set_error("%s:%d %s: %s", __FILE__, __LINE__, #call,                     \
                     nccl()->GetErrorString ? nccl()->GetErrorString(r__) : "nccl"); \
      return DLB_ERR_COMM;                                                          \
    }                                                                               \
  } while (0)

}  // namespace dlb

namespace dlb {

dlb_status comm_allgather_host(dlb_ctx *ctx, const void *mine, void *all, size_t bytes) {
  if (!nccl()->AllGather) {
    set_error("comm_allgather_host: the NCCL library has no ncclAllGather");
    return DLB_ERR_COMM;
  }
  char *dev = nullptr;
  DLB_CUDA(cudaMalloc(&dev, bytes * (size_t)(ctx->world + 1)));
  dlb_status st = DLB_OK;
  cudaError_t e = cudaMemcpyAsync(dev, mine, bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) {
    ncclResult_t r = nccl()->AllGather(dev, dev + bytes, bytes, ncclChar, ctx->comm, ctx->stream);
    if (r != ncclSuccess) {
      set_error("comm_allgather_host: %s", nccl()->GetErrorString ? nccl()->GetErrorString(r) : "nccl");
      st = DLB_ERR_COMM;
    }
  }
  if (e == cudaSuccess && st == DLB_OK)
    e = cudaMemcpyAsync(all, dev + bytes, bytes * (size_t)ctx->world, cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFree(dev);
  if (e != cudaSuccess) {
    set_error("comm_allgather_host: %s", cudaGetErrorString(e));
    return DLB_ERR_CUDA;
  }
  return st;
}

dlb_status comm_min_int(dlb_ctx *ctx, int *value) {
  int *dev = nullptr;
  DLB_CUDA(cudaMalloc(&dev, sizeof(int)));
  dlb_status st = DLB_OK;
  cudaError_t e = cudaMemcpyAsync(dev, value, sizeof(int), cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) {
    ncclResult_t r = nccl()->AllReduce(dev, dev, 1, ncclInt32, ncclMin, ctx->comm, ctx->stream);
    if (r != ncclSuccess) {
      set_error("comm_min_int: %s", nccl()->GetErrorString ? nccl()->GetErrorString(r) : "nccl");
      st = DLB_ERR_COMM;
    }
  }
  if (e == cudaSuccess && st == DLB_OK)
    e = cudaMemcpyAsync(value, dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  cudaFree(dev);
  if (e != cudaSuccess) {
    set_error("comm_min_int: %s", cudaGetErrorString(e));
    return DLB_ERR_CUDA;
  }
  return st;
}

}  // namespace dlb

using namespace dlb;

extern "C" {

const char *dlb_status_string(dlb_status s) {
  switch (s) {
    case DLB_OK: return "ok";
    case DLB_ERR_INVALID: return "invalid argument";
    case DLB_ERR_CUDA: return "CUDA error";
    case DLB_ERR_UNSUPPORTED: return "outside the supported path";
    case DLB_ERR_TIMEOUT: return "device-side wait timed out";
    case DLB_ERR_COMM: return "NCCL error";
    case DLB_ERR_NO_DEVICE: return "no sm_100 CUDA device (this library has no CPU path)";
    default: return "unknown status";
  }
}

const char *dlb_last_error(void) { return g_error; }

int dlb_version(void) { return 100; }

dlb_status dlb_ctx_create(dlb_ctx **out, int device) {
  DLB_REQUIRE(out, "dlb_ctx_create: null");
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0 || device < 0 || device >= count) {
    cudaGetLastError();
    set_error("dlb_ctx_create: CUDA device %d is not available (%d devices); libdlb200 has no CPU path",
              device, count);
    return DLB_ERR_NO_DEVICE;
  }
  cudaDeviceProp prop;
  DLB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    set_error("dlb_ctx_create: device %d is sm_%d%d; the kernels are built for sm_100a only", device,
              prop.major, prop.minor);
    return DLB_ERR_NO_DEVICE;
  }
  DLB_CUDA(cudaSetDevice(device));
  dlb_ctx *ctx = new dlb_ctx;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->tensor_core_ok = true;
  if (const char *e = getenv("DLB_TENSOR_CORE")) ctx->use_tensor_core = atoi(e) != 0;
  if (const char *e = getenv("DLB_GUARD_STRICT")) ctx->guard_strict = atoi(e) != 0;
  if (const char *e = getenv("DLB_GEMM_RESERVE_SMS")) ctx->gemm_reserve_sms = max(0, min(atoi(e), prop.multiProcessorCount - 1));
  if (const char *e = getenv("DLB_PDL")) ctx->use_pdl = atoi(e) != 0;
  if (const char *e = getenv("DLB_GEMM_KIND")) ctx->gemm_kind = e[0] == 't' ? DLB_GEMM_TF32X3 : DLB_GEMM_F16X3;
  cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&ctx->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, sizeof(int));
  if (e != cudaSuccess) {
    set_error("dlb_ctx_create: %s", cudaGetErrorString(e));
    delete ctx;
    return DLB_ERR_CUDA;
  }
  *out = ctx;
  return DLB_OK;
}

dlb_status dlb_ctx_destroy(dlb_ctx *ctx) {
  if (!ctx) return DLB_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->comm_stream) cudaStreamSynchronize(ctx->comm_stream);
  peer_teardown(ctx);
  if (ctx->comm && nccl() && nccl()->CommDestroy) nccl()->CommDestroy(ctx->comm);
  if (ctx->comm_stream) cudaStreamDestroy(ctx->comm_stream);
  if (ctx->ev_main) cudaEventDestroy(ctx->ev_main);
  if (ctx->ev_comm) cudaEventDestroy(ctx->ev_comm);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->d_status) cudaFree(ctx->d_status);
  planes_forget(ctx, 0, ~(size_t)0);
  if (ctx->scale_pool) cudaFree(ctx->scale_pool);
  if (ctx->d_guard) cudaFree(ctx->d_guard);
  if (ctx->timer_start) cudaEventDestroy(ctx->timer_start);
  if (ctx->timer_stop) cudaEventDestroy(ctx->timer_stop);
  for (auto &r : ctx->gemm_records) {
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return DLB_OK;
}

dlb_status dlb_ctx_sync(dlb_ctx *ctx, int *device_status) {
  DLB_REQUIRE(ctx, "dlb_ctx_sync: null");
  int st = 0;
  DLB_CUDA(cudaMemcpyAsync(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  if (device_status) *device_status = st;
  if (st != DLB_OK) {
    set_error("a kernel reported device status %d (%s)", st, dlb_status_string(st));
    return st;
  }
  return DLB_OK;
}

void *dlb_ctx_stream(dlb_ctx *ctx) { return ctx ? ctx->stream : nullptr; }

dlb_status dlb_ctx_set_tensor_core(dlb_ctx *ctx, int enable) {
  DLB_REQUIRE(ctx, "dlb_ctx_set_tensor_core: null");
  ctx->use_tensor_core = enable != 0;
  return DLB_OK;
}

uint64_t dlb_ctx_launch_count(dlb_ctx *ctx) { return ctx ? ctx->launches : 0; }

dlb_status dlb_ctx_timer_start(dlb_ctx *ctx) {
  DLB_REQUIRE(ctx, "dlb_ctx_timer_start: null");
  if (!ctx->timer_start) {
    DLB_CUDA(cudaEventCreate(&ctx->timer_start));
    DLB_CUDA(cudaEventCreate(&ctx->timer_stop));
  }
  DLB_CUDA(cudaEventRecord(ctx->timer_start, ctx->stream));
  return DLB_OK;
}

dlb_status dlb_ctx_timer_stop(dlb_ctx *ctx, float *milliseconds) {
  DLB_REQUIRE(ctx && milliseconds && ctx->timer_start, "dlb_ctx_timer_stop: no timer running");
  DLB_CUDA(cudaEventRecord(ctx->timer_stop, ctx->stream));
  DLB_CUDA(cudaEventSynchronize(ctx->timer_stop));
  DLB_CUDA(cudaEventElapsedTime(milliseconds, ctx->timer_start, ctx->timer_stop));
  return DLB_OK;
}

dlb_status dlb_ctx_gemm_profile(dlb_ctx *ctx, int enable) {
  DLB_REQUIRE(ctx, "dlb_ctx_gemm_profile: null");
  ctx->gemm_profile = enable != 0;
  return DLB_OK;
}

dlb_status dlb_ctx_gemm_profile_read(dlb_ctx *ctx, uint64_t *launches, double *milliseconds,
                                     double *flops) {
  DLB_REQUIRE(ctx && launches && milliseconds && flops, "dlb_ctx_gemm_profile_read: null");
  DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  *launches = 0;
  *milliseconds = 0.0;
  *flops = 0.0;
  ctx->join_wait_ms = ctx->exchange_ms = 0.0;
  ctx->join_waits = ctx->exchanges = 0;
  for (auto &r : ctx->gemm_records) {
    float ms = 0.f;
    DLB_CUDA(cudaEventElapsedTime(&ms, r.start, r.stop));
    if (r.kind == 1) {
      ctx->join_wait_ms += ms;
      ctx->join_waits += 1;
    } else if (r.kind == 2) {
      ctx->exchange_ms += ms;
      ctx->exchanges += 1;
    } else {
      *milliseconds += ms;
      *flops += r.flops;
      *launches += 1;
    }
    ctx->event_pool.push_back(r.start);
    ctx->event_pool.push_back(r.stop);
  }
  ctx->gemm_records.clear();
  return DLB_OK;
}

dlb_status dlb_ctx_comm_profile_read(dlb_ctx *ctx, uint64_t *join_waits, double *join_wait_ms,
                                     uint64_t *exchanges, double *exchange_ms) {
  DLB_REQUIRE(ctx && join_waits && join_wait_ms && exchanges && exchange_ms, "dlb_ctx_comm_profile_read: null");
  *join_waits = ctx->join_waits;
  *join_wait_ms = ctx->join_wait_ms;
  *exchanges = ctx->exchanges;
  *exchange_ms = ctx->exchange_ms;
  return DLB_OK;
}

dlb_status dlb_malloc(dlb_ctx *ctx, void **dev_ptr, size_t bytes) {
  DLB_REQUIRE(ctx && dev_ptr, "dlb_malloc: null");
  DLB_CUDA(cudaSetDevice(ctx->device));
  DLB_CUDA(cudaMalloc(dev_ptr, bytes ? bytes : 16));
  ctx->allocs[reinterpret_cast<uintptr_t>(*dev_ptr)] = bytes ? bytes : 16;
  return DLB_OK;
}

dlb_status dlb_free(dlb_ctx *ctx, void *dev_ptr) {
  DLB_REQUIRE(ctx, "dlb_free: null");
  if (!dev_ptr) return DLB_OK;
  DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  auto it = ctx->allocs.find(reinterpret_cast<uintptr_t>(dev_ptr));
  if (it != ctx->allocs.end()) {
    planes_forget(ctx, it->first, it->second);
    ctx->allocs.erase(it);
  }
  DLB_CUDA(cudaFree(dev_ptr));
  return DLB_OK;
}

dlb_status dlb_memset(dlb_ctx *ctx, void *dev_ptr, int value, size_t bytes) {
  DLB_REQUIRE(ctx && dev_ptr, "dlb_memset: null");
  DLB_CUDA(cudaMemsetAsync(dev_ptr, value, bytes, ctx->stream));
  return DLB_OK;
}

dlb_status dlb_memcpy_h2d(dlb_ctx *ctx, void *dev_dst, const void *host_src, size_t bytes) {
  DLB_REQUIRE(ctx && dev_dst && host_src, "dlb_memcpy_h2d: null");
  DLB_CUDA(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return DLB_OK;
}

dlb_status dlb_memcpy_d2h(dlb_ctx *ctx, void *host_dst, const void *dev_src, size_t bytes) {
  DLB_REQUIRE(ctx && host_dst && dev_src, "dlb_memcpy_d2h: null");
  DLB_CUDA(cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  DLB_CUDA(cudaStreamSynchronize(ctx->stream));
  return DLB_OK;
}

dlb_status dlb_memcpy_d2d(dlb_ctx *ctx, void *dev_dst, const void *dev_src, size_t bytes) {
  DLB_REQUIRE(ctx && dev_dst && dev_src, "dlb_memcpy_d2d: null");
  DLB_CUDA(cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return DLB_OK;
}

dlb_status dlb_device_mem_info(size_t *free_bytes, size_t *total_bytes) {
  DLB_REQUIRE(free_bytes && total_bytes, "dlb_device_mem_info: null");
  DLB_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
  return DLB_OK;
}

dlb_status dlb_host_alloc(void **host_ptr, size_t bytes) {
  DLB_REQUIRE(host_ptr, "dlb_host_alloc: null");
  DLB_CUDA(cudaMallocHost(host_ptr, bytes ? bytes : 16));
  return DLB_OK;
}

dlb_status dlb_host_free(void *host_ptr) {
  if (host_ptr) DLB_CUDA(cudaFreeHost(host_ptr));
  return DLB_OK;
}

// ---- FC products --------------------------------------------------------------

dlb_status dlb_fc_forward(dlb_ctx *ctx, const float *X, const float *X_lo, const float *W,
                          const float *W_lo, const float *bias, float *Z, int rows, int n_in,
                          int n_out) {
  DLB_REQUIRE(ctx && X && W && Z && rows > 0 && n_in > 0 && n_out > 0, "dlb_fc_forward");
  GemmOperand A{X, X_lo, n_in, 1};   // (m=b, k=i)
  GemmOperand B{W, W_lo, n_in, 1};   // (n=o, k=i)
  GemmEpilogue ep;
  ep.bias = bias;
  return gemm(ctx, A, B, Z, n_out, rows, n_out, n_in, ep);
}

dlb_status dlb_fc_backward_input(dlb_ctx *ctx, const float *delta, const float *delta_lo,
                                 const float *W, const float *W_lo, float *dX, int rows,
                                 int n_in, int n_out) {
  DLB_REQUIRE(ctx && delta && W && dX && rows > 0 && n_in > 0 && n_out > 0,
              "dlb_fc_backward_input");
  GemmOperand A{delta, delta_lo, n_out, 1};  // (m=b, k=o)
  GemmOperand B{W, W_lo, 1, n_in};           // (n=i, k=o): W[o,i]
  GemmEpilogue ep;
  return gemm(ctx, A, B, dX, n_in, rows, n_in, n_out, ep);
}

// Dropout of the fused forward: what the epilogue can apply (flags per unit, a
// factor, UOut draws).
static bool epilogue_dropout(const dlb_dropout_desc *d, FusedEpilogue *fe) {
  if (!d || d->type == DLB_DROPOUT_NONE) return true;
  switch (d->type) {
    case DLB_DROPOUT_BERNOULLI:
      if (!d->mask) return false;
      fe->mask = d->mask;
      return true;
    case DLB_DROPOUT_BERNOULLI_INVERTED:
      if (!d->mask || !(d->value > 0.f)) return false;
      fe->mask = d->mask;
      fe->keep_scale = 1.f / d->value;
      return true;
    case DLB_DROPOUT_UOUT:
      if (!d->noise) return false;
      fe->noise = d->noise;
      return true;
    default: return false;
  }
}

dlb_status dlb_fc_forward_activation(dlb_ctx *ctx, const float *X, const float *X_lo, const float *W,
                                     const float *W_lo, const float *bias, float *Z, int af,
                                     const dlb_dropout_desc *dropout, float *A_out, float *A_lo, int rows,
                                     int n_in, int n_out) {
  DLB_REQUIRE(ctx && X && W && Z && A_out && rows > 0 && n_in > 0 && n_out > 0, "dlb_fc_forward_activation");
  GemmOperand A{X, X_lo, n_in, 1};
  GemmOperand B{W, W_lo, n_in, 1};
  FusedEpilogue fe;
  fe.mode = EPI_ACTIVATION;
  fe.af = af;
  fe.out = A_out;
  if (A_lo && epilogue_dropout(dropout, &fe) && gemm_fused_supported(ctx, A, B, Z, n_out, rows, n_out, n_in)) {
    PlaneJob job;
    DLB_TRY(planes_open(ctx, A_out, A_lo, (size_t)rows * n_out, rows, n_out, true, &job));
    if (job.fused) {
      fe.sink = job.sink;
      GemmEpilogue ep;
      ep.bias = bias;
      ep.fused = &fe;
      DLB_TRY(gemm(ctx, A, B, Z, n_out, rows, n_out, n_in, ep));
      return planes_close(ctx, job);
    }
    // No scale to predict from yet (the buffer's first split): the two kernels below.
  }
  DLB_TRY(dlb_fc_forward(ctx, X, X_lo, W, W_lo, bias, Z, rows, n_in, n_out));
  return dlb_activation_forward(ctx, Z, nullptr, af, dropout, A_out, A_lo, rows, n_out);
}

dlb_status dlb_fc_backward_input_derivative(dlb_ctx *ctx, const float *delta, const float *delta_lo,
                                            const float *W, const float *W_lo, const float *Z_below,
                                            const float *A_below, int af_below, float *dX, float *dX_lo,
                                            int rows, int n_in, int n_out) {
  DLB_REQUIRE(ctx && delta && W && Z_below && A_below && dX && rows > 0 && n_in > 0 && n_out > 0,
              "dlb_fc_backward_input_derivative");
  GemmOperand A{delta, delta_lo, n_out, 1};
  GemmOperand B{W, W_lo, 1, n_in};
  if (dX_lo && gemm_fused_supported(ctx, A, B, dX, n_in, rows, n_in, n_out)) {
    PlaneJob job;
    DLB_TRY(planes_open(ctx, dX, dX_lo, (size_t)rows * n_in, rows, n_in, true, &job));
    if (job.fused) {
      FusedEpilogue fe;
      fe.mode = EPI_DERIVATIVE;
      fe.af = af_below;
      fe.z = Z_below;
      fe.a = A_below;
      fe.sink = job.sink;
      GemmEpilogue ep;
      ep.fused = &fe;
      DLB_TRY(gemm(ctx, A, B, dX, n_in, rows, n_in, n_out, ep));
      return planes_close(ctx, job);
    }
  }
  DLB_TRY(dlb_fc_backward_input(ctx, delta, delta_lo, W, W_lo, dX, rows, n_in, n_out));
  DLB_TRY(dlb_activation_backward(ctx, dX, Z_below, A_below, nullptr, af_below, rows, n_in, nullptr));
  if (dX_lo) DLB_TRY(dlb_split_planes_2d(ctx, dX, dX_lo, rows, n_in));
  return DLB_OK;
}

dlb_status dlb_fc_weight_gradient(dlb_ctx *ctx, const float *delta, const float *delta_lo,
                                  const float *X, const float *X_lo, float *dW, float *dbias,
                                  int rows, int n_in, int n_out, int accumulate) {
  return fc_weight_gradient_lines(ctx, delta, delta_lo, X, X_lo, dW, dbias, rows, n_in, n_out, accumulate, false);
}

}  // extern "C"

dlb_status dlb::fc_weight_gradient_lines(dlb_ctx *ctx, const float *delta, const float *delta_lo, const float *X,
                                         const float *X_lo, float *dW, float *dbias, int rows, int n_in, int n_out,
                                         int accumulate, bool rescale_lines) {
  DLB_REQUIRE(ctx && delta && X && dW && rows > 0 && n_in > 0 && n_out > 0,
              "dlb_fc_weight_gradient");
  GemmOperand A{delta, delta_lo, 1, n_out};  // (m=o, k=b): delta[b,o]
  GemmOperand B{X, X_lo, 1, n_in};           // (n=i, k=b): X[b,i]
  A.rescale_lines = rescale_lines;
  GemmEpilogue ep;
  ep.accumulate = accumulate;
  DLB_TRY(gemm(ctx, A, B, dW, n_in, n_out, n_in, rows, ep));
  if (dbias) DLB_TRY(bias_gradient(ctx, delta, rows, n_out, dbias, accumulate));
  return DLB_OK;
}

extern "C" {

// ---- NCCL -----------------------------------------------------------------------


dlb_status dlb_comm_unique_id(char out_id[128]) {
  DLB_REQUIRE(out_id, "dlb_comm_unique_id: null");
  if (!nccl()) {
    set_error("dlb_comm_unique_id: libnccl.so.2 could not be loaded");
    return DLB_ERR_COMM;
  }
  ncclUniqueId id;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  DLB_NCCL(nccl()->GetUniqueId(&id));
  memcpy(out_id, &id, 128);
  return DLB_OK;
}

dlb_status dlb_comm_init(dlb_ctx *ctx, const char id[128], int rank, int world) {
  DLB_REQUIRE(ctx && id && world >= 1 && rank >= 0 && rank < world, "dlb_comm_init");
  if (!nccl()) {
    set_error("dlb_comm_init: libnccl.so.2 could not be loaded");
    return DLB_ERR_COMM;
  }
  DLB_CUDA(cudaSetDevice(ctx->device));
  ncclUniqueId uid;
  memcpy(&uid, id, 128);
  DLB_NCCL(nccl()->CommInitRank(&ctx->comm, world, uid, rank));
  ctx->rank = rank;
  ctx->world = world;
  return peer_setup(ctx);
}

int dlb_comm_world(dlb_ctx *ctx) { return ctx ? ctx->world : 1; }
int dlb_comm_rank(dlb_ctx *ctx) { return ctx ? ctx->rank : 0; }

dlb_status dlb_allreduce_f32(dlb_ctx *ctx, float *buf, size_t n) {
  DLB_REQUIRE(ctx && (buf || n == 0), "dlb_allreduce_f32");
  if (!ctx->comm || ctx->world == 1 || n == 0) return DLB_OK;
  DLB_NCCL(nccl()->AllReduce(buf, buf, n, ncclFloat32, ncclSum, ctx->comm, ctx->stream));
  return DLB_OK;
}

dlb_status dlb_allreduce_f32_overlapped(dlb_ctx *ctx, float *buf, size_t n) {
  DLB_REQUIRE(ctx && (buf || n == 0), "dlb_allreduce_f32_overlapped");
  if (!ctx->comm || ctx->world == 1 || n == 0) return DLB_OK;
  if (!ctx->comm_stream) {
    DLB_CUDA(cudaStreamCreateWithFlags(&ctx->comm_stream, cudaStreamNonBlocking));
    DLB_CUDA(cudaEventCreateWithFlags(&ctx->ev_main, cudaEventDisableTiming));
    DLB_CUDA(cudaEventCreateWithFlags(&ctx->ev_comm, cudaEventDisableTiming));
  }
  DLB_CUDA(cudaEventRecord(ctx->ev_main, ctx->stream));
  DLB_CUDA(cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_main, 0));
  DLB_NCCL(nccl()->AllReduce(buf, buf, n, ncclFloat32, ncclSum, ctx->comm, ctx->comm_stream));
  ctx->comm_pending = true;
  return DLB_OK;
}

}  // extern "C"

// ---- owner-computes update: the pieces of one weight matrix -----------------
static dlb_status comm_stream_ready(dlb_ctx *ctx) {
  if (ctx->comm_stream) return DLB_OK;
  DLB_CUDA(cudaStreamCreateWithFlags(&ctx->comm_stream, cudaStreamNonBlocking));
  DLB_CUDA(cudaEventCreateWithFlags(&ctx->ev_main, cudaEventDisableTiming));
  DLB_CUDA(cudaEventCreateWithFlags(&ctx->ev_comm, cudaEventDisableTiming));
  return DLB_OK;
}

static dlb_status comm_mark(dlb_ctx *ctx, cudaEvent_t *done) {
  if (!*done) DLB_CUDA(cudaEventCreateWithFlags(done, cudaEventDisableTiming));
  DLB_CUDA(cudaEventRecord(*done, ctx->comm_stream));
  ctx->comm_pending = true;
  return DLB_OK;
}

bool dlb::comm_can_shard(dlb_ctx *ctx) {
  return ctx->comm && ctx->world > 1 && nccl() && nccl()->ReduceScatter && nccl()->AllGather;
}

dlb_status dlb::comm_reduce_scatter_begin(dlb_ctx *ctx, float *buf, size_t per_rank, cudaEvent_t *done) {
  DLB_REQUIRE(comm_can_shard(ctx) && buf && per_rank > 0 && done, "comm_reduce_scatter_begin");
  DLB_TRY(comm_stream_ready(ctx));
  DLB_CUDA(cudaEventRecord(ctx->ev_main, ctx->stream));
  DLB_CUDA(cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_main, 0));
  DLB_NCCL(nccl()->ReduceScatter(buf, buf + (size_t)ctx->rank * per_rank, per_rank, ncclFloat32, ncclSum, ctx->comm,
                                 ctx->comm_stream));
  return comm_mark(ctx, done);
}

dlb_status dlb::comm_all_gather_begin(dlb_ctx *ctx, float *buf, size_t per_rank, float *clear, cudaEvent_t *done) {
  DLB_REQUIRE(comm_can_shard(ctx) && buf && per_rank > 0 && done, "comm_all_gather_begin");
  DLB_TRY(comm_stream_ready(ctx));
  DLB_CUDA(cudaEventRecord(ctx->ev_main, ctx->stream));
  DLB_CUDA(cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_main, 0));
  DLB_NCCL(nccl()->AllGather(buf + (size_t)ctx->rank * per_rank, buf, per_rank, ncclFloat32, ctx->comm,
                             ctx->comm_stream));
  if (clear) {
    const size_t before = (size_t)ctx->rank * per_rank, after = (size_t)(ctx->world - ctx->rank - 1) * per_rank;
    if (before) DLB_CUDA(cudaMemsetAsync(clear, 0, before * sizeof(float), ctx->comm_stream));
    if (after) DLB_CUDA(cudaMemsetAsync(clear + before + per_rank, 0, after * sizeof(float), ctx->comm_stream));
  }
  return comm_mark(ctx, done);
}

dlb_status dlb::comm_wait(dlb_ctx *ctx, cudaEvent_t done) {
  DLB_REQUIRE(ctx && done, "comm_wait");
  ProfileSpan span;  // counted with the time the main stream stands still for transfers
  DLB_TRY(span.begin(ctx, 1, 0.0));
  DLB_CUDA(cudaStreamWaitEvent(ctx->stream, done, 0));
  return span.end();
}

dlb_status dlb::comm_all_gather(dlb_ctx *ctx, float *buf, size_t per_rank) {
  DLB_REQUIRE(comm_can_shard(ctx) && buf && per_rank > 0, "comm_all_gather");
  DLB_NCCL(nccl()->AllGather(buf + (size_t)ctx->rank * per_rank, buf, per_rank, ncclFloat32, ctx->comm, ctx->stream));
  return DLB_OK;
}

extern "C" {

dlb_status dlb_comm_join(dlb_ctx *ctx) {
  DLB_REQUIRE(ctx, "dlb_comm_join");
  if (!ctx->comm_pending) return DLB_OK;
  DLB_CUDA(cudaEventRecord(ctx->ev_comm, ctx->comm_stream));
  ProfileSpan span;  // how long the main stream stands still for the transfers
  DLB_TRY(span.begin(ctx, 1, 0.0));
  DLB_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_comm, 0));
  DLB_TRY(span.end());
  ctx->comm_pending = false;
  return DLB_OK;
}

dlb_status dlb_allreduce_f64(dlb_ctx *ctx, double *buf, size_t n) {
  DLB_REQUIRE(ctx && (buf || n == 0), "dlb_allreduce_f64");
  if (!ctx->comm || ctx->world == 1 || n == 0) return DLB_OK;
  ProfileSpan span;
  DLB_TRY(span.begin(ctx, 2, 0.0));
  if (peer_exchange_fits(ctx, n)) {
    DLB_TRY(peer_exchange_f64(ctx, buf, n));
  } else {
    DLB_NCCL(nccl()->AllReduce(buf, buf, n, ncclFloat64, ncclSum, ctx->comm, ctx->stream));
  }
  return span.end();
}

}  // extern "C"
