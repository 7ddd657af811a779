// Internal definitions shared by the kernels and the C ABI of libdlb200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <map>
#include <vector>

#include "dlb200.h"

typedef struct ncclComm *ncclComm_t;

struct dlb_ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  int *d_status = nullptr;      // sticky device status word
  void *scratch = nullptr;      // arena for reduction partials / residual planes
  size_t scratch_bytes = 0;
  ncclComm_t comm = nullptr;
  int rank = 0;
  int world = 1;
  cudaStream_t comm_stream = nullptr;   // overlapped gradient all-reduces
  cudaEvent_t ev_main = nullptr, ev_comm = nullptr;
  bool comm_pending = false;
  bool use_tensor_core = true;
  bool tensor_core_ok = false;  // device is sm_100
  // Operand form of the tensor-core products: DLB_GEMM_TF32X3 or DLB_GEMM_F16X3.
  int gemm_kind = DLB_GEMM_F16X3;
  // SMs the persistent GEMM leaves free while a communicator is bound
  // (DLB_GEMM_RESERVE_SMS), so that an overlapped all-reduce can run beside it.
  int gemm_reserve_sms = 8;
  // fp16 plane buffers, keyed by the buffer's address: the tensor they were
  // split from, its element count (the lo plane starts n halfs after the hi
  // plane), its shape when the producer gave one, the device slot of its scale
  // and flags, and the per-row / per-column maxima the producers leave for the
  // range check (rows + cols words, zero between uses).
  struct PlaneEntry {
    const float *x;
    size_t n;
    float *scale;
    int rows = 0, cols = 0;
    unsigned *lines = nullptr;  // [rows] row maxima, then [cols] column maxima (raw bits of |x|)
    bool seen = false;          // a split has completed: the slot holds a scale predicted for the next one
  };
  std::map<uintptr_t, PlaneEntry> planes;
  bool guard_strict = false;        // no exemptions (dlb_ctx_set_guard_strict)
  std::map<uintptr_t, size_t> rows_exempt;  // plane buffers (address, bytes) of tensors whose small rows are not guarded
  // Bumped by dlb_ctx_set_gemm_kind, which also drops every registration above:
  // a model compares it with the value it last split its weights under and
  // splits them again in the new form.
  uint64_t plane_generation = 0;
  // TMA descriptors of the operands seen so far (the shapes of a model repeat
  // every step), keyed by everything cuTensorMapEncodeTiled is given.
  struct TmapKey {
    uintptr_t ptr;
    uint64_t mn, k, ld;
    uint32_t box_k, box_mn;
    int es, mn_major;
    bool operator<(const TmapKey &o) const {
      if (ptr != o.ptr) return ptr < o.ptr;
      if (mn != o.mn) return mn < o.mn;
      if (k != o.k) return k < o.k;
      if (ld != o.ld) return ld < o.ld;
      if (box_k != o.box_k) return box_k < o.box_k;
      if (box_mn != o.box_mn) return box_mn < o.box_mn;
      if (es != o.es) return es < o.es;
      return mn_major < o.mn_major;
    }
  };
  struct TmapBlob {
    alignas(64) unsigned char bytes[128];
  };
  std::map<TmapKey, TmapBlob> tmaps;
  float *scale_pool = nullptr;   // SCALE_SLOTS slots of SLOT_WORDS words (planes.cuh)
  // Range guard of the fp16 operand form: [0] operand tensors found unsafe for it,
  // [1] products that therefore ran on the fp32 CUDA-core kernel, [2] tensors
  // split again after outgrowing their predicted scale.
  unsigned long long *d_guard = nullptr;
  std::vector<int> scale_free;
  std::map<uintptr_t, size_t> allocs;  // dlb_malloc'd blocks, to retire plane entries on free
  // Exchange of small fp64 vectors through peer memory: every rank's buffer
  // mapped by every rank of the node (peer.cu).
  struct Peer {
    bool ready = false;
    void *local = nullptr;
    void *mapped[8] = {};   // by rank; mapped[rank] == local
    uint32_t seq = 0;       // exchanges so far, the same on every rank
  } peer;
  uint64_t launches = 0;
  // Programmatic dependent launch for the library's kernels (DLB_PDL=0 turns it off).
  bool use_pdl = true;
  cudaEvent_t timer_start = nullptr, timer_stop = nullptr;
  // Optional per-launch record of the tensor-core GEMM.
  struct GemmRecord {
    cudaEvent_t start, stop;
    double flops;
    int kind;  // 0: FC product, 1: wait of the main stream for the overlapped all-reduces, 2: exchange of sums
  };
  bool gemm_profile = false;
  std::vector<GemmRecord> gemm_records;
  std::vector<cudaEvent_t> event_pool;
  // Totals of the last dlb_ctx_gemm_profile_read for kinds 1 and 2.
  double join_wait_ms = 0.0, exchange_ms = 0.0;
  uint64_t join_waits = 0, exchanges = 0;
};

namespace dlb {

void set_error(const char *fmt, ...);

#define DLB_CUDA(call)                                                         \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) {                                                  \
      dlb::set_error("%s:%d %s: %s", __FILE__, __LINE__, #call,                \
                     cudaGetErrorString(e__));                                 \
      return DLB_ERR_CUDA;                                                     \
    }                                                                          \
  } while (0)

#define DLB_REQUIRE(cond, what)                                                \
  do {                                                                         \
    if (!(cond)) {                                                             \
      dlb::set_error("%s:%d invalid argument: %s", __FILE__, __LINE__, what);  \
      return DLB_ERR_INVALID;                                                  \
    }                                                                          \
  } while (0)

#define DLB_TRY(expr)                                                          \
  do {                                                                         \
    dlb_status s__ = (expr);                                                   \
    if (s__ != DLB_OK) return s__;                                             \
  } while (0)

// Every kernel of the library begins with pdl_enter(): it waits until the kernels
// before it in the stream have completed and their writes are visible
// (griddepcontrol.wait; nothing to wait for under an ordinary launch), then lets
// the kernel behind it be scheduled (griddepcontrol.launch_dependents).  Launched
// with programmatic stream serialization (DLB_LAUNCH_KERNEL), the blocks of the
// next kernel take the places the last blocks of this one leave, run up to their
// own wait and start the moment this kernel is complete: the launch latency and
// the ramp of the block scheduler, a few microseconds per kernel boundary,
// disappear from a step of sixty kernels.  The hardware dispatches all blocks of
// a grid before any block of the next, so a waiting block never takes a place a
// working block needs.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class... P, class... A>
inline cudaError_t launch_kernel(dlb_ctx *ctx, void (*kernel)(P...), dim3 grid, dim3 block, size_t smem,
                                 A &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
#define DLB_LAUNCH_KERNEL(ctx, kernel, grid, block, smem, ...) \
  dlb::launch_kernel((ctx), (kernel), dim3(grid), dim3(block), (size_t)(smem), __VA_ARGS__)
#endif

// After a kernel launch: count it and surface launch-configuration errors.
#define DLB_LAUNCHED(ctx)                                                      \
  do {                                                                         \
    (ctx)->launches++;                                                         \
    DLB_CUDA(cudaGetLastError());                                              \
  } while (0)

// Returns at least `bytes` of 256-byte aligned scratch, growing the arena if
// needed (growth synchronises the stream; steady state never grows).
dlb_status scratch(dlb_ctx *ctx, size_t bytes, void **out);

// Internal dropout code of the inference pass (dlb_dropout_desc.type): every
// activation times dlb_dropout_desc.value, the keep probability
// (Forward_Pass__Dropout__Bernoulli__Inference__OpenMP, fwp_mp.cpp L:4870-4892).
constexpr int DROPOUT_INFERENCE_SCALE = 100;

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// GEMM C[m,n] (+)= sum_k A(m,k) * B(n,k) with element strides; the three FC
// products are three stride assignments of this one contract.
struct GemmOperand {
  const float *ptr;     // fp32 values (what the tensor core sees truncated)
  const float *lo;      // TF32 residual plane or nullptr
  long long stride_mn;  // elements between consecutive m (or n)
  long long stride_k;   // elements between consecutive k
  // fp16 planes of s * x (hi = fp16(s x), lo = fp16(s x - hi)) with the strides
  // of the tensor, and the device scalar s (a power of two); when all three are
  // set the product runs on kind::f16 instead of kind::tf32.
  const uint16_t *h_hi = nullptr;
  const uint16_t *h_lo = nullptr;
  const float *scale = nullptr;
  // Word that is non-zero when the planes cannot stand for the tensor (range
  // guard, planes.cuh): the tensor-core kernel then computes the product from
  // the fp32 tensors on the CUDA cores instead.
  const unsigned *guard = nullptr;
  // Bits of that word this operand's use in the product cares about: overflow,
  // and the small lines along its free dimension.
  unsigned guard_mask = 7u;
  // Strides of `ptr` where they differ from the planes' (planes transposed into
  // scratch for the product); 0: the same.
  long long fp32_stride_mn = 0, fp32_stride_k = 0;
  // Planes with a scale of their own per mn line (k-contiguous planes made for
  // one product): 1 / scale of every line; `scale` is then not read.
  const float *line_inv = nullptr;
  // Asked by the caller: make such planes for this product (A of a weight
  // gradient whose columns differ widely in size, e.g. the classes of a softmax
  // error).  Also done where TMA cannot tile the operand as it lies.
  bool rescale_lines = false;
};
// Flag bits (planes.cuh) a product looks at for an operand with these strides
// whose planes belong to a row-major [rows, cols] tensor.
inline unsigned guard_mask_of(const GemmOperand &o) {
  if (o.stride_k == 1) return 1u | 2u;   // mn runs over the tensor's rows
  if (o.stride_mn == 1) return 1u | 4u;  // mn runs over its columns
  return 7u;
}
struct FusedEpilogue;
struct GemmEpilogue {
  const float *bias = nullptr;   // per-n bias added to every row
  float *colsum = nullptr;       // per-n sum over m of C (db), written/accumulated
  int accumulate = 0;            // C += result
  // Work of the kernel that would follow the product, done on the tile while the
  // drain warps hold it (2-CTA fp16-plane kernel only: ask gemm_fused_supported).
  const FusedEpilogue *fused = nullptr;
};

dlb_status gemm(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                long long ldc, int M, int N, int K, const GemmEpilogue &ep);
dlb_status gemm_simt(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                     long long ldc, int M, int N, int K, const GemmEpilogue &ep);
// Returns DLB_ERR_UNSUPPORTED (without touching C) when the shape or alignment
// is outside what the TMA descriptors can express.
dlb_status gemm_tcgen05(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, float *C,
                        long long ldc, int M, int N, int K, const GemmEpilogue &ep);
bool gemm_tcgen05_supported(const GemmOperand &A, const GemmOperand &B, const float *C,
                            long long ldc, int M, int N, int K);
bool gemm_f16_supported(const GemmOperand &A, const GemmOperand &B, const float *C, long long ldc,
                        int M, int N, int K);
// Peer-memory exchange (peer.cu) and the two communicator calls its set-up
// needs (ctx.cu): every rank's `bytes` gathered into recv[world][bytes] on the
// host, and the minimum of one int over the ranks.
constexpr int PEER_MAX = 8;          // ranks of one node
constexpr int PEER_CTAS = 32;        // blocks of one exchange
constexpr size_t PEER_CAP = 32768;   // doubles per exchanged vector
dlb_status peer_setup(dlb_ctx *ctx);
void peer_teardown(dlb_ctx *ctx);
bool peer_exchange_fits(dlb_ctx *ctx, size_t n);
dlb_status peer_exchange_f64(dlb_ctx *ctx, double *buf, size_t n);
dlb_status comm_allgather_host(dlb_ctx *ctx, const void *mine, void *all, size_t bytes);
dlb_status comm_min_int(dlb_ctx *ctx, int *value);

// Owner-computes update of a weight matrix across ranks (ctx.cu).  buf holds
// world * per_rank floats, rank r owns [r * per_rank, (r + 1) * per_rank).
// *_begin: the transfer starts on the second stream once the kernels enqueued
// so far are done; *done is recorded behind it (created on first use) and
// comm_wait makes the main stream wait for it.  comm_all_gather_begin also
// clears, behind the gather, the slices of `clear` this rank does not own.
// dlb_comm_join waits for everything still in flight.
bool comm_can_shard(dlb_ctx *ctx);
dlb_status comm_reduce_scatter_begin(dlb_ctx *ctx, float *buf, size_t per_rank, cudaEvent_t *done);
dlb_status comm_all_gather_begin(dlb_ctx *ctx, float *buf, size_t per_rank, float *clear, cudaEvent_t *done);
dlb_status comm_wait(dlb_ctx *ctx, cudaEvent_t done);
dlb_status comm_all_gather(dlb_ctx *ctx, float *buf, size_t per_rank);  // on the main stream, in order

// Fills o.h_hi / h_lo / scale / guard from the plane buffer registered for
// (o.ptr, aux), if there is one and the planes are 16-byte aligned.
bool planes_lookup(dlb_ctx *ctx, const float *aux, GemmOperand *o);
// Marks (or unmarks) the plane buffer [planes, planes + bytes) as that of an error tensor of
// the backward pass whose rows are the examples of a batch: the range guard
// then leaves its small rows alone (planes.cuh), unless the context is strict.
void planes_rows_exempt(dlb_ctx *ctx, const float *planes, size_t bytes, bool on);
// x [K, M] with row pitch `pitch` (mn contiguous) -> fp16 planes [M, kp] (k
// contiguous), line m scaled by a power of two of its own taken from the
// line's largest |x| (`cmax`, M words of scratch); line_inv[m] = 1 / scale.
dlb_status planes_transpose_scaled(dlb_ctx *ctx, const float *x, long long pitch, int K, int M, uint16_t *hi_t,
                                   uint16_t *lo_t, long long kp, unsigned *cmax, float *line_inv);
// Drops the plane buffers registered at addresses in [base, base + bytes).
void planes_forget(dlb_ctx *ctx, uintptr_t base, size_t bytes);

// What a kernel that produces a GEMM operand is handed to write the operand's
// fp16 planes and range statistics in the same pass (device side: planes.cuh).
struct PlaneSink {
  uint16_t *hi = nullptr, *lo = nullptr;   // null: the kernel writes no planes
  float *slot = nullptr;                   // scale slot; null: nothing to track
  unsigned *rowmax = nullptr, *colmax = nullptr;   // where the producer leaves row / column maxima (null: not wanted)
  unsigned *lines = nullptr;               // the array both live in: n_rows words, then the columns'
  int n_rows = 0;
  int n_lines = 0;                         // rows + cols (0: no line statistics)
  int predicted = 0;                       // planes use the scale predicted from the previous split
  unsigned long long *guard = nullptr;     // counter of tensors the range guard flagged
  int rows_exempt = 0;                     // small rows are not flagged (planes.cuh)
  const float *x = nullptr;                // the tensor the planes are of, n elements: read again
  size_t n = 0;                            //   when it outgrew its predicted scale
};
// Elementwise work fused into the store of a product C[M, N] (all tensors dense,
// row pitch N).
//   EPI_ACTIVATION: C receives the sums (+ bias), `out` = dropout(f(C)): the
//     forward of a layer without normalization (Forward_Pass__FC_AF__OpenMP and
//     the dropout forwards, v1/learner/fwp_mp.cpp L:4741-4770, L:4809-4985).
//   EPI_DERIVATIVE: C receives product * f'(z, a): the error of the layer below
//     a dX product when that layer has no normalization
//     (Backward_Pass__FC__DF__OpenMP, v1/learner/bwp_mp.cpp L:1150-1186).
// `sink`, when it has planes, receives the fp16 planes and range statistics of
// the produced operand (`out`, or C) in the same pass.
enum { EPI_PLAIN = 0, EPI_ACTIVATION = 1, EPI_DERIVATIVE = 2 };
struct FusedEpilogue {
  int mode = EPI_PLAIN;
  int af = 0;
  const uint8_t *mask = nullptr;  // EPI_ACTIVATION: Bernoulli flags per unit, or null
  float keep_scale = 1.f;         //   factor of a kept unit (1, or 1 / keep probability)
  const float *noise = nullptr;   //   UOut draws [M, N], or null
  float *out = nullptr;           //   the activation [M, N]
  const float *z = nullptr;       // EPI_DERIVATIVE: pre-activation and activation [M, N] of the
  const float *a = nullptr;       //   layer whose error C is
  PlaneSink sink;
};
// dlb_fc_weight_gradient with a say on the planes of the error: rescale_lines
// asks for planes with a scale per unit (per output row of dW), made for this
// product (gemm() in ctx.cu).
dlb_status fc_weight_gradient_lines(dlb_ctx *ctx, const float *delta, const float *delta_lo, const float *X,
                                    const float *X_lo, float *dW, float *dbias, int rows, int n_in, int n_out,
                                    int accumulate, bool rescale_lines);
bool gemm_pair_enabled();  // the 2-CTA kernel is on (DLB_GEMM_PAIR)
int gemm_pair_chunk();     // its chunk of k-blocks per accumulator drain
// Whether gemm() would run this product on the kernel that takes a fused epilogue.
bool gemm_fused_supported(dlb_ctx *ctx, const GemmOperand &A, const GemmOperand &B, const float *C, long long ldc,
                          int M, int N, int K);

// One split of a tensor into its plane buffer.  planes_open registers the
// buffer and decides the form: `fused` (the producing kernel writes planes and
// statistics itself, with the scale predicted from the buffer's previous split)
// when the kernel can and such a scale exists, else the kernel only tracks
// max |x| (sink.slot) and planes_close runs the split pass.  planes_close then
// launches the check that sets the slot's scale and guard flag for the
// consumers and the prediction for the next split (planes_finalize_kernel).
struct PlaneJob {
  PlaneSink sink;
  const float *x = nullptr;
  float *planes = nullptr;
  size_t n = 0;
  int rows = 0, cols = 0;
  bool fused = false, active = false;
};
dlb_status planes_open(dlb_ctx *ctx, const float *x, float *planes, size_t n, int rows, int cols,
                       bool kernel_can_fuse, PlaneJob *job);
dlb_status planes_close(dlb_ctx *ctx, const PlaneJob &job);
// max |x| of a tensor no kernel of the library produced (inputs, fresh weights).
dlb_status planes_absmax(dlb_ctx *ctx, const float *x, size_t n, float *slot);
// Split into caller storage outside the registry (scratch): planes, slot of
// SLOT_WORDS words and rows + cols words of line maxima, all zeroed here.
dlb_status planes_split_adhoc(dlb_ctx *ctx, const float *x, size_t n, int rows, int cols, uint16_t *hi,
                              uint16_t *lo, float *slot, unsigned *lines);
dlb_status optimizer_step_amax(dlb_ctx *ctx, int rule, const dlb_optimizer_scalars *s, float *p, float *g,
                               float *first, float *second, float *second_hat, const float *wd_mask, size_t n,
                               unsigned *amax);
dlb_status optimizer_step_sink(dlb_ctx *ctx, int rule, const dlb_optimizer_scalars *s, float *p, float *g,
                               float *first, float *second, float *second_hat, const float *wd_mask, int rows,
                               int cols, const PlaneSink &sink);
constexpr int SCALE_SLOTS = 8192;
constexpr int SLOT_WORDS = 8;    // words of one scale slot (layout: planes.cuh)
constexpr int MAX_DEVICES = 64;  // device indices a process may hold contexts on

}  // namespace dlb
