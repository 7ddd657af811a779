// Exchange of small fp64 vectors (the batch-renormalization sums of a layer,
// 2 x units doubles forward and backward) between the ranks of one node
// through peer memory instead of a library collective.
//
// Every rank owns one buffer that all ranks of the node map (CUDA IPC):
//
//   inbox [2][PEER_MAX][PEER_CAP] of 16 bytes   inbox[q][s][i]: element i of
//       rank s's vector in an exchange whose sequence number is q mod 2, as
//       two 8-byte words {low half of the double, seq} {high half, seq}
//
// One exchange is one kernel per rank.  A thread of rank r stores element i of
// r's vector, tagged with the exchange's sequence number, into inbox[seq & 1][r]
// of every rank (its own included); it then reads inbox[seq & 1][s][i] of its
// own buffer for s = 0 .. W-1, each until both words carry seq, and adds the W
// values in rank order, so that every rank forms the same sum bit for bit.
// An 8-byte store arrives whole, so a word that carries seq carries the data
// of seq: no fence, no separate flag and no second trip over the link.  A rank
// can run at most one exchange ahead of the slowest (it needs everybody's
// vector of exchange seq to finish seq), which is why two inbox halves are
// enough, and a thread waits for remote stores only, never for a block of its
// own grid, so the grid need not be co-resident.  Waits are bounded by the
// global timer; a wait that runs out sets the context's device status to
// DLB_ERR_TIMEOUT.
//
// The reference sums these statistics over its OpenMP threads
// (Forward_Pass__Batch_Renormalization__Training__OpenMP, fwp_mp.cpp
// L:4647-4663, and the backward sums of bwp_mp.cpp L:1520-1621); across GPUs
// the same sums cross NVLink.
#include <string.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "common.cuh"

namespace dlb {

namespace {

constexpr size_t PEER_BYTES = 2 * (size_t)PEER_MAX * PEER_CAP * sizeof(ulonglong2);
constexpr unsigned long long PEER_WAIT_NS = 20ull * 1000 * 1000 * 1000;  // 20 s

struct PeerView {
  char *base[PEER_MAX];
  int rank, world;
};

__device__ __forceinline__ ulonglong2 *inbox(char *base, int parity, int src) {
  return reinterpret_cast<ulonglong2 *>(base) + ((size_t)parity * PEER_MAX + src) * PEER_CAP;
}
__device__ __forceinline__ void store_words(ulonglong2 *p, ulonglong2 v) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(v.x), "l"(v.y) : "memory");
}
__device__ __forceinline__ ulonglong2 load_words(const ulonglong2 *p) {
  ulonglong2 v;
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// EMULATED: all ranks are rows of one grid (blockIdx.y = rank) over buffers of
// one device, launched cooperatively so that the rows are co-resident; this is
// how the protocol runs where there is one GPU.  Otherwise the rank is the
// process's and every other rank's kernel runs on a GPU of its own.
template <bool EMULATED>
__global__ void __launch_bounds__(256)
peer_exchange_f64_kernel(double *buf, double *const *bufs, int n, PeerView v, uint32_t seq,
                         unsigned long long wait_ns, int absent, int *status) {
  const int rank = EMULATED ? (int)blockIdx.y : v.rank;
  const int W = v.world;
  if (EMULATED) {
    if (rank == absent) return;  // a rank that never delivers: the others' waits run out
    buf = bufs[rank];
  }
  const int parity = (int)(seq & 1u);
  const int first = (int)(blockIdx.x * blockDim.x + threadIdx.x), step = (int)(gridDim.x * blockDim.x);
  const unsigned long long tag = (unsigned long long)seq << 32;

  for (int i = first; i < n; i += step) {
    const unsigned long long bits = (unsigned long long)__double_as_longlong(buf[i]);
    const ulonglong2 words = make_ulonglong2((bits & 0xffffffffull) | tag, (bits >> 32) | tag);
    for (int p = 0; p < W; ++p) store_words(inbox(v.base[p], parity, rank) + i, words);
  }

  const unsigned long long t0 = global_ns();
  bool gave_up = false;
  for (int i = first; i < n; i += step) {
    double sum = 0.0;
    for (int r = 0; r < W; ++r) {
      const ulonglong2 *src = inbox(v.base[rank], parity, r) + i;
      ulonglong2 w = load_words(src);
      for (unsigned spins = 0; (uint32_t)(w.x >> 32) != seq || (uint32_t)(w.y >> 32) != seq; ++spins) {
        if (gave_up || ((spins & 255u) == 255u && global_ns() - t0 > wait_ns)) {
          gave_up = true;
          break;
        }
        if (spins > 64) __nanosleep(100);
        w = load_words(src);
      }
      sum += __longlong_as_double((long long)((w.x & 0xffffffffull) | (w.y << 32)));
    }
    buf[i] = sum;
  }
  if (gave_up) atomicCAS(status, (int)DLB_OK, (int)DLB_ERR_TIMEOUT);
}

int exchange_blocks(size_t n) { return (int)std::min<size_t>(PEER_CTAS, (n + 255) / 256); }

// What a rank tells the others about itself when the communicator is set up.
struct PeerCard {
  cudaIpcMemHandle_t handle;
  char host[64];
  char bus[32];
  int wanted;
  int pad[3];
};

void peer_release(dlb_ctx *ctx) {
  for (int r = 0; r < PEER_MAX; ++r) {
    if (ctx->peer.mapped[r] && r != ctx->rank) cudaIpcCloseMemHandle(ctx->peer.mapped[r]);
    ctx->peer.mapped[r] = nullptr;
  }
  if (ctx->peer.local) cudaFree(ctx->peer.local);
  ctx->peer.local = nullptr;
  ctx->peer.ready = false;
  cudaGetLastError();
}

}  // namespace

void peer_teardown(dlb_ctx *ctx) { peer_release(ctx); }

// Called by every rank once the library communicator exists.  Leaves
// ctx->peer.ready false (the sums then go through the library all-reduce)
// unless every rank is on the same host, on a device of its own, asked for the
// exchange and could map every other rank's buffer; the ranks agree on that
// through the communicator, so that either all of them use the exchange or
// none does.
dlb_status peer_setup(dlb_ctx *ctx) {
  const int W = ctx->world, rank = ctx->rank;
  if (W < 2) return DLB_OK;
  PeerCard mine;
  memset(&mine, 0, sizeof(mine));
  const char *env = getenv("DLB_PEER_EXCHANGE");
  mine.wanted = (W <= PEER_MAX && !(env && atoi(env) == 0)) ? 1 : 0;
  gethostname(mine.host, sizeof(mine.host) - 1);
  DLB_CUDA(cudaDeviceGetPCIBusId(mine.bus, sizeof(mine.bus), ctx->device));
  if (mine.wanted) {
    if (cudaMalloc(&ctx->peer.local, PEER_BYTES) != cudaSuccess ||
        cudaMemset(ctx->peer.local, 0, PEER_BYTES) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&mine.handle, ctx->peer.local) != cudaSuccess) {
      cudaGetLastError();
      mine.wanted = 0;
    }
  }
  std::vector<PeerCard> cards((size_t)W);
  DLB_TRY(comm_allgather_host(ctx, &mine, cards.data(), sizeof(PeerCard)));
  int ok = 1;
  for (int r = 0; r < W && ok; ++r) {
    if (!cards[r].wanted || strncmp(cards[r].host, mine.host, sizeof(mine.host)) != 0) ok = 0;
    for (int q = 0; q < r && ok; ++q)
      if (strncmp(cards[r].bus, cards[q].bus, sizeof(mine.bus)) == 0) ok = 0;  // two ranks, one GPU
  }
  if (ok) {
    for (int r = 0; r < W && ok; ++r) {
      if (r == rank) {
        ctx->peer.mapped[r] = ctx->peer.local;
        continue;
      }
      if (cudaIpcOpenMemHandle(&ctx->peer.mapped[r], cards[r].handle, cudaIpcMemLazyEnablePeerAccess) !=
          cudaSuccess) {
        cudaGetLastError();
        ctx->peer.mapped[r] = nullptr;
        ok = 0;
      }
    }
  }
  int all_ok = ok;
  DLB_TRY(comm_min_int(ctx, &all_ok));
  if (!all_ok) {
    // Nobody uses the exchange.  The second round keeps a rank from unmapping
    // a buffer that another rank is still opening.
    int done = 1;
    DLB_TRY(comm_min_int(ctx, &done));
    peer_release(ctx);
    return DLB_OK;
  }
  ctx->peer.seq = 0;
  ctx->peer.ready = true;
  return DLB_OK;
}

bool peer_exchange_fits(dlb_ctx *ctx, size_t n) { return ctx->peer.ready && n > 0 && n <= PEER_CAP; }

dlb_status peer_exchange_f64(dlb_ctx *ctx, double *buf, size_t n) {
  PeerView v;
  for (int r = 0; r < PEER_MAX; ++r) v.base[r] = static_cast<char *>(ctx->peer.mapped[r]);
  v.rank = ctx->rank;
  v.world = ctx->world;
  const uint32_t seq = ++ctx->peer.seq;
  peer_exchange_f64_kernel<false><<<exchange_blocks(n), 256, 0, ctx->stream>>>(
      buf, nullptr, (int)n, v, seq, PEER_WAIT_NS, -1, ctx->d_status);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // namespace dlb

using namespace dlb;

extern "C" {

int dlb_comm_peer_exchange(dlb_ctx *ctx) { return ctx && ctx->peer.ready ? 1 : 0; }

// The exchange protocol with `world` emulated ranks on this one device: the
// ranks are the rows of one cooperative grid.  vectors: [world][n] on the
// host, in: each rank's vector, out: what each rank holds afterwards (every
// row the same sum).  `rounds` exchanges run back to back on the same
// buffers (round k exchanges the vectors scaled by k + 1), `absent` >= 0 names
// a rank whose row returns without delivering: the others then give up after
// wait_ms and the call returns DLB_ERR_TIMEOUT with the context still usable.
dlb_status dlb_peer_exchange_emulated(dlb_ctx *ctx, int world, size_t n, int rounds, const double *in,
                                      double *out, int absent, unsigned wait_ms) {
  DLB_REQUIRE(ctx && in && out && world >= 1 && world <= PEER_MAX && n > 0 && n <= PEER_CAP && rounds >= 1 &&
                  absent < world,
              "dlb_peer_exchange_emulated");
  DLB_CUDA(cudaSetDevice(ctx->device));
  const int blocks = exchange_blocks(n);
  int coop = 0, per_sm = 0;
  DLB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
  DLB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, peer_exchange_f64_kernel<true>, 256, 0));
  if (!coop || blocks * world > per_sm * ctx->sm_count) {
    set_error("dlb_peer_exchange_emulated: %d blocks cannot be co-resident on this device", blocks * world);
    return DLB_ERR_UNSUPPORTED;
  }
  std::vector<void *> owned;
  auto cleanup = [&]() {
    cudaStreamSynchronize(ctx->stream);
    for (void *p : owned) cudaFree(p);
  };
  auto alloc = [&](size_t bytes) -> void * {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
    owned.push_back(p);
    return p;
  };
  PeerView v;
  memset(&v, 0, sizeof(v));
  v.world = world;
  std::vector<double *> vec((size_t)world);
  for (int r = 0; r < world; ++r) {
    v.base[r] = static_cast<char *>(alloc(PEER_BYTES));
    vec[r] = static_cast<double *>(alloc(n * sizeof(double)));
    if (!v.base[r] || !vec[r]) {
      cleanup();
      set_error("dlb_peer_exchange_emulated: out of device memory");
      return DLB_ERR_CUDA;
    }
    cudaMemsetAsync(v.base[r], 0, PEER_BYTES, ctx->stream);
  }
  double **table = static_cast<double **>(alloc(world * sizeof(double *)));
  if (!table) {
    cleanup();
    return DLB_ERR_CUDA;
  }
  cudaMemcpyAsync(table, vec.data(), world * sizeof(double *), cudaMemcpyHostToDevice, ctx->stream);
  std::vector<double> scaled(n);
  dlb_status result = DLB_OK;
  for (int k = 0; k < rounds && result == DLB_OK; ++k) {
    for (int r = 0; r < world; ++r) {
      for (size_t i = 0; i < n; ++i) scaled[i] = in[(size_t)r * n + i] * (double)(k + 1);
      cudaMemcpyAsync(vec[r], scaled.data(), n * sizeof(double), cudaMemcpyHostToDevice, ctx->stream);
      cudaStreamSynchronize(ctx->stream);
    }
    uint32_t seq = (uint32_t)(k + 1);
    int nn = (int)n;
    double *none = nullptr;
    double *const *tbl = table;
    unsigned long long wait_ns = (unsigned long long)wait_ms * 1000000ull;
    int *status = ctx->d_status;
    void *args[] = {&none, &tbl, &nn, &v, &seq, &wait_ns, &absent, &status};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(peer_exchange_f64_kernel<true>),
                                                dim3(blocks, world), dim3(256), args, 0, ctx->stream);
    if (e != cudaSuccess) {
      set_error("dlb_peer_exchange_emulated: %s", cudaGetErrorString(e));
      result = DLB_ERR_CUDA;
      break;
    }
    ctx->launches++;
    int st = 0;
    cudaMemcpyAsync(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
      set_error("dlb_peer_exchange_emulated: %s", cudaGetErrorString(cudaGetLastError()));
      result = DLB_ERR_CUDA;
      break;
    }
    if (st != DLB_OK) {
      // Report and clear: the context stays usable.
      cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
      set_error("dlb_peer_exchange_emulated: a rank gave up waiting (device status %d)", st);
      result = (dlb_status)st;
      break;
    }
    if (k == rounds - 1)
      for (int r = 0; r < world; ++r)
        cudaMemcpyAsync(out + (size_t)r * n, vec[r], n * sizeof(double), cudaMemcpyDeviceToHost, ctx->stream);
  }
  cleanup();
  return result;
}

}  // extern "C"
