// LSTM layer (memory blocks of cells with peephole connections), the part that is
// not a matrix product.
//
// ref: Forward_Pass__LSTM__Gates_CIF_AF_State__OpenMP, ..__Output__OpenMP,
// ..__States_AF__OpenMP (v1/learner/fwp_rec_mp.cpp L:985-1526);
// Backward_Pass__LSTM_Derivative__Output / __Cell_State_AF /
// __Gates_CIF_AF_State__OpenMP (v1/learner/bwp_rec_mp.cpp L:1112-1582);
// the peephole part of Recurrent__Update_Derivative_Weight__LSTM__OpenMP
// (v1/learner/update_derivative_rec_mp.cpp L:489-726).
//
// The reference keeps a block's parameters together: per cell [W_z | R_z], then
// W_i, W_f, W_o, R_i, R_f, R_o, p_i, p_f, p_o (connections_prepare.cpp L:83-225),
// rows of two different lengths in one range.  The products need matrices, so
// the layer works on packed copies: Wff [G, I] and Wrec [G, C] with G = C + 3 B
// rows in the order {z of every cell, i, f, o of every block}, gathered from the
// parameter vector before the forward pass and scattered back (added) into the
// gradient vector after the weight gradients.  The gates' sums of a time step
// are one row of G values in that order; so are the gates' errors.
#include "common.cuh"

namespace dlb {

__device__ __forceinline__ float sigmoid_ref(float x) { return 1.f / (1.f + expf(-x)); }
// The reference's tanh: 2 / (1 + exp(-2 x)) - 1 (v1/ops/activations/functions.hpp L:44).
__device__ __forceinline__ float tanh_ref(float x) { return 2.f / (1.f + expf(-2.f * x)) - 1.f; }

// dst[r, :] = src[offset[r] ...], rows of `width` floats.
__global__ void gather_rows_kernel(const float *__restrict__ src, const unsigned long long *__restrict__ offset,
                                   float *__restrict__ dst, size_t rows, int width) {
  pdl_enter();
  const size_t total = rows * (size_t)width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = src[offset[i / width] + i % width];
}

// dst[offset[r] + j] += src[r, j].  Offsets may repeat (the reference's bias
// indices alias): atomics keep every contribution.
__global__ void scatter_add_rows_kernel(const float *__restrict__ src, const unsigned long long *__restrict__ offset,
                                        float *__restrict__ dst, size_t rows, int width) {
  pdl_enter();
  const size_t total = rows * (size_t)width;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    atomicAdd(dst + offset[i / width] + i % width, src[i]);
}

struct LstmStep {
  // sums of this time step, rows of G = C + 3 B values {z | i | f | o}
  const float *g_in;   // W x_t
  const float *g_rec;  // R h_{t-1}, null at t = 0
  const float *bias;   // [G]
  const float *peep;   // [3, C]: p_i, p_f, p_o per cell
  const float *c_prev; // [rows, C], null at t = 0
  float *z, *c, *ca, *h;   // [rows, C]
  float *gi, *gf, *go;     // [rows, B]
};

// One thread per (row, block).
__global__ void lstm_forward_kernel(LstmStep s, int rows, int B, int K) {
  pdl_enter();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * B) return;
  const int n = idx / B, b = idx % B;
  const int C = B * K, G = C + 3 * B;
  const float *gin = s.g_in + (size_t)n * G, *grec = s.g_rec ? s.g_rec + (size_t)n * G : nullptr;
  const size_t cell0 = (size_t)n * C + (size_t)b * K;
  const float *pi = s.peep + b * K, *pf = s.peep + C + b * K, *po = s.peep + 2 * C + b * K;
  // Gates: input + recurrent + bias, then the peepholes in cell order
  // (fwp_rec_mp.cpp L:1041-1062).
  float si = gin[C + b] + (grec ? grec[C + b] : 0.f) + s.bias[C + b];
  float sf = 0.f;
  if (s.c_prev) {
    sf = gin[C + B + b] + grec[C + B + b] + s.bias[C + B + b];
    for (int k = 0; k < K; ++k) {
      const float cp = s.c_prev[cell0 + k];
      si += cp * pi[k];
      sf += cp * pf[k];
    }
  }
  const float i_gate = sigmoid_ref(si);
  const float f_gate = s.c_prev ? sigmoid_ref(sf) : 0.f;
  s.gi[(size_t)n * B + b] = i_gate;
  s.gf[(size_t)n * B + b] = f_gate;
  float so = gin[C + 2 * B + b] + (grec ? grec[C + 2 * B + b] : 0.f) + s.bias[C + 2 * B + b];
  for (int k = 0; k < K; ++k) {
    const int cc = b * K + k;
    const float sz = gin[cc] + (grec ? grec[cc] : 0.f) + s.bias[cc];
    const float z = tanh_ref(sz);
    float c = z * i_gate;
    if (s.c_prev) c += s.c_prev[cell0 + k] * f_gate;
    s.z[cell0 + k] = z;
    s.c[cell0 + k] = c;
    s.ca[cell0 + k] = tanh_ref(c);
    so += c * po[k];   // peephole from the new state (L:1330-1336)
  }
  const float o_gate = sigmoid_ref(so);
  s.go[(size_t)n * B + b] = o_gate;
  for (int k = 0; k < K; ++k) s.h[cell0 + k] = s.ca[cell0 + k] * o_gate;
}

struct LstmBackStep {
  const float *dH;      // [rows, C] error of the outputs of this time step (recurrent part included)
  const float *z, *ca, *gi, *gf, *go;   // this time step (gf unused at t = 0)
  const float *c_prev;  // c_{t-1}, null at t = 0
  const float *gf_next; // f_{t+1}, null at the last time step
  const float *dC_next; // [rows, C]
  const float *d_next;  // gates' errors of t + 1, rows of G values; null at the last time step
  const float *peep;
  float *dC;            // [rows, C]
  float *d;             // gates' errors of this time step, rows of G values {dz | di | df | do}
};

__global__ void lstm_backward_kernel(LstmBackStep s, int rows, int B, int K) {
  pdl_enter();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * B) return;
  const int n = idx / B, b = idx % B;
  const int C = B * K, G = C + 3 * B;
  const size_t cell0 = (size_t)n * C + (size_t)b * K;
  const float *pi = s.peep + b * K, *pf = s.peep + C + b * K, *po = s.peep + 2 * C + b * K;
  float *d = s.d + (size_t)n * G;
  const float o_gate = s.go[(size_t)n * B + b], i_gate = s.gi[(size_t)n * B + b];
  // Output gate: sigm'(o) * sum_k dH tanh(c) (bwp_rec_mp.cpp L:1199-1212).
  float eo = 0.f;
  for (int k = 0; k < K; ++k) eo += s.dH[cell0 + k] * s.ca[cell0 + k];
  const float d_o = o_gate * (1.f - o_gate) * eo;
  d[C + 2 * B + b] = d_o;
  const bool last = s.d_next == nullptr;
  const float di_next = last ? 0.f : s.d_next[(size_t)n * G + C + b];
  const float df_next = last ? 0.f : s.d_next[(size_t)n * G + C + B + b];
  const float f_next = last ? 0.f : s.gf_next[(size_t)n * B + b];
  float ei = 0.f, ef = 0.f;
  for (int k = 0; k < K; ++k) {
    const float ca = s.ca[cell0 + k], z = s.z[cell0 + k];
    // Cell state: through the output, the three peepholes and the next state
    // (L:1257-1309, L:1372-1384).
    float e = s.dH[cell0 + k] * o_gate * (1.f - ca * ca);
    e += po[k] * d_o;
    if (!last) {
      e += pi[k] * di_next;
      e += pf[k] * df_next;
      e += s.dC_next[cell0 + k] * f_next;
    }
    s.dC[cell0 + k] = e;
    d[b * K + k] = e * i_gate * (1.f - z * z);
    ei += e * z;
    if (s.c_prev) ef += e * s.c_prev[cell0 + k];
  }
  d[C + b] = ei * i_gate * (1.f - i_gate);
  // No forget gate at t = 0 (L:1440-1500).
  float d_f = 0.f;
  if (s.c_prev) {
    const float f = s.gf[(size_t)n * B + b];
    d_f = ef * f * (1.f - f);
  }
  d[C + B + b] = d_f;
}

// Peephole gradients, one block per cell: dp_o[c] = sum_{t, n} do_t c_t,
// dp_i[c] = sum_{t < T - 1, n} di_{t+1} c_t, dp_f likewise
// (update_derivative_rec_mp.cpp L:596-612, L:655-660).  Sums in double, a fixed
// tree over the block's threads.
__global__ void __launch_bounds__(256)
    lstm_peephole_grad_kernel(const float *__restrict__ d, const float *__restrict__ c, float *__restrict__ out,
                              int T, int rows, int B, int K) {
  pdl_enter();
  __shared__ double red[3][256];
  const int cell = blockIdx.x, b = cell / K;
  const int C = B * K, G = C + 3 * B;
  double si = 0.0, sf = 0.0, so = 0.0;
  const size_t total = (size_t)T * rows;
  for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
    const size_t t = i / rows;
    const double cv = c[i * C + cell];
    so += (double)d[i * G + C + 2 * B + b] * cv;
    if (t + 1 < (size_t)T) {
      const size_t nx = i + rows;   // the same example one time step later
      si += (double)d[nx * G + C + b] * cv;
      sf += (double)d[nx * G + C + B + b] * cv;
    }
  }
  red[0][threadIdx.x] = si;
  red[1][threadIdx.x] = sf;
  red[2][threadIdx.x] = so;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w)
      for (int j = 0; j < 3; ++j) red[j][threadIdx.x] += red[j][threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x < 3) out[threadIdx.x * C + cell] = (float)red[threadIdx.x][0];
}

static int flat_grid(dlb_ctx *ctx, size_t items) {
  return (int)std::max<size_t>(1, std::min<size_t>((items + 255) / 256, (size_t)ctx->sm_count * 8));
}

}  // namespace dlb

using namespace dlb;

extern "C" {

dlb_status dlb_gather_rows(dlb_ctx *ctx, const float *src, const unsigned long long *offsets, float *dst,
                           size_t rows, int width) {
  DLB_REQUIRE(ctx && src && offsets && dst && rows > 0 && width > 0, "dlb_gather_rows");
  DLB_LAUNCH_KERNEL(ctx, gather_rows_kernel, flat_grid(ctx, rows * width), 256, 0, src, offsets, dst, rows, width);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_scatter_add_rows(dlb_ctx *ctx, const float *src, const unsigned long long *offsets, float *dst,
                                size_t rows, int width) {
  DLB_REQUIRE(ctx && src && offsets && dst && rows > 0 && width > 0, "dlb_scatter_add_rows");
  DLB_LAUNCH_KERNEL(ctx, scatter_add_rows_kernel, flat_grid(ctx, rows * width), 256, 0, src, offsets, dst, rows, width);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_lstm_forward_step(dlb_ctx *ctx, const float *g_in, const float *g_rec, const float *bias,
                                 const float *peep, const float *c_prev, float *z, float *c, float *ca, float *h,
                                 float *gi, float *gf, float *go, int rows, int blocks, int cells) {
  DLB_REQUIRE(ctx && g_in && bias && peep && z && c && ca && h && gi && gf && go && rows > 0 && blocks > 0 && cells > 0,
              "dlb_lstm_forward_step");
  DLB_REQUIRE((g_rec == nullptr) == (c_prev == nullptr),
              "dlb_lstm_forward_step: the first time step has neither recurrent sums nor a previous state");
  LstmStep s{g_in, g_rec, bias, peep, c_prev, z, c, ca, h, gi, gf, go};
  DLB_LAUNCH_KERNEL(ctx, lstm_forward_kernel, ceil_div(rows * blocks, 128), 128, 0, s, rows, blocks, cells);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_lstm_backward_step(dlb_ctx *ctx, const float *dH, const float *z, const float *ca, const float *gi,
                                  const float *gf, const float *go, const float *c_prev, const float *gf_next,
                                  const float *dC_next, const float *d_next, const float *peep, float *dC, float *d,
                                  int rows, int blocks, int cells) {
  DLB_REQUIRE(ctx && dH && z && ca && gi && go && peep && dC && d && rows > 0 && blocks > 0 && cells > 0,
              "dlb_lstm_backward_step");
  DLB_REQUIRE((d_next == nullptr) == (dC_next == nullptr) && (d_next == nullptr) == (gf_next == nullptr),
              "dlb_lstm_backward_step: the last time step has nothing after it");
  DLB_REQUIRE(!c_prev || gf, "dlb_lstm_backward_step: forget gate of this time step");
  LstmBackStep s{dH, z, ca, gi, gf, go, c_prev, gf_next, dC_next, d_next, peep, dC, d};
  DLB_LAUNCH_KERNEL(ctx, lstm_backward_kernel, ceil_div(rows * blocks, 128), 128, 0, s, rows, blocks, cells);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

dlb_status dlb_lstm_peephole_gradient(dlb_ctx *ctx, const float *d, const float *c, float *out, int seq_w, int rows,
                                      int blocks, int cells) {
  DLB_REQUIRE(ctx && d && c && out && seq_w > 0 && rows > 0 && blocks > 0 && cells > 0, "dlb_lstm_peephole_gradient");
  DLB_LAUNCH_KERNEL(ctx, lstm_peephole_grad_kernel, blocks * cells, 256, 0, d, c, out, seq_w, rows, blocks, cells);
  DLB_LAUNCHED(ctx);
  return DLB_OK;
}

}  // extern "C"
